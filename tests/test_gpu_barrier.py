"""The cross-GPU barrier (`mok_barrier_all`, called through the C ABI) on one GPU: the counter arithmetic the
reference pins (tests/test_misc.py:1730-1771: after two calls target == buffer == 2 * ep_size) and the bounded wait.
The wait is made to run out the harmless way: with ep_size = 2 the second "peer" counter is another local word, so
the polled counter only ever receives this rank's own +1 and can never reach the target; the kernel gives up after
`timeout_ms`, sets the status bit and returns.  Nothing faults, traps or spins for ever."""
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import mok  # noqa: F401
    return torch.device("cuda", 0)


def _barrier(dev, counter, peers, target, timeout_ms):
    from mok import _native as nat
    nat.check(nat.lib().mok_barrier_all(nat.ptr(counter), nat.ptr_array([int(p.data_ptr()) for p in peers]), len(peers),
                                        nat.ptr(target), nat.ptr(nat.status_word(dev)), timeout_ms, nat.stream_ptr(dev)),
              "barrier_all")


def test_barrier_counter_known_answer(dev):
    """Both peer addresses name the local counter, so every call delivers ep_size arrivals to it: after two calls the
    target and the counter both read 2 * ep_size and no wait ran out."""
    from mok import _native as nat
    for ep in (2, 4, 8):
        counter = torch.zeros(1, dtype=torch.int32, device=dev)
        target = torch.zeros(1, dtype=torch.int32, device=dev)
        for _ in range(2):
            _barrier(dev, counter, [counter] * ep, target, 1000)
        torch.cuda.synchronize()
        assert int(target.item()) == 2 * ep and int(counter.item()) == 2 * ep
        nat.check_status(dev)


def test_barrier_wait_runs_out_and_reports(dev):
    from mok import _native as nat
    counter = torch.zeros(1, dtype=torch.int32, device=dev)
    elsewhere = torch.zeros(1, dtype=torch.int32, device=dev)    # stands in for a peer that never arrives here
    target = torch.zeros(1, dtype=torch.int32, device=dev)
    t0 = time.time()
    _barrier(dev, counter, [counter, elsewhere], target, 50)
    torch.cuda.synchronize()                                      # the kernel returned by itself
    assert time.time() - t0 < 10.0
    assert int(target.item()) == 2 and int(counter.item()) == 1 and int(elsewhere.item()) == 1
    with pytest.raises(RuntimeError, match="barrier wait ran out"):
        nat.check_status(dev)
    nat.check_status(dev)                                         # the word was reset by the failed check
    # the context is intact: a barrier whose arrivals do come completes and leaves the status clean
    counter.zero_()
    target.zero_()
    _barrier(dev, counter, [counter, counter], target, 1000)
    torch.cuda.synchronize()
    assert int(counter.item()) == 2
    nat.check_status(dev)
