"""GPU parity of the MXFP8 kernels through the C ABI: the block-scaled grouped GEMM forms against fp32 math on the
DEQUANTIZED operands (the exact value the tensor core is asked to compute; bound rel-L2 <= 1e-2, observed ~2e-3
from the bf16 output rounding), and against the unquantized product within the format's noise (rel-L2 <= 6e-2)."""
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import mok  # noqa: F401
    return torch.device("cuda", 0)


def _rel_l2(ref, got):
    ref, got = ref.double(), got.double()
    return ((ref - got).norm() / ref.norm().clamp_min(1e-30)).item()


def _quant(x):
    q, sc = O.mxfp8_quantize_rows_oracle(x)
    return q, sc, O.mxfp8_dequantize_oracle(q, sc)


@pytest.mark.parametrize("counts,N,K", [
    (None, 256, 128),                 # one tile, one K step
    (None, 256, 512),
    ([256, 512, 0, 256], 512, 384),   # uneven experts, an empty one
    ([1024, 256], 768, 1024),
])
def test_mxfp8_grouped_gemm(dev, counts, N, K):
    from mok import _native as nat
    g = torch.Generator().manual_seed(21)
    rows = 256 if counts is None else sum(counts)
    E = 1 if counts is None else len(counts)
    A = (torch.randn(rows, K, generator=g) * 0.7).to(torch.bfloat16)
    B = (torch.randn(E, N, K, generator=g) * 0.1).to(torch.bfloat16)
    Aq, Asc, Adq = _quant(A)
    Bq, Bsc, Bdq = _quant(B)
    D = torch.full((rows, N), float("nan"), device=dev, dtype=torch.bfloat16)
    tpe = None if counts is None else torch.tensor(counts, dtype=torch.int32, device=dev)
    nt = None if counts is None else torch.tensor([rows], dtype=torch.int32, device=dev)
    dA, dAs, dB, dBs = Aq.to(dev), Asc.to(dev), Bq.to(dev), Bsc.to(dev)
    nat.check(nat.lib().mok_grouped_gemm_mxfp8(nat.ptr(dA), nat.ptr(dAs), nat.ptr(dB), nat.ptr(dBs), nat.ptr(D), nat.ptr(tpe),
                                               nat.ptr(nt), E, rows, N, K, nat.ptr(nat.status_word(dev)), nat.stream_ptr(dev)),
              "grouped_gemm_mxfp8")
    torch.cuda.synchronize()
    nat.check_status(dev)
    ref = torch.empty(rows, N)
    plain = torch.empty(rows, N)
    off = 0
    for e, n in enumerate([rows] if counts is None else counts):
        ref[off:off + n] = Adq[off:off + n] @ Bdq[e].T
        plain[off:off + n] = A[off:off + n].float() @ B[e].float().T
        off += n
    got = D.float().cpu()
    assert not torch.isnan(got).any(), "unwritten output tile"
    assert _rel_l2(ref, got) <= 1e-2, f"vs dequantized operands: {_rel_l2(ref, got):.3e}"
    assert _rel_l2(plain, got) <= 6e-2, f"vs unquantized operands: {_rel_l2(plain, got):.3e}"


@pytest.mark.parametrize("counts,M,N", [(None, 256, 256), ([256, 0, 768], 256, 512), ([512, 512], 512, 256)])
def test_mxfp8_grouped_wgrad(dev, counts, M, N):
    from mok import _native as nat
    g = torch.Generator().manual_seed(23)
    rows = 512 if counts is None else sum(counts)
    E = 1 if counts is None else len(counts)
    A = (torch.randn(rows, M, generator=g) * 0.3).to(torch.bfloat16)
    B = (torch.randn(rows, N, generator=g) * 0.3).to(torch.bfloat16)
    Atq, Atsc, Atdq = _quant(A.T.contiguous())     # [M, rows], scales along the rows of the schedule
    Btq, Btsc, Btdq = _quant(B.T.contiguous())
    D = torch.full((E, M, N), float("nan"), device=dev, dtype=torch.bfloat16)
    tpe = None if counts is None else torch.tensor(counts, dtype=torch.int32, device=dev)
    nt = None if counts is None else torch.tensor([rows], dtype=torch.int32, device=dev)
    dA, dAs, dB, dBs = Atq.to(dev), Atsc.to(dev), Btq.to(dev), Btsc.to(dev)
    nat.check(nat.lib().mok_grouped_wgrad_mxfp8(nat.ptr(dA), nat.ptr(dAs), nat.ptr(dB), nat.ptr(dBs), nat.ptr(D), nat.ptr(tpe),
                                                nat.ptr(nt), E, rows, M, N, nat.ptr(nat.status_word(dev)), nat.stream_ptr(dev)),
              "grouped_wgrad_mxfp8")
    torch.cuda.synchronize()
    nat.check_status(dev)
    off = 0
    for e, n in enumerate([rows] if counts is None else counts):
        if n == 0:
            assert torch.isnan(D[e].float()).all()
            continue
        ref = Atdq[:, off:off + n] @ Btdq[:, off:off + n].T
        err = _rel_l2(ref, D[e].float().cpu())
        assert err <= 1e-2, f"expert {e}: {err:.3e}"
        off += n
