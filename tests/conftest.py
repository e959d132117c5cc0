"""Shared pytest configuration: the `gpu` marker, import paths, and small helpers."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "mixture-of-kittens_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (sm_100a)")


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")


@pytest.fixture(scope="session")
def dist_ctx():
    """(rank, world_size, device) with an NCCL process group; world_size 1 unless launched by torchrun."""
    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if not dist.is_initialized():
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    yield rank, world, device
    import mok
    mok.functional.clear_workspace_cache()
    if dist.is_initialized():
        dist.destroy_process_group()
