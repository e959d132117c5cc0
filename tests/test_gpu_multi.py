"""Expert parallelism over several GPUs of one node: spawns one process per GPU (EP = 2, and 4 / 8 when the box
has them) and checks schedule, outputs and gradients of every rank against the CPU oracle (see multi_gpu_worker.py)."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_parallel_layer_matches_oracle(world):
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    import multi_gpu_worker
    mp.spawn(multi_gpu_worker.run, args=(world, 29600 + world), nprocs=world, join=True)
