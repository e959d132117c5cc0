"""The grouped GEMM's tile lists, walked on the CPU: `tests/tile_math_host.cu` includes the kernels' own header
(`csrc/gemm_tiles.cuh`) and calls the same `decode_tile` / `total_tiles` the device code runs, over random expert row
counts, window sizes and both K steps.  It checks that the rows form produces every output tile exactly once inside
one expert's range, and that the weight-gradient form's K ranges over all windows cover each expert's occupied rows
once, in schedule order, with the accumulate flag set exactly where an earlier window held the expert's first rows."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_tile_lists_cover_every_row_once(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("needs nvcc to build the host harness")
    exe = str(tmp_path / "tile_math_host")
    build = subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "--expt-relaxed-constexpr", "-O1",
                            "-o", exe, os.path.join(ROOT, "tests", "tile_math_host.cu")], capture_output=True, text=True, timeout=600)
    assert build.returncode == 0, build.stderr[-3000:]
    run = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0 and run.stdout.startswith("ok"), run.stdout[-2000:] + run.stderr[-2000:]
