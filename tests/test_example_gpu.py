"""The runnable copy of the reference's example script (examples/example.py), launched as a user
would: at its own size (M = 7680, K = N = 8192) on one rank, and as the 960-row shard that each of 8
ranks gets there (not a multiple of the 128-row tile: the edge the reference kernel leaves unguarded,
distributed-kernels/bf16_gemm/kernel.cpp:76-77)."""
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def _run(*extra):
    r = subprocess.run([sys.executable, str(ROOT / "examples" / "example.py"), *extra], capture_output=True,
                       text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "PASSED" in r.stdout
    return r.stdout


def test_example_at_its_own_size_one_rank():
    out = _run()
    assert "7680x8192 @ 8192x8192" in out


@pytest.mark.parametrize("rank", [0, 7])
def test_example_shard_of_eight_ranks(rank):
    out = _run("--as-rank", str(rank), "--of", "8")
    assert "960 rows" in out and f"Rank {rank}:" in out


def test_reference_bench_shapes_run():
    sys.path.insert(0, str(ROOT / "examples"))
    import bench_gemm
    rows = bench_gemm.run(iters=3)
    assert len(rows) == 8 and all(r["tflops"] > 0 for r in rows)
