"""Multi-GPU parity of the row-sharded (fused peer-store exchange and NCCL all-to-all),
table-sharded and replica embedding steps.
Runs tests/sharded_worker.py under torchrun on 2 (or up to 4) GPUs; skipped on one GPU.
ANNC_TEST_WORLD=8 lifts the cap to eight ranks on a box that has them."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
import torch
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("mode", ["row", "row_hot", "row_whole", "row_nccl", "table", "table_nccl", "replica"])
def test_sharded_pipeline_matches_oracle(mode):
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    n = min(n, int(os.environ.get("ANNC_TEST_WORLD", "4")))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29531",
           os.path.join(ROOT, "tests", "sharded_worker.py"), mode]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
