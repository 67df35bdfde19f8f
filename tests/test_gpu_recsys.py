"""Parity of the large row-sharded recsys step (hashed tables, mean pooling, BF16 MLP) on 1 rank
and, where the box has them, 2 ranks: tests/recsys_worker.py under torchrun."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("shard", ["row", "row_hot", "table"])
@pytest.mark.parametrize("ranks", [1, 2])
def test_recsys_pipeline_matches_oracle(ranks, shard):
    if torch.cuda.device_count() < ranks:
        pytest.skip("needs %d GPUs" % ranks)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={ranks}",
           "--master-addr", "127.0.0.1", "--master-port", "29537",
           os.path.join(ROOT, "tests", "recsys_worker.py"), shard]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
