"""Worker run under torchrun by test_gpu_recsys.py: builds the row-sharded recsys pipeline on
this rank's GPU (hashed tables filled on the device, mean pooling, BF16 MLP) and checks it
against the CPU oracle on this rank's own batch.  Exit code 0 = parity.
Bounds: table rows bit-exact; pooled means (stored as bf16) within one bf16 rounding step of
the fp32 oracle; predictions within 1e-2 (BF16 GEMM bound) of the fp32 MLP."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from annc_b200 import synth  # noqa: E402
from annc_b200.recsys import RecsysPipeline  # noqa: E402
from oracle import oracle  # noqa: E402


def main():
    shard = sys.argv[1] if len(sys.argv) > 1 else "row"
    rank, local = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    world = int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    model = synth.recsys_model(seed=3, tables=5, rows=50_001, dim=128, batch=512, max_bag=50,
                               zipf_a=1.2, hidden=(256, 128, 1), input_seed=200 + rank, threads=2)
    hot = 0
    if shard == "row_hot":  # row sharding with the rows of each table's 100 most popular ids replicated
        shard, hot = "row", 100
    pipe = RecsysPipeline(model, dev, shard=shard, hot_rows=hot)
    got = pipe.forward().cpu().numpy()
    assert pipe.embed_error_bits() == 0
    again = pipe.forward().cpu().numpy()  # second receive buffer
    assert np.array_equal(got, again)
    T, R, D, B = model.tables, model.rows, model.dim, model.batch
    # 1. the device-filled shard equals the numpy restatement of the hash
    probe = np.array([0, 1, 7, pipe.local_rows - 1])
    if shard == "row":
        for t in (0, T - 1):
            want_rows = synth.hashed_table_rows(model.seed, t, rank + world * probe, D)
            np.testing.assert_array_equal(pipe.table_mem[t][torch.from_numpy(probe).to(dev)].cpu().numpy(), want_rows)
    else:
        for j, t in enumerate(pipe.owned):
            want_rows = synth.hashed_table_rows(model.seed, t, probe, D)
            np.testing.assert_array_equal(pipe.table_mem[j][torch.from_numpy(probe).to(dev)].cpu().numpy(), want_rows)
    # 2. pooled means
    pooled = np.zeros((B, T, D), np.float32)
    for t, bag in enumerate(model.bags):
        bucket = (bag.raw_ids.view(np.uint64) % np.uint64(R)).astype(np.int64)
        uniq, inv = np.unique(bucket, return_inverse=True)
        data = synth.hashed_table_rows(model.seed, t, uniq, D)
        want, _ = oracle.sparse_segment_reduce(data, inv.astype(np.int64), bag.slice_input,
                                               np.array([0, 0], np.int32), np.array([0], np.int32), 1)
        pooled[:want.shape[0], t, :] = want
    x0 = pipe.x0.float().cpu().numpy().reshape(B, T, D)
    assert np.abs(x0 - pooled).max() <= 2.0 ** -8 * np.abs(pooled).max() + 1e-7
    # 3. predictions against the fp32 MLP
    x = pooled.reshape(B, T * D)
    for i, (w, b) in enumerate(model.mlp):
        x = oracle.matmul(x, w) + b
        x = 1 / (1 + np.exp(-x)) if i == len(model.mlp) - 1 else np.maximum(x, 0)
    err = float(np.abs(got - x).max())
    assert err <= 1e-2, err
    assert pipe.kernel_names[0] == "tcgen05_pair_bf16", pipe.kernel_names
    dist.barrier()
    pipe.close()
    dist.destroy_process_group()
    print(f"rank {rank} recsys {shard} ok err {err:.2e}")


if __name__ == "__main__":
    main()
