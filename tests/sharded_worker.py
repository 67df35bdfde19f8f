"""Worker run under torchrun by test_gpu_sharded.py: builds the sharded DLRM pipeline in the
given mode on this rank's GPU and checks its predictions and pooled vectors against the CPU
oracle evaluated on this rank's own batch.  Exit code 0 = parity."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from annc_b200 import synth  # noqa: E402
from annc_b200.sharded import ShardedDlrmPipeline  # noqa: E402
from oracle import oracle  # noqa: E402


def main():
    mode = sys.argv[1]
    rank, local = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    model = synth.dlrm_model(seed=5, batch=2048, tables=7, max_rows=2e5, input_seed=100 + rank)
    # "row_hot": row sharding with the rows of each table's 300 most popular ids replicated;
    # "row_whole": 20000 replicated rows, which is all of the smaller tables: those stay out of
    # the exchange and are pooled by the one-GPU kernel into their own slots of z
    hot = {"row_hot": 300, "row_whole": 20000}.get(mode, 0)
    pipe = ShardedDlrmPipeline(model, dev, "row" if mode.startswith("row_") and hot else mode, hot_rows=hot)
    if mode == "row_whole":
        assert pipe.whole_tables and pipe.part_tables, (pipe.whole_tables, pipe.part_tables)
    mode = "row_hot" if mode == "row_whole" else mode
    got = pipe.forward().cpu().numpy()
    assert pipe.embed_error_bits() == 0
    if mode in ("row", "row_hot", "table"):
        # lists, masks and receive slabs are reused: a second and third step must agree
        for _ in range(2):
            again = pipe.forward().cpu().numpy()
            assert np.array_equal(again, got), "row-sharded steps differ from one step to the next"
    if mode in ("row", "row_hot"):
        # the issue orders for back-to-back batches: dense part under the next embedding part,
        # then also the sum of the parts on the dense stream (pooling kernels back to back on
        # the main stream, with and without a block per SM left free); same predictions
        for split, ctas, side in ((False, 0, 0), (True, 0, 0), (True, -1, 0), (True, -2, 2), (False, 0, 0)):
            pipe.rowbags.ex.set_pool_ctas_per_sm(ctas)
            # side: the tables replicated whole pooled on the side stream beside the exchange
            pipe.whole_on_side = side if pipe.whole_tables else 0
            outs = []
            for _ in range(5):
                outs.append(pipe.forward_pipelined(split=split))
            pipe.sync_pipeline()
            torch.cuda.synchronize()
            for o in outs[-2:]:  # the two buffer sets
                assert np.array_equal(o.cpu().numpy(), got), f"pipelined steps (split={split}) differ"
            assert pipe.embed_error_bits() == 0
        pipe.rowbags.ex.set_pool_ctas_per_sm(0)
        pipe.whole_on_side = 0
        again = pipe.forward().cpu().numpy()
        assert np.array_equal(again, got), "a plain step after pipelined ones differs"
        st = pipe.rowbags.exchange_stats()
        print(f"rank {rank} {mode}: remote parts per bag {st['remote_parts_per_bag']:.2f}, "
              f"NVLink bytes {st['nvlink_bytes']}, hot bytes {st['hot_bytes']}")
    want = oracle.dlrm_forward(model, threads=4)
    z = pipe.z.cpu().numpy()
    emb = model.emb
    zw = np.zeros_like(z)
    oracle.embed_bags_tables(emb.tables, [t.shape[0] for t in emb.tables], [b.raw_ids for b in emb.bags],
                             [b.slice_input for b in emb.bags], emb.batch, emb.dim, zw, z.shape[1], 1)
    scale = np.abs(zw[:, 1:]).max()
    perr = float(np.abs(z[:, 1:] - zw[:, 1:]).max() / scale)
    if mode in ("table", "table_nccl", "replica"):
        assert np.array_equal(z[:, 1:], zw[:, 1:]), "pooled vectors must be bit-exact"
    assert perr <= 1e-5, perr          # fp32 pooling tolerance under row sharding
    assert np.abs(got - want).max() <= 2e-3  # TF32 MLP
    dist.barrier()
    pipe.close_exchange()
    dist.destroy_process_group()
    print(f"rank {rank} mode {mode} ok pooled_err {perr:.2e}")


if __name__ == "__main__":
    main()
