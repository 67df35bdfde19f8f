"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations (numpy, host memory).  No dataset is used: the reference's own
end-to-end models are not available, these tensors stand in for them.

One child stream per tensor is spawned from ``default_rng(seed)`` in a fixed order,
so the GPU arm, the CPU arm and the tests see identical values."""
from __future__ import annotations

import concurrent.futures as cf
from dataclasses import dataclass, field
from typing import List, Tuple

import numpy as np


def _children(seed: int, n: int):
    return np.random.default_rng(seed).spawn(n)


# ---------------------------------------------------------------- GEMM configs

def matmul_add_relu_case(seed: int = 0, m: int = 512, k: int = 1024, n: int = 1024):
    """X[m,k] ~ U(-1,1), W[k,n] ~ N(0,(1/32)^2), bias[n] ~ N(0,0.1^2) broadcast to the
    [m,n] addend the custom-call ABI carries; the max operand is zeros."""
    r = _children(seed, 3)
    x = r[0].uniform(-1, 1, (m, k)).astype(np.float32)
    w = (r[1].standard_normal((k, n)) / 32).astype(np.float32)
    bias = (r[2].standard_normal(n) * 0.1).astype(np.float32)
    addend = np.ascontiguousarray(np.broadcast_to(bias, (m, n)))
    return x, w, bias, addend, np.zeros((m, n), np.float32)


def layout_matmul_case(seed: int = 0, m: int = 8192, k: int = 2048, n: int = 4096):
    """W[k,n] ~ N(0,(1/64)^2) (to be kn4-packed), X[m,k] ~ N(0,1)."""
    r = _children(seed, 2)
    w = (r[0].standard_normal((k, n), dtype=np.float32) / np.float32(64))
    x = r[1].standard_normal((m, k), dtype=np.float32)
    return x, w


def batch_matmul_softmax_case(seed: int = 0, b: int = 64, m: int = 256, k: int = 64, n: int = 256):
    """Q[b,m,k], K^T[b,k,n] ~ N(0,1)/8."""
    r = _children(seed, 2)
    q = r[0].standard_normal((b, m, k), dtype=np.float32) / np.float32(8)
    kt = r[1].standard_normal((b, k, n), dtype=np.float32) / np.float32(8)
    return q, kt


# ---------------------------------------------------------------- embedding configs

@dataclass
class BagInputs:
    """Lookups of one table: raw 64-bit ids and the COO matrix whose column 0 is the
    sample (segment) id and column 1 the position inside the bag.  `lut` is the table's
    popularity map: the lookup of Zipf rank r carries the id lut[r mod 2^22]."""
    raw_ids: np.ndarray      # int64[nnz], values in [0, 2^62)
    slice_input: np.ndarray  # int64[nnz, 2]
    lut: np.ndarray | None = None

    def popular_rows(self, k: int, rows: int) -> np.ndarray:
        """Rows (hash buckets) of the k most popular ids of this table, ascending and unique:
        the replicated hot set of a row-sharded run is chosen from them."""
        if k <= 0:
            return np.zeros(0, np.int64)
        if k >= rows:
            return np.arange(rows, dtype=np.int64)
        ids = self.lut[1:min(k, self.lut.shape[0] - 1) + 1]
        return np.unique((ids.view(np.uint64) % np.uint64(rows)).astype(np.int64))


_LUT_BITS = 22


def _bag_inputs(rng: np.random.Generator, batch: int, max_bag: int, zipf_a: float,
                table_rng: np.random.Generator | None = None) -> BagInputs:
    """`rng` draws the bag lengths and the Zipf ranks.  The rank -> id map belongs to the
    table, not to the batch: with `table_rng` (ranks of a multi-GPU run, which draw their own
    batches from their own `rng`) it is taken from that stream at the position the
    single-stream form draws it, so every rank sees the same popular ids for a table."""
    lens = rng.integers(1, max_bag + 1, batch)
    nnz = int(lens.sum())
    seg = np.repeat(np.arange(batch, dtype=np.int64), lens)
    starts = np.cumsum(lens) - lens
    pos = np.arange(nnz, dtype=np.int64) - np.repeat(starts, lens)
    # uniform 62-bit values with Zipf frequencies: rank r -> a fixed random 62-bit id
    if table_rng is None:
        lut = rng.integers(0, 1 << 62, 1 << _LUT_BITS, dtype=np.int64)
    else:
        table_rng.integers(1, max_bag + 1, batch)  # the draw that precedes the map in that stream
        lut = table_rng.integers(0, 1 << 62, 1 << _LUT_BITS, dtype=np.int64)
    ranks = rng.zipf(zipf_a, nnz)
    raw = lut[(ranks.astype(np.uint64) & np.uint64((1 << _LUT_BITS) - 1)).astype(np.int64)]
    return BagInputs(raw_ids=np.ascontiguousarray(raw),
                     slice_input=np.ascontiguousarray(np.stack([seg, pos], axis=1)), lut=lut)


def _table(rng: np.random.Generator, rows: int, dim: int) -> np.ndarray:
    t = rng.random((rows, dim), dtype=np.float32)
    t *= np.float32(0.1)
    t -= np.float32(0.05)
    return t


@dataclass
class EmbeddingWorkload:
    tables: List[np.ndarray]
    bags: List[BagInputs]
    batch: int
    dim: int

    @property
    def nnz(self) -> int:
        return int(sum(b.raw_ids.shape[0] for b in self.bags))

    def algorithmic_bytes(self) -> int:
        """Per batch: row read + raw id + segment id per lookup, one output row per bag."""
        return self.nnz * (4 * self.dim + 8 + 8) + len(self.tables) * self.batch * 4 * self.dim


def embedding_workload(seed: int, rows: List[int], dim: int, batch: int, max_bag: int,
                       zipf_a: float, threads: int = 8, input_seed: int | None = None
                       ) -> EmbeddingWorkload:
    """Tables come from ``seed``; the lookups too unless ``input_seed`` is given (ranks of a
    multi-GPU run share the tables and draw their own batches)."""
    n = len(rows)
    ch = _children(seed, 2 * n)
    own = _children(input_seed, n) if input_seed is not None else None

    def make(t):
        if own is None:
            return _table(ch[2 * t], rows[t], dim), _bag_inputs(ch[2 * t + 1], batch, max_bag, zipf_a)
        return _table(ch[2 * t], rows[t], dim), _bag_inputs(own[t], batch, max_bag, zipf_a,
                                                            table_rng=ch[2 * t + 1])

    with cf.ThreadPoolExecutor(max_workers=max(1, threads)) as ex:
        res = list(ex.map(make, range(n)))
    return EmbeddingWorkload([r[0] for r in res], [r[1] for r in res], batch, dim)


def hash_bucket_bag_case(seed: int = 0, tables: int = 26, rows: int = 1_000_000, dim: int = 64,
                         batch: int = 16384, max_bag: int = 20, zipf_a: float = 1.05):
    """26 tables x 1M rows x dim 64 ~ U(-0.05, 0.05); batch 16384; bags U{1..20}; sum pool."""
    return embedding_workload(seed, [rows] * tables, dim, batch, max_bag, zipf_a)


# ---------------------------------------------------------------- DLRM-style model

@dataclass
class DlrmModel:
    """fp32 weights; W are [fan_in, fan_out] row-major as XLA holds them."""
    bottom: List[Tuple[np.ndarray, np.ndarray]]
    top: List[Tuple[np.ndarray, np.ndarray]]
    emb: EmbeddingWorkload
    dense: np.ndarray  # f32[batch, 13]
    table_rows: List[int] = field(default_factory=list)


def _mlp(rngs, sizes):
    layers = []
    for i in range(len(sizes) - 1):
        w = (rngs[2 * i].standard_normal((sizes[i], sizes[i + 1]))
             / np.sqrt(sizes[i])).astype(np.float32)
        b = (rngs[2 * i + 1].standard_normal(sizes[i + 1]) * 0.01).astype(np.float32)
        layers.append((w, b))
    return layers


def dlrm_model(seed: int = 0, batch: int = 65536, tables: int = 26, dim: int = 64,
               min_rows: float = 1e3, max_rows: float = 1e7, max_bag: int = 20,
               zipf_a: float = 1.05, dense_features: int = 13,
               bottom=(512, 256, 64), top=(512, 256, 1), input_seed: int | None = None
               ) -> DlrmModel:
    """13 dense ~ N(0,1); bottom MLP 13-512-256-64 ReLU; `tables` tables with log-uniform
    rows in [min_rows, max_rows]; dot interaction of the 27 vectors; top MLP
    415-512-256-1 with a final sigmoid."""
    root = np.random.default_rng(seed)
    r_rows, r_dense, r_emb = root.spawn(3)
    rows = [int(round(10 ** u)) for u in r_rows.uniform(np.log10(min_rows), np.log10(max_rows), tables)]
    if input_seed is not None:
        r_dense = np.random.default_rng(input_seed + 7919)
    dense = r_dense.standard_normal((batch, dense_features), dtype=np.float32)
    f = tables + 1
    inter = dim + f * (f - 1) // 2
    mlp_rngs = root.spawn(2 * (len(bottom) + len(top)))
    bsz = (dense_features,) + tuple(bottom)
    tsz = (inter,) + tuple(top)
    bl = _mlp(mlp_rngs[:2 * len(bottom)], bsz)
    tl = _mlp(mlp_rngs[2 * len(bottom):], tsz)
    emb_seed = int(r_emb.integers(0, 2 ** 31))
    emb = embedding_workload(emb_seed, rows, dim, batch, max_bag, zipf_a, input_seed=input_seed)
    return DlrmModel(bl, tl, emb, dense, rows)


def dlrm_flops_per_sample(m: DlrmModel) -> int:
    f = len(m.emb.tables) + 1
    fl = 0
    for w, _ in m.bottom + m.top:
        fl += 2 * w.shape[0] * w.shape[1]
    fl += 2 * f * f * m.emb.dim
    return fl


# ---------------------------------------------------------------- hashed tables (large recsys)

_M64 = (1 << 64) - 1


def _splitmix64(z: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = z + np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def hashed_table_rows(seed: int, table_id: int, rows: np.ndarray, dim: int) -> np.ndarray:
    """f32[len(rows), dim]: the values annc_synth_fill_rows_dev writes for these global rows
    of table `table_id`, bit for bit (same integer steps, one fp32 multiply, one subtract)."""
    rows = np.asarray(rows, dtype=np.uint64).reshape(-1, 1)
    cols = np.arange(dim, dtype=np.uint64).reshape(1, -1)
    with np.errstate(over="ignore"):
        base = np.uint64(seed & _M64) ^ np.uint64((table_id * 0x9E3779B97F4A7C15) & _M64)
        ctr = base + rows * np.uint64(0xD1B54A32D192ED03) + cols * np.uint64(0x8CB92BA72F3D8DD7)
    u = (_splitmix64(ctr) >> np.uint64(40)).astype(np.float32)
    scale = np.float32(0.1) * np.float32(2.0 ** -24)
    return u * scale - np.float32(0.05)


@dataclass
class RecsysModel:
    """Large row-sharded recsys configuration: `tables` hashed tables of `rows` x `dim`, mean
    pooling, concat -> MLP (bias + ReLU, last layer sigmoid).  Weights fp32 [fan_in, fan_out]."""
    seed: int
    tables: int
    rows: int
    dim: int
    batch: int
    bags: List[BagInputs]
    mlp: List[Tuple[np.ndarray, np.ndarray]]

    @property
    def nnz(self) -> int:
        return int(sum(b.raw_ids.shape[0] for b in self.bags))


def recsys_model(seed: int = 0, tables: int = 64, rows: int = 20_000_000, dim: int = 128,
                 batch: int = 16384, max_bag: int = 50, zipf_a: float = 1.2,
                 hidden=(1024, 512, 1), input_seed: int | None = None, threads: int = 8) -> RecsysModel:
    """`batch` is this rank's share of the global batch; ranks pass their own input_seed."""
    root = np.random.default_rng(seed)
    r_mlp, r_in = root.spawn(2)
    sizes = (tables * dim,) + tuple(hidden)
    mlp = _mlp(r_mlp.spawn(2 * len(hidden)), sizes)
    table_rngs = r_in.spawn(tables)
    own = np.random.default_rng(input_seed).spawn(tables) if input_seed is not None else None

    def make(t):
        if own is None:
            return _bag_inputs(table_rngs[t], batch, max_bag, zipf_a)
        return _bag_inputs(own[t], batch, max_bag, zipf_a, table_rng=table_rngs[t])

    with cf.ThreadPoolExecutor(max_workers=max(1, threads)) as ex:
        bags = list(ex.map(make, range(tables)))
    return RecsysModel(seed, tables, rows, dim, batch, bags, mlp)
