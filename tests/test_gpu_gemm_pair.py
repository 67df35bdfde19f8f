"""The persistent CTA-pair tcgen05 GEMM (TF32 and BF16) against the fp32 OpenBLAS oracle:
both B layouts, tails in M, N and K, every epilogue, strided batches, bf16 output and the
fused row softmax.  Bounds (normwise max|y - ref| / max|ref|): 2e-3 TF32, 1e-2 BF16;
softmax 1e-5 absolute on the probabilities of TF32-rounded logits is not meaningful, so the
fused softmax is compared with the softmax of this kernel's own logits (1e-6) and with the
oracle's probabilities within the TF32 bound."""
import numpy as np
import pytest

from oracle import oracle

pytestmark = pytest.mark.gpu

import torch
import annc_b200  # noqa: F401,E402  (no fallback: a missing library fails the collection)
from annc_b200 import device  # noqa: E402
from annc_b200._lib import (ACT_NONE, ACT_RELU, ACT_SIGMOID, IO_A_BF16, IO_B_BF16, IO_C_BF16,  # noqa: E402
                            IO_PAIR, IO_SOFTMAX, MATH_BF16, MATH_TF32)


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def nerr(got, want):
    return float(np.abs(got.float().cpu().numpy() - want).max() / np.abs(want).max())


SHAPES = [(256, 256, 32), (256, 256, 256), (512, 512, 96), (300, 200, 100), (1000, 520, 264),
          (257, 192, 36), (2048, 1024, 1024), (4096, 512, 416), (640, 768, 2048), (8192, 256, 64)]


@pytest.mark.parametrize("m,n,k", SHAPES)
@pytest.mark.parametrize("bsrc", ["nk", "kn"])
def test_pair_tf32(m, n, k, bsrc):
    rng = np.random.default_rng(m + 7 * n + 13 * k)
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((k, n)).astype(np.float32)
    want = oracle.matmul(a, b)
    c = torch.full((m, n), float("nan"), device="cuda")
    if bsrc == "nk":
        name = device.gemm(_dev(a), _dev(b.T), c, m=m, n=n, k=k, trans_b=True, math=MATH_TF32, io_flags=IO_PAIR)
    else:
        name = device.gemm(_dev(a), _dev(b), c, m=m, n=n, k=k, math=MATH_TF32, io_flags=IO_PAIR)
    assert name == "tcgen05_pair_tf32"
    assert not device.gemm_timed_out()
    assert nerr(c, want) <= 2e-3


@pytest.mark.parametrize("act", [ACT_NONE, ACT_RELU, ACT_SIGMOID])
@pytest.mark.parametrize("with_addend,with_bias,alpha,beta", [(False, True, 1.0, 0.0), (True, False, 1.0, 0.0),
                                                              (True, True, 0.5, 2.0), (False, False, 2.0, -1.0)])
def test_pair_epilogues(act, with_addend, with_bias, alpha, beta):
    m, n, k = 600, 328, 96
    rng = np.random.default_rng(act + 10)
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((k, n)).astype(np.float32)
    c0 = rng.standard_normal((m, n)).astype(np.float32)
    add = rng.standard_normal((m, n)).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    pre = alpha * (a @ b) + beta * c0
    want = pre.copy()
    if with_addend:
        want = want + add
    if with_bias:
        want = want + bias
    if act == ACT_RELU:
        want = np.maximum(want, 0)
    elif act == ACT_SIGMOID:
        want = 1 / (1 + np.exp(-want))
    c = _dev(c0)
    name = device.gemm(_dev(a), _dev(b), c, m=m, n=n, k=k, alpha=alpha, beta=beta,
                       addend=_dev(add) if with_addend else None, bias=_dev(bias) if with_bias else None,
                       activation=act, math=MATH_TF32, io_flags=IO_PAIR)
    assert name == "tcgen05_pair_tf32" and not device.gemm_timed_out()
    assert np.abs(c.cpu().numpy() - want).max() <= 2e-3 * np.abs(pre).max()


def test_pair_strided_batch_and_pitched_output():
    bsz, m, n, k = 5, 300, 256, 64
    rng = np.random.default_rng(2)
    a = rng.standard_normal((bsz, m, k)).astype(np.float32)
    b = rng.standard_normal((bsz, k, n)).astype(np.float32)
    want = np.matmul(a, b)
    c = torch.full((bsz, m, n + 8), 9.0, device="cuda")
    name = device.gemm(_dev(a), _dev(b), c, m=m, n=n, k=k, batch=bsz, stride_a=m * k, stride_b=k * n,
                       stride_c=m * (n + 8), ldc=n + 8, math=MATH_TF32, io_flags=IO_PAIR)
    assert name == "tcgen05_pair_tf32" and not device.gemm_timed_out()
    got = c.cpu().numpy()
    assert (got[:, :, n:] == 9.0).all()
    assert np.abs(got[:, :, :n] - want).max() <= 2e-3 * np.abs(want).max()


@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (1000, 520, 264), (4096, 1024, 8192), (8192, 64, 512)])
@pytest.mark.parametrize("c_bf16", [False, True])
def test_pair_bf16(m, n, k, c_bf16):
    rng = np.random.default_rng(m + n + k)
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = (rng.standard_normal((k, n)) / np.sqrt(k)).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    want = np.maximum(oracle.matmul(a, b) + bias, 0)
    a16 = device.cast_bf16(_dev(a))
    b16 = device.bf16_weight(_dev(b))
    assert torch.equal(a16, _dev(a).to(torch.bfloat16)) and torch.equal(b16, _dev(b).t().contiguous().to(torch.bfloat16))
    c = torch.full((m, n), float("nan"), device="cuda", dtype=torch.bfloat16 if c_bf16 else torch.float32)
    flags = IO_A_BF16 | IO_B_BF16 | (IO_C_BF16 if c_bf16 else 0)
    name = device.gemm(a16, b16, c, m=m, n=n, k=k, trans_b=True, bias=_dev(bias), activation=ACT_RELU,
                       math=MATH_BF16, io_flags=flags)
    assert name == "tcgen05_pair_bf16" and not device.gemm_timed_out()
    assert nerr(c, want) <= 1e-2


@pytest.mark.parametrize("n", [256, 100])
def test_pair_batch_matmul_softmax(n):
    """batch_matmul Q K^T followed by the row softmax in one kernel."""
    bsz, m, k = 8, 256, 64
    rng = np.random.default_rng(n)
    q = (rng.standard_normal((bsz, m, k)) / 8).astype(np.float32)
    kt = rng.standard_normal((bsz, k, n)).astype(np.float32)
    logits = torch.empty((bsz, m, n), device="cuda")
    probs = torch.full((bsz, m, n), float("nan"), device="cuda")
    kw = dict(m=m, n=n, k=k, batch=bsz, stride_a=m * k, stride_b=k * n, stride_c=m * n, math=MATH_TF32)
    device.gemm(_dev(q), _dev(kt), logits, io_flags=IO_PAIR, **kw)
    name = device.gemm(_dev(q), _dev(kt), probs, io_flags=IO_SOFTMAX, **kw)
    assert name == "tcgen05_pair_tf32" and not device.gemm_timed_out()
    own = oracle.softmax(logits.cpu().numpy().reshape(-1, n)).reshape(bsz, m, n)
    assert np.abs(probs.cpu().numpy() - own).max() <= 1e-6
    ref = oracle.softmax(np.matmul(q, kt).reshape(-1, n)).reshape(bsz, m, n)
    assert np.abs(probs.cpu().numpy() - ref).max() <= 2e-3
