"""The tcgen05 (TF32) GEMM route against the fp32 OpenBLAS oracle: all three B sources
([N,K] by TMA, [K,N] and kn4 by the cp.async loader), tails in M, N and K, every
epilogue.  Bound: normwise 2e-3 (TF32)."""
import numpy as np
import pytest

from oracle import oracle

pytestmark = pytest.mark.gpu

import torch
import annc_b200  # noqa: F401,E402  (no fallback: a missing library fails the collection)
from annc_b200 import device  # noqa: E402
from annc_b200._lib import (ACT_NONE, ACT_RELU, ACT_SIGMOID, B_KN4, B_PLAIN, MATH_FP32,  # noqa: E402
                            MATH_TF32)

TF32_TOL = 2e-3


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def nerr(got, want):
    return float(np.abs(got.cpu().numpy() - want).max() / np.abs(want).max())


SHAPES = [(128, 128, 32), (128, 128, 64), (256, 256, 128), (64, 16, 32), (100, 132, 36),
          (129, 260, 100), (1000, 520, 264), (512, 1024, 1024), (4096, 512, 416), (300, 64, 2048)]


@pytest.mark.parametrize("m,n,k", SHAPES)
@pytest.mark.parametrize("bsrc", ["nk_tma", "kn", "kn4"])
def test_tf32_gemm_sources(m, n, k, bsrc):
    rng = np.random.default_rng(m * 3 + n * 5 + k)
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((k, n)).astype(np.float32)
    want = oracle.matmul(a, b)
    c = torch.full((m, n), float("nan"), device="cuda")
    if bsrc == "nk_tma":
        name = device.gemm(_dev(a), _dev(b.T), c, m=m, n=n, k=k, trans_b=True, math=MATH_TF32)
    elif bsrc == "kn":
        name = device.gemm(_dev(a), _dev(b), c, m=m, n=n, k=k, math=MATH_TF32)
    else:
        name = device.gemm(_dev(a), _dev(oracle.kn4_pack(b)), c, m=m, n=n, k=k, b_format=B_KN4, math=MATH_TF32)
    assert name.startswith("tcgen05") and name.endswith("tf32")
    assert not device.gemm_timed_out()
    assert nerr(c, want) <= TF32_TOL


def test_tf32_is_not_fp32():
    """Guards against a silent route change: the TF32 result must differ from the fp32 one."""
    rng = np.random.default_rng(0)
    a = rng.standard_normal((256, 512)).astype(np.float32)
    b = rng.standard_normal((512, 256)).astype(np.float32)
    c1 = torch.empty((256, 256), device="cuda")
    c2 = torch.empty((256, 256), device="cuda")
    device.gemm(_dev(a), _dev(b), c1, m=256, n=256, k=512, math=MATH_TF32)
    device.gemm(_dev(a), _dev(b), c2, m=256, n=256, k=512, math=MATH_FP32)
    d = (c1 - c2).abs().max().item()
    assert 0 < d < 0.2


@pytest.mark.parametrize("act", [ACT_NONE, ACT_RELU, ACT_SIGMOID])
@pytest.mark.parametrize("with_addend,with_bias,alpha,beta", [(False, True, 1.0, 0.0), (True, False, 1.0, 0.0),
                                                              (True, True, 0.5, 2.0), (False, False, 2.0, -1.0)])
def test_tf32_epilogues(act, with_addend, with_bias, alpha, beta):
    m, n, k = 300, 200, 96
    rng = np.random.default_rng(act)
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((k, n)).astype(np.float32)
    c0 = rng.standard_normal((m, n)).astype(np.float32)
    add = rng.standard_normal((m, n)).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    want = alpha * (a @ b) + beta * c0
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
                       activation=act, math=MATH_TF32)
    assert name.startswith("tcgen05") and name.endswith("tf32") and not device.gemm_timed_out()
    pre = alpha * (a @ b) + beta * c0
    scale = np.abs(pre).max()
    assert np.abs(c.cpu().numpy() - want).max() <= TF32_TOL * scale


def test_tf32_strided_output():
    """ldc larger than n: the bottom MLP writes slot 0 of the [batch, 27, 64] interaction input."""
    m, n, k = 512, 64, 256
    rng = np.random.default_rng(1)
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((k, n)).astype(np.float32)
    z = torch.full((m, 27, 64), 5.0, device="cuda")
    device.gemm(_dev(a), _dev(b), z, m=m, n=n, k=k, ldc=27 * 64, math=MATH_TF32)
    got = z.cpu().numpy()
    assert (got[:, 1:, :] == 5.0).all()
    assert np.abs(got[:, 0, :] - a @ b).max() <= TF32_TOL * np.abs(a @ b).max()


def test_layout_matmul_full_config_properties():
    """BASELINE config W[2048,4096] kn4-packed, X[8192,2048]: checked on sampled rows against
    the oracle and through linearity (doubling X doubles Y exactly)."""
    from annc_b200 import synth
    x, w = synth.layout_matmul_case(0)
    packed = device.kn4_pack(_dev(w))
    xd = _dev(x)
    y = torch.empty((8192, 4096), device="cuda")
    name = device.gemm(xd, packed, y, m=8192, n=4096, k=2048, b_format=B_KN4)
    assert name.startswith("tcgen05") and name.endswith("tf32") and not device.gemm_timed_out()
    rows = np.random.default_rng(0).integers(0, 8192, 64)
    want = x[rows] @ w
    assert np.abs(y[torch.from_numpy(rows).cuda()].cpu().numpy() - want).max() <= TF32_TOL * np.abs(want).max()
    y2 = torch.empty_like(y)
    device.gemm(xd * 2, packed, y2, m=8192, n=4096, k=2048, b_format=B_KN4)
    assert torch.equal(y2, y * 2)


def test_kn4_with_workspace_matches_direct_route():
    """With a workspace the packed weight is re-laid on the device first; the result must be
    bit-identical to the plain-layout GEMM and within TF32 of the oracle."""
    m, n, k = 1024, 520, 708
    rng = np.random.default_rng(3)
    a = rng.standard_normal((m, k)).astype(np.float32)
    w = rng.standard_normal((k, n)).astype(np.float32)
    packed = _dev(oracle.kn4_pack(w))
    ws = torch.empty((k, n), device="cuda")
    c_ws = torch.empty((m, n), device="cuda")
    c_plain = torch.empty((m, n), device="cuda")
    c_direct = torch.empty((m, n), device="cuda")
    device.gemm(_dev(a), packed, c_ws, m=m, n=n, k=k, b_format=B_KN4, workspace=ws)
    device.gemm(_dev(a), _dev(w), c_plain, m=m, n=n, k=k)
    device.gemm(_dev(a), packed, c_direct, m=m, n=n, k=k, b_format=B_KN4)
    assert torch.equal(ws, _dev(w))
    assert torch.equal(c_ws, c_plain)
    assert nerr(c_direct, a @ w) <= TF32_TOL and nerr(c_ws, a @ w) <= TF32_TOL


def test_kn4_with_workspace_takes_the_k_major_route_for_long_k():
    """K >= 1024, K % 4 == 0 and enough 256 x 256 tiles to occupy the SM pairs: the packed weight
    is re-laid as [N,K] and the CTA-pair kernel runs its K-major TMA route; the workspace then
    holds the transposed weight."""
    m, n, k = 4096, 1300, 1032
    rng = np.random.default_rng(4)
    a = rng.standard_normal((m, k)).astype(np.float32)
    w = rng.standard_normal((k, n)).astype(np.float32)
    packed = _dev(oracle.kn4_pack(w))
    ws = torch.zeros((n, k), device="cuda")
    c = torch.full((m, n), float("nan"), device="cuda")
    device.gemm(_dev(a), packed, c, m=m, n=n, k=k, b_format=B_KN4, workspace=ws)
    assert not device.gemm_timed_out()
    assert torch.equal(ws, _dev(w).t().contiguous())
    assert nerr(c, a @ w) <= TF32_TOL


@pytest.mark.parametrize("m,n,k", [(512, 1024, 1024), (128, 256, 1000), (100, 132, 2052), (192, 384, 4100),
                                   (128, 4096, 2048), (256, 512, 288), (64, 128, 8192)])
@pytest.mark.parametrize("bsrc", ["nk_tma", "kn", "kn4"])
def test_split_k_cluster_route(m, n, k, bsrc):
    """Few output tiles and a long K: the CTAs of a cluster share a tile, split its K range and
    add their partial tiles through distributed shared memory (k-step counts that do not
    divide by the split, ragged M and N, every epilogue).  The result must be the same from
    run to run (ranks are added in a fixed order)."""
    rng = np.random.default_rng(m + 7 * n + k)
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = (rng.standard_normal((k, n)) / np.sqrt(k)).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    addend = rng.standard_normal((m, n)).astype(np.float32)
    want = np.maximum(oracle.matmul(a, b) * np.float32(0.5) + addend + bias, 0)
    kw = dict(m=m, n=n, k=k, math=MATH_TF32, alpha=0.5, bias=_dev(bias), addend=_dev(addend), activation=ACT_RELU)
    if bsrc == "nk_tma":
        bd, kw2 = _dev(b.T), dict(trans_b=True)
    elif bsrc == "kn":
        bd, kw2 = _dev(b), {}
    else:
        bd, kw2 = _dev(oracle.kn4_pack(b)), dict(b_format=B_KN4)
    c1 = torch.full((m, n), float("nan"), device="cuda")
    c2 = torch.full((m, n), float("nan"), device="cuda")
    device.gemm(_dev(a), bd, c1, **kw, **kw2)
    device.gemm(_dev(a), bd, c2, **kw, **kw2)
    assert not device.gemm_timed_out()
    assert nerr(c1, want) <= TF32_TOL
    assert torch.equal(c1, c2)
