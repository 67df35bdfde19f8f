"""End-to-end parity of the DLRM-style step with the CPU oracle."""
import numpy as np
import pytest

from oracle import oracle

pytestmark = pytest.mark.gpu

import torch
import annc_b200  # noqa: F401,E402  (no fallback: a missing library fails the collection)
from annc_b200 import synth  # noqa: E402
from annc_b200._lib import MATH_AUTO, MATH_FP32  # noqa: E402
from annc_b200.dlrm import DlrmPipeline  # noqa: E402


@pytest.mark.parametrize("math,tol", [(MATH_FP32, 2e-5), (MATH_AUTO, 2e-3)])
def test_dlrm_step_matches_oracle(math, tol):
    model = synth.dlrm_model(seed=3, batch=4096, max_rows=3e5)
    pipe = DlrmPipeline(model, torch.device("cuda:0"), math=math, keep_host_inputs=True)
    got = pipe.forward().cpu().numpy()
    assert pipe.embed_error_bits() == 0
    want = oracle.dlrm_forward(model, threads=oracle.host_threads())
    assert np.abs(got - want).max() <= tol  # sigmoid outputs in (0,1): absolute == normwise
    # the end-to-end entry (host buffers in, host result out) gives the same answer
    pipe.ids_all.zero_()
    pipe.seg_all.zero_()
    pipe.dense.zero_()
    h = pipe.forward_e2e()
    torch.cuda.synchronize()
    np.testing.assert_array_equal(h.numpy(), got)


def test_smoke_entry():
    import __graft_entry__ as g
    g.smoke()
