"""MEX forward on the library's own fixed scratch (simnets_mex_forward_static_scratch), for hosts that
cannot pass a workspace because every byte of device memory already belongs to their runtime.

Checked through the C ABI against simnets_mex_forward (caller workspace) on two calls in a row that
use different shapes, so the second call meets whatever the first one left in the shared array.
This file sorts last on purpose: a run that stops at the first failure has then run everything else.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import cases
from simnets_tf_b200 import _lib, abi

pytestmark = pytest.mark.gpu


def _both(lib, c, seed):
    d = cases.mex_desc(c)
    g = abi.MexGeometry()
    assert lib.simnets_mex_dims(C.byref(d), C.byref(g)) == 0
    rng = np.random.default_rng(seed)
    x = torch.from_numpy(rng.normal(size=c["shape"]).astype(np.float32)).cuda()
    off = torch.from_numpy(rng.normal(0, 0.3, size=(g.num_regions, c["M"], g.block_c, g.block_h, g.block_w)).astype(np.float32)).cuda()
    shape = (c["shape"][0], g.channels_out_total, g.height_out, g.width_out)
    y_ws = torch.full(shape, float("nan"), device="cuda")
    y_static = torch.full(shape, float("nan"), device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    n = lib.simnets_mex_workspace_bytes(C.byref(d))
    ws = torch.empty(n, dtype=torch.uint8, device="cuda")
    assert lib.simnets_mex_forward(C.byref(d), x.data_ptr(), off.data_ptr(), y_ws.data_ptr(), ws.data_ptr(), n, stream) == 0
    before = torch.cuda.memory_allocated()
    assert lib.simnets_mex_forward_static_scratch(C.byref(d), x.data_ptr(), off.data_ptr(), y_static.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    return y_ws.cpu().numpy(), y_static.cpu().numpy()


def test_static_scratch_forward_matches_workspace_forward_twice(cuda_lib):
    first = cases.mex_case("static_a", (8, 32, 16, 16), 64, (32, 1, 1), (32, 1, 1), softmax=True, unshared_region=(2,))
    second = cases.mex_case("static_b", (3, 12, 9, 10), 5, (4, 2, 3), (4, 2, 1), (0, 1, 1), eps=0.5, unshared=False, shared_region=(2,))
    for i, c in enumerate((first, second, first)):
        a, b = _both(cuda_lib, c, seed=40 + i)
        assert np.isfinite(a).all()
        cases.assert_parity(b, a, tol=1e-6, what="static scratch vs workspace, call %d" % i)


def test_static_scratch_rejects_problems_beyond_its_capacity(cuda_lib):
    big = cases.mex_case("static_big", (256, 256, 32, 32), 256, (4, 2, 2), (4, 2, 2), eps=0.5, softmax=True, unshared=False)
    d = cases.mex_desc(big)
    assert cuda_lib.simnets_mex_workspace_bytes(C.byref(d)) > 8 << 20
    dummy = torch.zeros(16, device="cuda")
    rc = cuda_lib.simnets_mex_forward_static_scratch(C.byref(d), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
                                                     torch.cuda.current_stream().cuda_stream)
    assert rc == abi.E_TOO_LARGE
    assert b"capacity" in cuda_lib.simnets_status_string(rc)
