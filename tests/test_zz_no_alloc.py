"""MEX forward on the library's own fixed scratch (simnets_mex_forward_static_scratch), for hosts that
cannot pass a workspace because every byte of device memory already belongs to their runtime.

Checked through the C ABI against the CPU oracle and against simnets_mex_forward (caller workspace) on
calls in a row that use different shapes, so each call meets whatever the one before left in the
shared array.  The entry point always runs the CUDA-core kernels; tolerance 1e-5 * max(1, |ref|).
This file sorts last on purpose: a run that stops at the first failure has then run everything else.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import cases
from simnets_tf_b200 import _lib, abi

pytestmark = pytest.mark.gpu


def _both(lib, c, seed, port=None, flags=None):
    d = cases.mex_desc(c) if flags is None else cases.mex_desc(c, flags=flags)
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
    if port is not None:
        ref = port.mex_forward(cases.mex_desc(c), x.cpu().numpy(), off.cpu().numpy())
        cases.assert_parity(y_static.cpu().numpy(), ref, tol=1e-5, what="static scratch vs oracle (%s)" % c["name"])
    return y_ws.cpu().numpy(), y_static.cpu().numpy()


def test_static_scratch_forward_matches_workspace_forward_twice(cuda_lib, port):
    first = cases.mex_case("static_a", (8, 32, 16, 16), 64, (32, 1, 1), (32, 1, 1), softmax=True, unshared_region=(2,))
    second = cases.mex_case("static_b", (3, 12, 9, 10), 5, (4, 2, 3), (4, 2, 1), (0, 1, 1), eps=0.5, unshared=False, shared_region=(2,))
    for i, c in enumerate((first, second, first)):
        a, b = _both(cuda_lib, c, seed=40 + i, port=port)
        assert np.isfinite(a).all()
        cases.assert_parity(b, a, tol=1e-5, what="static scratch vs workspace, call %d" % i)


def test_static_scratch_keeps_the_callers_flags_and_matches_the_oracle_on_a_tensor_core_shape(cuda_lib, port):
    """A shape simnets_mex_forward sends to the tensor cores (K=64, M=128, unshared regions) and a caller flag
    (per-term exp form): the static entry runs its CUDA-core route and stays within the float32 bound of the
    oracle and of the workspace call."""
    c = cases.mex_case("static_tc", (4, 64, 8, 8), 128, (64, 1, 1), (64, 1, 1), softmax=True, unshared_region=(2,))
    a, b = _both(cuda_lib, c, seed=47, port=port)
    cases.assert_parity(b, a, tol=1e-5, what="static scratch vs tensor-core workspace call")
    small = cases.mex_case("static_smallk", (4, 3, 8, 8), 16, (3, 1, 1), (3, 1, 1), softmax=True, unshared=False)
    a, b = _both(cuda_lib, small, seed=48, port=port, flags=abi.FLAG_MEX_EXACT)
    cases.assert_parity(b, a, tol=1e-5, what="static scratch vs workspace, caller flag kept")


def test_static_scratch_rejects_problems_beyond_its_capacity(cuda_lib):
    big = cases.mex_case("static_big", (256, 256, 32, 32), 256, (4, 2, 2), (4, 2, 2), eps=0.5, softmax=True, unshared=False)
    d = cases.mex_desc(big)
    assert cuda_lib.simnets_mex_workspace_bytes(C.byref(d)) > 8 << 20
    dummy = torch.zeros(16, device="cuda")
    rc = cuda_lib.simnets_mex_forward_static_scratch(C.byref(d), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
                                                     torch.cuda.current_stream().cuda_stream)
    assert rc == abi.E_TOO_LARGE
    assert b"capacity" in cuda_lib.simnets_status_string(rc)
