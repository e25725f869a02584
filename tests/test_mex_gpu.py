"""GPU parity of the MEX op family against the CPU oracle, through the C ABI."""
import os

import importlib

import numpy as np
import pytest
import torch

import cases
import gpu_util
from simnets_tf_b200 import abi
mex_ops = importlib.import_module("simnets_tf_b200.ops.mex")

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("c", cases.MEX_SMALL, ids=lambda c: c["name"])
def test_small_grid(port, c):
    gpu_util.check_mex(port, c, f64_tiebreak=True)


@pytest.mark.parametrize("c", cases.MEX_SMALL, ids=lambda c: c["name"])
def test_small_grid_direct_kernels(port, c):
    gpu_util.check_mex(port, c, flags=abi.FLAG_FORCE_DIRECT, f64_tiebreak=True)


@pytest.mark.parametrize("c", cases.MEX_SMALL, ids=lambda c: c["name"])
def test_small_grid_exact_evaluation(port, c):
    gpu_util.check_mex(port, c, flags=abi.FLAG_MEX_EXACT, f64_tiebreak=True)


@pytest.mark.parametrize("c", [c for c in cases.MEX_SMALL + cases.MEX_CONFIGS if c["name"].startswith(("tc_", "cfg5_mex"))],
                         ids=lambda c: c["name"])
def test_tensor_core_shapes_one_tile_kernels(port, c):
    """The one-tile-per-CTA tensor-core kernels (SIMNETS_FLAG_MEX_TC_ONE_TILE) must agree with the oracle as well."""
    gpu_util.check_mex(port, c, flags=abi.FLAG_MEX_TC_ONE_TILE, f64_tiebreak=True)


_PAIRED = [c for c in cases.MEX_SMALL + cases.MEX_CONFIGS if c["name"].startswith(("tc_", "cfg5_mex", "cfg2", "cfg3_mex"))] + cases.MEX_PAIR


@pytest.mark.parametrize("c", cases.MEX_PAIR, ids=lambda c: c["name"])
def test_pair_tile_shapes(port, c):
    """Layers whose sibling regions alternate along the width take the pair-tile kernels (8-byte accesses of pixel pairs)."""
    gpu_util.check_mex(port, c, f64_tiebreak=True)
    gpu_util.check_mex_pooled_dy(port, c)          # (None for an odd output height)


@pytest.mark.parametrize("c", _PAIRED, ids=lambda c: c["name"])
def test_pair_tile_shapes_on_one_region_kernels(port, c):
    """SIMNETS_FLAG_MEX_NO_PAIR_TILES keeps such layers on the kernels that give a CTA the positions of one region."""
    gpu_util.check_mex(port, c, flags=abi.FLAG_MEX_NO_PAIR_TILES, f64_tiebreak=True)
    gpu_util.check_mex_pooled_dy(port, c, flags=abi.FLAG_MEX_NO_PAIR_TILES)


@pytest.mark.parametrize("c", cases.MEX_ROWS, ids=lambda c: c["name"])
def test_row_tiling_blocks(port, c):
    """Blocks as wide as their stride that tile the input rows: per-position extrema from whole block rows."""
    gpu_util.check_mex(port, c, f64_tiebreak=True)


@pytest.mark.parametrize("c", cases.MEX_HEAD, ids=lambda c: c["name"])
def test_head_shapes(port, c):
    """Whole-sample patches under few instances and one offsets region: the head kernels."""
    gpu_util.check_mex(port, c, f64_tiebreak=True)


@pytest.mark.parametrize("c", cases.MEX_HEAD + [c for c in cases.MEX_CONFIGS if c["name"] == "cfg5_head_sub"], ids=lambda c: c["name"])
def test_head_gradients_from_the_forward_pass_workspace(port, c):
    """The head's forward kernel leaves the per-position maxima in the workspace; primed gradients must not change."""
    d = cases.mex_desc(c)
    x, off, dy = cases.mex_inputs(c, port.mex_offsets_shape(d), port.mex_out_shape(d))
    xd, od, dyd = (gpu_util.dev(a) for a in (x, off, dy))
    attrs = cases.mex_attrs(c)
    ws = mex_ops.mex_layer_workspace(xd, c["M"], **attrs)
    yd = mex_ops.mex_forward(xd, od, c["M"], workspace=ws, **attrs)
    ry = port.mex_forward(d, x, off)
    cases.assert_parity(yd.cpu().numpy(), ry, what="y")
    ryd = gpu_util.dev(ry)
    mex_ops.mex_forward(xd, od, c["M"], workspace=ws, **attrs)
    dx, doff = mex_ops.mex_backward(xd, od, ryd, dyd, c["M"], primed_workspace=ws, **attrs)
    cases.assert_parity(dx.cpu().numpy(), port.mex_input_grad(d, x, off, ry, dy), tol=2e-5, what="dx")
    cases.assert_parity(doff.cpu().numpy(), port.mex_offsets_grad(d, x, off, ry, dy), tol=2e-5, what="doff")
    cases.assert_parity(mex_ops.mex_input_grad(xd, od, ryd, dyd, c["M"], primed_workspace=ws, **attrs).cpu().numpy(),
                        port.mex_input_grad(d, x, off, ry, dy), tol=2e-5, what="dx alone")
    cases.assert_parity(mex_ops.mex_offsets_grad(xd, od, ryd, dyd, c["M"], primed_workspace=ws, **attrs).cpu().numpy(),
                        port.mex_offsets_grad(d, x, off, ry, dy), tol=2e-5, what="doff alone")


def test_pair_tiles_need_8_byte_alignment(port):
    """Tensors that start on an odd float cannot be read as pixel pairs: the library takes the one-region kernels."""
    c = cases.MEX_PAIR[0]
    d = cases.mex_desc(c)
    x, off, dy = cases.mex_inputs(c, port.mex_offsets_shape(d), port.mex_out_shape(d))
    ry = port.mex_forward(d, x, off)

    def odd(a):
        buf = torch.empty(a.size + 1, device="cuda")
        v = buf[1:].view(a.shape)
        v.copy_(torch.from_numpy(a))
        assert v.data_ptr() % 8 == 4 and v.is_contiguous()
        return v
    xd, dyd, ryd = odd(x), odd(dy), odd(ry)
    od = gpu_util.dev(off)
    attrs = cases.mex_attrs(c)
    cases.assert_parity(mex_ops.mex_forward(xd, od, c["M"], **attrs).cpu().numpy(), ry, what="y")
    dx, doff = mex_ops.mex_backward(xd, od, ryd, dyd, c["M"], **attrs)
    cases.assert_parity(dx.cpu().numpy(), port.mex_input_grad(d, x, off, ry, dy), what="dx")
    cases.assert_parity(doff.cpu().numpy(), port.mex_offsets_grad(d, x, off, ry, dy), tol=2e-5, what="doff")


def test_a_wait_that_runs_out_is_reported_and_recomputed(port, cuda_lib):
    """SIMNETS_FLAG_MEX_TEST_EXPIRE_WAIT: the tensor-core forward kernel's MMA role withholds one completion signal and
    all waits are short, so a bounded wait runs out.  The kernel must return (no hang, no fault), word 1 of the
    workspace status must be set, and the output must still be right because the exact kernel behind redoes it."""
    import ctypes as C
    c = next(c for c in cases.MEX_CONFIGS if c["name"] == "cfg5_mex1_sub")
    d = cases.mex_desc(c)
    x, off, _ = cases.mex_inputs(c, port.mex_offsets_shape(d), port.mex_out_shape(d))
    xd, od = gpu_util.dev(x), gpu_util.dev(off)
    attrs = cases.mex_attrs(c)
    ry = port.mex_forward(d, x, off)
    stream = torch.cuda.current_stream().cuda_stream
    status = (C.c_int32 * 2)(7, 7)
    for flags, want in ((0, 0), (abi.FLAG_MEX_TEST_EXPIRE_WAIT, 1), (0, 0)):
        ws = mex_ops.mex_layer_workspace(xd, c["M"], flags=flags, **attrs)
        y = mex_ops.mex_forward(xd, od, c["M"], flags=flags, workspace=ws, **attrs)
        assert cuda_lib.simnets_mex_workspace_status(ws.data_ptr(), stream, status) == 0
        torch.cuda.synchronize()
        assert (status[0], status[1]) == (0, want)
        cases.assert_parity(y.cpu().numpy(), ry, what="y with flags %d" % flags)


@pytest.mark.parametrize("c", cases.MEX_SMALL[::3], ids=lambda c: c["name"])
def test_small_grid_float64(port, c):
    gpu_util.check_mex(port, c, dtype=abi.F64, tol=1e-12)


@pytest.mark.parametrize("c", cases.MEX_CONFIGS, ids=lambda c: c["name"])
def test_baseline_configs(port, c):
    errs = gpu_util.check_mex(port, c, f64_tiebreak=True)
    print(c["name"], errs)


def test_golden_vectors(cuda_lib):
    """The committed vectors were produced by the reference project's own CPU templates."""
    golden = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "mex_small.npz"))
    by_name = {c["name"]: c for c in cases.MEX_SMALL}
    for name in sorted({k.split("/")[0] for k in golden.files}):
        c = by_name[name]
        g = {k: golden["%s/%s" % (name, k)] for k in ("x", "off", "dy", "y", "dx", "doff")}
        xd, od, dyd, yd = (gpu_util.dev(g[k]) for k in ("x", "off", "dy", "y"))
        attrs = cases.mex_attrs(c)
        cases.assert_parity(mex_ops.mex_forward(xd, od, c["M"], **attrs).cpu().numpy(), g["y"], what=name + " y")
        cases.assert_parity(mex_ops.mex_input_grad(xd, od, yd, dyd, c["M"], **attrs).cpu().numpy(), g["dx"], what=name + " dx")
        cases.assert_parity(mex_ops.mex_offsets_grad(xd, od, yd, dyd, c["M"], **attrs).cpu().numpy(), g["doff"], tol=2e-5, what=name + " doff")


def test_autograd_wiring_matches_grad_ops(port):
    """`mex(...)` is differentiable and its backward is the two grad ops (reference ops/mex.py:47-81)."""
    c = next(c for c in cases.MEX_SMALL if c["name"] == "blocks_bug")
    d = cases.mex_desc(c)
    x, off, dy = cases.mex_inputs(c, port.mex_offsets_shape(d), port.mex_out_shape(d))
    xd, od = (gpu_util.dev(a).requires_grad_(True) for a in (x, off))
    y = mex_ops.mex(xd, od, c["M"], **cases.mex_attrs(c))
    y.backward(gpu_util.dev(dy))
    ry = port.mex_forward(d, x, off)
    cases.assert_parity(xd.grad.cpu().numpy(), port.mex_input_grad(d, x, off, ry, dy), tol=2e-5, what="dx")
    cases.assert_parity(od.grad.cpu().numpy(), port.mex_offsets_grad(d, x, off, ry, dy), tol=2e-5, what="doff")


@pytest.mark.parametrize("name", ["blocks_bug", "eps_half", "tiled_regions", "head_disjoint", "wide_M_K", "eps_pinf"])
def test_fused_backward_equals_the_two_gradient_ops(port, name):
    """simnets_mex_backward shares the prepasses between the two gradients; results must not change."""
    c = next(c for c in cases.MEX_SMALL if c["name"] == name)
    d = cases.mex_desc(c)
    x, off, dy = cases.mex_inputs(c, port.mex_offsets_shape(d), port.mex_out_shape(d))
    xd, od, dyd = (gpu_util.dev(a) for a in (x, off, dy))
    yd = gpu_util.dev(port.mex_forward(d, x, off))
    attrs = cases.mex_attrs(c)
    dx, doff = mex_ops.mex_backward(xd, od, yd, dyd, c["M"], **attrs)
    assert torch.equal(dx, mex_ops.mex_input_grad(xd, od, yd, dyd, c["M"], **attrs))
    assert torch.equal(doff, mex_ops.mex_offsets_grad(xd, od, yd, dyd, c["M"], **attrs))


@pytest.mark.parametrize("c", cases.MEX_SMALL + cases.MEX_CONFIGS, ids=lambda c: c["name"])
def test_gradients_from_the_forward_pass_workspace(port, c):
    """SIMNETS_FLAG_MEX_WORKSPACE_PRIMED: gradients that reuse what the forward pass left in the layer's own
    workspace are the gradients computed from scratch (full and pooled dy, all three entry points)."""
    d = cases.mex_desc(c)
    oshape = port.mex_out_shape(d)
    x, off, dy = cases.mex_inputs(c, port.mex_offsets_shape(d), oshape)
    xd, od, dyd = (gpu_util.dev(a) for a in (x, off, dy))
    attrs, fl = cases.mex_attrs(c), c["flags"]
    pooled_ok = oshape[0] > 0 and oshape[2] % 2 == 0 and oshape[3] % 2 == 0
    for pooled in ([False, True] if pooled_ok else [False]):
        g = dyd[:, :, ::2, ::2].contiguous() if pooled else dyd
        ws = mex_ops.mex_layer_workspace(xd, c["M"], pooled=pooled, flags=fl, **attrs)
        yd = mex_ops.mex_forward(xd, od, c["M"], flags=fl, workspace=ws, **attrs)
        y2 = mex_ops.mex_forward(xd, od, c["M"], flags=fl, **attrs)
        assert torch.equal(torch.nan_to_num(yd, nan=7.0), torch.nan_to_num(y2, nan=7.0))
        kw = dict(flags=fl, pooled=pooled, **attrs)
        want_dx = mex_ops.mex_input_grad(xd, od, yd, g, c["M"], **kw)
        want_doff = mex_ops.mex_offsets_grad(xd, od, yd, g, c["M"], **kw)
        # (equal bit for bit except where overlapping blocks take the kernels that add with atomics)
        same = lambda a, b: torch.allclose(a, b, rtol=1e-5, atol=1e-7, equal_nan=True)
        for _ in range(2):      # the gradient calls leave the workspace primed for one another
            dx, doff = mex_ops.mex_backward(xd, od, yd, g, c["M"], primed_workspace=ws, **kw)
            assert same(dx, want_dx) and same(doff, want_doff), c["name"]
            assert same(mex_ops.mex_input_grad(xd, od, yd, g, c["M"], primed_workspace=ws, **kw), want_dx), c["name"]
            assert same(mex_ops.mex_offsets_grad(xd, od, yd, g, c["M"], primed_workspace=ws, **kw), want_doff), c["name"]


@pytest.mark.parametrize("c", cases.MEX_SMALL + cases.MEX_CONFIGS, ids=lambda c: c["name"])
def test_pooled_output_gradient(port, c):
    """SIMNETS_FLAG_MEX_DY_POOLED2: dy at half resolution stands for its 2x nearest upsampling."""
    if gpu_util.check_mex_pooled_dy(port, c) is None:
        pytest.skip("odd output size")


@pytest.mark.parametrize("c", cases.MEX_SMALL[::2], ids=lambda c: c["name"])
def test_pooled_output_gradient_direct_and_f64(port, c):
    if gpu_util.check_mex_pooled_dy(port, c, flags=abi.FLAG_FORCE_DIRECT) is None:
        pytest.skip("odd output size")
    gpu_util.check_mex_pooled_dy(port, c, dtype=abi.F64, tol=1e-12)


def test_pooled_gradient_rejects_odd_output():
    x = torch.randn(2, 4, 5, 5, device="cuda")
    off = torch.zeros(1, 3, 4, 1, 1, device="cuda")
    attrs = dict(blocks=[4, 1, 1], strides=[4, 1, 1], use_unshared_regions=False, shared_offset_region=[-1])
    y = mex_ops.mex_forward(x, off, 3, **attrs)
    with pytest.raises(RuntimeError):
        mex_ops.mex_input_grad(x, off, y, torch.zeros(2, 3, 2, 2, device="cuda"), 3, pooled=True, **attrs)


@pytest.mark.parametrize("shape", [(3, 5, 8, 12), (2, 3, 6, 6), (1, 1, 2, 2), (4, 7, 10, 14), (0, 3, 4, 4)])
def test_sum_pool2x2_kernel(shape):
    """The library's 2x2 sum pooling equals 4 * avg_pool2d (16-byte path: width % 4 == 0; scalar path otherwise)."""
    torch.manual_seed(1)
    x = torch.randn(*shape, device="cuda")
    got = mex_ops.sum_pool2x2(x)
    want = torch.nn.functional.avg_pool2d(x, 2) * 4.0 if shape[0] else torch.empty(shape[:2] + (shape[2] // 2, shape[3] // 2), device="cuda")
    assert got.shape == want.shape
    assert torch.allclose(got, want, rtol=1e-6, atol=1e-6)
    # unaligned view (offset by one float): takes the scalar path
    if shape[0]:
        flat = torch.randn(x.numel() + 1, device="cuda")[1:].reshape(shape)
        assert torch.allclose(mex_ops.sum_pool2x2(flat), torch.nn.functional.avg_pool2d(flat, 2) * 4.0, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("shape", [(4, 5, 3, 2, 2), (1, 1, 1, 1, 1), (2, 10, 8192, 1, 1), (3, 7, 33, 1, 1), (0, 4, 2, 1, 1)])
def test_normalize_offsets_kernels(shape):
    """The library's normalize_offsets (forward and gradient) against the composed torch expression, in float64."""
    from simnets_tf_b200 import keras as layers
    torch.manual_seed(2)
    off = torch.randn(*shape, device="cuda") * 3
    if off.numel() > 8:
        off.view(-1)[3] = float("-inf")                    # a log-space zero probability
    a = off.clone().requires_grad_(True)
    out = layers._NormalizeOffsets.apply(a)
    b = off.double().clone().requires_grad_(True)
    flat = b.reshape(shape[0] * shape[1], shape[2] * shape[3] * shape[4])
    want = (flat - torch.logsumexp(flat, dim=1, keepdim=True)).reshape(shape)
    assert out.shape == want.shape
    fin = torch.isfinite(want)
    assert torch.equal(torch.isfinite(out), fin)
    assert torch.allclose(out[fin].double(), want[fin], rtol=1e-6, atol=1e-6)
    g = torch.randn(*shape, device="cuda")
    out.backward(g)
    want.backward(g.double())
    if off.numel():
        assert torch.allclose(a.grad.double(), b.grad, rtol=1e-5, atol=1e-6)


def test_mex_sum_pool2_equals_mex_then_pooling():
    """The fused MEX + 2x2 sum pooling op: same forward bits, same gradients as the two ops chained."""
    torch.manual_seed(3)
    x = torch.randn(6, 64, 8, 8, device="cuda")
    off = (0.3 * torch.randn(4, 96, 64, 1, 1, device="cuda"))
    kw = dict(blocks=[64, 1, 1], strides=[64, 1, 1], softmax_mode=True, use_unshared_regions=True, unshared_offset_region=[2])
    outs = []
    for fused in (True, False):
        xa, oa = x.clone().requires_grad_(True), off.clone().requires_grad_(True)
        if fused:
            z = mex_ops.mex_sum_pool2(xa, oa, 96, **kw)
        else:
            z = torch.nn.functional.avg_pool2d(mex_ops.mex(xa, oa, 96, **kw), 2) * 4.0
        (z * torch.linspace(-1, 1, z.numel(), device="cuda").reshape(z.shape)).sum().backward()
        outs.append((z.detach(), xa.grad, oa.grad))
    assert cases.rel_err(outs[0][0].cpu().numpy(), outs[1][0].cpu().numpy()) < 1e-6
    assert cases.rel_err(outs[0][1].cpu().numpy(), outs[1][1].cpu().numpy()) < 1e-6
    assert cases.rel_err(outs[0][2].cpu().numpy(), outs[1][2].cpu().numpy()) < 1e-6


def test_rows_past_the_last_position_do_not_leak(port):
    """A region with fewer positions than a tile leaves tile rows without a position.  Such a row once read the y of
    an unrelated position while its dy was forced to 0; with outputs around -400 that is 0 * 2^(+577) = NaN in the
    offsets gradient.  Inputs shifted far from zero make the leak visible."""
    c = next(c for c in cases.MEX_CONFIGS if c["name"] == "cfg3_mex4_sub")
    d = cases.mex_desc(c)
    x, off, dy = cases.mex_inputs(c, port.mex_offsets_shape(d), port.mex_out_shape(d))
    x = (x - 400.0).astype(np.float32)
    ry = port.mex_forward(d, x, off)
    assert ry.max() < -300
    xd, od, dyd, ryd = (gpu_util.dev(a) for a in (x, off, dy, ry))
    attrs = cases.mex_attrs(c)
    # inputs near -400 carry 3e-5 of float32 spacing, so the float32 oracle is itself that far from exact arithmetic:
    # judge against the float64 oracle as the acceptance rule allows
    d64 = cases.mex_desc(c, dtype=abi.F64)
    x64, o64, dy64 = (a.astype(np.float64) for a in (x, off, dy))
    y64 = port.mex_forward(d64, x64, o64)
    dx64, doff64 = port.mex_input_grad(d64, x64, o64, y64, dy64), port.mex_offsets_grad(d64, x64, o64, y64, dy64)
    for flags in (0, abi.FLAG_MEX_TC_ONE_TILE):
        dx, doff = mex_ops.mex_backward(xd, od, ryd, dyd, c["M"], flags=flags, **attrs)
        cases.assert_parity(dx.cpu().numpy(), port.mex_input_grad(d, x, off, ry, dy), dx64, tol=2e-5, what="dx")
        cases.assert_parity(doff.cpu().numpy(), port.mex_offsets_grad(d, x, off, ry, dy), doff64, tol=2e-5, what="doff")
        cases.assert_parity(mex_ops.mex_forward(xd, od, c["M"], flags=flags, **attrs).cpu().numpy(), ry, y64, what="y")


def test_wide_dynamic_range_takes_the_exact_route(port):
    """Offsets and inputs spanning hundreds of units (and -inf entries) would underflow a factorised
    evaluation; results must still match the oracle, whichever route the library picks."""
    c = cases.mex_case("range", (2, 6, 6, 6), 5, (6, 1, 1), (6, 1, 1), softmax=True, unshared_region=(2,), seed=77)
    d = cases.mex_desc(c)
    x, off, dy = cases.mex_inputs(c, port.mex_offsets_shape(d), port.mex_out_shape(d))
    x = (x * 150).astype(np.float32)
    off = (off * 150).astype(np.float32)
    off[0, 0, 0] = -np.inf
    x[0, 1, 2, 2] = -np.inf
    xd, od, dyd = (gpu_util.dev(a) for a in (x, off, dy))
    ry = port.mex_forward(d, x, off)
    attrs = cases.mex_attrs(c)
    cases.assert_parity(mex_ops.mex_forward(xd, od, c["M"], **attrs).cpu().numpy(), ry, what="y")
    ryd = gpu_util.dev(ry)
    cases.assert_parity(mex_ops.mex_input_grad(xd, od, ryd, dyd, c["M"], **attrs).cpu().numpy(),
                        port.mex_input_grad(d, x, off, ry, dy), what="dx")
    cases.assert_parity(mex_ops.mex_offsets_grad(xd, od, ryd, dyd, c["M"], **attrs).cpu().numpy(),
                        port.mex_offsets_grad(d, x, off, ry, dy), what="doff")


def test_full_size_properties():
    """Config-4 MEX at full output size (4 GiB): properties that need no oracle.
    (1) with all offsets equal to a constant a and softmax_mode, y = a + logsumexp_eps(block), checked
    against torch on a slice; (2) a sample's output does not depend on its batch neighbours;
    (3) per-block softmax weights sum to one, so sum over taps of dx equals sum of dy per block."""
    torch.manual_seed(0)
    B, C, H, M = 256, 256, 32, 256
    x = torch.randn(B, C, H, H, device="cuda")
    attrs = dict(softmax_mode=True, blocks=[4, 2, 2], strides=[4, 2, 2], epsilon=0.5, use_unshared_regions=False,
                 shared_offset_region=[-1])
    off = torch.full((1, M, 4, 2, 2), 0.25, device="cuda")
    y = mex_ops.mex_forward(x, off, M, **attrs)
    assert y.shape == (B, M * 64, 16, 16)
    blocks = x[:2].reshape(2, 64, 4, 16, 2, 16, 2).permute(0, 1, 3, 5, 2, 4, 6).reshape(2, 64, 16, 16, 16)
    want = 0.25 + torch.logsumexp(0.5 * blocks.double(), dim=-1) / 0.5
    got = y[:2].reshape(2, M, 64, 16, 16)
    assert cases.rel_err(got[:, 0].cpu().numpy(), want.cpu().numpy()) < 1e-5
    assert cases.rel_err(got[:, M - 1].cpu().numpy(), want.cpu().numpy()) < 1e-5
    del got, want, blocks
    y_tail = mex_ops.mex_forward(x[B - 2:], off, M, **attrs)
    assert torch.equal(y[B - 2:], y_tail)
    del y_tail
    nb = 8
    off2 = 0.1 * torch.randn(1, M, 4, 2, 2, device="cuda")
    y2 = mex_ops.mex_forward(x[:nb], off2, M, **attrs)
    dy = torch.randn_like(y2)
    dx = mex_ops.mex_input_grad(x[:nb], off2, y2, dy, M, **attrs)
    per_block_dx = dx.reshape(nb, 64, 4, 16, 2, 16, 2).sum(dim=(2, 4, 6))
    per_block_dy = dy.reshape(nb, M, 64, 16, 16).sum(dim=1)
    assert cases.rel_err(per_block_dx.cpu().numpy(), per_block_dy.cpu().numpy()) < 1e-4
    doff = mex_ops.mex_offsets_grad(x[:nb], off2, y2, dy, M, **attrs)
    assert cases.rel_err(doff.sum(dim=(2, 3, 4)).flatten().cpu().numpy(), dy.reshape(nb, M, -1).sum(dim=(0, 2)).cpu().numpy()) < 1e-4


# ---- forward with the 2x2 sum pooling of its output (simnets_mex_forward_pool2x2)
def _pool2(a):
    a = a.astype(np.float64)
    return (a[:, :, 0::2, 0::2] + a[:, :, 0::2, 1::2]) + (a[:, :, 1::2, 0::2] + a[:, :, 1::2, 1::2])


_POOLABLE = [c for c in cases.MEX_PAIR + cases.MEX_CONFIGS + cases.MEX_SMALL[::4]]


@pytest.mark.parametrize("c", _POOLABLE, ids=lambda c: c["name"])
def test_forward_with_pooled_output(port, c):
    """y as the plain forward gives it, and the 2x2 sum pooling of y, from one library call: fused into the epilogue
    on the pair-tile kernels, a pooling launch behind the forward kernels elsewhere."""
    d = cases.mex_desc(c)
    x, off, _ = cases.mex_inputs(c, port.mex_offsets_shape(d), port.mex_out_shape(d))
    ry = port.mex_forward(d, x, off)
    if ry.shape[2] % 2 or ry.shape[3] % 2:
        with pytest.raises(RuntimeError):
            mex_ops.mex_forward_pool2(gpu_util.dev(x), gpu_util.dev(off), c["M"], **cases.mex_attrs(c))
        return
    for flags in (0, abi.FLAG_MEX_NO_PAIR_TILES):
        y, yp = mex_ops.mex_forward_pool2(gpu_util.dev(x), gpu_util.dev(off), c["M"], flags=c["flags"] | flags, **cases.mex_attrs(c))
        cases.assert_parity(y.cpu().numpy(), ry, what="y")
        cases.assert_parity(yp.cpu().numpy(), _pool2(ry).astype(np.float32), tol=1e-5, what="pooled y (flags %d)" % flags)


def test_pooled_output_on_the_recomputing_routes(port, cuda_lib):
    """The pooled output must also be right when the exact kernels redo the forward pass: offsets with a spread that makes
    the factorisation unsafe (status word 0), and a bounded wait that runs out (status word 1)."""
    import ctypes as C
    c = next(c for c in cases.MEX_CONFIGS if c["name"] == "cfg5_mex1_sub")
    d = cases.mex_desc(c)
    x, off, _ = cases.mex_inputs(c, port.mex_offsets_shape(d), port.mex_out_shape(d))
    attrs = cases.mex_attrs(c)
    stream = torch.cuda.current_stream().cuda_stream
    status = (C.c_int32 * 2)(7, 7)
    wide = off.copy()
    wide[0, 0, 0] = 300.0
    for o, flags, want in ((off, abi.FLAG_MEX_TEST_EXPIRE_WAIT, (0, 1)), (wide, 0, (1, 0)), (off, 0, (0, 0))):
        ry = port.mex_forward(d, x, o)
        xd, od = gpu_util.dev(x), gpu_util.dev(o)
        ws = mex_ops.mex_layer_workspace(xd, c["M"], flags=flags, **attrs)
        y, yp = mex_ops.mex_forward_pool2(xd, od, c["M"], flags=flags, workspace=ws, **attrs)
        assert cuda_lib.simnets_mex_workspace_status(ws.data_ptr(), stream, status) == 0
        torch.cuda.synchronize()
        assert (status[0], status[1]) == want
        cases.assert_parity(y.cpu().numpy(), ry, what="y")
        cases.assert_parity(yp.cpu().numpy(), _pool2(ry).astype(np.float32), tol=1e-5, what="pooled y")


# ---- raw offsets, normalised inside the op (SIMNETS_FLAG_MEX_NORMALIZED_OFFSETS)
def _normalise(off):
    o = off.astype(np.float64)
    flat = o.reshape(o.shape[0] * o.shape[1], -1)
    m = flat.max(axis=1, keepdims=True)
    lse = m + np.log(np.exp(flat - m).sum(axis=1, keepdims=True))
    return (flat - lse).reshape(o.shape), np.exp(flat - lse)          # normalised offsets, softmax of every row


_RAW = cases.MEX_PAIR[::2] + cases.MEX_HEAD[::2] + [c for c in cases.MEX_CONFIGS if not c["name"].startswith("cfg4")] + cases.MEX_SMALL[::5]


@pytest.mark.parametrize("c", _RAW, ids=lambda c: c["name"])
def test_raw_offsets_are_normalised_inside_the_op(port, c):
    """Forward and input gradient as with offsets - logsumexp(row) in front of the op; the offsets gradient comes back with
    respect to the raw values: d - softmax(row) * sum(d) of the oracle's gradient d."""
    d = cases.mex_desc(c)
    x, off, dy = cases.mex_inputs(c, port.mex_offsets_shape(d), port.mex_out_shape(d))
    offn64, soft = _normalise(off)
    offn = offn64.astype(np.float32)
    ry = port.mex_forward(d, x, offn)
    rdx = port.mex_input_grad(d, x, offn, ry, dy)
    de = port.mex_offsets_grad(cases.mex_desc(c, dtype=abi.F64), x.astype(np.float64), offn64, ry.astype(np.float64), dy.astype(np.float64))
    flat = de.reshape(soft.shape)
    rdoff = (flat - soft * flat.sum(axis=1, keepdims=True)).reshape(off.shape)
    xd, od, dyd, ryd = (gpu_util.dev(a) for a in (x, off, dy, ry))
    attrs = cases.mex_attrs(c)
    fl = c["flags"] | abi.FLAG_MEX_NORMALIZED_OFFSETS
    cases.assert_parity(mex_ops.mex_forward(xd, od, c["M"], flags=fl, **attrs).cpu().numpy(), ry, what="y")
    cases.assert_parity(mex_ops.mex_input_grad(xd, od, ryd, dyd, c["M"], flags=fl, **attrs).cpu().numpy(), rdx, tol=2e-5, what="dx")
    cases.assert_parity(mex_ops.mex_offsets_grad(xd, od, ryd, dyd, c["M"], flags=fl, **attrs).cpu().numpy(), rdoff.astype(np.float32), tol=3e-5,
                        what="doff (raw)")
    bdx, bdoff = mex_ops.mex_backward(xd, od, ryd, dyd, c["M"], flags=fl, **attrs)
    cases.assert_parity(bdx.cpu().numpy(), rdx, tol=2e-5, what="dx (fused call)")
    cases.assert_parity(bdoff.cpu().numpy(), rdoff.astype(np.float32), tol=3e-5, what="doff (fused call)")
    # accumulate into a caller tensor
    acc = torch.full(off.shape, 2.0, device="cuda")
    mex_ops.mex_offsets_grad(xd, od, ryd, dyd, c["M"], flags=fl | abi.FLAG_ACCUMULATE, out=acc, **attrs)
    cases.assert_parity(acc.cpu().numpy() - 2.0, rdoff.astype(np.float32), tol=1e-4, what="doff accumulated")


def test_raw_offsets_on_the_exact_route(port):
    """A row spread that makes the factorisation unsafe: the exact kernels work on the normalised rows kept in the workspace."""
    c = next(c for c in cases.MEX_CONFIGS if c["name"] == "cfg5_mex1_sub")
    d = cases.mex_desc(c)
    x, off, dy = cases.mex_inputs(c, port.mex_offsets_shape(d), port.mex_out_shape(d))
    off = off.copy()
    off[0, 0, 0] = 300.0
    offn64, soft = _normalise(off)
    offn = offn64.astype(np.float32)
    ry = port.mex_forward(d, x, offn)
    de = port.mex_offsets_grad(cases.mex_desc(c, dtype=abi.F64), x.astype(np.float64), offn64, ry.astype(np.float64), dy.astype(np.float64))
    flat = de.reshape(soft.shape)
    rdoff = (flat - soft * flat.sum(axis=1, keepdims=True)).reshape(off.shape)
    xd, od, dyd, ryd = (gpu_util.dev(a) for a in (x, off, dy, ry))
    attrs = cases.mex_attrs(c)
    fl = abi.FLAG_MEX_NORMALIZED_OFFSETS
    cases.assert_parity(mex_ops.mex_forward(xd, od, c["M"], flags=fl, **attrs).cpu().numpy(), ry, what="y")
    dx, doff = mex_ops.mex_backward(xd, od, ryd, dyd, c["M"], flags=fl, **attrs)
    cases.assert_parity(dx.cpu().numpy(), port.mex_input_grad(d, x, offn, ry, dy), tol=2e-5, what="dx")
    cases.assert_parity(doff.cpu().numpy(), rdoff.astype(np.float32), tol=3e-5, what="doff (raw)")
    with pytest.raises(RuntimeError):
        mex_ops.mex_forward(xd, od, c["M"], flags=fl | abi.FLAG_FORCE_DIRECT, **attrs)


def test_layer_with_fused_and_separate_normalisation():
    from simnets_tf_b200 import keras as layers
    torch.manual_seed(0)
    x = torch.randn(4, 64, 8, 8, device="cuda")
    kw = dict(num_instances=96, blocks=[64, 1, 1], strides=[64, 1, 1], softmax_mode=True, unshared_offset_region=[2], normalize_offsets=True)
    a, b = layers.Mex(**kw), layers.Mex(**kw)
    a.build(tuple(x.shape), device=x.device)
    b.build(tuple(x.shape), device=x.device)
    with torch.no_grad():
        b.offsets.copy_(a.offsets)
    ya = a(x, sum_pool2=True)
    b._op_flags = lambda dtype, device: 0                 # the separate normalisation kernels in front of and behind the op
    yb = b(x, sum_pool2=True)
    assert torch.allclose(ya, yb, rtol=1e-5, atol=1e-5 * float(yb.abs().max()))
    g = torch.randn_like(ya)
    ya.backward(g)
    yb.backward(g)
    assert torch.allclose(a.offsets.grad, b.offsets.grad, rtol=1e-4, atol=3e-5 * float(b.offsets.grad.abs().max()))


@pytest.mark.parametrize("shape,M", [((6, 32, 16, 16), 64), ((4, 64, 32, 32), 128), ((5, 40, 8, 16), 70)], ids=["K32", "cfg5_mex1", "ragged"])
@pytest.mark.parametrize("norm", [0, abi.FLAG_MEX_NORMALIZED_OFFSETS], ids=["plain", "raw_offsets"])
def test_results_do_not_depend_on_what_the_workspace_held(shape, M, norm):
    """A forward call and the gradient calls that reuse its workspace (pooled dy) read nothing they did not write: a
    workspace poisoned with NaN bytes or with large values gives the bits of a zeroed one.  (A layout that depended on
    the pooled flag once made the gradient call look for the forward pass's tables in the wrong place.)"""
    torch.manual_seed(0)
    B, C, H, W = shape
    attrs = dict(blocks=[C, 1, 1], strides=[C, 1, 1], softmax_mode=True, unshared_offset_region=[2])
    x = torch.randn(B, C, H, W, device="cuda")
    off = torch.randn(4, M, C, 1, 1, device="cuda")
    dyp = torch.randn(B, M, H // 2, W // 2, device="cuda")

    def run(fill):
        ws = mex_ops.mex_layer_workspace(x, M, pooled=True, flags=norm, **attrs)
        ws.fill_(fill)
        y, yp = mex_ops.mex_forward_pool2(x, off, M, flags=norm, workspace=ws, **attrs)
        dx, doff = mex_ops.mex_backward(x, off, y, dyp, M, flags=norm, primed_workspace=ws, pooled=True, **attrs)
        return y, yp, dx, doff
    ref = run(0)
    for fill in (255, 127):
        for a, b in zip(run(fill), ref):
            assert torch.equal(a, b)
