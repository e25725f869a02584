"""GPU parity of the Similarity op family against the CPU oracle, through the C ABI."""
import os

import importlib

import numpy as np
import pytest
import torch

import cases
import gpu_util
from simnets_tf_b200 import abi
sim_ops = importlib.import_module("simnets_tf_b200.ops.similarity")

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("c", cases.SIM_SMALL, ids=lambda c: c["name"])
def test_small_grid(port, c):
    gpu_util.check_similarity(port, c, f64_tiebreak=True)


@pytest.mark.parametrize("c", cases.SIM_SMALL, ids=lambda c: c["name"])
def test_small_grid_direct_kernels(port, c):
    gpu_util.check_similarity(port, c, flags=abi.FLAG_FORCE_DIRECT, f64_tiebreak=True)


@pytest.mark.parametrize("c", cases.SIM_SMALL[::3], ids=lambda c: c["name"])
def test_small_grid_float64(port, c):
    gpu_util.check_similarity(port, c, dtype=abi.F64, tol=1e-12)


@pytest.mark.parametrize("c", cases.SIM_CONFIGS, ids=lambda c: c["name"])
def test_baseline_configs(port, c):
    errs = gpu_util.check_similarity(port, c, f64_tiebreak=True)
    print(c["name"], errs)


def test_golden_vectors(cuda_lib):
    """The committed vectors were produced by the reference project's own CPU templates."""
    golden = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "similarity_small.npz"))
    by_name = {c["name"]: c for c in cases.SIM_SMALL}
    for name in sorted({k.split("/")[0] for k in golden.files}):
        c = by_name[name]
        g = {k: golden["%s/%s" % (name, k)] for k in ("x", "t", "w", "dy", "y", "dx", "dt", "dw")}
        fl = c["flags"] | abi.FLAG_SIM_BATCH_CONST_QUIRK
        xd, td, wd, dyd = (gpu_util.dev(g[k]) for k in ("x", "t", "w", "dy"))
        attrs = cases.sim_attrs(c)
        cases.assert_parity(sim_ops.similarity_forward(xd, td, wd, flags=fl, **attrs).cpu().numpy(), g["y"], what=name + " y")
        cases.assert_parity(sim_ops.similarity_input_grad(xd, td, wd, dyd, flags=fl, **attrs).cpu().numpy(), g["dx"], what=name + " dx")
        dt, dw = sim_ops.similarity_parameters_grad(xd, td, wd, dyd, flags=fl, **attrs)
        cases.assert_parity(dt.cpu().numpy(), g["dt"], tol=2e-5, what=name + " dt")
        cases.assert_parity(dw.cpu().numpy(), g["dw"], tol=2e-5, what=name + " dw")


def test_autograd_wiring_matches_grad_ops(port):
    """`similarity(...)` is differentiable and its backward is the two grad ops (reference ops/similarity.py:18-45)."""
    c = next(c for c in cases.SIM_SMALL if c["name"] == "nan_pad1")
    d = cases.sim_desc(c)
    x, t, w, dy = cases.sim_inputs(c, port.sim_out_shape(d))
    xd, td, wd, dyd = (gpu_util.dev(a).requires_grad_(True) for a in (x, t, w, dy))
    y = sim_ops.similarity(xd, td, wd, **cases.sim_attrs(c))
    y.backward(dyd)
    cases.assert_parity(xd.grad.cpu().numpy(), port.similarity_input_grad(d, x, t, w, dy), what="dx")
    rdt, rdw = port.similarity_params_grad(d, x, t, w, dy)
    cases.assert_parity(td.grad.cpu().numpy(), rdt, what="dt")
    cases.assert_parity(wd.grad.cpu().numpy(), rdw, what="dw")


def test_accumulate_flag_adds_into_destination(port):
    c = next(c for c in cases.SIM_SMALL if c["name"] == "l1_3x3")
    d = cases.sim_desc(c)
    x, t, w, dy = cases.sim_inputs(c, port.sim_out_shape(d))
    xd, td, wd, dyd = (gpu_util.dev(a) for a in (x, t, w, dy))
    bucket = torch.full((2, t.size), 3.0, device="cuda")
    sim_ops.similarity_parameters_grad(xd, td, wd, dyd, flags=abi.FLAG_ACCUMULATE, out=(bucket[0], bucket[1]), **cases.sim_attrs(c))
    rdt, rdw = port.similarity_params_grad(d, x, t, w, dy)
    cases.assert_parity(bucket[0].cpu().numpy().reshape(t.shape) - 3.0, rdt, tol=1e-4, what="dt+3")
    cases.assert_parity(bucket[1].cpu().numpy().reshape(t.shape) - 3.0, rdw, tol=1e-4, what="dw+3")


def test_full_size_properties():
    """Config-4 shapes at a size the CPU oracle cannot finish: properties that need no oracle.
    (1) the op is a sum over taps, so an all-NaN input with ignore_nan_input gives exactly 0;
    (2) outputs of a sample do not depend on its batch neighbours; (3) gradients are linear in dy."""
    torch.manual_seed(0)
    B, C, H, M = 16, 64, 32, 256
    x = torch.randn(B, C, H, H, device="cuda")
    x[torch.rand_like(x) < 0.2] = float("nan")
    t = 0.1 * torch.randn(M, C, 3, 3, device="cuda")
    w = (1 + 0.1 * torch.randn(M, C, 3, 3, device="cuda")).abs() + 1e-3
    attrs = dict(similarity_function="L2", blocks=[3, 3], strides=[1, 1], padding=[1, 1], normalization_term=True,
                 ignore_nan_input=True, out_of_bounds_value=0.0)
    y = sim_ops.similarity_forward(x, t, w, **attrs)
    assert torch.isfinite(y).all()
    assert (sim_ops.similarity_forward(torch.full_like(x[:1], float("nan")), t, w, **dict(attrs, out_of_bounds_value=float("nan"))) == 0).all()
    y_tail = sim_ops.similarity_forward(x[B - 3:], t, w, **attrs)
    assert torch.equal(y[B - 3:], y_tail)
    dy1, dy2 = torch.randn_like(y), torch.randn_like(y)
    g1 = sim_ops.similarity_parameters_grad(x, t, w, dy1, **attrs)
    g2 = sim_ops.similarity_parameters_grad(x, t, w, dy2, **attrs)
    g12 = sim_ops.similarity_parameters_grad(x, t, w, dy1 + 2 * dy2, **attrs)
    for a, b, ab in zip(g1, g2, g12):
        assert cases.rel_err((a + 2 * b).cpu().numpy(), ab.cpu().numpy()) < 1e-4
    dx1 = sim_ops.similarity_input_grad(x, t, w, dy1, **attrs)
    dx12 = sim_ops.similarity_input_grad(x, t, w, 3 * dy1, **attrs)
    assert (dx1[torch.isnan(x)] == 0).all()
    assert cases.rel_err((3 * dx1).cpu().numpy(), dx12.cpu().numpy()) < 1e-5


# ---- opt-in tensor-core evaluation of L2 (SIMNETS_FLAG_SIM_L2_TENSORCORE): tolerance 1e-3 of the largest output magnitude
SIM_TC = [
    cases.sim_case("tc_cfg5_layer", (8, 3, 32, 32), 64, "L2", (3, 3), (1, 1), (1, 1), seed=601, x_dist="uniform"),
    cases.sim_case("tc_cfg4_style", (2, 64, 32, 32), 256, "L2", (3, 3), (1, 1), (1, 1), seed=602),
    cases.sim_case("tc_norm_stride2", (3, 5, 13, 11), 70, "L2", (3, 2), (2, 2), (1, 0), norm=True, seed=603),
    cases.sim_case("tc_few_instances_oob", (5, 2, 9, 9), 5, "L2", (2, 2), (1, 1), (1, 1), oob=0.7, seed=604),
    cases.sim_case("tc_ragged_tile", (1, 7, 20, 19), 130, "L2", (1, 1), (1, 1), (0, 0), norm=True, seed=605),
]


@pytest.mark.parametrize("c", SIM_TC, ids=lambda c: c["name"])
def test_tensor_core_l2_forward_within_its_stated_tolerance(port, cuda_lib, c):
    import ctypes as C
    d = cases.sim_desc(c)
    x, t, w, dy = cases.sim_inputs(c, port.sim_out_shape(d))
    xd, td, wd = (gpu_util.dev(a) for a in (x, t, w))
    attrs = cases.sim_attrs(c)
    ref = port.similarity_forward(d, x, t, w)
    y = sim_ops.similarity_forward(xd, td, wd, flags=abi.FLAG_SIM_L2_TENSORCORE, **attrs).cpu().numpy()
    err = cases.assert_parity(y, ref, tol=1e-3, what=c["name"] + " y (tensor cores)")
    print(c["name"], "tensor-core L2 relative error", err)
    # through the C ABI once more, to read the status words: no bounded wait ran out, nothing was redone
    dd = cases.sim_desc(c, flags=abi.FLAG_SIM_L2_TENSORCORE)
    n = cuda_lib.simnets_similarity_workspace_bytes(C.byref(dd))
    ws = torch.empty(n, dtype=torch.uint8, device="cuda")
    y2 = torch.empty(ref.shape, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    assert cuda_lib.simnets_similarity_forward(C.byref(dd), xd.data_ptr(), td.data_ptr(), wd.data_ptr(), y2.data_ptr(), ws.data_ptr(), n, stream) == 0
    status = (C.c_int32 * 2)(7, 7)
    assert cuda_lib.simnets_similarity_workspace_status(ws.data_ptr(), stream, status) == 0
    torch.cuda.synchronize()
    assert list(status) == [0, 0]
    assert np.array_equal(y2.cpu().numpy(), y)


def test_tensor_core_flag_is_ignored_where_the_expansion_does_not_apply(port):
    """L1, and L2 with ignore_nan_input, keep their term-by-term kernels: same bits with and without the flag."""
    for name in ("l1_stride2", "params_norm_nan"):
        c = next(c for c in cases.SIM_SMALL if c["name"] == name)
        d = cases.sim_desc(c)
        x, t, w, dy = cases.sim_inputs(c, port.sim_out_shape(d))
        xd, td, wd = (gpu_util.dev(a) for a in (x, t, w))
        a = sim_ops.similarity_forward(xd, td, wd, flags=c["flags"], **cases.sim_attrs(c)).cpu().numpy()
        b = sim_ops.similarity_forward(xd, td, wd, flags=c["flags"] | abi.FLAG_SIM_L2_TENSORCORE, **cases.sim_attrs(c)).cpu().numpy()
        assert np.array_equal(a, b, equal_nan=True)


def test_cfg4_parameter_gradients_summed_over_eight_samples(port):
    """The batch-summed parameter gradients of the cfg4 layer (8 x 1024 positions per sum: 8192 terms) against the
    float64 oracle, beside the two-sample cases of test_baseline_configs."""
    c = dict(next(c for c in cases.SIM_CONFIGS if c["name"] == "cfg4a_sub"), shape=(8, 64, 32, 32), name="cfg4a_b8")
    d32, d64 = cases.sim_desc(c), cases.sim_desc(c, dtype=abi.F64)
    x, t, w, dy = cases.sim_inputs(c, port.sim_out_shape(d32))
    xd, td, wd, dyd = (gpu_util.dev(a) for a in (x, t, w, dy))
    dt, dw = sim_ops.similarity_parameters_grad(xd, td, wd, dyd, flags=c["flags"], **cases.sim_attrs(c))
    r64 = port.similarity_params_grad(d64, *(a.astype(np.float64) for a in (x, t, w, dy)))
    for name, ours, ref in (("dt", dt, r64[0]), ("dw", dw, r64[1])):
        err = cases.rel_err(ours.cpu().numpy(), ref)
        print("cfg4a batch 8 %s: %.2e from the float64 oracle" % (name, err))
        assert err <= 1e-5, (name, err)
