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
