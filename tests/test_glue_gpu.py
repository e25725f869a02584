"""Glue of the reference's Keras layers and example networks as library kernels: |weights| inside the Similarity ops
(python/simnets/keras.py:65) and the softmax cross-entropy of the example networks (README.md:108-111)."""
import importlib

import numpy as np
import pytest
import torch

import cases
import gpu_util
from simnets_tf_b200 import abi

sim_ops = importlib.import_module("simnets_tf_b200.ops.similarity")
loss_ops = importlib.import_module("simnets_tf_b200.ops.loss")

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["dims05", "params_norm_nan", "l1_stride2", "wide_M_K", "norm_batch3_quirk"])
@pytest.mark.parametrize("flags", [0, abi.FLAG_FORCE_DIRECT], ids=["tiled", "direct"])
def test_abs_weights_flag_equals_abs_in_front_of_the_op(port, name, flags):
    """Raw weights of both signs (and one exact zero): forward and input gradient as with |w|, weight gradient times
    sign(w), all against the oracle run on |w|."""
    c = next(c for c in cases.SIM_SMALL if c["name"] == name)
    d = cases.sim_desc(c)
    x, t, w, dy = cases.sim_inputs(c, port.sim_out_shape(d))
    rng = np.random.default_rng(77)
    sign = np.where(rng.random(w.shape) < 0.5, -1.0, 1.0).astype(np.float32)
    raw = (w * sign).astype(np.float32)
    raw.reshape(-1)[3] = 0.0
    sign.reshape(-1)[3] = 0.0
    wabs = np.abs(raw)
    xd, td, rd, dyd = (gpu_util.dev(a) for a in (x, t, raw, dy))
    fl = c["flags"] | flags | abi.FLAG_SIM_ABS_WEIGHTS
    attrs = cases.sim_attrs(c)
    cases.assert_parity(sim_ops.similarity_forward(xd, td, rd, flags=fl, **attrs).cpu().numpy(), port.similarity_forward(d, x, t, wabs), what="y")
    cases.assert_parity(sim_ops.similarity_input_grad(xd, td, rd, dyd, flags=fl, **attrs).cpu().numpy(),
                        port.similarity_input_grad(d, x, t, wabs, dy), tol=2e-5, what="dx")
    dt, dw = sim_ops.similarity_parameters_grad(xd, td, rd, dyd, flags=fl, **attrs)
    rdt, rdw = port.similarity_params_grad(d, x, t, wabs, dy)
    cases.assert_parity(dt.cpu().numpy(), rdt, tol=2e-5, what="dt")
    cases.assert_parity(dw.cpu().numpy(), rdw * sign, tol=2e-5, what="dw_raw")


def test_raw_weights_op_is_differentiable_like_abs_then_similarity():
    c = next(c for c in cases.SIM_SMALL if c["name"] == "dims05")
    rng = np.random.default_rng(5)
    B, C_, H, W = c["shape"]
    x = torch.from_numpy(rng.normal(size=c["shape"]).astype(np.float32)).cuda()
    t = torch.from_numpy(rng.normal(size=(c["M"], C_) + c["blocks"]).astype(np.float32)).cuda().requires_grad_(True)
    raw = torch.from_numpy(rng.normal(size=(c["M"], C_) + c["blocks"]).astype(np.float32)).cuda().requires_grad_(True)
    attrs = cases.sim_attrs(c)
    ya = sim_ops.similarity(x, t, torch.abs(raw), **attrs)
    ga = torch.autograd.grad(ya.square().sum(), [t, raw])
    yb = sim_ops.similarity_of_raw_weights(x, t, raw, **attrs)
    gb = torch.autograd.grad(yb.square().sum(), [t, raw])
    assert torch.equal(ya, yb)
    for a, b in zip(ga, gb):
        assert torch.allclose(a, b, rtol=1e-5, atol=1e-5 * float(a.abs().max()))


@pytest.mark.parametrize("batch,classes", [(1, 1), (7, 10), (256, 10), (2048, 10), (33, 1000), (5000, 3)])
def test_softmax_cross_entropy_matches_float64(batch, classes):
    rng = np.random.default_rng(batch * 31 + classes)
    logits = (rng.normal(size=(batch, classes)) * 4.0).astype(np.float32)
    labels = rng.integers(0, classes, size=batch).astype(np.int64)
    scale = 1.0 / (3 * batch)
    l64 = logits.astype(np.float64)
    lse = np.log(np.exp(l64 - l64.max(axis=1, keepdims=True)).sum(axis=1)) + l64.max(axis=1)
    ref_loss = scale * float((lse - l64[np.arange(batch), labels]).sum())
    ref_grad = np.exp(l64 - lse[:, None])
    ref_grad[np.arange(batch), labels] -= 1.0
    ref_grad *= scale
    loss, grad = loss_ops.softmax_cross_entropy_with_grad(torch.from_numpy(logits).cuda(), torch.from_numpy(labels).cuda(), scale)
    assert abs(float(loss) - ref_loss) <= 1e-5 * max(1.0, abs(ref_loss))
    cases.assert_parity(grad.cpu().numpy(), ref_grad, tol=1e-5, what="dlogits")
    # twice in a row on the same workspace: the ticket counter is left clean
    loss2, _ = loss_ops.softmax_cross_entropy_with_grad(torch.from_numpy(logits).cuda(), torch.from_numpy(labels).cuda(), scale)
    assert float(loss2) == float(loss)


def test_softmax_cross_entropy_autograd_and_ignored_labels():
    logits = torch.randn(9, 6, device="cuda", requires_grad=True)
    labels = torch.tensor([0, 5, 2, -1, 3, 6, 1, 1, 4], device="cuda")
    keep = (labels >= 0) & (labels < 6)
    ref = torch.nn.functional.cross_entropy(logits[keep], labels[keep], reduction="sum") * 0.25
    (gr,) = torch.autograd.grad(ref, logits)
    ours = loss_ops.softmax_cross_entropy(logits, labels, 0.25)
    (go,) = torch.autograd.grad(ours * 2.0, logits)
    assert torch.allclose(ours, ref, rtol=1e-5, atol=1e-6)
    assert torch.allclose(go, 2.0 * gr, rtol=1e-5, atol=1e-6)
