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


# ---- per-pixel extrema of the Similarity output handed to the MEX layer behind it
@pytest.mark.parametrize("name", ["dims05", "l1_stride2", "wide_M_K", "params_norm_nan"])
def test_similarity_forward_extrema(port, name):
    c = next(c for c in cases.SIM_SMALL if c["name"] == name)
    d = cases.sim_desc(c)
    x, t, w, _ = cases.sim_inputs(c, port.sim_out_shape(d))
    ref = port.similarity_forward(d, x, t, w)
    B, M, oh, ow = ref.shape
    hi = torch.full((B, oh, ow), 7.0, device="cuda")
    lo = torch.full((B, oh, ow), 7.0, device="cuda")
    y = sim_ops.similarity_forward(gpu_util.dev(x), gpu_util.dev(t), gpu_util.dev(w), flags=c["flags"], extrema=(hi.data_ptr(), lo.data_ptr()),
                                   **cases.sim_attrs(c))
    cases.assert_parity(y.cpu().numpy(), ref, what="y")
    # the extrema are those of the tensor the call wrote, NaN entries ignored
    yn = y.cpu().numpy()
    assert np.array_equal(hi.cpu().numpy(), np.fmax.reduce(yn, axis=1, initial=-np.inf))
    assert np.array_equal(lo.cpu().numpy(), np.fmin.reduce(yn, axis=1, initial=np.inf))


def test_mex_forward_takes_given_maxima(port, cuda_lib):
    """SIMNETS_FLAG_MEX_MAXIMA_GIVEN: the per-position extrema are in the workspace already (here written by torch), the
    forward pass skips its own pass over the input and gives the same bits."""
    mex_ops = importlib.import_module("simnets_tf_b200.ops.mex")
    for cname, eps in (("cfg5_mex1_sub", None), ("pair_eps_neg", None)):
        c = next(c for c in cases.MEX_CONFIGS + cases.MEX_PAIR if c["name"] == cname)
        d = cases.mex_desc(c)
        x, off, _ = cases.mex_inputs(c, port.mex_offsets_shape(d), port.mex_out_shape(d))
        xd, od = gpu_util.dev(x), gpu_util.dev(off)
        attrs = cases.mex_attrs(c)
        plain = mex_ops.mex_forward(xd, od, c["M"], **attrs)
        ws = mex_ops.mex_layer_workspace(xd, c["M"], **attrs)
        ptr = mex_ops.mex_workspace_maxima(tuple(xd.shape), xd.dtype, c["M"], ws, **attrs)
        assert ptr is not None and ws.data_ptr() <= ptr < ws.data_ptr() + ws.numel()
        ext = xd.amax(dim=1) if c["eps"] > 0 else xd.amin(dim=1)                     # [B, H, W]: blocks span all channels of a pixel
        slot = ws[ptr - ws.data_ptr():ptr - ws.data_ptr() + 4 * ext.numel()].view(torch.float32)
        slot.copy_(ext.reshape(-1))
        given = mex_ops.mex_forward(xd, od, c["M"], flags=abi.FLAG_MEX_MAXIMA_GIVEN, workspace=ws, **attrs)
        assert torch.equal(plain, given)
        cases.assert_parity(given.cpu().numpy(), port.mex_forward(d, x, off), what="y")


def test_network_with_and_without_the_extrema_hand_over():
    from simnets_tf_b200.simnet import SimNet, SPECS
    spec = SPECS["cfg5"]
    rng = np.random.default_rng(3)
    x = torch.from_numpy(rng.uniform(-0.5, 0.5, size=(6,) + tuple(spec["input_shape"])).astype(np.float32)).cuda()
    labels = torch.from_numpy(rng.integers(0, spec["classes"], size=6)).cuda()
    outs = []
    for fuse in (True, False):
        net = SimNet(spec, seed=2)
        net.fuse_extrema = fuse
        loss = net.loss(x, labels)
        loss.backward()
        outs.append([loss.detach()] + [p.grad.clone() for p in net.parameters()])
    for a, b in zip(*outs):
        assert torch.equal(a, b)
