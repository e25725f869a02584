"""Helpers of the GPU parity tests: run one op family through the torch-facing wrappers (which call
the C ABI) and compare every output with the CPU oracle under the acceptance rule of cases.py."""
import importlib

import numpy as np
import torch

import cases
from simnets_tf_b200 import abi
mex_ops = importlib.import_module("simnets_tf_b200.ops.mex")
sim_ops = importlib.import_module("simnets_tf_b200.ops.similarity")


def dev(a, dtype=torch.float32):
    return torch.as_tensor(np.ascontiguousarray(a)).to(device="cuda", dtype=dtype)


def check_similarity(port, c, flags=0, f64_tiebreak=False, tol=1e-5, dtype=abi.F32):
    npdt, tdt = (np.float32, torch.float32) if dtype == abi.F32 else (np.float64, torch.float64)
    d = cases.sim_desc(c, dtype=dtype)
    x, t, w, dy = cases.sim_inputs(c, port.sim_out_shape(d), npdt)
    attrs = cases.sim_attrs(c)
    fl = c["flags"] | flags
    xd, td, wd, dyd = (dev(a, tdt) for a in (x, t, w, dy))
    y = sim_ops.similarity_forward(xd, td, wd, flags=fl, **attrs).cpu().numpy()
    dx = sim_ops.similarity_input_grad(xd, td, wd, dyd, flags=fl, **attrs).cpu().numpy()
    dt, dw = (g.cpu().numpy() for g in sim_ops.similarity_parameters_grad(xd, td, wd, dyd, flags=fl, **attrs))
    ry = port.similarity_forward(d, x, t, w)
    rdx = port.similarity_input_grad(d, x, t, w, dy)
    rdt, rdw = port.similarity_params_grad(d, x, t, w, dy)
    r64 = [None] * 4
    if f64_tiebreak:
        d64 = cases.sim_desc(c, dtype=abi.F64)
        a64 = [a.astype(np.float64) for a in (x, t, w, dy)]
        r64 = [port.similarity_forward(d64, *a64[:3]), port.similarity_input_grad(d64, *a64)] + list(port.similarity_params_grad(d64, *a64))
    errs = {}
    for name, ours, ref, ref64 in (("y", y, ry, r64[0]), ("dx", dx, rdx, r64[1]), ("dt", dt, rdt, r64[2]), ("dw", dw, rdw, r64[3])):
        errs[name] = cases.assert_parity(ours, ref, ref64, tol=tol, what="%s %s" % (c["name"], name))
    return errs


def check_mex(port, c, flags=0, f64_tiebreak=False, tol=1e-5, dtype=abi.F32):
    npdt, tdt = (np.float32, torch.float32) if dtype == abi.F32 else (np.float64, torch.float64)
    d = cases.mex_desc(c, dtype=dtype)
    x, off, dy = cases.mex_inputs(c, port.mex_offsets_shape(d), port.mex_out_shape(d), npdt)
    attrs = cases.mex_attrs(c)
    fl = c["flags"] | flags
    xd, od, dyd = (dev(a, tdt) for a in (x, off, dy))
    ry = port.mex_forward(d, x, off)
    y = mex_ops.mex_forward(xd, od, c["M"], flags=fl, **attrs).cpu().numpy()
    # gradients are taken at the oracle's forward output, as the reference's grad ops take orig_output as an input
    ryd = dev(ry, tdt)
    dx = mex_ops.mex_input_grad(xd, od, ryd, dyd, c["M"], flags=fl, **attrs).cpu().numpy()
    doff = mex_ops.mex_offsets_grad(xd, od, ryd, dyd, c["M"], flags=fl, **attrs).cpu().numpy()
    bdx, bdoff = (a.cpu().numpy() for a in mex_ops.mex_backward(xd, od, ryd, dyd, c["M"], flags=fl, **attrs))
    rdx = port.mex_input_grad(d, x, off, ry, dy)
    rdoff = port.mex_offsets_grad(d, x, off, ry, dy)
    r64 = [None] * 3
    if f64_tiebreak:
        d64 = cases.mex_desc(c, dtype=abi.F64)
        x64, o64, dy64 = (a.astype(np.float64) for a in (x, off, dy))
        y64 = port.mex_forward(d64, x64, o64)
        r64 = [y64, port.mex_input_grad(d64, x64, o64, y64, dy64), port.mex_offsets_grad(d64, x64, o64, y64, dy64)]
    errs = {}
    for name, ours, ref, ref64 in (("y", y, ry, r64[0]), ("dx", dx, rdx, r64[1]), ("doff", doff, rdoff, r64[2]),
                                   ("backward dx", bdx, rdx, r64[1]), ("backward doff", bdoff, rdoff, r64[2])):
        errs[name] = cases.assert_parity(ours, ref, ref64, tol=tol, what="%s %s" % (c["name"], name))
    return errs


def check_mex_pooled_dy(port, c, flags=0, tol=1e-5, dtype=abi.F32):
    """Gradients taken from a dy given at half resolution (the gradient of a 2x2 sum pooling of the output) must
    equal the oracle's gradients for the explicitly upsampled dy.  Returns None for odd output sizes."""
    npdt, tdt = (np.float32, torch.float32) if dtype == abi.F32 else (np.float64, torch.float64)
    d = cases.mex_desc(c, dtype=dtype)
    oshape = port.mex_out_shape(d)
    if oshape[2] % 2 or oshape[3] % 2 or oshape[0] == 0:
        return None
    x, off, _ = cases.mex_inputs(c, port.mex_offsets_shape(d), oshape, npdt)
    dyp = np.random.default_rng(c["seed"] + 5).standard_normal((oshape[0], oshape[1], oshape[2] // 2, oshape[3] // 2)).astype(npdt)
    dy = np.repeat(np.repeat(dyp, 2, axis=2), 2, axis=3)
    attrs = cases.mex_attrs(c)
    fl = c["flags"] | flags
    ry = port.mex_forward(d, x, off)
    xd, od, dypd, ryd = (dev(a, tdt) for a in (x, off, dyp, ry))
    dx = mex_ops.mex_input_grad(xd, od, ryd, dypd, c["M"], flags=fl, pooled=True, **attrs)
    doff = mex_ops.mex_offsets_grad(xd, od, ryd, dypd, c["M"], flags=fl, pooled=True, **attrs)
    dx2, doff2 = mex_ops.mex_backward(xd, od, ryd, dypd, c["M"], flags=fl, pooled=True, **attrs)
    rdx = port.mex_input_grad(d, x, off, ry, dy)
    rdoff = port.mex_offsets_grad(d, x, off, ry, dy)
    r64 = [None, None]
    if dtype == abi.F32:
        d64 = cases.mex_desc(c, dtype=abi.F64)
        x64, o64, dy64 = (a.astype(np.float64) for a in (x, off, dy))
        y64 = port.mex_forward(d64, x64, o64)
        r64 = [port.mex_input_grad(d64, x64, o64, y64, dy64), port.mex_offsets_grad(d64, x64, o64, y64, dy64)]
    return {"dx": cases.assert_parity(dx.cpu().numpy(), rdx, r64[0], tol=tol, what=c["name"] + " pooled dx"),
            "doff": cases.assert_parity(doff.cpu().numpy(), rdoff, r64[1], tol=tol, what=c["name"] + " pooled doff"),
            "backward dx": cases.assert_parity(dx2.cpu().numpy(), rdx, r64[0], tol=tol, what=c["name"] + " pooled backward dx"),
            "backward doff": cases.assert_parity(doff2.cpu().numpy(), rdoff, r64[1], tol=tol, what=c["name"] + " pooled backward doff")}
