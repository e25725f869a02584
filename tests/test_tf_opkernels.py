"""The C++ host side: TensorFlow GPU OpKernels on the C ABI (simnets_tf_b200/tf_opkernels), compiled against a
TensorFlow test double and the reference's own kernel-common headers, then run through the double.

CPU part: the sources compile, register the six ops of the reference for float and double, and the reference's own
constructors reject what they reject in TensorFlow.  GPU part: Compute() on device buffers against the oracle.
The check library is built where a reference checkout exists and travels as a built file; without it the tests skip."""
import ctypes as C
import os
import sys

import numpy as np
import pytest

import cases

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "tf_double"))
import build as tf_double_build  # noqa: E402

OPS = ["Similarity", "SimilarityInputGrad", "SimilarityParametersGrad", "Mex", "MexInputGrad", "MexOffsetsGrad"]


@pytest.fixture(scope="module")
def tfk(cuda_lib):
    path = tf_double_build.build()
    if path is None:
        pytest.skip("no reference checkout and no prebuilt check library")
    lib = C.CDLL(path)
    lib.tfk_run.argtypes = [C.c_char_p, C.c_int, C.c_char_p, C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_int), C.POINTER(C.c_longlong),
                            C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_int), C.POINTER(C.c_longlong), C.c_void_p, C.c_ulonglong,
                            C.c_void_p, C.c_char_p, C.c_int]
    lib.tfk_has.argtypes = [C.c_char_p, C.c_char_p, C.c_int]
    return lib


def _attr_text(**kw):
    def fmt(v):
        if isinstance(v, bool):
            return "1" if v else "0"
        if isinstance(v, (list, tuple)):
            return ",".join(str(int(e)) for e in v)
        return repr(float(v)) if isinstance(v, float) else str(v)
    return ";".join("%s=%s" % (k, fmt(v)) for k, v in kw.items()).encode()


def sim_attrs(c):
    return _attr_text(similarity_function=c["fn"], blocks=c["blocks"], strides=c["strides"], padding=c["padding"],
                      normalization_term=c["norm"], normalization_term_fudge=0.001,
                      ignore_nan_input=c["ignore_nan"], out_of_bounds_value=float(c["oob"]))


def mex_attrs(c):
    return _attr_text(num_instances=c["M"], softmax_mode=c["softmax"], padding=c["padding"], strides=c["strides"], blocks=c["blocks"],
                      epsilon=float(c["eps"]), blocks_out_of_bounds_value=float(c["oob"]), blocks_round_down=c["round_down"],
                      use_unshared_regions=c["unshared"], shared_offset_region=c["shared_region"],
                      unshared_offset_region=c["unshared_region"])


def run(lib, op, attrs, inputs, out_shapes, scratch_bytes=64 << 20):
    """inputs: torch CUDA tensors; out_shapes: upper bounds used to size the output buffers.  Returns (rc, message, outputs)."""
    import torch
    dt = inputs[0].dtype
    outs = [torch.empty(s, dtype=dt, device="cuda") for s in out_shapes]
    scratch = torch.empty(scratch_bytes, dtype=torch.uint8, device="cuda")
    n_in, n_out = len(inputs), len(outs)
    in_ptrs = (C.c_void_p * n_in)(*[t.data_ptr() for t in inputs])
    in_ranks = (C.c_int * n_in)(*[t.dim() for t in inputs])
    in_dims = (C.c_longlong * (5 * n_in))(*[(list(t.shape) + [0] * 5)[a] for t in inputs for a in range(5)])
    out_ptrs = (C.c_void_p * n_out)(*[t.data_ptr() for t in outs])
    out_ranks = (C.c_int * n_out)()
    out_dims = (C.c_longlong * (5 * n_out))()
    err = C.create_string_buffer(512)
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.tfk_run(op.encode(), int(dt == torch.float64), attrs, n_in, in_ptrs, in_ranks, in_dims, n_out, out_ptrs, out_ranks, out_dims,
                     scratch.data_ptr(), scratch_bytes, stream, err, 512)
    torch.cuda.synchronize()
    shapes = [tuple(out_dims[5 * i + a] for a in range(out_ranks[i])) for i in range(n_out)]
    return rc, err.value.decode(), [o.reshape(-1)[:int(np.prod(s))].reshape(s) if rc == 0 else o for o, s in zip(outs, shapes)]


def test_opkernels_compile_and_register_the_reference_ops(tfk):
    assert tfk.tfk_count() == 12
    for op in OPS:
        for is_double in (0, 1):
            assert tfk.tfk_has(op.encode(), b"GPU", is_double) == 1
        assert tfk.tfk_has(op.encode(), b"CPU", 0) == 0        # no CPU kernels in the GPU build


def test_reference_constructors_still_validate(tfk):
    """Attr validation is the reference's own code (SimilarityKernelCommon / MEXKernelCommon constructors)."""
    null = (C.c_void_p * 1)()
    ranks, dims, err = (C.c_int * 1)(), (C.c_longlong * 5)(), C.create_string_buffer(512)

    def construct(op, attrs):
        rc = tfk.tfk_run(op.encode(), 0, attrs, 0, null, ranks, dims, 0, null, ranks, dims, None, 0, None, err, 512)
        return rc, err.value.decode()

    base = dict(similarity_function="L1", blocks=[3, 3], strides=[1, 1], padding=[0, 0], normalization_term=True,
                normalization_term_fudge=0.001, ignore_nan_input=False, out_of_bounds_value=0.0)
    rc, msg = construct("Similarity", _attr_text(**base))
    assert rc == 1 and "normalization_term is relevant only if similarity_function is L2" in msg
    rc, msg = construct("Similarity", _attr_text(**dict(base, similarity_function="L2", normalization_term=False, ignore_nan_input=True)))
    assert rc == 1 and "ignore_nan" in msg
    rc, msg = construct("Similarity", _attr_text(**dict(base, blocks=[3])))
    assert rc == 1 and "blocks" in msg
    mex = dict(num_instances=0, softmax_mode=True, padding=[0, 0, 0], strides=[1, 1, 1], blocks=[1, 1, 1], epsilon=1.0,
               blocks_out_of_bounds_value=0.0, blocks_round_down=True, use_unshared_regions=True, shared_offset_region=[-1],
               unshared_offset_region=[-1])
    rc, msg = construct("Mex", _attr_text(**mex))
    assert rc == 1 and "num_instances must be positive" in msg
    rc, msg = construct("Mex", _attr_text(**dict(mex, num_instances=3, strides=[1, 1])))
    assert rc == 1 and "strides" in msg


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["dims00", "params_norm_nan", "l1_stride2", "nan_pad1", "nan_propagates", "wide_M_K"])
def test_similarity_opkernels_match_the_oracle(tfk, port, name):
    import gpu_util
    c = next(c for c in cases.SIM_SMALL if c["name"] == name)
    if c["flags"]:
        pytest.skip("case uses library-only flags")
    d = cases.sim_desc(c)
    x, t, w, dy = cases.sim_inputs(c, port.sim_out_shape(d))
    xd, td, wd, dyd = (gpu_util.dev(a) for a in (x, t, w, dy))
    attrs = sim_attrs(c)
    rc, msg, (y,) = run(tfk, "Similarity", attrs, [xd, td, wd], [dy.shape])
    assert rc == 0, msg
    assert tuple(y.shape) == dy.shape
    cases.assert_parity(y.cpu().numpy(), port.similarity_forward(d, x, t, w), what="y")
    rc, msg, (dx,) = run(tfk, "SimilarityInputGrad", attrs, [xd, td, wd, dyd], [x.shape])
    assert rc == 0, msg
    cases.assert_parity(dx.cpu().numpy(), port.similarity_input_grad(d, x, t, w, dy), tol=2e-5, what="dx")
    rc, msg, (dt, dw) = run(tfk, "SimilarityParametersGrad", attrs, [xd, td, wd, dyd], [t.shape, w.shape])
    assert rc == 0, msg
    rdt, rdw = port.similarity_params_grad(d, x, t, w, dy)
    cases.assert_parity(dt.cpu().numpy(), rdt, tol=2e-5, what="dt")
    cases.assert_parity(dw.cpu().numpy(), rdw, tol=2e-5, what="dw")


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["blocks_bug", "tiled_regions", "tc_unshared", "head_disjoint", "eps_pinf"])
def test_mex_opkernels_match_the_oracle(tfk, port, name):
    import gpu_util
    c = next(c for c in cases.MEX_SMALL if c["name"] == name)
    d = cases.mex_desc(c)
    x, off, dy = cases.mex_inputs(c, port.mex_offsets_shape(d), port.mex_out_shape(d))
    ry = port.mex_forward(d, x, off)
    xd, od, dyd, ryd = (gpu_util.dev(a) for a in (x, off, dy, ry))
    attrs = mex_attrs(c)
    rc, msg, (y,) = run(tfk, "Mex", attrs, [xd, od], [ry.shape])
    assert rc == 0, msg
    assert tuple(y.shape) == ry.shape
    cases.assert_parity(y.cpu().numpy(), ry, what="y")
    rc, msg, (dx,) = run(tfk, "MexInputGrad", attrs, [xd, od, ryd, dyd], [x.shape])
    assert rc == 0, msg
    cases.assert_parity(dx.cpu().numpy(), port.mex_input_grad(d, x, off, ry, dy), tol=2e-5, what="dx")
    rc, msg, (doff,) = run(tfk, "MexOffsetsGrad", attrs, [xd, od, ryd, dyd], [off.shape])
    assert rc == 0, msg
    cases.assert_parity(doff.cpu().numpy(), port.mex_offsets_grad(d, x, off, ry, dy), tol=2e-5, what="doff")


@pytest.mark.gpu
def test_mex_opkernel_reports_bad_offsets_shape(tfk, port):
    import torch
    x = torch.randn(2, 4, 6, 6, device="cuda")
    off = torch.zeros(1, 3, 4, 1, 2, device="cuda")          # block_w should be 1
    attrs = _attr_text(num_instances=3, softmax_mode=True, padding=[0, 0, 0], strides=[4, 1, 1], blocks=[4, 1, 1], epsilon=1.0,
                       blocks_out_of_bounds_value=0.0, blocks_round_down=True, use_unshared_regions=False, shared_offset_region=[-1],
                       unshared_offset_region=[-1])
    rc, msg, _ = run(tfk, "Mex", attrs, [x, off], [(2, 3, 6, 6)])
    assert rc == 2 and "offsets must be" in msg


@pytest.mark.gpu
def test_mex_opkernel_takes_a_two_entry_padding_as_the_reference_does(tfk, port):
    """padding=[h, w] means [-1, h, w] (ExpandDimSpec, src/kernels/mex_kernel_common.cpp:8-27): the channel padding
    becomes the channel count.  The oracle is given the expanded form."""
    import gpu_util
    c = dict(next(c for c in cases.MEX_SMALL if c["name"] == "tiled_regions"))
    C_ = c["shape"][1]
    c["padding"] = (C_, 1, 1)
    d = cases.mex_desc(c)
    x, off, dy = cases.mex_inputs(c, port.mex_offsets_shape(d), port.mex_out_shape(d))
    ry = port.mex_forward(d, x, off)
    xd, od, dyd, ryd = (gpu_util.dev(a) for a in (x, off, dy, ry))
    attrs = mex_attrs(dict(c, padding=(1, 1)))
    rc, msg, (y,) = run(tfk, "Mex", attrs, [xd, od], [ry.shape])
    assert rc == 0, msg
    assert tuple(y.shape) == ry.shape
    cases.assert_parity(y.cpu().numpy(), ry, what="y")
    rc, msg, (dx,) = run(tfk, "MexInputGrad", attrs, [xd, od, ryd, dyd], [x.shape])
    assert rc == 0, msg
    cases.assert_parity(dx.cpu().numpy(), port.mex_input_grad(d, x, off, ry, dy), tol=2e-5, what="dx")
    rc, msg, _ = run(tfk, "Mex", mex_attrs(dict(c, padding=(1,))), [xd, od], [ry.shape])
    assert rc == 2 and "padding should be" in msg


@pytest.mark.gpu
def test_mex_grad_opkernels_reject_a_wrong_output_shape(tfk, port):
    import gpu_util
    c = next(c for c in cases.MEX_SMALL if c["name"] == "tiled_regions")
    d = cases.mex_desc(c)
    x, off, dy = cases.mex_inputs(c, port.mex_offsets_shape(d), port.mex_out_shape(d))
    ry = port.mex_forward(d, x, off)
    xd, od, dyd, ryd = (gpu_util.dev(a) for a in (x, off, dy, ry))
    attrs = mex_attrs(c)
    short = ryd[:, :, :-1].contiguous()
    for op, out in (("MexInputGrad", x.shape), ("MexOffsetsGrad", off.shape)):
        rc, msg, _ = run(tfk, op, attrs, [xd, od, short, dyd], [out])
        assert rc == 2 and "orig_output must have" in msg, (op, rc, msg)
        rc, msg, _ = run(tfk, op, attrs, [xd, od, ryd, short], [out])
        assert rc == 2 and "output_grad must have" in msg, (op, rc, msg)


@pytest.mark.gpu
def test_similarity_opkernels_reject_wrong_block_and_gradient_shapes(tfk, port):
    import gpu_util
    c = next(c for c in cases.SIM_SMALL if c["name"] == "dims00")
    d = cases.sim_desc(c)
    x, t, w, dy = cases.sim_inputs(c, port.sim_out_shape(d))
    xd, td, wd, dyd = (gpu_util.dev(a) for a in (x, t, w, dy))
    attrs = sim_attrs(c)
    import torch
    wide = torch.zeros(t.shape[:3] + (t.shape[3] + 1,), device="cuda")
    rc, msg, _ = run(tfk, "Similarity", attrs, [xd, wide, wide], [dy.shape])
    assert rc == 2 and "mismatch" in msg
    rc, msg, _ = run(tfk, "Similarity", attrs, [xd, td, wide], [dy.shape])
    assert rc == 2 and "mismatch" in msg
    short = dyd[:, :, :-1].contiguous()
    rc, msg, _ = run(tfk, "SimilarityInputGrad", attrs, [xd, td, wd, short], [x.shape])
    assert rc == 2 and "output_grad must have" in msg
    rc, msg, _ = run(tfk, "SimilarityParametersGrad", attrs, [xd, td, wd, short], [t.shape, w.shape])
    assert rc == 2 and "output_grad must have" in msg


_LEGACY_CHILD = r"""
import os, sys
sys.path.insert(0, {tests!r}); sys.path.insert(0, {root!r})
import numpy as np, torch
import cases, test_tf_opkernels as T
import ctypes as C
from simnets_tf_b200 import abi
from oracle import oracle
port = oracle.load("port")
lib = C.CDLL(T.tf_double_build.build())
lib.tfk_run.argtypes = [C.c_char_p, C.c_int, C.c_char_p, C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_int), C.POINTER(C.c_longlong),
                        C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_int), C.POINTER(C.c_longlong), C.c_void_p, C.c_ulonglong,
                        C.c_void_p, C.c_char_p, C.c_int]
c = next(c for c in cases.SIM_SMALL if c["name"] == "norm_batch3_quirk")
d = cases.sim_desc(c, flags=abi.FLAG_SIM_BATCH_CONST_QUIRK)
x, t, w, dy = cases.sim_inputs(c, port.sim_out_shape(d))
rc, msg, (y,) = T.run(lib, "Similarity", T.sim_attrs(c), [torch.from_numpy(a).cuda() for a in (x, t, w)], [dy.shape])
assert rc == 0, msg
cases.assert_parity(y.cpu().numpy(), port.similarity_forward(d, x, t, w), what="y with the batch constant of the fast op")
print("LEGACY_OK")
"""


@pytest.mark.gpu
def test_legacy_batch_constant_switch_reproduces_the_fast_op(tfk):
    """SIMNETS_B200_LEGACY_BATCH_CONSTANT=1 is read once per process, so the check runs in a child process."""
    import subprocess
    root = os.path.dirname(HERE)
    env = dict(os.environ, SIMNETS_B200_LEGACY_BATCH_CONSTANT="1")
    out = subprocess.run([sys.executable, "-c", _LEGACY_CHILD.format(tests=HERE, root=root)], env=env, capture_output=True, text=True,
                         timeout=600)
    assert "LEGACY_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]
