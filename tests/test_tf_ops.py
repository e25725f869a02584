"""The reference's op registrations (src/ops/similarity_op.cpp, src/ops/mex_op.cpp), compiled unchanged against the
TensorFlow double: all eight ops register with the inputs, outputs, attrs and defaults the drop-in boundary promises to
keep, and their shape functions give the shapes the layers expect
(reference python/simnets/test/keras/__init__.py:12-140 for the expectations).  CPU only."""
import ctypes as C
import os
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "tf_double"))


@pytest.fixture(scope="module")
def ops_lib():
    import build as tf_double_build
    path = tf_double_build.build_ops()
    if path is None:
        pytest.skip("tests/tf_double/_build/libtf_ops_check.so not built (needs a checkout of the reference project)")
    return C.CDLL(path)


def _registry(lib):
    out = {}
    buf = C.create_string_buffer(1 << 16)
    for i in range(lib.tfop_count()):
        assert lib.tfop_describe(i, buf, len(buf)) == 0
        name, ins, outs, attrs, has_fn = buf.value.decode().split("|")
        a = {}
        for item in attrs.split(";"):
            key, rest = item.split(":", 1)
            typ, _, default = rest.partition("=")
            a[key] = (typ, default if "=" in rest else None)
        out[name] = dict(inputs=[s.split(":")[0] for s in ins.split(";")], outputs=[s.split(":")[0] for s in outs.split(";")],
                         attrs=a, shape_fn=has_fn == "1")
    return out


SIM_ATTRS = {"T": ("{float32, float64}", None), "similarity_function": ("{'L1', 'L2'}", "'L2'"), "blocks": ("list(int)", "[3,3]"),
             "strides": ("list(int)", "[2,2]"), "padding": ("list(int)", "[0,0]"), "normalization_term": ("bool", "false"),
             "normalization_term_fudge": ("float", "0.001"), "ignore_nan_input": ("bool", "false"),
             "out_of_bounds_value": ("float", "0.0")}
MEX_ATTRS = {"T": ("{float32, float64}", None), "num_instances": ("int", None), "softmax_mode": ("bool", "false"),
             "padding": ("list(int)", "[0, 0, 0]"), "strides": ("list(int)", "[1, 1, 1]"), "blocks": ("list(int)", "[1, 1, 1]"),
             "epsilon": ("float", "1.0"), "blocks_out_of_bounds_value": ("float", "0.0"), "blocks_round_down": ("bool", "true"),
             "use_unshared_regions": ("bool", "true"), "shared_offset_region": ("list(int)", "[-1]"),
             "unshared_offset_region": ("list(int)", "[-1]")}


def test_all_eight_ops_register_with_the_kept_interface(ops_lib):
    reg = _registry(ops_lib)
    assert sorted(reg) == ["Mex", "MexInputGrad", "MexOffsetsGrad", "MexRef", "Similarity", "SimilarityInputGrad",
                           "SimilarityParametersGrad", "SimilarityRef"]
    for name in ("Similarity", "SimilarityRef", "SimilarityInputGrad", "SimilarityParametersGrad"):
        assert reg[name]["attrs"] == SIM_ATTRS, name
    for name in ("Mex", "MexRef", "MexInputGrad", "MexOffsetsGrad"):
        assert reg[name]["attrs"] == MEX_ATTRS, name
    assert reg["Similarity"]["inputs"] == ["input", "templates", "weights"] and reg["Similarity"]["outputs"] == ["output"]
    assert reg["SimilarityInputGrad"]["inputs"] == ["input", "templates", "weights", "input_grad"]
    assert reg["SimilarityParametersGrad"]["outputs"] == ["templates_grad", "weights_grad"]
    assert reg["Mex"]["inputs"] == ["input", "offsets"] and reg["Mex"]["outputs"] == ["output"]
    assert reg["MexInputGrad"]["inputs"] == ["input", "offsets", "orig_output", "output_grad"]
    assert reg["MexOffsetsGrad"]["inputs"] == ["input", "offsets", "orig_output", "output_grad"]
    assert reg["Similarity"]["shape_fn"] and reg["Mex"]["shape_fn"]


def _shape(lib, op, attrs, *inputs):
    ranks = (C.c_int * len(inputs))(*[len(s) for s in inputs])
    dims = (C.c_longlong * (5 * len(inputs)))()
    for i, s in enumerate(inputs):
        for j, d in enumerate(s):
            dims[5 * i + j] = d
    n_out, out_ranks, out_dims = C.c_int(0), (C.c_int * 4)(), (C.c_longlong * 20)()
    err = C.create_string_buffer(512)
    rc = lib.tfop_shape(op.encode(), attrs.encode(), len(inputs), ranks, dims, 4, C.byref(n_out), out_ranks, out_dims, err, len(err))
    if rc:
        return rc, err.value.decode()
    return 0, [tuple(out_dims[5 * i + j] for j in range(out_ranks[i])) for i in range(n_out.value)]


def test_similarity_shape_function(ops_lib):
    # the Keras test's expectations: 'SAME' padding (block // 2) keeps the size at stride 1, 'VALID' shrinks it
    rc, out = _shape(ops_lib, "Similarity", "blocks=3,3;strides=1,1;padding=1,1", (2, 3, 28, 28), (10, 3, 3, 3), (10, 3, 3, 3))
    assert rc == 0 and out == [(2, 10, 28, 28)]
    rc, out = _shape(ops_lib, "Similarity", "blocks=3,3;strides=1,1;padding=0,0", (2, 3, 28, 28), (10, 3, 3, 3), (10, 3, 3, 3))
    assert rc == 0 and out == [(2, 10, 26, 26)]
    rc, out = _shape(ops_lib, "Similarity", "blocks=2,2;strides=2,2;padding=2,2", (64, 1, 28, 28), (32, 1, 2, 2), (32, 1, 2, 2))
    assert rc == 0 and out == [(64, 32, 16, 16)]
    rc, msg = _shape(ops_lib, "Similarity", "strides=1,1,1", (2, 3, 8, 8), (4, 3, 3, 3), (4, 3, 3, 3))
    assert rc == 1 and "stride" in msg
    rc, msg = _shape(ops_lib, "Similarity", "", (2, 3, 8, 8), (4, 5, 3, 3), (4, 5, 3, 3))        # channel mismatch
    assert rc == 1
    rc, out = _shape(ops_lib, "SimilarityParametersGrad", "", (2, 3, 8, 8), (4, 3, 3, 3), (4, 3, 3, 3), (2, 4, 3, 3))
    assert rc == 0 and out == [(4, 3, 3, 3), (4, 3, 3, 3)]


def test_mex_shape_function_agrees_with_the_library(ops_lib):
    from simnets_tf_b200 import _lib, abi
    for shape, inst, blocks, strides, padding, round_down in (((2, 64, 32, 32), 128, (64, 1, 1), (64, 1, 1), (0, 0, 0), True),
                                                               ((2, 256, 32, 32), 256, (4, 2, 2), (4, 2, 2), (0, 0, 0), True),
                                                               ((3, 5, 9, 10), 7, (2, 3, 3), (1, 2, 2), (1, 1, 1), False)):
        attrs = "num_instances=%d;blocks=%s;strides=%s;padding=%s;blocks_round_down=%s" % (
            inst, ",".join(map(str, blocks)), ",".join(map(str, strides)), ",".join(map(str, padding)), "true" if round_down else "false")
        rc, out = _shape(ops_lib, "Mex", attrs, shape, (1, inst) + blocks)
        assert rc == 0
        d = abi.make_mex_desc(shape, inst, True, padding, strides, blocks, 1.0, 0.0, round_down, False, (-1,), (-1,))
        g = abi.MexGeometry()
        assert _lib.lib().simnets_mex_dims(C.byref(d), C.byref(g)) == 0
        assert out == [(shape[0], g.channels_out_total, g.height_out, g.width_out)]
