"""ctypes mirror of include/simnets_b200.h: descriptors, flags and status codes.

Field order and types follow the C header exactly; `tests/test_abi.py` checks the struct sizes
against the values the shared library reports.
"""
import ctypes as C
import math

F32, F64 = 0, 1
SIM_L1, SIM_L2 = 0, 1

FLAG_ACCUMULATE = 1 << 0
FLAG_FORCE_DIRECT = 1 << 1
FLAG_MEX_EXACT = 1 << 2
FLAG_SIM_BATCH_CONST_QUIRK = 1 << 3
FLAG_SIM_L1_SKIP_NAN = 1 << 4
FLAG_MEX_NO_TENSORCORE = 1 << 5
FLAG_MEX_DY_POOLED2 = 1 << 6
FLAG_MEX_TC_ONE_TILE = 1 << 7
FLAG_MEX_WORKSPACE_PRIMED = 1 << 8
FLAG_MEX_NO_PAIR_TILES = 1 << 9
FLAG_MEX_TEST_EXPIRE_WAIT = 1 << 10
FLAG_SIM_L2_TENSORCORE = 1 << 11
FLAG_SIM_ABS_WEIGHTS = 1 << 12
FLAG_MEX_MAXIMA_GIVEN = 1 << 13
FLAG_MEX_NORMALIZED_OFFSETS = 1 << 14

OK = 0
E_NULL, E_DESC, E_DTYPE, E_WORKSPACE, E_UNSUPPORTED, E_TOO_LARGE = -1, -2, -3, -4, -5, -6


class SimDesc(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32),
        ("batch", C.c_int32), ("channels", C.c_int32), ("height", C.c_int32), ("width", C.c_int32),
        ("num_instances", C.c_int32),
        ("block_h", C.c_int32), ("block_w", C.c_int32),
        ("stride_h", C.c_int32), ("stride_w", C.c_int32),
        ("pad_h", C.c_int32), ("pad_w", C.c_int32),
        ("similarity_function", C.c_int32),
        ("normalization_term", C.c_int32),
        ("ignore_nan_input", C.c_int32),
        ("normalization_term_fudge", C.c_float),
        ("out_of_bounds_value", C.c_float),
        ("flags", C.c_uint32),
    ]


class MexDesc(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32),
        ("batch", C.c_int32), ("channels", C.c_int32), ("height", C.c_int32), ("width", C.c_int32),
        ("num_instances", C.c_int32),
        ("blocks", C.c_int32 * 3), ("strides", C.c_int32 * 3), ("padding", C.c_int32 * 3),
        ("epsilon", C.c_float),
        ("softmax_mode", C.c_int32),
        ("blocks_out_of_bounds_value", C.c_float),
        ("blocks_round_down", C.c_int32),
        ("use_unshared_regions", C.c_int32),
        ("shared_offset_region", C.c_int32 * 3), ("n_shared_offset_region", C.c_int32),
        ("unshared_offset_region", C.c_int32 * 3), ("n_unshared_offset_region", C.c_int32),
        ("flags", C.c_uint32),
    ]


class MexGeometry(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "block_c", "block_h", "block_w", "stride_c", "stride_h", "stride_w", "pad_c", "pad_h", "pad_w",
        "channels_out", "height_out", "width_out", "channels_out_total",
        "region_c", "region_h", "region_w", "offsets_c", "offsets_h", "offsets_w",
        "num_regions", "region_size", "M", "K", "N", "is_1x1")]

    def as_dict(self):
        return {n: getattr(self, n) for n, _ in self._fields_}


def _two(v, name):
    v = [int(e) for e in v]
    if len(v) != 2:
        raise ValueError("%s must be a list with two elements" % name)
    return v


def make_sim_desc(input_shape, num_instances, similarity_function="L2", blocks=(3, 3), strides=(2, 2),
                  padding=(0, 0), normalization_term=False, normalization_term_fudge=0.001,
                  ignore_nan_input=False, out_of_bounds_value=0.0, dtype=F32, flags=0):
    """Descriptor for the Similarity op family; defaults are the op's attr defaults
    (reference src/ops/similarity_op.cpp:61-75)."""
    b, c, h, w = [int(e) for e in input_shape]
    blocks, strides, padding = _two(blocks, "blocks"), _two(strides, "stride"), _two(padding, "padding")
    fn = {"L1": SIM_L1, "L2": SIM_L2}.get(str(similarity_function).upper())
    if fn is None:
        raise ValueError("similarity_function must be 'L1' or 'L2', got %r" % (similarity_function,))
    return SimDesc(dtype, b, c, h, w, int(num_instances), blocks[0], blocks[1], strides[0], strides[1],
                   padding[0], padding[1], fn, int(bool(normalization_term)), int(bool(ignore_nan_input)),
                   float(normalization_term_fudge), float(out_of_bounds_value), int(flags))


def _three(v, name):
    v = [int(e) for e in v]
    if len(v) == 1:
        v = v * 3
    elif len(v) == 2:
        v = [-1] + v
    if len(v) != 3:
        raise ValueError("%s should be a list with 3 elements" % name)
    return v


def _region(v, name):
    v = [int(e) for e in v]
    if len(v) not in (1, 3):
        raise ValueError("%s should be a list with 1 or 3 elements" % name)
    return (C.c_int32 * 3)(*(v + [0, 0])[:3]), len(v)


def make_mex_desc(input_shape, num_instances, softmax_mode=False, padding=(0, 0, 0), strides=(1, 1, 1),
                  blocks=(1, 1, 1), epsilon=1.0, blocks_out_of_bounds_value=0.0, blocks_round_down=True,
                  use_unshared_regions=True, shared_offset_region=(-1,), unshared_offset_region=(-1,),
                  dtype=F32, flags=0):
    """Descriptor for the Mex op family; defaults are the op's attr defaults
    (reference src/ops/mex_op.cpp:58-74)."""
    b, c, h, w = [int(e) for e in input_shape]
    blocks = [int(e) for e in blocks]
    if len(blocks) != 3:
        raise ValueError("blocks should be a list with 3 elements")
    sh, nsh = _region(shared_offset_region, "shared_offset_region")
    un, nun = _region(unshared_offset_region, "unshared_offset_region")
    eps = float(epsilon)
    if math.isnan(eps) or eps == 0.0:
        raise ValueError("epsilon must be non-zero and not NaN")
    return MexDesc(dtype, b, c, h, w, int(num_instances), (C.c_int32 * 3)(*blocks),
                   (C.c_int32 * 3)(*_three(strides, "strides")), (C.c_int32 * 3)(*_three(padding, "padding")),
                   eps, int(bool(softmax_mode)), float(blocks_out_of_bounds_value), int(bool(blocks_round_down)),
                   int(bool(use_unshared_regions)), sh, nsh, un, nun, int(flags))
