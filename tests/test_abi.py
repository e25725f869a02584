"""CPU-only checks of the boundary: the CUDA library loads without a GPU, exports every symbol
the public header declares, and its host-only entry points (dimensions, validation, the legacy
region-count helper) behave like the reference's."""
import ctypes as C
import os
import re

import pytest

import cases
from simnets_tf_b200 import _lib, abi
from simnets_tf_b200.ops.mex import _expand_dim_specification, _mex_dims_helper

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_every_declared_symbol_is_exported(cuda_lib):
    header = open(os.path.join(ROOT, "include", "simnets_b200.h")).read()
    declared = set(re.findall(r"SIMNETS_API\s+[\w\s\*]+?\b(\w+)\s*\(", header))
    assert {"simnets_similarity_forward", "simnets_mex_forward", "get_mex_offsets_nregions", "simnets_mex_offsets_grad"} <= declared
    for name in sorted(declared):
        assert hasattr(cuda_lib, name), "library does not export " + name
    assert cuda_lib.simnets_abi_version() == 1


def test_struct_layout_matches_header():
    assert C.sizeof(abi.SimDesc) == 18 * 4
    assert C.sizeof(abi.MexDesc) == (6 + 9 + 1 + 1 + 1 + 1 + 1 + 4 + 4 + 1) * 4
    assert C.sizeof(abi.MexGeometry) == 25 * 4


def test_similarity_validation_follows_the_reference_constructor(cuda_lib):
    oh, ow = C.c_int32(), C.c_int32()

    def dims(**kw):
        d = abi.make_sim_desc((2, 3, 10, 10), 4, **kw)
        return cuda_lib.simnets_similarity_output_dims(C.byref(d), C.byref(oh), C.byref(ow))

    assert dims(similarity_function="L2", blocks=(3, 3), strides=(2, 2), padding=(1, 1)) == 0 and (oh.value, ow.value) == (5, 5)
    # "normalization_term is relevant only if similarity_function is L2"
    assert dims(similarity_function="L1", normalization_term=True) == abi.E_DESC
    # "ignore_nan is relevant only if normalization_term is true"
    assert dims(similarity_function="L2", ignore_nan_input=True) == abi.E_DESC
    assert dims(similarity_function="L2", blocks=(11, 3)) == abi.E_DESC
    d = abi.make_sim_desc((2, 3, 10, 10), 4, dtype=7)
    assert cuda_lib.simnets_similarity_output_dims(C.byref(d), C.byref(oh), C.byref(ow)) == abi.E_DTYPE
    assert cuda_lib.simnets_similarity_output_dims(None, C.byref(oh), C.byref(ow)) == abi.E_NULL
    with pytest.raises(ValueError):
        abi.make_sim_desc((2, 3, 10, 10), 4, blocks=(3, 3, 3))
    assert b"descriptor" in cuda_lib.simnets_status_string(abi.E_DESC)


def test_keras_layer_shape_expectations_of_the_reference(cuda_lib):
    """Output shapes the reference's Keras tests expect (python/simnets/test/keras/__init__.py:46-55, 110-119)."""
    oh, ow = C.c_int32(), C.c_int32()
    for M, pad, st, bl, inp, want in ((10, [0, 1], [1, 1], [2, 2], (3, 10, 13), (10, 9, 14)),
                                      (10, [1, 1], [3, 2], [2, 2], (3, 10, 13), (10, 4, 7)),
                                      (2, [1, 1], [3, 2], [2, 2], (1, 10, 13), (2, 4, 7))):
        d = abi.make_sim_desc((1,) + inp, M, "L1", bl, st, pad)
        assert cuda_lib.simnets_similarity_output_dims(C.byref(d), C.byref(oh), C.byref(ow)) == 0
        assert (M, oh.value, ow.value) == want
    g = abi.MexGeometry()
    for M, pad, st, bl, inp, want in ((10, [1, 0, 1], [1, 1, 1], [1, 2, 2], (3, 10, 13), (50, 9, 14)),
                                      (10, [2, 1, 1], [1, 3, 2], [1, 2, 2], (3, 10, 13), (70, 5, 8)),
                                      (2, [1, 1, 1], [1, 3, 2], [1, 2, 2], (1, 10, 13), (6, 5, 8))):
        d = abi.make_mex_desc((1,) + inp, M, True, pad, st, bl, 2.0, 1.0, False, False, [2], [4])
        assert cuda_lib.simnets_mex_dims(C.byref(d), C.byref(g)) == 0
        assert (g.channels_out_total, g.height_out, g.width_out) == want


def test_mex_geometry_matches_oracle_on_all_cases(cuda_lib, port):
    for c in cases.MEX_SMALL + cases.MEX_CONFIGS:
        d = cases.mex_desc(c)
        g = abi.MexGeometry()
        assert cuda_lib.simnets_mex_dims(C.byref(d), C.byref(g)) == 0, c["name"]
        assert g.as_dict() == port.mex_dims(d).as_dict(), c["name"]


def test_mex_geometry_of_baseline_configs(cuda_lib):
    g = abi.MexGeometry()
    d = cases.mex_desc(cases.MEX_CONFIGS[0])     # config 2
    assert cuda_lib.simnets_mex_dims(C.byref(d), C.byref(g)) == 0
    assert (g.num_regions, g.region_size, g.M, g.K, g.N, g.is_1x1) == (4, 64, 64, 32, 256, 1)
    d = cases.mex_desc(cases.MEX_CONFIGS[1])     # config 4
    assert cuda_lib.simnets_mex_dims(C.byref(d), C.byref(g)) == 0
    assert (g.num_regions, g.M, g.K, g.N, g.channels_out_total) == (1, 256, 16, 16384, 16384)


def test_mex_validation(cuda_lib):
    g = abi.MexGeometry()

    def rc(**kw):
        d = abi.make_mex_desc((1, 4, 8, 8), kw.pop("num_instances", 3), **kw)
        return cuda_lib.simnets_mex_dims(C.byref(d), C.byref(g))

    assert rc(blocks=(4, 1, 1)) == 0
    assert rc(blocks=(5, 1, 1)) == abi.E_DESC              # "block depth must be smaller than input depth"
    assert rc(num_instances=0, blocks=(1, 1, 1)) == abi.E_DESC   # "num_instances must be positive"
    d = abi.make_mex_desc((1, 4, 8, 8), 3, blocks=(1, 1, 1))
    d.n_shared_offset_region = 2                           # "... should be a list with 1 or 3 elements"
    assert cuda_lib.simnets_mex_dims(C.byref(d), C.byref(g)) == abi.E_DESC
    with pytest.raises(ValueError):
        abi.make_mex_desc((1, 4, 8, 8), 3, blocks=(1, 1))
    with pytest.raises(ValueError):
        abi.make_mex_desc((1, 4, 8, 8), 3, blocks=(1, 1, 1), epsilon=float("nan"))


def test_legacy_region_count_helper():
    """get_mex_offsets_nregions keeps the reference's symbol and argument order (src/kernels/mex_dims_helper.cpp:8-44)."""
    assert _mex_dims_helper([32, 16, 16], 64, [32, 1, 1], [0, 0, 0], [32, 1, 1], unshared_offset_region=[2]) == 4
    assert _mex_dims_helper([3, 41, 40], 2, [1, 3, 3], [0, 1, 0], [1, 4, 4], use_unshared_regions=False, shared_offset_region=[3]) == 16
    assert _mex_dims_helper([3, 41, 40], 2, [1, 3, 3], [0, 1, 0], [1, 1, 1], unshared_offset_region=[1, 5, 4]) == 20
    assert _mex_dims_helper([512, 1, 1], 10, [512, 1, 1]) == 1          # length-1 padding/strides defaults are broadcast
    assert _mex_dims_helper([3, 8, 8], 2, [1, 3]) == -1                 # blocks must have three entries


def test_expand_dim_specification():
    assert _expand_dim_specification([3, 10, 13], [2, 2]) == [3, 2, 2]
    assert _expand_dim_specification([None, 3, 10, 13], [-1, 1, -1]) == [3, 1, 13]
    with pytest.raises(ValueError):
        _expand_dim_specification([3, 10, 13], [1])


def test_ops_refuse_cpu_tensors():
    import torch
    from simnets_tf_b200.ops import mex, similarity
    with pytest.raises(RuntimeError, match="no CPU kernels"):
        similarity(torch.zeros(1, 1, 4, 4), torch.zeros(2, 1, 3, 3), torch.ones(2, 1, 3, 3))
    with pytest.raises(RuntimeError, match="no CPU kernels"):
        mex(torch.zeros(1, 2, 4, 4), torch.zeros(1, 3, 2, 1, 1), 3, blocks=[2, 1, 1])
