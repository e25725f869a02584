"""Loader for the CUDA library (libsimnets_b200.so) and thin ctypes prototypes of its C ABI.

There is no CPU path: if the library has not been built the import of an operator fails with an
error that says how to build it, and operators reject tensors that do not live on a CUDA device.
"""
import ctypes as C
import os

from . import abi

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libsimnets_b200.so")
_lib = None

_P = C.c_void_p


class SimnetsError(RuntimeError):
    def __init__(self, status, message):
        super(SimnetsError, self).__init__("simnets_b200: %s (status %d)" % (message, status))
        self.status = status


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("%s is missing: build it with `python -m simnets_tf_b200.build` "
                              "(this package has no CPU fallback)" % LIB_PATH)
        l = C.CDLL(LIB_PATH)
        sd, md = C.POINTER(abi.SimDesc), C.POINTER(abi.MexDesc)
        l.simnets_status_string.restype = C.c_char_p
        l.simnets_status_string.argtypes = [C.c_int]
        l.simnets_launch_count.restype = C.c_uint64
        l.simnets_abi_version.restype = C.c_int
        l.simnets_similarity_output_dims.argtypes = [sd, C.POINTER(C.c_int32), C.POINTER(C.c_int32)]
        l.simnets_similarity_workspace_bytes.restype = C.c_size_t
        l.simnets_similarity_workspace_bytes.argtypes = [sd]
        l.simnets_similarity_forward.argtypes = [sd, _P, _P, _P, _P, _P, C.c_size_t, _P]
        l.simnets_similarity_input_grad.argtypes = [sd, _P, _P, _P, _P, _P, _P, C.c_size_t, _P]
        l.simnets_similarity_params_grad.argtypes = [sd, _P, _P, _P, _P, _P, _P, _P, C.c_size_t, _P]
        l.simnets_mex_dims.argtypes = [md, C.POINTER(abi.MexGeometry)]
        l.simnets_mex_workspace_bytes.restype = C.c_size_t
        l.simnets_mex_workspace_bytes.argtypes = [md]
        l.simnets_mex_forward.argtypes = [md, _P, _P, _P, _P, C.c_size_t, _P]
        l.simnets_mex_workspace_status.argtypes = [_P, _P, C.POINTER(C.c_int32)]
        l.simnets_mex_forward_pool2x2.argtypes = [md, _P, _P, _P, _P, _P, C.c_size_t, _P]
        l.simnets_mex_workspace_maxima.restype = C.c_void_p
        l.simnets_mex_workspace_maxima.argtypes = [md, _P]
        l.simnets_similarity_forward_extrema.argtypes = [sd, _P, _P, _P, _P, _P, _P, _P, C.c_size_t, _P]
        l.simnets_similarity_workspace_status.argtypes = [_P, _P, C.POINTER(C.c_int32)]
        l.simnets_softmax_cross_entropy_workspace_bytes.restype = C.c_size_t
        l.simnets_softmax_cross_entropy_workspace_bytes.argtypes = [C.c_int32]
        l.simnets_softmax_cross_entropy.argtypes = [C.c_int32, C.c_int32, C.c_float, _P, _P, _P, _P, _P, C.c_size_t, _P]
        l.simnets_mex_forward_static_scratch.argtypes = [md, _P, _P, _P, _P]
        l.simnets_mex_input_grad.argtypes = [md, _P, _P, _P, _P, _P, _P, C.c_size_t, _P]
        l.simnets_mex_offsets_grad.argtypes = [md, _P, _P, _P, _P, _P, _P, C.c_size_t, _P]
        l.simnets_mex_backward.argtypes = [md, _P, _P, _P, _P, _P, _P, _P, C.c_size_t, _P]
        l.simnets_normalize_offsets_forward.argtypes = [C.c_int64, C.c_int32, _P, _P, _P]
        l.simnets_normalize_offsets_backward.argtypes = [C.c_int64, C.c_int32, _P, _P, _P, _P]
        l.simnets_sum_pool2x2_forward.argtypes = [C.c_int64, C.c_int32, C.c_int32, _P, _P, _P]
        l.simnets_fp32_fma_probe.restype = C.c_int64
        l.simnets_fp32_fma_probe.argtypes = [C.c_int32, C.c_int32, _P, _P]
        l.get_mex_offsets_nregions.restype = C.c_int
        _lib = l
    return _lib


def check(status):
    if status != 0:
        msg = lib().simnets_status_string(int(status)).decode()
        if status in (abi.E_DESC, abi.E_DTYPE, abi.E_NULL):
            raise ValueError("simnets_b200: %s (status %d)" % (msg, status))
        raise SimnetsError(status, msg)


def launch_count():
    return int(lib().simnets_launch_count())
