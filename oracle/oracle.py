"""TEST INFRASTRUCTURE: numpy front end for the two CPU checkers built by oracle/Makefile.

`load("port")` is the restatement (oracle/liboracle.so); `load("reference")` is the reference
project's own CPU templates (oracle/_ref/libsimnets_ref.so).  Both export the same entry points.
Only tests, the smoke check and the benchmark's CPU-baseline leg may import this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

from simnets_tf_b200 import abi

_HERE = os.path.dirname(os.path.abspath(__file__))
_PATHS = {"port": os.path.join(_HERE, "liboracle.so"), "reference": os.path.join(_HERE, "_ref", "libsimnets_ref.so")}
_CACHE = {}


def build(reference_dir=None):
    """Compile the checkers (g++ only).  The reference build is skipped unless `reference_dir` exists."""
    cmd = ["make", "-s", "-C", _HERE]
    if reference_dir and os.path.isdir(reference_dir):
        cmd.append("REFERENCE_DIR=" + reference_dir)
    subprocess.check_call(cmd)


def available(kind):
    return os.path.exists(_PATHS[kind])


class Oracle(object):
    def __init__(self, kind):
        self.kind = kind
        self.lib = C.CDLL(_PATHS[kind])
        self.lib.oracle_kind.restype = C.c_char_p
        assert self.lib.oracle_kind().decode() == kind

    @staticmethod
    def _np(d):
        return np.float32 if d.dtype == abi.F32 else np.float64

    @staticmethod
    def _p(a):
        return a.ctypes.data_as(C.c_void_p)

    def _in(self, d, *arrs):
        return [np.ascontiguousarray(a, dtype=self._np(d)) for a in arrs]

    @staticmethod
    def _check(rc):
        if rc != 0:
            raise ValueError("oracle rejected the call: status %d" % rc)

    # -- Similarity
    def sim_out_shape(self, d):
        oh, ow = C.c_int32(), C.c_int32()
        self._check(self.lib.oracle_similarity_output_dims(C.byref(d), C.byref(oh), C.byref(ow)))
        return (d.batch, d.num_instances, oh.value, ow.value)

    def similarity_forward(self, d, x, t, w, naive=False):
        x, t, w = self._in(d, x, t, w)
        y = np.empty(self.sim_out_shape(d), dtype=self._np(d))
        fn = self.lib.oracle_similarity_naive if naive else self.lib.oracle_similarity_forward
        self._check(fn(C.byref(d), self._p(x), self._p(t), self._p(w), self._p(y)))
        return y

    def similarity_input_grad(self, d, x, t, w, dy):
        x, t, w, dy = self._in(d, x, t, w, dy)
        dx = np.empty_like(x)
        self._check(self.lib.oracle_similarity_input_grad(C.byref(d), self._p(x), self._p(t), self._p(w), self._p(dy), self._p(dx)))
        return dx

    def similarity_params_grad(self, d, x, t, w, dy):
        x, t, w, dy = self._in(d, x, t, w, dy)
        dt, dw = np.empty_like(t), np.empty_like(w)
        self._check(self.lib.oracle_similarity_params_grad(C.byref(d), self._p(x), self._p(t), self._p(w), self._p(dy),
                                                           self._p(dt), self._p(dw)))
        return dt, dw

    # -- MEX
    def mex_dims(self, d):
        g = abi.MexGeometry()
        self._check(self.lib.oracle_mex_dims(C.byref(d), C.byref(g)))
        return g

    def mex_out_shape(self, d):
        g = self.mex_dims(d)
        return (d.batch, g.channels_out_total, g.height_out, g.width_out)

    def mex_offsets_shape(self, d):
        g = self.mex_dims(d)
        return (g.num_regions, d.num_instances, g.block_c, g.block_h, g.block_w)

    def mex_forward(self, d, x, off, naive=False):
        x, off = self._in(d, x, off)
        y = np.empty(self.mex_out_shape(d), dtype=self._np(d))
        fn = self.lib.oracle_mex_naive if naive else self.lib.oracle_mex_forward
        self._check(fn(C.byref(d), self._p(x), self._p(off), self._p(y)))
        return y

    def mex_input_grad(self, d, x, off, y, dy):
        x, off, y, dy = self._in(d, x, off, y, dy)
        dx = np.empty_like(x)
        self._check(self.lib.oracle_mex_input_grad(C.byref(d), self._p(x), self._p(off), self._p(y), self._p(dy), self._p(dx)))
        return dx

    def mex_offsets_grad(self, d, x, off, y, dy):
        x, off, y, dy = self._in(d, x, off, y, dy)
        doff = np.empty_like(off)
        self._check(self.lib.oracle_mex_offsets_grad(C.byref(d), self._p(x), self._p(off), self._p(y), self._p(dy), self._p(doff)))
        return doff


def load(kind="port"):
    if kind not in _CACHE:
        if not available(kind):
            raise FileNotFoundError("%s is not built; run `make -C oracle`" % _PATHS[kind])
        _CACHE[kind] = Oracle(kind)
    return _CACHE[kind]
