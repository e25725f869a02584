"""TEST INFRASTRUCTURE: the benchmark networks on the CPU checkers.

Runs a layer specification of `simnets_tf_b200.simnet` with the oracle's operators (numpy in, numpy
out) under torch's CPU autograd, which supplies the glue the reference leaves to TensorFlow (abs of
the weights, normalize_offsets, sum pooling, softmax cross-entropy).  The operators' batch loop is
independent per sample, so a call is split into one shard per thread (ctypes releases the GIL);
parameter-gradient shards are summed afterwards.  Used by tests and by the benchmark's CPU legs only.
"""
import os
from concurrent.futures import ThreadPoolExecutor

import numpy as np
import torch
import torch.nn.functional as F

from simnets_tf_b200 import abi
from simnets_tf_b200 import netspec


def host_cores():
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return os.cpu_count() or 1


class CpuOps(object):
    def __init__(self, oracle, threads=1, dtype=abi.F32):
        self.o = oracle
        self.dtype = dtype
        self.threads = max(1, int(threads))
        self.pool = ThreadPoolExecutor(self.threads) if self.threads > 1 else None

    def _shards(self, batch):
        n = min(self.threads, max(1, batch))
        edges = np.linspace(0, batch, n + 1).astype(int)
        return [(int(a), int(b)) for a, b in zip(edges[:-1], edges[1:]) if b > a]

    def _map(self, fn, batch):
        sh = self._shards(batch)
        if self.pool is None or len(sh) == 1:
            return [fn(a, b) for a, b in sh]
        return list(self.pool.map(lambda ab: fn(*ab), sh))

    # ---- Similarity
    def _sd(self, kw, shape):
        return abi.make_sim_desc(shape, kw["num_instances"], kw.get("similarity_function", "L2"), kw["blocks"], kw["strides"],
                                 kw["padding"], kw.get("normalization_term", False), kw.get("normalization_term_fudge", 0.001),
                                 kw.get("ignore_nan_input", False), kw.get("out_of_bounds_value", 0.0), dtype=self.dtype)

    def sim_fwd(self, kw, x, t, w):
        return np.concatenate(self._map(lambda a, b: self.o.similarity_forward(self._sd(kw, x[a:b].shape), x[a:b], t, w), len(x)))

    def sim_dx(self, kw, x, t, w, dy):
        return np.concatenate(self._map(lambda a, b: self.o.similarity_input_grad(self._sd(kw, x[a:b].shape), x[a:b], t, w, dy[a:b]), len(x)))

    def sim_dp(self, kw, x, t, w, dy):
        parts = self._map(lambda a, b: self.o.similarity_params_grad(self._sd(kw, x[a:b].shape), x[a:b], t, w, dy[a:b]), len(x))
        return sum(p[0] for p in parts), sum(p[1] for p in parts)

    # ---- MEX
    def _md(self, kw, shape):
        return abi.make_mex_desc(shape, kw["num_instances"], kw.get("softmax_mode", False), kw.get("padding", [0, 0, 0]),
                                 kw.get("strides", [1, 1, 1]), kw["blocks"], kw.get("epsilon", 1.0),
                                 kw.get("blocks_out_of_bounds_value", 0.0), kw.get("blocks_round_down", True),
                                 kw.get("use_unshared_regions", True), kw.get("shared_offset_region", [-1]),
                                 kw.get("unshared_offset_region", [-1]), dtype=self.dtype)

    def mex_fwd(self, kw, x, off):
        return np.concatenate(self._map(lambda a, b: self.o.mex_forward(self._md(kw, x[a:b].shape), x[a:b], off), len(x)))

    def mex_dx(self, kw, x, off, y, dy):
        return np.concatenate(self._map(lambda a, b: self.o.mex_input_grad(self._md(kw, x[a:b].shape), x[a:b], off, y[a:b], dy[a:b]), len(x)))

    def mex_doff(self, kw, x, off, y, dy):
        return sum(self._map(lambda a, b: self.o.mex_offsets_grad(self._md(kw, x[a:b].shape), x[a:b], off, y[a:b], dy[a:b]), len(x)))


def _np(t):
    return np.ascontiguousarray(t.detach().numpy())


class _SimFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ops, kw, x, t, w):
        ctx.ops, ctx.kw = ops, kw
        ctx.save_for_backward(x, t, w)
        return torch.from_numpy(ops.sim_fwd(kw, _np(x), _np(t), _np(w)))

    @staticmethod
    def backward(ctx, dy):
        x, t, w = ctx.saved_tensors
        gx = torch.from_numpy(ctx.ops.sim_dx(ctx.kw, _np(x), _np(t), _np(w), _np(dy))) if ctx.needs_input_grad[2] else None
        gt, gw = ctx.ops.sim_dp(ctx.kw, _np(x), _np(t), _np(w), _np(dy))
        return None, None, gx, torch.from_numpy(gt), torch.from_numpy(gw)


class _MexFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ops, kw, x, off):
        y = torch.from_numpy(ops.mex_fwd(kw, _np(x), _np(off)))
        ctx.ops, ctx.kw = ops, kw
        ctx.save_for_backward(x, off, y)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, off, y = ctx.saved_tensors
        gx = torch.from_numpy(ctx.ops.mex_dx(ctx.kw, _np(x), _np(off), _np(y), _np(dy))) if ctx.needs_input_grad[2] else None
        go = torch.from_numpy(ctx.ops.mex_doff(ctx.kw, _np(x), _np(off), _np(y), _np(dy)))
        return None, None, gx, go


class CpuSimNet(object):
    """Same parameters (by seed) and same arithmetic order of layers as `simnets_tf_b200.simnet.SimNet`."""

    def __init__(self, spec, oracle, seed=0, threads=1, dtype=np.float32):
        self.spec = spec
        self.dtype = np.dtype(dtype)
        self.ops = CpuOps(oracle, threads, abi.F64 if self.dtype == np.float64 else abi.F32)
        self.params = []

        def nregions(chw, num_instances, blocks, strides, kw):      # the checker's own dimension code, not the CUDA library's
            d = abi.make_mex_desc([1] + list(chw), num_instances, kw.get("softmax_mode", False), [0, 0, 0], strides, blocks,
                                  kw.get("epsilon", 1.0), 0.0, True, kw.get("use_unshared_regions", True),
                                  kw.get("shared_offset_region", [-1]), kw.get("unshared_offset_region", [-1]))
            return oracle.mex_dims(d).num_regions

        for entry, values in zip(spec["layers"], netspec.init_parameters(spec, seed, nregions)):
            if values is None:
                self.params.append(None)
            else:
                self.params.append({k: torch.from_numpy(v.astype(self.dtype)).requires_grad_(True) for k, v in values.items()})

    def parameters(self):
        """In the order torch lists them for SimNet: per layer (weights, templates) / (offsets)."""
        out = []
        for p in self.params:
            if p is None:
                continue
            out.extend([p["weights"], p["templates"]] if "templates" in p else [p["offsets"]])
        return out

    def forward(self, x):
        for entry, p in zip(self.spec["layers"], self.params):
            kind = entry[0]
            if kind == "similarity":
                x = _SimFn.apply(self.ops, entry[1], x, p["templates"], torch.abs(p["weights"]))
            elif kind == "mex":
                off = p["offsets"]
                kw = dict(entry[1], blocks=list(off.shape[2:]))
                if entry[1].get("normalize_offsets"):
                    flat = off.reshape(off.shape[0] * off.shape[1], -1)
                    off = (flat - torch.logsumexp(flat, dim=1, keepdim=True)).reshape(off.shape)
                kw["strides"] = [kw["blocks"][i] if s == -1 else s for i, s in enumerate(kw["strides"])]
                x = _MexFn.apply(self.ops, kw, x, off)
            elif kind == "sumpool":
                x = F.avg_pool2d(x, entry[1]) * float(entry[1] * entry[1])
            elif kind == "flatten":
                x = x.flatten(1)
        return x

    def step(self, x, labels, global_batch=None):
        """One forward + backward; returns (loss, [gradients in parameters() order])."""
        for p in self.parameters():
            p.grad = None
        logits = self.forward(torch.from_numpy(np.ascontiguousarray(x, dtype=self.dtype)))
        loss = F.cross_entropy(logits, torch.from_numpy(np.asarray(labels)).long(), reduction="sum") / float(global_batch or len(x))
        loss.backward()
        return float(loss.detach()), [p.grad.numpy() for p in self.parameters()]
