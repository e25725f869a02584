"""Plumbing between torch tensors and the C ABI: dtype codes, pointers, the current stream and a
per-(device, stream) scratch workspace that grows on demand."""

import torch

from . import abi

_WORKSPACES = {}

# Descriptor flags OR-ed into every op call of this process; 0 unless a program sets it (an A/B measurement that
# wants, say, abi.FLAG_MEX_NO_PAIR_TILES on every layer assigns it before the first call).
DEFAULT_FLAGS = 0


def dtype_code(t):
    if t.dtype == torch.float32:
        return abi.F32
    if t.dtype == torch.float64:
        return abi.F64
    raise TypeError("simnets ops are registered for float32 and float64 only, got %s" % t.dtype)


def require_cuda(*tensors):
    dev = tensors[0].device
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("simnets_b200 has no CPU kernels: every tensor must live on a CUDA device")
        if t.device != dev:
            raise RuntimeError("all tensors of one op call must be on the same device")
        if t.dtype != tensors[0].dtype:
            raise TypeError("all tensors of one op call must share a dtype")
    return dev


def stream_ptr(dev):
    return torch.cuda.current_stream(dev).cuda_stream


def workspace(dev, nbytes):
    """A scratch buffer of at least `nbytes` for the current stream of `dev` (contents undefined)."""
    key = (dev.index, stream_ptr(dev))
    buf = _WORKSPACES.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=dev)
        _WORKSPACES[key] = buf
    return buf


class OpProfile(object):
    """Optional per-op device timing: when enabled, every operator call is bracketed by CUDA events on
    the stream it launches on, together with the algorithmic bytes and term count of that call."""

    def __init__(self):
        self.enabled = False
        self.rows = {}

    def start(self):
        self.enabled, self.rows = True, {}

    def stop(self):
        """Stop recording and return {key: dict(calls, ms, bytes, terms)} (synchronises)."""
        self.enabled = False
        torch.cuda.synchronize()
        out = {}
        for key, recs in self.rows.items():
            out[key] = dict(calls=len(recs), ms=sum(s.elapsed_time(e) for s, e, _, _ in recs),
                            bytes=sum(r[2] for r in recs), terms=sum(r[3] for r in recs))
        self.rows = {}
        return out


PROFILE = OpProfile()


class timed(object):
    """`with timed(op, signature, algorithmic_bytes, terms):` around one C-ABI call."""

    def __init__(self, op, sig, nbytes, terms):
        self.key, self.nbytes, self.terms = "%s[%s]" % (op, sig), nbytes, terms

    def __enter__(self):
        if PROFILE.enabled:
            self.s = torch.cuda.Event(enable_timing=True)
            self.e = torch.cuda.Event(enable_timing=True)
            self.s.record()
        return self

    def __exit__(self, *exc):
        if PROFILE.enabled and exc[0] is None:
            self.e.record()
            PROFILE.rows.setdefault(self.key, []).append((self.s, self.e, self.nbytes, self.terms))
        return False
