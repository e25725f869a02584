"""Plumbing between torch tensors and the C ABI: dtype codes, pointers, the current stream and a
per-(device, stream) scratch workspace that grows on demand."""
import torch

from . import abi

_WORKSPACES = {}


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
