"""Softmax cross-entropy over logit rows as one library kernel (loss and gradient in the same launch): the loss the
reference's example networks train with (HUJI-Deep/simnets-tf README.md:108-111)."""
import ctypes as C

import torch

from .. import _lib
from .._torch_glue import require_cuda, stream_ptr, workspace


def softmax_cross_entropy_with_grad(logits, labels, scale=1.0):
    """(loss, dlogits): loss = scale * sum_b (logsumexp(logits[b]) - logits[b, labels[b]]) as a 0-d tensor and its
    gradient with respect to the logits.  float32 CUDA logits [batch, classes], int64 CUDA labels [batch]."""
    dev = require_cuda(logits)
    if not labels.is_cuda or labels.device != dev:
        raise RuntimeError("labels must live on the device of the logits")
    if logits.dtype != torch.float32 or labels.dtype != torch.int64 or logits.dim() != 2 or labels.shape != logits.shape[:1]:
        raise ValueError("logits must be float32 [batch, classes] and labels int64 [batch]")
    logits, labels = logits.contiguous(), labels.contiguous()
    loss = torch.empty((), dtype=torch.float32, device=dev)
    dlogits = torch.empty_like(logits)
    lib = _lib.lib()
    with torch.cuda.device(dev):
        n = lib.simnets_softmax_cross_entropy_workspace_bytes(logits.shape[0])
        ws = workspace(dev, n)
        _lib.check(lib.simnets_softmax_cross_entropy(logits.shape[0], logits.shape[1], C.c_float(scale), logits.data_ptr(), labels.data_ptr(),
                                                     loss.data_ptr(), dlogits.data_ptr(), ws.data_ptr(), ws.numel(), stream_ptr(dev)))
    return loss, dlogits


class _SoftmaxCrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, labels, scale):
        loss, dlogits = softmax_cross_entropy_with_grad(logits, labels, scale)
        ctx.save_for_backward(dlogits)
        return loss

    @staticmethod
    def backward(ctx, grad):
        (dlogits,) = ctx.saved_tensors
        return dlogits * grad, None, None


def softmax_cross_entropy(logits, labels, scale=1.0):
    """Differentiable (w.r.t. the logits) form of softmax_cross_entropy_with_grad."""
    return _SoftmaxCrossEntropy.apply(logits, labels, float(scale))
