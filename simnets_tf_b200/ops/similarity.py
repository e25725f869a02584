"""`similarity` and its gradient ops, with the signature of the reference's python wrapper
(HUJI-Deep/simnets-tf python/simnets/ops/similarity.py:48-121) and the gradient wiring of its
`_similarity_grad` (same file, :18-45).  Tensors are torch CUDA tensors; the work is done by the
CUDA library through the C ABI.
"""
import ctypes as C

import torch

from .. import _lib, abi
from .. import _torch_glue
from .._torch_glue import dtype_code, require_cuda, stream_ptr, timed, workspace

_DEFAULTS = dict(similarity_function="L2", blocks=[3, 3], strides=[2, 2], padding=[0, 0], normalization_term=False,
                 normalization_term_fudge=0.001, ignore_nan_input=False, out_of_bounds_value=0.0)


def _attrs(**given):
    """Op attrs with the op registration's defaults (reference src/ops/similarity_op.cpp:61-75) for every None."""
    out = dict(_DEFAULTS)
    for k, v in given.items():
        if v is not None:
            out[k] = v
    return out


def _desc(input, templates, weights, attrs, flags=0):
    if input.dim() != 4 or templates.dim() != 4 or weights.dim() != 4:
        raise ValueError("input, templates and weights must be 4-D")
    if templates.shape != weights.shape:
        raise ValueError("templates and weights must have the same shape")
    if templates.shape[1] != input.shape[1]:
        raise ValueError("Number of channels mismatch between input and template")
    blocks = list(attrs["blocks"])
    if list(templates.shape[2:]) != [int(b) for b in blocks]:
        raise ValueError("templates spatial shape %s does not match blocks %s" % (list(templates.shape[2:]), blocks))
    return abi.make_sim_desc(input.shape, templates.shape[0], attrs["similarity_function"], blocks, attrs["strides"],
                             attrs["padding"], attrs["normalization_term"], attrs["normalization_term_fudge"],
                             attrs["ignore_nan_input"], attrs["out_of_bounds_value"], dtype=dtype_code(input), flags=flags | _torch_glue.DEFAULT_FLAGS)


def _cost(d, y_numel, kind):
    """(signature, algorithmic bytes, terms) of one call: bytes = every input read once + every output written once."""
    k = d.channels * d.block_h * d.block_w
    x, p, e = d.batch * d.channels * d.height * d.width, d.num_instances * k, 4 if d.dtype == abi.F32 else 8
    nbytes = {"fwd": x + 2 * p + y_numel, "dx": 2 * x + 2 * p + y_numel, "dp": x + y_numel + 4 * p}[kind] * e
    sig = "B%d C%d %dx%d M%d K%d" % (d.batch, d.channels, d.height, d.width, d.num_instances, k)
    return sig, nbytes, y_numel * k


def _ws(d, dev):
    n = _lib.lib().simnets_similarity_workspace_bytes(C.byref(d))
    buf = workspace(dev, n)
    return buf.data_ptr(), buf.numel()


def similarity_forward(input, templates, weights, flags=0, extrema=None, **attrs):
    """The `Similarity` op: [batch, templates, out_h, out_w].  `extrema=(max_ptr, min_ptr)`: device addresses (or None)
    that receive the per-pixel maximum / minimum of the output over the templates, float32 [batch, out_h, out_w]."""
    attrs = _attrs(**attrs)
    dev = require_cuda(input, templates, weights)
    input, templates, weights = input.contiguous(), templates.contiguous(), weights.contiguous()
    d = _desc(input, templates, weights, attrs, flags)
    oh, ow = C.c_int32(), C.c_int32()
    _lib.check(_lib.lib().simnets_similarity_output_dims(C.byref(d), C.byref(oh), C.byref(ow)))
    y = torch.empty((input.shape[0], templates.shape[0], oh.value, ow.value), dtype=input.dtype, device=dev)
    with torch.cuda.device(dev):
        ws, n = _ws(d, dev)
        with timed("similarity_forward", *_cost(d, y.numel(), "fwd")):
            if extrema is not None and (extrema[0] or extrema[1]):
                _lib.check(_lib.lib().simnets_similarity_forward_extrema(C.byref(d), input.data_ptr(), templates.data_ptr(), weights.data_ptr(),
                                                                         y.data_ptr(), extrema[0], extrema[1], ws, n, stream_ptr(dev)))
            else:
                _lib.check(_lib.lib().simnets_similarity_forward(C.byref(d), input.data_ptr(), templates.data_ptr(), weights.data_ptr(),
                                                                 y.data_ptr(), ws, n, stream_ptr(dev)))
    return y


def similarity_input_grad(input, templates, weights, input_grad, flags=0, **attrs):
    """The `SimilarityInputGrad` op (its fourth input is the gradient w.r.t. the op's output)."""
    attrs = _attrs(**attrs)
    dev = require_cuda(input, templates, weights, input_grad)
    input, templates, weights, dy = input.contiguous(), templates.contiguous(), weights.contiguous(), input_grad.contiguous()
    d = _desc(input, templates, weights, attrs, flags)
    dx = torch.empty_like(input)
    with torch.cuda.device(dev):
        ws, n = _ws(d, dev)
        with timed("similarity_input_grad", *_cost(d, dy.numel(), "dx")):
            _lib.check(_lib.lib().simnets_similarity_input_grad(C.byref(d), input.data_ptr(), templates.data_ptr(), weights.data_ptr(),
                                                                dy.data_ptr(), dx.data_ptr(), ws, n, stream_ptr(dev)))
    return dx


def similarity_parameters_grad(input, templates, weights, output_grad, flags=0, out=None, **attrs):
    """The `SimilarityParametersGrad` op: (templates_grad, weights_grad).

    `out=(dt, dw)` writes into caller-owned tensors (e.g. slices of a data-parallel gradient
    bucket); with `flags & FLAG_ACCUMULATE` the results are added to them."""
    attrs = _attrs(**attrs)
    dev = require_cuda(input, templates, weights, output_grad)
    input, templates, weights, dy = input.contiguous(), templates.contiguous(), weights.contiguous(), output_grad.contiguous()
    d = _desc(input, templates, weights, attrs, flags)
    if out is None:
        dt, dw = torch.empty_like(templates), torch.empty_like(weights)
    else:
        dt, dw = out
        assert dt.is_contiguous() and dw.is_contiguous() and dt.numel() == templates.numel() and dw.numel() == weights.numel()
    with torch.cuda.device(dev):
        ws, n = _ws(d, dev)
        with timed("similarity_params_grad", *_cost(d, dy.numel(), "dp")):
            _lib.check(_lib.lib().simnets_similarity_params_grad(C.byref(d), input.data_ptr(), templates.data_ptr(), weights.data_ptr(),
                                                                 dy.data_ptr(), dt.data_ptr(), dw.data_ptr(), ws, n, stream_ptr(dev)))
    return dt, dw


class _Similarity(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, templates, weights, attrs, flags=0, extrema=None, grad_sinks=None):
        ctx.attrs, ctx.flags, ctx.grad_sinks = attrs, flags, grad_sinks
        ctx.save_for_backward(input, templates, weights)
        return similarity_forward(input, templates, weights, flags=flags, extrema=extrema, **attrs)

    @staticmethod
    def backward(ctx, grad):
        input, templates, weights = ctx.saved_tensors
        gi = gt = gw = None
        if ctx.needs_input_grad[0]:
            gi = similarity_input_grad(input, templates, weights, grad, flags=ctx.flags, **ctx.attrs)
        if ctx.needs_input_grad[1] or ctx.needs_input_grad[2]:
            if ctx.grad_sinks is not None:          # both parameter gradients are added straight into the caller's tensors
                similarity_parameters_grad(input, templates, weights, grad, flags=ctx.flags | abi.FLAG_ACCUMULATE, out=ctx.grad_sinks, **ctx.attrs)
            else:
                gt, gw = similarity_parameters_grad(input, templates, weights, grad, flags=ctx.flags, **ctx.attrs)
        return gi, gt, gw, None, None, None, None


def similarity(input, templates, weights, similarity_function=None, blocks=None, strides=None, padding=None,
               normalization_term=None, normalization_term_fudge=None, ignore_nan_input=None, out_of_bounds_value=None,
               name=None, ksize=None):
    """Computes a similarity measure given 4-D `input`, `templates` and `weights` tensors.

    Same arguments, defaults and result as the reference's `simnets.ops.similarity.similarity`; `name`
    is accepted and ignored, `ksize` is an alias of `blocks` (the name the reference's README uses).
    Differentiable w.r.t. all three tensors.
    """
    if blocks is None and ksize is not None:
        blocks = ksize
    attrs = _attrs(similarity_function=similarity_function, blocks=blocks, strides=strides, padding=padding,
                   normalization_term=normalization_term, normalization_term_fudge=normalization_term_fudge,
                   ignore_nan_input=ignore_nan_input, out_of_bounds_value=out_of_bounds_value)
    return _Similarity.apply(input, templates, weights, attrs)


def similarity_of_raw_weights(input, templates, raw_weights, flags=0, extrema=None, grad_sinks=None, **attrs):
    """`similarity(input, templates, abs(raw_weights), ...)`, differentiable w.r.t. all three tensors, with the absolute
    value and its gradient taken inside the library's kernels (abi.FLAG_SIM_ABS_WEIGHTS): what the reference's Keras
    layer computes with `K.abs(self.sweights)` in front of the op (python/simnets/keras.py:65)."""
    return _Similarity.apply(input, templates, raw_weights, _attrs(**attrs), flags | abi.FLAG_SIM_ABS_WEIGHTS, extrema, grad_sinks)
