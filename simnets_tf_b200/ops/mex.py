"""`mex` and its gradient ops, with the signature of the reference's python wrapper
(HUJI-Deep/simnets-tf python/simnets/ops/mex.py:114-195), its `_mex_dims_helper` (:17-38),
`_expand_dim_specification` (:84-112) and the gradient wiring of `_mex_grad` (:47-81).
"""
import ctypes as C

import torch

from .. import _lib, abi
from .. import _torch_glue
from .._torch_glue import dtype_code, require_cuda, stream_ptr, timed, workspace

_DEFAULTS = dict(softmax_mode=False, padding=[0, 0, 0], strides=[1, 1, 1], blocks=[1, 1, 1], epsilon=1.0,
                 blocks_out_of_bounds_value=0.0, blocks_round_down=True, use_unshared_regions=True,
                 shared_offset_region=[-1], unshared_offset_region=[-1])


def _attrs(**given):
    """Op attrs with the op registration's defaults (reference src/ops/mex_op.cpp:58-74) for every None."""
    out = dict(_DEFAULTS)
    for k, v in given.items():
        if v is not None:
            out[k] = v
    return out


def _mex_dims_helper(input_dim, num_instances, blocks, padding=[0], strides=[1], blocks_round_down=True,
                     use_unshared_regions=True, shared_offset_region=[-1], unshared_offset_region=[-1]):
    """Number of offset regions for an input of shape `input_dim` = [C, H, W] (or -1 if invalid)."""
    args = []

    def add_array(l):
        l = [int(e) for e in l]
        args.extend([C.c_int(len(l)), (C.c_int * len(l))(*l)])

    add_array(input_dim)
    add_array(padding)
    add_array(strides)
    args.extend([C.c_int(num_instances), C.c_int(blocks_round_down), C.c_int(use_unshared_regions)])
    add_array(blocks)
    add_array(shared_offset_region)
    add_array(unshared_offset_region)
    return _lib.lib().get_mex_offsets_nregions(*args)


def _expand_dim_specification(image_shape, dim_spec):
    """Expand a 2- or 3-long dimension specification: prepend -1 to a pair, then replace every -1
    with the corresponding image dimension (`image_shape` has 3 entries, or 4 with the batch)."""
    if len(dim_spec) != 2 and len(dim_spec) != 3:
        raise ValueError('Bad dimensions specifications, should be a list of two or three, got %s' % dim_spec)
    image_shape = list(image_shape)
    if len(image_shape) == 3:
        image_shape = [None] + image_shape
    dim_spec = list(dim_spec)
    if len(dim_spec) == 2:
        dim_spec = [-1] + dim_spec
    for i in range(3):
        if dim_spec[i] == -1:
            dim_spec[i] = image_shape[i + 1]
    return dim_spec


def _desc_of(shape, dtype, num_instances, attrs, flags=0):
    if len(shape) != 4:
        raise ValueError("input must be 4-D")
    return abi.make_mex_desc(shape, num_instances, attrs["softmax_mode"], attrs["padding"], attrs["strides"],
                             attrs["blocks"], attrs["epsilon"], attrs["blocks_out_of_bounds_value"], attrs["blocks_round_down"],
                             attrs["use_unshared_regions"], attrs["shared_offset_region"], attrs["unshared_offset_region"],
                             dtype=abi.F32 if dtype == torch.float32 else abi.F64, flags=flags | _torch_glue.DEFAULT_FLAGS)


def _desc(input, num_instances, attrs, flags=0):
    dtype_code(input)           # (rejects anything but float32 / float64)
    return _desc_of(tuple(input.shape), input.dtype, num_instances, attrs, flags)


def _geometry(d):
    g = abi.MexGeometry()
    _lib.check(_lib.lib().simnets_mex_dims(C.byref(d), C.byref(g)))
    return g


def _check_dy(dy, input, g, pooled):
    """dy has the op's output shape, or half its height and width when it is given pooled."""
    k = 2 if pooled else 1
    want = (input.shape[0], g.channels_out_total, g.height_out // k, g.width_out // k)
    if tuple(dy.shape) != want:
        raise ValueError("output_grad must have shape %s, got %s" % (want, tuple(dy.shape)))


def _check_offsets(offsets, g, num_instances):
    want = (g.num_regions, num_instances, g.block_c, g.block_h, g.block_w)
    if tuple(offsets.shape) != want:
        raise ValueError("offsets must have shape %s, got %s" % (want, tuple(offsets.shape)))


def _cost(d, g, kind):
    """(signature, algorithmic bytes, terms) of one call: bytes = every input read once + every output written once."""
    x, o, y = d.batch * d.channels * d.height * d.width, g.num_regions * g.M * g.K, d.batch * g.M * g.N
    e = 4 if d.dtype == abi.F32 else 8
    nbytes = {"fwd": x + o + y, "dx": 2 * x + o + 2 * y, "doff": x + 2 * o + 2 * y, "bwd": 2 * x + 2 * o + 2 * y}[kind] * e
    sig = "B%d C%d %dx%d M%d K%d N%d R%d" % (d.batch, d.channels, d.height, d.width, g.M, g.K, g.N, g.num_regions)
    return sig, nbytes, y * g.K


def _ws(d, dev, own=None):
    n = _lib.lib().simnets_mex_workspace_bytes(C.byref(d))
    if own is not None:
        if own.dtype != torch.uint8 or own.device != dev or not own.is_contiguous() or own.numel() < n:
            raise ValueError("workspace: need a contiguous uint8 tensor of at least %d bytes on %s" % (n, dev))
        return own.data_ptr(), own.numel()
    buf = workspace(dev, n)
    return buf.data_ptr(), buf.numel()


def mex_layer_workspace(input, num_instances, pooled=False, flags=0, **attrs):
    """A workspace of one layer's own, large enough for its forward and gradient calls: give it to `mex_forward`
    as `workspace=` and to the gradient ops as `primed_workspace=`, and they reuse the per-position maxima and
    the offsets tables of the forward pass instead of computing them again."""
    return mex_layer_workspace_for(tuple(input.shape), input.dtype, require_cuda(input), num_instances, pooled=pooled, flags=flags, **attrs)


def mex_layer_workspace_for(input_shape, dtype, device, num_instances, pooled=False, flags=0, **attrs):
    """`mex_layer_workspace` for an input that does not exist yet (shape, dtype and device given)."""
    attrs = _attrs(**attrs)
    n = 256
    for f in (flags, flags | (abi.FLAG_MEX_DY_POOLED2 if pooled else 0)):
        d = _desc_of(input_shape, dtype, num_instances, attrs, f)
        n = max(n, int(_lib.lib().simnets_mex_workspace_bytes(C.byref(d))))
    return torch.empty(n, dtype=torch.uint8, device=device)


def mex_workspace_maxima(input_shape, dtype, num_instances, workspace, flags=0, **attrs):
    """Device address inside `workspace` (a tensor from `mex_layer_workspace`) where the forward pass of this layer reads the
    per-position extrema of its patches, or None for shapes that find them on the fly.  A layer in front that writes them
    there (ops.similarity.similarity_forward(..., extrema=...)) lets `mex_forward(..., flags=FLAG_MEX_MAXIMA_GIVEN)` skip
    its own pass over the input; only valid when every patch is exactly the channels of one pixel."""
    d = _desc_of(tuple(input_shape), dtype, num_instances, _attrs(**attrs), flags)
    p = _lib.lib().simnets_mex_workspace_maxima(C.byref(d), workspace.data_ptr())
    return int(p) if p else None


def _primed(flags, primed_workspace):
    return flags | (abi.FLAG_MEX_WORKSPACE_PRIMED if primed_workspace is not None else 0)


def mex_forward(input, offsets, num_instances, flags=0, workspace=None, **attrs):
    """The `Mex` op: [batch, num_instances * channels_out, height_out, width_out].  `workspace`: a buffer from
    `mex_layer_workspace` to run in instead of the stream's shared scratch."""
    attrs = _attrs(**attrs)
    dev = require_cuda(input, offsets)
    input, offsets = input.contiguous(), offsets.contiguous()
    d = _desc(input, num_instances, attrs, flags)
    g = _geometry(d)
    _check_offsets(offsets, g, num_instances)
    y = torch.empty((input.shape[0], g.channels_out_total, g.height_out, g.width_out), dtype=input.dtype, device=dev)
    with torch.cuda.device(dev):
        ws, n = _ws(d, dev, workspace)
        with timed("mex_forward", *_cost(d, g, "fwd")):
            _lib.check(_lib.lib().simnets_mex_forward(C.byref(d), input.data_ptr(), offsets.data_ptr(), y.data_ptr(), ws, n, stream_ptr(dev)))
    return y


def mex_forward_pool2(input, offsets, num_instances, flags=0, workspace=None, **attrs):
    """The `Mex` op and the 2x2 sum pooling of its output in one library call: (y, y_pooled).  float32, even output
    height and width.  On the pair-tile kernels the forward kernel's epilogue does the pooling."""
    attrs = _attrs(**attrs)
    dev = require_cuda(input, offsets)
    input, offsets = input.contiguous(), offsets.contiguous()
    d = _desc(input, num_instances, attrs, flags)
    g = _geometry(d)
    _check_offsets(offsets, g, num_instances)
    y = torch.empty((input.shape[0], g.channels_out_total, g.height_out, g.width_out), dtype=input.dtype, device=dev)
    yp = torch.empty((input.shape[0], g.channels_out_total, g.height_out // 2, g.width_out // 2), dtype=input.dtype, device=dev)
    with torch.cuda.device(dev):
        ws, n = _ws(d, dev, workspace)
        with timed("mex_forward", *_cost(d, g, "fwd")):
            _lib.check(_lib.lib().simnets_mex_forward_pool2x2(C.byref(d), input.data_ptr(), offsets.data_ptr(), y.data_ptr(), yp.data_ptr(),
                                                              ws, n, stream_ptr(dev)))
    return y, yp


def mex_input_grad(input, offsets, orig_output, output_grad, num_instances, flags=0, primed_workspace=None, pooled=False, **attrs):
    """The `MexInputGrad` op.  pooled=True: `output_grad` is the gradient of a 2x2 sum pooling of the output
    (half height and width); the library reads it in place of its 2x upsampling."""
    attrs = _attrs(**attrs)
    flags = _primed(flags | (abi.FLAG_MEX_DY_POOLED2 if pooled else 0), primed_workspace)
    dev = require_cuda(input, offsets, orig_output, output_grad)
    input, offsets, y, dy = input.contiguous(), offsets.contiguous(), orig_output.contiguous(), output_grad.contiguous()
    d = _desc(input, num_instances, attrs, flags)
    g = _geometry(d)
    _check_offsets(offsets, g, num_instances)
    _check_dy(dy, input, g, pooled)
    dx = torch.empty_like(input)
    with torch.cuda.device(dev):
        ws, n = _ws(d, dev, primed_workspace)
        with timed("mex_input_grad", *_cost(d, g, "dx")):
            _lib.check(_lib.lib().simnets_mex_input_grad(C.byref(d), input.data_ptr(), offsets.data_ptr(), y.data_ptr(), dy.data_ptr(),
                                                         dx.data_ptr(), ws, n, stream_ptr(dev)))
    return dx


def mex_offsets_grad(input, offsets, orig_output, output_grad, num_instances, flags=0, primed_workspace=None, out=None, pooled=False, **attrs):
    """The `MexOffsetsGrad` op.  `out` / FLAG_ACCUMULATE as in `similarity_parameters_grad`; `pooled` as in
    `mex_input_grad`."""
    attrs = _attrs(**attrs)
    flags = _primed(flags | (abi.FLAG_MEX_DY_POOLED2 if pooled else 0), primed_workspace)
    dev = require_cuda(input, offsets, orig_output, output_grad)
    input, offsets, y, dy = input.contiguous(), offsets.contiguous(), orig_output.contiguous(), output_grad.contiguous()
    d = _desc(input, num_instances, attrs, flags)
    g = _geometry(d)
    _check_offsets(offsets, g, num_instances)
    _check_dy(dy, input, g, pooled)
    if out is None:
        doff = torch.empty_like(offsets)
    else:
        doff = out
        assert doff.is_contiguous() and doff.numel() == offsets.numel()
    with torch.cuda.device(dev):
        ws, n = _ws(d, dev, primed_workspace)
        with timed("mex_offsets_grad", *_cost(d, g, "doff")):
            _lib.check(_lib.lib().simnets_mex_offsets_grad(C.byref(d), input.data_ptr(), offsets.data_ptr(), y.data_ptr(), dy.data_ptr(),
                                                           doff.data_ptr(), ws, n, stream_ptr(dev)))
    return doff


def mex_backward(input, offsets, orig_output, output_grad, num_instances, flags=0, primed_workspace=None, pooled=False, doff_out=None, **attrs):
    """`MexInputGrad` and `MexOffsetsGrad` in one library call: (input_grad, offsets_grad).  `pooled` as in
    `mex_input_grad`.  `primed_workspace` (all three gradient ops): the buffer that `mex_forward` ran in for the same
    input and offsets, untouched since."""
    attrs = _attrs(**attrs)
    flags = _primed(flags | (abi.FLAG_MEX_DY_POOLED2 if pooled else 0), primed_workspace)
    dev = require_cuda(input, offsets, orig_output, output_grad)
    input, offsets, y, dy = input.contiguous(), offsets.contiguous(), orig_output.contiguous(), output_grad.contiguous()
    d = _desc(input, num_instances, attrs, flags)
    g = _geometry(d)
    _check_offsets(offsets, g, num_instances)
    _check_dy(dy, input, g, pooled)
    dx = torch.empty_like(input)
    if doff_out is None:
        doff = torch.empty_like(offsets)
    else:                                   # (with FLAG_ACCUMULATE in `flags` the offsets gradient is added to it)
        doff = doff_out
        assert doff.is_contiguous() and doff.numel() == offsets.numel() and doff.dtype == offsets.dtype
    with torch.cuda.device(dev):
        ws, n = _ws(d, dev, primed_workspace)
        sig, nbytes, terms = _cost(d, g, "bwd")     # fused: x, offsets, y, dy read once, dx and doffsets written
        if pooled:
            sig, nbytes = sig + " dy/4", nbytes - 3 * dy.numel() * dy.element_size()
        with timed("mex_backward", sig, nbytes, 2 * terms):
            _lib.check(_lib.lib().simnets_mex_backward(C.byref(d), input.data_ptr(), offsets.data_ptr(), y.data_ptr(), dy.data_ptr(),
                                                       dx.data_ptr(), doff.data_ptr(), ws, n, stream_ptr(dev)))
    return dx, doff


def _gradients(ctx, grad, pooled):
    input, offsets, y = ctx.saved_tensors
    gi = go = None
    kw = dict(pooled=pooled, primed_workspace=ctx.layer_ws, flags=ctx.op_flags, **ctx.attrs)
    sink = ctx.grad_sink
    if sink is not None:                    # the offsets gradient is added straight into the caller's tensor (a gradient bucket)
        kw["flags"] = kw["flags"] | abi.FLAG_ACCUMULATE
    if ctx.needs_input_grad[0] and ctx.needs_input_grad[1]:
        gi, go = mex_backward(input, offsets, y, grad, ctx.num_instances, doff_out=sink, **kw)
    elif ctx.needs_input_grad[0]:
        gi = mex_input_grad(input, offsets, y, grad, ctx.num_instances, **kw)
    elif ctx.needs_input_grad[1]:
        go = mex_offsets_grad(input, offsets, y, grad, ctx.num_instances, out=sink, **kw)
    if sink is not None:
        go = None                           # nothing left for autograd to accumulate
    return gi, go, None, None


def _forward_for_autograd(ctx, input, offsets, num_instances, attrs, pooled, layer_ws=None, fwd_flags=0, op_flags=0, grad_sink=None):
    # a differentiated layer runs in a workspace of its own, which its gradient pass then finds primed
    # (layer_ws: the caller made that workspace already, e.g. to have the layer in front fill in the extrema)
    ctx.layer_ws, ctx.op_flags, ctx.grad_sink = layer_ws, op_flags, grad_sink
    fwd_flags |= op_flags
    if layer_ws is None and (ctx.needs_input_grad[0] or ctx.needs_input_grad[1]) and input.is_cuda and input.shape[0] > 0:
        ctx.layer_ws = mex_layer_workspace(input, num_instances, pooled=pooled, flags=op_flags, **attrs)
    if pooled and input.dtype == torch.float32 and input.shape[0] > 0:
        y, out = mex_forward_pool2(input, offsets, num_instances, flags=fwd_flags, workspace=ctx.layer_ws, **attrs)
    else:
        y = out = mex_forward(input, offsets, num_instances, flags=fwd_flags, workspace=ctx.layer_ws, **attrs)
        if pooled:
            out = torch.nn.functional.avg_pool2d(y, 2) * 4.0
    ctx.attrs, ctx.num_instances = attrs, num_instances
    ctx.save_for_backward(input, offsets, y)
    return out


class _Mex(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, offsets, num_instances, attrs, layer_ws=None, fwd_flags=0, op_flags=0, grad_sink=None):
        return _forward_for_autograd(ctx, input, offsets, num_instances, attrs, False, layer_ws, fwd_flags, op_flags, grad_sink)

    @staticmethod
    def backward(ctx, grad):
        return _gradients(ctx, grad, False) + (None, None, None, None)


def sum_pool2x2(y):
    """2x2 / stride-2 sum pooling of a float32 CUDA tensor [B, C, H, W] with even H and W (the library's kernel)."""
    dev = require_cuda(y)
    y = y.contiguous()
    out = torch.empty(y.shape[:2] + (y.shape[2] // 2, y.shape[3] // 2), dtype=y.dtype, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().simnets_sum_pool2x2_forward(y.shape[0] * y.shape[1], y.shape[2], y.shape[3], y.data_ptr(), out.data_ptr(),
                                                          stream_ptr(dev)))
    return out


class _MexSumPool2(torch.autograd.Function):
    """MEX followed by a 2x2 / stride-2 sum pooling.  The pooling's gradient (every dy value copied to the four
    positions it summed) is never written out: the MEX gradient kernels read the pooled dy directly."""

    @staticmethod
    def forward(ctx, input, offsets, num_instances, attrs, layer_ws=None, fwd_flags=0, op_flags=0, grad_sink=None):
        return _forward_for_autograd(ctx, input, offsets, num_instances, attrs, True, layer_ws, fwd_flags, op_flags, grad_sink)

    @staticmethod
    def backward(ctx, grad):
        return _gradients(ctx, grad, True) + (None, None, None, None)


def mex(input, offsets, num_instances, softmax_mode=None, padding=None, strides=None, blocks=None, epsilon=None,
        blocks_out_of_bounds_value=None, blocks_round_down=None, use_unshared_regions=None, shared_offset_region=None,
        unshared_offset_region=None, name=None):
    """Computes the MEX layer given a 4-D `input` and 5-D `offsets`
    ([num_regions, num_instances, block_c, block_h, block_w]).

    Same arguments, defaults and result as the reference's `simnets.ops.mex.mex`; `name` is accepted
    and ignored.  Differentiable w.r.t. `input` and `offsets`.
    """
    attrs = _attrs(softmax_mode=softmax_mode, padding=padding, strides=strides, blocks=blocks, epsilon=epsilon,
                   blocks_out_of_bounds_value=blocks_out_of_bounds_value, blocks_round_down=blocks_round_down,
                   use_unshared_regions=use_unshared_regions, shared_offset_region=shared_offset_region,
                   unshared_offset_region=unshared_offset_region)
    return _Mex.apply(input, offsets, num_instances, attrs)


def mex_sum_pool2(input, offsets, num_instances, layer_ws=None, fwd_flags=0, op_flags=0, grad_sink=None, **kwargs):
    """`mex(...)` followed by a 2x2 sum pooling (the MEX + pooling pair of the reference's example networks,
    README.md:114-131, where the pooling is `4 * AveragePooling2D(2)`), with the pooling's backward folded into
    the MEX gradient kernels.  Same keyword arguments as `mex`.  Falls back to the two separate ops when the
    MEX output height or width is odd."""
    attrs = _attrs(**{k: v for k, v in kwargs.items() if k != "name"})
    g = _geometry(_desc(input, num_instances, attrs))
    if g.height_out % 2 or g.width_out % 2:
        return torch.nn.functional.avg_pool2d(_Mex.apply(input, offsets, num_instances, attrs, layer_ws, fwd_flags, op_flags, grad_sink), 2) * 4.0
    return _MexSumPool2.apply(input, offsets, num_instances, attrs, layer_ws, fwd_flags, op_flags, grad_sink)


def mex_in_workspace(input, offsets, num_instances, layer_ws=None, fwd_flags=0, op_flags=0, sum_pool2=False, grad_sink=None, **kwargs):
    """`mex(...)` (or `mex_sum_pool2(...)`) with the library's extras: a layer workspace the caller made
    (`mex_layer_workspace_for`), flags for the forward call only (abi.FLAG_MEX_MAXIMA_GIVEN after the layer in front has
    filled in the extrema), flags for the forward and the gradient calls (abi.FLAG_MEX_NORMALIZED_OFFSETS: `offsets` are raw
    and the gradient comes back with respect to them), a tensor that the offsets gradient is ADDED to instead of being
    handed to autograd (`grad_sink`: the offsets' slice of a data-parallel gradient bucket)."""
    attrs = _attrs(**{k: v for k, v in kwargs.items() if k != "name"})
    if sum_pool2:
        return mex_sum_pool2(input, offsets, num_instances, layer_ws=layer_ws, fwd_flags=fwd_flags, op_flags=op_flags, grad_sink=grad_sink, **attrs)
    return _Mex.apply(input, offsets, num_instances, attrs, layer_ws, fwd_flags, op_flags, grad_sink)
