"""Layer classes with the constructor arguments, attribute handling and `get_config` keys of the
reference's Keras layers (HUJI-Deep/simnets-tf python/simnets/keras.py:19-188).

Keras and TensorFlow are not part of this stack; the layers are `torch.nn.Module`s that create their
variables on first call (the counterpart of Keras' `build(input_shape)`) and run the CUDA operators.
`perform_unsupervised_init` (k-means / GMM initialisation of Similarity layers) lives in `unsupervised.py`, built on the
Similarity operators; the reference's PCA branch serves Keras convolution layers, which do not exist here.
"""
import ctypes as C
import math

import numpy as np
import torch

from . import _lib, abi
from .ops.mex import _expand_dim_specification, _mex_dims_helper
from .ops.mex import mex as _mex
from .ops.mex import mex_sum_pool2 as _mex_sum_pool2
from .ops.mex import mex_in_workspace as _mex_in_workspace, mex_layer_workspace_for as _mex_layer_workspace_for
from .ops.mex import mex_workspace_maxima as _mex_workspace_maxima
from .ops.similarity import similarity_of_raw_weights as _similarity_of_raw_weights


def _sinks(*params):
    """The tensors that a data-parallel gradient bucket asked these parameters' gradients to be added to (dp.GradBucket), or
    None unless every one of them has one and still holds it as its `.grad`."""
    out = []
    for p in params:
        s = getattr(p, "_simnets_grad_sink", None)
        if s is None or p.grad is None or p.grad.data_ptr() != s.data_ptr() or not torch.is_grad_enabled() or not p.requires_grad:
            return None
        out.append(s)
    return tuple(out)


def _init_tensor(spec, shape, device, dtype, generator=None):
    """Keras initializer names the reference's layers use ('random_normal' = N(0, 0.05), 'ones', 'zeros')
    or a callable `(shape, dtype) -> array-like`."""
    if callable(spec):
        return torch.as_tensor(np.asarray(spec(shape, dtype=None)), dtype=dtype).to(device)
    name = str(spec).lower()
    if name == "ones":
        return torch.ones(shape, dtype=dtype, device=device)
    if name == "zeros":
        return torch.zeros(shape, dtype=dtype, device=device)
    if name == "random_normal":
        return (0.05 * torch.randn(shape, dtype=dtype, device="cpu", generator=generator)).to(device)
    raise ValueError("unknown initializer %r" % (spec,))


class Similarity(torch.nn.Module):
    """Similarity layer; `weights` enter the op as their absolute value, as in the reference's `call`."""

    def __init__(self, num_instances=None, similarity_function='L2', strides=[1, 1], blocks=[3, 3], padding='SAME',
                 normalization_term=False, normalization_term_fudge=0.001, ignore_nan_input=False,
                 out_of_bounds_value=0, templates_initializer='random_normal', weights_initializer='ones',
                 channels_last=False, **kwargs):
        super(Similarity, self).__init__()
        assert num_instances is not None
        self.num_instances = num_instances
        self.similarity_function = similarity_function
        self.strides = list(strides)
        self.blocks = list(blocks)
        if isinstance(padding, str):
            if padding.upper() not in ['SAME', 'VALID']:
                raise ValueError('Padding must be one of SAME, VALID (or a list of ints)')
            self.padding = [0, 0] if padding.upper() == 'VALID' else [e // 2 for e in blocks]
        else:
            self.padding = list(padding)
        self.normalization_term = normalization_term
        self.normalization_term_fudge = normalization_term_fudge
        self.ignore_nan_input = ignore_nan_input
        self.out_of_bounds_value = out_of_bounds_value
        self.templates_initializer = templates_initializer
        self.weights_initializer = weights_initializer
        self.channels_last = channels_last
        self.generator = kwargs.pop("generator", None)
        self.sweights = None
        self.templates = None

    def build(self, input_shape, device=None, dtype=torch.float32):
        num_channels = input_shape[3] if self.channels_last else input_shape[1]
        shape = (self.num_instances, num_channels, self.blocks[0], self.blocks[1])
        self.sweights = torch.nn.Parameter(_init_tensor(self.weights_initializer, shape, device, dtype, self.generator))
        self.templates = torch.nn.Parameter(_init_tensor(self.templates_initializer, shape, device, dtype, self.generator))

    def compute_output_shape(self, input_shape):
        """Shape of the layer's output for `input_shape` (batch first), as the Similarity op's shape function infers it
        in the reference (src/ops/similarity_op.cpp:8-59)."""
        shape = list(input_shape)
        if self.channels_last:
            shape = [shape[0], shape[3], shape[1], shape[2]]
        d = abi.make_sim_desc([max(int(shape[0]), 1)] + shape[1:], self.num_instances, self.similarity_function, self.blocks,
                              self.strides, self.padding, self.normalization_term, self.normalization_term_fudge,
                              self.ignore_nan_input, self.out_of_bounds_value)
        oh, ow = C.c_int32(), C.c_int32()
        _lib.check(_lib.lib().simnets_similarity_output_dims(C.byref(d), C.byref(oh), C.byref(ow)))
        out = [shape[0], self.num_instances, oh.value, ow.value]
        return tuple([out[0], out[2], out[3], out[1]] if self.channels_last else out)

    def forward(self, x, extrema=None):
        """extrema=(max_address, min_address): also write the per-pixel maximum / minimum of the output over the
        templates to those device addresses (see Mex.extrema_slot)."""
        if self.templates is None:
            self.build(tuple(x.shape), x.device, x.dtype)
        if self.channels_last:
            x = x.permute(0, 3, 1, 2)
        # |weights| and its gradient are taken inside the op's kernels
        y = _similarity_of_raw_weights(x, self.templates, self.sweights, similarity_function=self.similarity_function,
                                       blocks=self.blocks, strides=self.strides, padding=self.padding,
                                       normalization_term=self.normalization_term,
                                       normalization_term_fudge=self.normalization_term_fudge,
                                       ignore_nan_input=self.ignore_nan_input, out_of_bounds_value=self.out_of_bounds_value,
                                       extrema=extrema, grad_sinks=_sinks(self.templates, self.sweights))
        return y.permute(0, 2, 3, 1) if self.channels_last else y

    def get_config(self):
        names = ['num_instances', 'similarity_function', 'strides', 'blocks', 'padding', 'normalization_term',
                 'normalization_term_fudge', 'ignore_nan_input', 'out_of_bounds_value', 'templates_initializer',
                 'weights_initializer', 'channels_last']
        return {k: getattr(self, k) for k in names}


class DirichletInit(object):
    """log of Dirichlet(alpha) samples over each (region, instance) block."""

    def __init__(self, alpha=1.0, seed=None):
        self.alpha = alpha
        self.rng = np.random.default_rng(seed)

    def __call__(self, shape, dtype=None):
        num_regions, num_instances, block_c, block_h, block_w = shape
        k = block_c * block_h * block_w
        init = self.rng.dirichlet([self.alpha] * k, size=(num_regions, num_instances))
        with np.errstate(divide="ignore"):
            init = np.log(init)
        return init.reshape(shape).astype(np.float32 if dtype is None else dtype)

    def get_config(self):
        return {'alpha': self.alpha}


dirichlet_init = DirichletInit


class _NormalizeOffsets(torch.autograd.Function):
    """offsets[r, m, ...] minus the log-sum-exp over the block (the `normalize_offsets` option)."""

    @staticmethod
    def forward(ctx, offsets):
        from . import _lib
        from ._torch_glue import stream_ptr
        off = offsets.contiguous()
        rows, k = off.shape[0] * off.shape[1], int(math.prod(off.shape[2:]))
        out = torch.empty_like(off)
        with torch.cuda.device(off.device):
            _lib.check(_lib.lib().simnets_normalize_offsets_forward(rows, k, off.data_ptr(), out.data_ptr(), stream_ptr(off.device)))
        ctx.save_for_backward(off)
        return out

    @staticmethod
    def backward(ctx, grad):
        from . import _lib
        from ._torch_glue import stream_ptr
        off, = ctx.saved_tensors
        grad = grad.contiguous()
        rows, k = off.shape[0] * off.shape[1], int(math.prod(off.shape[2:]))
        doff = torch.empty_like(off)
        with torch.cuda.device(off.device):
            _lib.check(_lib.lib().simnets_normalize_offsets_backward(rows, k, off.data_ptr(), grad.data_ptr(), doff.data_ptr(),
                                                                     stream_ptr(off.device)))
        return doff


class Mex(torch.nn.Module):
    """MEX layer; `normalize_offsets` subtracts a per-(region, instance) logsumexp from the offsets variable."""

    def __init__(self, num_instances=None, padding=[0, 0, 0], strides=[1, 1, 1], blocks=[1, 1, 1],
                 epsilon=1.0, use_unshared_regions=True, shared_offset_region=[-1],
                 unshared_offset_region=[-1], softmax_mode=False, blocks_out_of_bounds_value=0.0,
                 blocks_round_down=True, normalize_offsets=False, offsets_initializer=None,
                 channels_last=False, **kwargs):
        super(Mex, self).__init__()
        assert num_instances is not None
        self.num_instances = num_instances
        self.padding = padding
        self.strides = list(strides)
        self.blocks = list(blocks)
        self.epsilon = epsilon
        self.use_unshared_regions = use_unshared_regions
        self.shared_offset_region = list(shared_offset_region)
        self.unshared_offset_region = list(unshared_offset_region)
        self.softmax_mode = softmax_mode
        self.blocks_out_of_bounds_value = blocks_out_of_bounds_value
        self.blocks_round_down = blocks_round_down
        self.normalize_offsets = normalize_offsets
        if offsets_initializer is None or (isinstance(offsets_initializer, str) and offsets_initializer == 'dirichlet'):
            offsets_initializer = dirichlet_init()
        self.offsets_initializer = offsets_initializer
        self.channels_last = channels_last
        self.offsets = None

    def build(self, input_shape, device=None, dtype=torch.float32):
        input_shape = list(input_shape)
        if self.channels_last:
            input_shape = [input_shape[0], input_shape[3], input_shape[1], input_shape[2]]
        self.blocks = _expand_dim_specification(input_shape, self.blocks)
        if isinstance(self.padding, str):
            if self.padding.upper() not in ['SAME', 'VALID']:
                raise ValueError('Padding must be one of SAME, VALID (or a list of ints)')
            self.padding = [0, 0, 0] if self.padding.upper() == 'VALID' else [e // 2 for e in self.blocks]
        nregions = _mex_dims_helper(input_shape[1:], self.num_instances, blocks=self.blocks, padding=self.padding,
                                    strides=self.strides, use_unshared_regions=self.use_unshared_regions,
                                    shared_offset_region=self.shared_offset_region,
                                    blocks_round_down=self.blocks_round_down,
                                    unshared_offset_region=self.unshared_offset_region)
        if nregions < 0:
            raise ValueError("invalid MEX geometry for input shape %s" % (input_shape,))
        shape = (nregions, self.num_instances) + tuple(self.blocks)
        self.offsets = torch.nn.Parameter(_init_tensor(self.offsets_initializer, shape, device, dtype))

    def compute_output_shape(self, input_shape):
        """Shape of the layer's output for `input_shape` (batch first), as the Mex op's shape function infers it in
        the reference (src/ops/mex_op.cpp:19-56): a matter of blocks, strides, padding and the rounding mode only,
        so it also answers for region lists the op's kernel would refuse."""
        if self.offsets is None:
            self.build(tuple(input_shape))
        shape = list(input_shape)
        if self.channels_last:
            shape = [shape[0], shape[3], shape[1], shape[2]]
        d = abi.make_mex_desc([max(int(shape[0]), 1)] + shape[1:], self.num_instances, padding=self.padding, strides=self.strides,
                              blocks=self.blocks, blocks_round_down=self.blocks_round_down)
        g = abi.MexGeometry()
        _lib.check(_lib.lib().simnets_mex_dims(C.byref(d), C.byref(g)))
        out = [shape[0], g.channels_out_total, g.height_out, g.width_out]
        return tuple([out[0], out[2], out[3], out[1]] if self.channels_last else out)

    def effective_offsets(self):
        if not self.normalize_offsets:
            return self.offsets
        if self.offsets.is_cuda and self.offsets.dtype == torch.float32:
            return _NormalizeOffsets.apply(self.offsets)             # one library kernel each way
        flat = self.offsets.reshape(self.offsets.shape[0] * self.offsets.shape[1], -1)
        return (flat - torch.logsumexp(flat, dim=1, keepdim=True)).reshape(self.offsets.shape)

    def _op_attrs(self):
        return dict(blocks=self.blocks, padding=self.padding, strides=self.strides, use_unshared_regions=self.use_unshared_regions,
                    shared_offset_region=self.shared_offset_region, blocks_out_of_bounds_value=self.blocks_out_of_bounds_value,
                    blocks_round_down=self.blocks_round_down, unshared_offset_region=self.unshared_offset_region,
                    epsilon=self.epsilon, softmax_mode=self.softmax_mode)

    def _op_flags(self, dtype, device):
        # float32 on the GPU: the op takes the raw offsets and normalises them in its own prepass (and its gradient comes back
        # with respect to the raw values); otherwise effective_offsets() does it in front of the op
        fused = self.normalize_offsets and dtype == torch.float32 and device.type == "cuda" and self.offsets is not None and \
            self.offsets.dtype == torch.float32 and self.offsets.is_cuda
        from . import _torch_glue
        if _torch_glue.DEFAULT_FLAGS & (abi.FLAG_FORCE_DIRECT | abi.FLAG_MEX_EXACT):
            fused = False           # those routes run without a workspace, which the fused normalisation needs
        return abi.FLAG_MEX_NORMALIZED_OFFSETS if fused else 0

    def extrema_slot(self, input_shape, dtype, device, sum_pool2=False):
        """For a layer whose every patch is exactly the channels of one pixel (blocks [C, 1, 1], unit spatial strides, no
        padding): (workspace, device address, want_max) -- a layer workspace made ahead of the call and the place in it
        where the forward pass expects the per-pixel maximum (epsilon > 0) or minimum of its input over the channels.
        The layer in front writes them there while it produces that input (`Similarity.forward(x, extrema=...)`), and
        `forward(x, layer_ws=workspace, maxima_given=True)` then skips its own pass over the input.  None otherwise."""
        if self.channels_last or dtype != torch.float32 or device.type != "cuda":
            return None
        if self.offsets is None:
            self.build(tuple(input_shape), device, dtype)
        b, c, h, w = [int(e) for e in input_shape]
        if list(self.blocks) != [c, 1, 1] or list(self.strides)[1:] != [1, 1] or any(int(p) != 0 for p in self.padding) or b == 0:
            return None
        ws = _mex_layer_workspace_for((b, c, h, w), dtype, device, self.num_instances, pooled=sum_pool2, flags=self._op_flags(dtype, device),
                                      **self._op_attrs())
        ptr = _mex_workspace_maxima((b, c, h, w), dtype, self.num_instances, ws, flags=self._op_flags(dtype, device), **self._op_attrs())
        return None if ptr is None else (ws, ptr, float(self.epsilon) > 0)

    def forward(self, x, sum_pool2=False, layer_ws=None, maxima_given=False):
        """sum_pool2=True returns the 2x2 sum pooling of the layer's output (pooling gradient fused into the
        MEX gradient kernels).  layer_ws / maxima_given: see extrema_slot."""
        if self.offsets is None:
            self.build(tuple(x.shape), x.device, x.dtype)
        if self.channels_last:
            x = x.permute(0, 3, 1, 2)
        op_flags = self._op_flags(x.dtype, x.device) if x.shape[0] > 0 else 0
        if layer_ws is not None or op_flags:
            sink = _sinks(self.offsets) if op_flags else None       # (the raw offsets are the op's own input only when it normalises them)
            y = _mex_in_workspace(x, self.offsets if op_flags else self.effective_offsets(), self.num_instances, layer_ws,
                                  fwd_flags=abi.FLAG_MEX_MAXIMA_GIVEN if maxima_given else 0, op_flags=op_flags, sum_pool2=sum_pool2,
                                  grad_sink=sink[0] if sink else None, **self._op_attrs())
            return y.permute(0, 2, 3, 1) if self.channels_last else y
        op = _mex_sum_pool2 if sum_pool2 else _mex
        y = op(x, self.effective_offsets(), self.num_instances, blocks=self.blocks, padding=self.padding,
                 strides=self.strides, use_unshared_regions=self.use_unshared_regions,
                 shared_offset_region=self.shared_offset_region,
                 blocks_out_of_bounds_value=self.blocks_out_of_bounds_value,
                 blocks_round_down=self.blocks_round_down,
                 unshared_offset_region=self.unshared_offset_region,
                 epsilon=self.epsilon, softmax_mode=self.softmax_mode)
        return y.permute(0, 2, 3, 1) if self.channels_last else y

    def get_config(self):
        names = ['num_instances', 'padding', 'strides', 'blocks', 'epsilon', 'use_unshared_regions', 'shared_offset_region',
                 'unshared_offset_region', 'softmax_mode', 'blocks_out_of_bounds_value', 'blocks_round_down',
                 'normalize_offsets', 'offsets_initializer', 'channels_last']
        return {k: getattr(self, k) for k in names}


def perform_unsupervised_init(model, kind='gmm', layers=[], data=None, batch_size=None, **kwargs):
    """python/simnets/keras.py:191-238 for Similarity layers; see unsupervised.perform_unsupervised_init."""
    from . import unsupervised
    return unsupervised.perform_unsupervised_init(model, kind=kind, layers=layers, data=data, batch_size=batch_size, **kwargs)
