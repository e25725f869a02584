"""The SimNet architectures of the benchmark configurations, as layer specifications plus a torch
module that runs them on the CUDA operators.

A specification is a list of ("similarity", kwargs) / ("mex", kwargs) / ("sumpool", k) / ("flatten",)
entries; the kwargs are those of the layer classes in `simnets_tf_b200.keras`.  The same lists drive
the CPU checker's network, so both sides build the identical model.

cfg3: the README / Keras example network of the reference (README.md:114-131,
      test/basic_net_with_keras.py:95-135) for 1x28x28 inputs.
cfg5: the deeper 3x32x32 network of the data-parallel configuration (last layer as in
      test/basic_net_mnist_tf_ll.py:149-154).
Sum pooling is a 2x2 average pool times 4, as the reference's README builds it.
"""
import numpy as np
import torch
import torch.nn.functional as F

from . import keras as layers
from .ops.loss import softmax_cross_entropy


from .netspec import SPECS  # noqa: F401
from . import netspec


def _library_nregions(input_chw, num_instances, blocks, strides, kw):
    return layers._mex_dims_helper(input_chw, num_instances, blocks, [0, 0, 0], strides,
                                   use_unshared_regions=kw.get("use_unshared_regions", True),
                                   shared_offset_region=kw.get("shared_offset_region", [-1]),
                                   unshared_offset_region=kw.get("unshared_offset_region", [-1]))


def init_parameters(spec, seed):
    """`netspec.init_parameters` with the library's `get_mex_offsets_nregions` for the region counts."""
    return netspec.init_parameters(spec, seed, _library_nregions)


class _SumPool(torch.autograd.Function):
    """k x k sum pooling (stride k).  The backward of a sum pool copies each output gradient to the k*k
    inputs it summed, which is a nearest-neighbour upsampling."""

    @staticmethod
    def forward(ctx, x, k):
        ctx.k = k
        return F.avg_pool2d(x, k) * float(k * k)

    @staticmethod
    def backward(ctx, dy):
        return F.interpolate(dy, scale_factor=ctx.k, mode="nearest"), None


def sum_pool(x, k):
    if x.shape[2] % k or x.shape[3] % k:
        return F.avg_pool2d(x, k) * float(k * k)
    return _SumPool.apply(x, k)


class SimNet(torch.nn.Module):
    """A specification instantiated on the CUDA operators."""

    def __init__(self, spec, seed=0, device="cuda", dtype=torch.float32):
        super(SimNet, self).__init__()
        self.spec = spec
        mods, init = [], init_parameters(spec, seed)
        for entry, values in zip(spec["layers"], init):
            if entry[0] == "similarity":
                m = layers.Similarity(**entry[1])
                m.sweights = torch.nn.Parameter(torch.from_numpy(values["weights"]).to(device=device, dtype=dtype))      # same order as build()
                m.templates = torch.nn.Parameter(torch.from_numpy(values["templates"]).to(device=device, dtype=dtype))
                mods.append(m)
            elif entry[0] == "mex":
                m = layers.Mex(**entry[1])
                m.blocks = list(values["offsets"].shape[2:])
                m.offsets = torch.nn.Parameter(torch.from_numpy(values["offsets"]).to(device=device, dtype=dtype))
                mods.append(m)
            else:
                mods.append(None)
        self.stages = torch.nn.ModuleList([m for m in mods if m is not None])
        self.fuse_pooling = True
        self.fuse_extrema = True
        self._plan = [(e, m) for e, m in zip(spec["layers"], mods)]

    def forward(self, x):
        return self.forward_range(x, 0, len(self._plan))

    def split_point(self):
        """Index into the layer plan that leaves the last two MEX layers (the largest offsets tensors) behind it: their
        gradients are the first that a backward pass finishes, so a data-parallel step can start reducing them while
        the layers in front are still being differentiated.  0 when the network has fewer than three MEX layers."""
        mex = [i for i, (e, _) in enumerate(self._plan) if e[0] == "mex"]
        return mex[-2] if len(mex) >= 3 else 0

    def parameters_from(self, begin):
        """Parameters of the layers plan[begin:], in `parameters()` order (they are its tail)."""
        out = []
        for _, m in self._plan[begin:]:
            if m is not None:
                out.extend(m.parameters())
        return out

    def forward_range(self, x, begin, end):
        """Layers plan[begin:end] (a MEX + sum-pool pair is never split: `begin` and `end` are layer starts)."""
        plan, i = self._plan, begin
        while i < end:
            entry, mod = plan[i]
            pooled_next = lambda j: self.fuse_pooling and j + 1 < len(plan) and plan[j + 1][0] == ("sumpool", 2)
            if entry[0] == "similarity" and self.fuse_extrema and i + 1 < end and plan[i + 1][0][0] == "mex":
                # Similarity -> MEX over the channels of each pixel: the Similarity kernel leaves the per-pixel extrema of its
                # output in the MEX layer's workspace, and the MEX forward pass skips its pass over that tensor
                nxt = plan[i + 1][1]
                slot = nxt.extrema_slot(mod.compute_output_shape(tuple(x.shape)), x.dtype, x.device, sum_pool2=pooled_next(i + 1))
                if slot is not None:
                    ws, ptr, up = slot
                    x = mod(x, extrema=(ptr, None) if up else (None, ptr))
                    x = nxt(x, sum_pool2=pooled_next(i + 1), layer_ws=ws, maxima_given=True)
                    i += 3 if pooled_next(i + 1) else 2
                    continue
            if entry[0] == "mex" and pooled_next(i):
                x = mod(x, sum_pool2=True)          # MEX + 2x2 sum pooling, pooling gradient inside the MEX gradient kernels
                i += 2
                continue
            if mod is not None:
                x = mod(x)
            elif entry[0] == "sumpool":
                x = sum_pool(x, entry[1])
            elif entry[0] == "flatten":
                x = x.flatten(1)
            i += 1
        return x

    def loss_of_logits(self, logits, labels, global_batch=None):
        n = float(global_batch if global_batch else logits.shape[0])
        if logits.is_cuda and logits.dtype == torch.float32 and labels.dtype == torch.int64:
            return softmax_cross_entropy(logits, labels, 1.0 / n)       # loss and gradient in one library launch
        return F.cross_entropy(logits, labels, reduction="sum") / n

    def loss(self, x, labels, global_batch=None):
        """Softmax cross-entropy summed over this shard and divided by the global batch."""
        return self.loss_of_logits(self.forward(x), labels, global_batch)
