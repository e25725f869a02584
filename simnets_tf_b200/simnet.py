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


def _mex_c(num_instances, channels):
    return ("mex", dict(num_instances=num_instances, blocks=[channels, 1, 1], strides=[channels, 1, 1], softmax_mode=True,
                        normalize_offsets=True, use_unshared_regions=True, unshared_offset_region=[2]))


SPECS = {
    "cfg3": dict(
        input_shape=(1, 28, 28), classes=10,
        layers=[("similarity", dict(num_instances=32, similarity_function="L2", blocks=[2, 2], strides=[2, 2], padding=[2, 2],
                                    normalization_term=True, ignore_nan_input=True, out_of_bounds_value=float("nan"))),
                _mex_c(64, 32), ("sumpool", 2), _mex_c(128, 64), ("sumpool", 2), _mex_c(256, 128), ("sumpool", 2),
                _mex_c(512, 256), ("sumpool", 2),
                ("mex", dict(num_instances=10, blocks=[512, 1, 1], strides=[512, 1, 1], softmax_mode=True, normalize_offsets=True,
                             use_unshared_regions=True, shared_offset_region=[1])),
                ("flatten",)]),
    "cfg5": dict(
        input_shape=(3, 32, 32), classes=10,
        layers=[("similarity", dict(num_instances=64, similarity_function="L2", blocks=[3, 3], strides=[1, 1], padding=[1, 1],
                                    normalization_term=False, ignore_nan_input=False, out_of_bounds_value=0.0)),
                _mex_c(128, 64), ("sumpool", 2), _mex_c(256, 128), ("sumpool", 2), _mex_c(512, 256), ("sumpool", 2),
                ("mex", dict(num_instances=10, blocks=[512, 4, 4], strides=[512, 4, 4], softmax_mode=True, normalize_offsets=True,
                             use_unshared_regions=True, unshared_offset_region=[-1])),
                ("flatten",)]),
}


def init_parameters(spec, seed):
    """Deterministic host-side initial values for every layer of a specification, in layer order:
    similarity -> (templates ~ N(0, 0.05), weights = 1); mex -> log Dirichlet(1) offsets.
    Returned as numpy arrays so that the CUDA network and the CPU checker start from the same bytes."""
    rng = np.random.default_rng(seed)
    c, h, w = spec["input_shape"]
    out = []
    for entry in spec["layers"]:
        kind = entry[0]
        if kind == "similarity":
            kw = entry[1]
            shape = (kw["num_instances"], c, kw["blocks"][0], kw["blocks"][1])
            out.append(dict(templates=rng.normal(0, 0.05, size=shape).astype(np.float32), weights=np.ones(shape, np.float32)))
            h = (h + 2 * kw["padding"][0] - kw["blocks"][0]) // kw["strides"][0] + 1
            w = (w + 2 * kw["padding"][1] - kw["blocks"][1]) // kw["strides"][1] + 1
            c = kw["num_instances"]
        elif kind == "mex":
            kw = entry[1]
            blocks = layers._expand_dim_specification([c, h, w], kw["blocks"])
            strides = layers._expand_dim_specification([c, h, w], kw["strides"])
            nreg = layers._mex_dims_helper([c, h, w], kw["num_instances"], blocks, [0, 0, 0], strides,
                                           use_unshared_regions=kw.get("use_unshared_regions", True),
                                           shared_offset_region=kw.get("shared_offset_region", [-1]),
                                           unshared_offset_region=kw.get("unshared_offset_region", [-1]))
            k = blocks[0] * blocks[1] * blocks[2]
            off = np.log(rng.dirichlet([1.0] * k, size=(nreg, kw["num_instances"]))).astype(np.float32)
            out.append(dict(offsets=off.reshape((nreg, kw["num_instances"]) + tuple(blocks))))
            co = (c - blocks[0]) // strides[0] + 1
            h = (h - blocks[1]) // strides[1] + 1
            w = (w - blocks[2]) // strides[2] + 1
            c = co * kw["num_instances"]
        elif kind == "sumpool":
            h //= entry[1]; w //= entry[1]
            out.append(None)
        else:
            out.append(None)
    return out


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
        self._plan = [(e, m) for e, m in zip(spec["layers"], mods)]

    def forward(self, x):
        plan, i = self._plan, 0
        while i < len(plan):
            entry, mod = plan[i]
            if entry[0] == "mex" and self.fuse_pooling and i + 1 < len(plan) and plan[i + 1][0] == ("sumpool", 2):
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

    def loss(self, x, labels, global_batch=None):
        """Softmax cross-entropy summed over this shard and divided by the global batch."""
        logits = self.forward(x)
        total = F.cross_entropy(logits, labels, reduction="sum")
        return total / float(global_batch if global_batch else x.shape[0])
