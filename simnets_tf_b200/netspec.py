"""Layer specifications of the benchmark SimNet architectures and their deterministic initial values.

Pure Python / numpy: nothing here loads the CUDA library, so the CPU checkers can build the identical
network without it.  The number of offset regions of a MEX layer comes from a caller-supplied function
(`simnets_tf_b200.simnet` passes the library's `get_mex_offsets_nregions`, the CPU checkers their own).

A specification is a list of ("similarity", kwargs) / ("mex", kwargs) / ("sumpool", k) / ("flatten",)
entries; the kwargs are those of the layer classes in `simnets_tf_b200.keras`.

cfg3: the README / Keras example network of the reference (README.md:114-131,
      test/basic_net_with_keras.py:95-135) for 1x28x28 inputs.
cfg5: the deeper 3x32x32 network of the data-parallel configuration (last layer as in
      test/basic_net_mnist_tf_ll.py:149-154).
"""
import numpy as np


def expand_dim_specification(image_shape, dim_spec):
    """[C, H, W] image shape and a 2- or 3-long specification -> 3 entries with every -1 replaced by the image
    dimension (reference python/simnets/ops/mex.py:84-112)."""
    dim_spec = list(dim_spec)
    if len(dim_spec) == 2:
        dim_spec = [-1] + dim_spec
    if len(dim_spec) != 3:
        raise ValueError('Bad dimensions specifications, should be a list of two or three, got %s' % dim_spec)
    return [image_shape[i] if dim_spec[i] == -1 else dim_spec[i] for i in range(3)]


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


def init_parameters(spec, seed, nregions):
    """Deterministic host-side initial values for every layer of a specification, in layer order:
    similarity -> (templates ~ N(0, 0.05), weights = 1); mex -> log Dirichlet(1) offsets.
    Returned as numpy arrays so that the CUDA network and the CPU checker start from the same bytes.
    `nregions(input_chw, num_instances, blocks, strides, layer_kwargs)` -> number of offset regions."""
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
            blocks = expand_dim_specification([c, h, w], kw["blocks"])
            strides = expand_dim_specification([c, h, w], kw["strides"])
            nreg = nregions([c, h, w], kw["num_instances"], blocks, strides, kw)
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


