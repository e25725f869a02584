"""Single-operator micro-benchmark on synthetic data of a named layer shape.

    python -m simnets_tf_b200.opbench --layer cfg5_mex2 --op forward --batch 512 --iters 20

Prints one JSON line: device time per call (CUDA events on the launching stream, after warm-up),
algorithmic GB/s (every input read once, every output written once) and G terms/s (one term = one
(instance, tap, position) triple).  Used for profiling one kernel family at a time; the end-to-end
numbers come from bench.py.
"""
import argparse
import importlib
import json

import torch

from . import _lib
from ._torch_glue import PROFILE

mex_ops = importlib.import_module("simnets_tf_b200.ops.mex")
sim_ops = importlib.import_module("simnets_tf_b200.ops.similarity")

NAN = float("nan")

# name -> (kind, input CHW, instances, attrs, default batch, fraction of NaN inputs)
LAYERS = {
    "cfg1_sim": ("sim", (1, 28, 28), 32, dict(similarity_function="L2", blocks=[2, 2], strides=[2, 2], padding=[2, 2],
                                              normalization_term=True, ignore_nan_input=True, out_of_bounds_value=NAN), 64, 0.0),
    "cfg4_sim": ("sim", (64, 32, 32), 256, dict(similarity_function="L2", blocks=[3, 3], strides=[1, 1], padding=[1, 1],
                                                normalization_term=True, ignore_nan_input=True, out_of_bounds_value=0.0), 256, 0.2),
    "cfg4_sim_l1": ("sim", (64, 32, 32), 256, dict(similarity_function="L1", blocks=[3, 3], strides=[1, 1], padding=[1, 1]), 256, 0.0),
    "cfg4_sim_l2": ("sim", (64, 32, 32), 256, dict(similarity_function="L2", blocks=[3, 3], strides=[1, 1], padding=[1, 1]), 256, 0.0),
    "cfg5_sim": ("sim", (3, 32, 32), 64, dict(similarity_function="L2", blocks=[3, 3], strides=[1, 1], padding=[1, 1]), 2048, 0.0),
    "cfg2_mex": ("mex", (32, 16, 16), 64, dict(blocks=[32, 1, 1], strides=[32, 1, 1], softmax_mode=True, unshared_offset_region=[2]), 64, 0.0),
    "cfg4_mex": ("mex", (256, 32, 32), 256, dict(blocks=[4, 2, 2], strides=[4, 2, 2], epsilon=0.5, softmax_mode=True,
                                                 use_unshared_regions=False, shared_offset_region=[-1]), 256, 0.0),
    "cfg5_mex1": ("mex", (64, 32, 32), 128, dict(blocks=[64, 1, 1], strides=[64, 1, 1], softmax_mode=True, unshared_offset_region=[2]), 2048, 0.0),
    "cfg5_mex2": ("mex", (128, 16, 16), 256, dict(blocks=[128, 1, 1], strides=[128, 1, 1], softmax_mode=True, unshared_offset_region=[2]), 2048, 0.0),
    "cfg5_mex3": ("mex", (256, 8, 8), 512, dict(blocks=[256, 1, 1], strides=[256, 1, 1], softmax_mode=True, unshared_offset_region=[2]), 2048, 0.0),
    # diagnostics: the cfg5_mex1 GEMM sizes on maps whose sibling regions are laid out differently in memory
    "diag_rows_contiguous": ("mex", (64, 16, 64), 128, dict(blocks=[64, 1, 1], strides=[64, 1, 1], softmax_mode=True, unshared_offset_region=[1, 1, 2]), 2048, 0.0),
    "diag_rows_256B": ("mex", (64, 16, 64), 128, dict(blocks=[64, 1, 1], strides=[64, 1, 1], softmax_mode=True, unshared_offset_region=[2]), 2048, 0.0),
    "cfg5_head": ("mex", (512, 4, 4), 10, dict(blocks=[512, 4, 4], strides=[512, 4, 4], softmax_mode=True), 2048, 0.0),
}


def run(layer, op, batch, iters, warmup, flags=0, seed=0):
    kind, chw, inst, attrs, default_batch, nan_frac = LAYERS[layer]
    batch = batch or default_batch
    dev = torch.device("cuda")
    gen = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn((batch,) + chw, generator=gen).to(dev)
    if nan_frac:
        x[torch.rand(x.shape, generator=gen).to(dev) < nan_frac] = NAN
    if kind == "sim":
        t = (0.1 * torch.randn((inst, chw[0]) + tuple(attrs["blocks"]), generator=gen)).to(dev)
        w = ((1 + 0.1 * torch.randn(t.shape, generator=gen)).abs() + 1e-3).to(dev)
        y = sim_ops.similarity_forward(x, t, w, flags=flags, **attrs)
        dy = torch.randn(y.shape, generator=gen).to(dev)
        calls = {"forward": lambda: sim_ops.similarity_forward(x, t, w, flags=flags, **attrs),
                 "input_grad": lambda: sim_ops.similarity_input_grad(x, t, w, dy, flags=flags, **attrs),
                 "params_grad": lambda: sim_ops.similarity_parameters_grad(x, t, w, dy, flags=flags, **attrs)}
    else:
        g = mex_ops._geometry(mex_ops._desc(x, inst, mex_ops._attrs(**attrs)))
        off = (0.1 * torch.randn((g.num_regions, inst, g.block_c, g.block_h, g.block_w), generator=gen)).to(dev)
        y = mex_ops.mex_forward(x, off, inst, flags=flags, **attrs)
        dy = torch.randn(y.shape, generator=gen).to(dev)
        calls = {"forward": lambda: mex_ops.mex_forward(x, off, inst, flags=flags, **attrs),
                 "input_grad": lambda: mex_ops.mex_input_grad(x, off, y, dy, inst, flags=flags, **attrs),
                 "offsets_grad": lambda: mex_ops.mex_offsets_grad(x, off, y, dy, inst, flags=flags, **attrs),
                 "backward": lambda: mex_ops.mex_backward(x, off, y, dy, inst, flags=flags, **attrs)}
        if g.height_out % 2 == 0 and g.width_out % 2 == 0:
            dyp = torch.randn(y.shape[:2] + (y.shape[2] // 2, y.shape[3] // 2), generator=gen).to(dev)
            calls["backward_pooled"] = lambda: mex_ops.mex_backward(x, off, y, dyp, inst, flags=flags, pooled=True, **attrs)
    fn = calls[op]
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    launches = _lib.launch_count()
    PROFILE.start()
    for _ in range(iters):
        fn()
    rows = PROFILE.stop()
    launches = _lib.launch_count() - launches
    (key, r), = rows.items()
    ms = r["ms"] / r["calls"]
    return {"layer": layer, "op": key, "batch": batch, "iters": iters, "ms_per_call": ms,
            "GBps": r["bytes"] / r["calls"] / (ms * 1e-3) / 1e9, "Gterms_per_s": r["terms"] / r["calls"] / (ms * 1e-3) / 1e9,
            "algorithmic_bytes": r["bytes"] // r["calls"], "terms": r["terms"] // r["calls"], "kernel_launches_per_call": launches / iters}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layer", choices=sorted(LAYERS), required=True)
    ap.add_argument("--op", default="forward", choices=["forward", "input_grad", "params_grad", "offsets_grad", "backward", "backward_pooled"])
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--flags", type=lambda v: int(v, 0), default=0)
    a = ap.parse_args()
    print(json.dumps(run(a.layer, a.op, a.batch, a.iters, a.warmup, a.flags)))


if __name__ == "__main__":
    main()
