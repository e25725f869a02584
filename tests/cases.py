"""Shared case tables, seeded input generators and the acceptance rule of the parity tests.

The small grids re-express the reference's own unit-test grids
(HUJI-Deep/simnets-tf python/simnets/test/__init__.py:106-154 for Similarity, :299-372 for MEX) and
add what those never exercise: real NaNs, partial padding, epsilon != 1, epsilon = +-inf,
softmax_mode off, round-up output sizes, non-zero padding values, batch > 1 with normalization.
"""
import itertools
import math

import numpy as np

from simnets_tf_b200 import abi

NAN = float("nan")
INF = float("inf")


# ----------------------------------------------------------------------------- Similarity
def sim_case(name, shape, M, fn="L2", blocks=(3, 3), strides=(1, 1), padding=(0, 0), norm=False, ignore_nan=False,
             oob=0.0, nan_frac=0.0, seed=0, flags=0, x_dist="normal"):
    return dict(name=name, shape=tuple(shape), M=M, fn=fn, blocks=tuple(blocks), strides=tuple(strides), padding=tuple(padding),
                norm=norm, ignore_nan=ignore_nan, oob=oob, nan_frac=nan_frac, seed=seed, flags=flags, x_dist=x_dist)


def sim_attrs(c):
    return dict(similarity_function=c["fn"], blocks=list(c["blocks"]), strides=list(c["strides"]), padding=list(c["padding"]),
                normalization_term=c["norm"], normalization_term_fudge=0.001, ignore_nan_input=c["ignore_nan"],
                out_of_bounds_value=c["oob"])


def sim_desc(c, dtype=abi.F32, flags=None):
    return abi.make_sim_desc(c["shape"], c["M"], c["fn"], c["blocks"], c["strides"], c["padding"], c["norm"], 0.001,
                             c["ignore_nan"], c["oob"], dtype=dtype, flags=c["flags"] if flags is None else flags)


def sim_inputs(c, out_shape, dtype=np.float32):
    rng = np.random.default_rng(c["seed"])
    B, C, H, W = c["shape"]
    if c["x_dist"] == "uniform":
        x = rng.uniform(-0.5, 0.5, size=c["shape"])
    else:
        x = rng.normal(size=c["shape"])
    if c["nan_frac"] > 0:
        x[rng.random(c["shape"]) < c["nan_frac"]] = np.nan
    t = rng.normal(0, 0.1 if c["x_dist"] == "uniform" else 1.0, size=(c["M"], C) + c["blocks"])
    w = np.abs(rng.normal(1, 0.1, size=t.shape)) + 1e-3
    dy = rng.normal(size=out_shape)
    return [a.astype(dtype) for a in (x, t, w, dy)]


def _sim_small():
    cases = []
    # reference grid test_reference_dimensions (:106-116), reduced image, float32 instead of float64
    for i, (st, B, C, bl, pad) in enumerate(itertools.product((1, 2), (1, 2), (1, 3), (1, 3), ("SAME", "VALID"))):
        p = (bl // 2, bl // 2) if pad == "SAME" else (0, 0)
        cases.append(sim_case("dims%02d" % i, (B, C, 12, 11), 4, "L2", (bl, bl), (st, st), p, seed=100 + i))
    # reference grid test_reference_params (:119-129): normalization x ignore_nan, 3x3/2 SAME
    cases.append(sim_case("params_norm", (1, 3, 14, 13), 5, "L2", (3, 3), (2, 2), (1, 1), norm=True, seed=130))
    cases.append(sim_case("params_norm_nan", (1, 3, 14, 13), 5, "L2", (3, 3), (2, 2), (1, 1), norm=True, ignore_nan=True, seed=131))
    # L1, beyond the reference's single 1x1x1x1 element (:131-141)
    cases.append(sim_case("l1_1x1x1x1", (1, 1, 1, 1), 1, "L1", (1, 1), (1, 1), (0, 0), seed=140))
    cases.append(sim_case("l1_3x3", (2, 3, 10, 10), 6, "L1", (3, 3), (1, 1), (1, 1), seed=141))
    cases.append(sim_case("l1_stride2", (2, 2, 9, 12), 3, "L1", (2, 3), (2, 1), (0, 2), oob=0.75, seed=142))
    # what the reference never feeds: NaNs, NaN padding, partial padding, batch>1 with normalization
    cases.append(sim_case("nan_pad1", (3, 2, 9, 9), 7, "L2", (3, 3), (1, 1), (1, 1), norm=True, ignore_nan=True, oob=NAN, nan_frac=0.2, seed=150))
    cases.append(sim_case("nan_pad2_s2", (2, 1, 8, 8), 5, "L2", (2, 2), (2, 2), (2, 2), norm=True, ignore_nan=True, oob=NAN, seed=151, x_dist="uniform"))
    cases.append(sim_case("nan_propagates", (2, 2, 7, 8), 4, "L2", (3, 3), (1, 1), (1, 1), nan_frac=0.05, seed=152))
    cases.append(sim_case("nan_propagates_l1", (2, 2, 7, 8), 4, "L1", (3, 3), (1, 1), (1, 1), nan_frac=0.05, seed=153))
    cases.append(sim_case("norm_batch3", (3, 2, 8, 8), 4, "L2", (3, 3), (1, 1), (1, 1), norm=True, seed=154))
    cases.append(sim_case("norm_batch3_quirk", (3, 2, 8, 8), 4, "L2", (3, 3), (1, 1), (1, 1), norm=True, seed=154,
                          flags=abi.FLAG_SIM_BATCH_CONST_QUIRK))
    cases.append(sim_case("oob_value", (2, 3, 6, 7), 3, "L2", (3, 3), (2, 2), (2, 2), oob=-1.5, seed=155))
    cases.append(sim_case("one_by_one", (2, 5, 6, 7), 9, "L2", (1, 1), (1, 1), (0, 0), seed=156))
    cases.append(sim_case("stride_gt_block", (2, 2, 11, 11), 3, "L2", (2, 2), (3, 3), (0, 0), seed=157))
    cases.append(sim_case("wide_M_K", (2, 8, 9, 9), 70, "L2", (3, 3), (1, 1), (1, 1), norm=True, ignore_nan=True, nan_frac=0.1, seed=158))
    cases.append(sim_case("empty_batch", (0, 2, 6, 6), 3, "L2", (3, 3), (1, 1), (1, 1), seed=159))
    # enough channels for the tiled input-gradient kernel (C >= 16), with NaNs, stride 2 and L1
    cases.append(sim_case("dx_tiled_nan", (2, 20, 9, 10), 12, "L2", (3, 3), (1, 1), (1, 1), norm=True, ignore_nan=True, nan_frac=0.1, seed=160))
    cases.append(sim_case("dx_tiled_l1_s2", (2, 17, 8, 8), 6, "L1", (3, 3), (2, 2), (1, 1), seed=161))
    cases.append(sim_case("dx_tiled_l2", (3, 16, 7, 9), 70, "L2", (2, 3), (1, 2), (1, 1), oob=0.25, seed=162))
    return cases


SIM_SMALL = _sim_small()

# BASELINE configs (seeded synthetic stand-ins): cfg1 at full size, cfg4 variants at a sub-batch,
# cfg5's first layer at a sub-batch.
SIM_CONFIGS = [
    sim_case("cfg1", (64, 1, 28, 28), 32, "L2", (2, 2), (2, 2), (2, 2), norm=True, ignore_nan=True, oob=NAN, seed=0, x_dist="uniform"),
    sim_case("cfg4a_sub", (2, 64, 32, 32), 256, "L2", (3, 3), (1, 1), (1, 1), norm=True, ignore_nan=True, oob=0.0, nan_frac=0.2, seed=3),
    sim_case("cfg4b_sub", (2, 64, 32, 32), 256, "L1", (3, 3), (1, 1), (1, 1), seed=3),
    sim_case("cfg4c_sub", (2, 64, 32, 32), 256, "L1", (3, 3), (1, 1), (1, 1), nan_frac=0.2, seed=3, flags=abi.FLAG_SIM_L1_SKIP_NAN),
    sim_case("cfg5_sim_sub", (8, 3, 32, 32), 64, "L2", (3, 3), (1, 1), (1, 1), seed=4, x_dist="uniform"),
]


# ------------------------------------------------------------------------------------ MEX
def mex_case(name, shape, M, blocks, strides=(1, 1, 1), padding=(0, 0, 0), eps=1.0, softmax=False, oob=0.0, round_down=True,
             unshared=True, shared_region=(-1,), unshared_region=(-1,), seed=0, flags=0, normalize=False):
    return dict(name=name, shape=tuple(shape), M=M, blocks=tuple(blocks), strides=tuple(strides), padding=tuple(padding), eps=eps,
                softmax=softmax, oob=oob, round_down=round_down, unshared=unshared, shared_region=tuple(shared_region),
                unshared_region=tuple(unshared_region), seed=seed, flags=flags, normalize=normalize)


def mex_attrs(c):
    return dict(softmax_mode=c["softmax"], padding=list(c["padding"]), strides=list(c["strides"]), blocks=list(c["blocks"]),
                epsilon=c["eps"], blocks_out_of_bounds_value=c["oob"], blocks_round_down=c["round_down"],
                use_unshared_regions=c["unshared"], shared_offset_region=list(c["shared_region"]),
                unshared_offset_region=list(c["unshared_region"]))


def mex_desc(c, dtype=abi.F32, flags=None):
    return abi.make_mex_desc(c["shape"], c["M"], c["softmax"], c["padding"], c["strides"], c["blocks"], c["eps"], c["oob"],
                             c["round_down"], c["unshared"], c["shared_region"], c["unshared_region"], dtype=dtype,
                             flags=c["flags"] if flags is None else flags)


def mex_inputs(c, offsets_shape, out_shape, dtype=np.float32):
    rng = np.random.default_rng(c["seed"])
    x = rng.normal(size=c["shape"])
    off = rng.normal(0, 0.1 if c["normalize"] else 1.0, size=offsets_shape)
    if c["normalize"]:
        # the Keras layer's normalize_offsets (reference python/simnets/keras.py:155-160)
        flat = off.reshape(offsets_shape[0] * offsets_shape[1], -1)
        mx = flat.max(axis=1, keepdims=True)
        flat = flat - (mx + np.log(np.exp(flat - mx).sum(axis=1, keepdims=True)))
        off = flat.reshape(offsets_shape)
    dy = rng.normal(size=out_shape)
    return [a.astype(dtype) for a in (x, off, dy)]


def _mex_small():
    cases = []
    i = 0
    # reference grids test_reference_dimensions_shared / _unshared (:299-327), image shrunk from 41x40
    for st, B, C, H, bw in itertools.product((1, 4), (1, 2), (1, 3), (13, 12), (1, 3)):
        for unshared, region in ((False, (2,)), (False, (3,)), (True, (1, 5, 4)), (True, (2,))):
            if (i % 3) == 0:    # every third combination keeps the table small
                cases.append(mex_case("grid%03d" % i, (B, C, H, 12), 2, (1, bw, 3), (1, st, st), (0, 1, 0), softmax=True,
                                      unshared=unshared, shared_region=region if not unshared else (-1,),
                                      unshared_region=region if unshared else (-1,), seed=200 + i))
            i += 1
    # the "blocks bug" regression of the reference (:359-372)
    cases.append(mex_case("blocks_bug", (2, 3, 16, 16), 3, (3, 8, 8), (1, 1, 1), (0, 4, 4), softmax=True, seed=300))
    # numerics the reference only attribute-checks
    cases.append(mex_case("eps_half", (2, 4, 8, 8), 5, (4, 2, 2), (4, 2, 2), eps=0.5, softmax=True, unshared=False, seed=301))
    cases.append(mex_case("eps_neg", (2, 4, 8, 8), 5, (2, 2, 2), (2, 1, 1), eps=-2.0, seed=302))
    cases.append(mex_case("eps_pinf", (2, 4, 7, 8), 3, (4, 3, 3), (4, 1, 1), (0, 1, 1), eps=INF, unshared_region=(2,), seed=303))
    cases.append(mex_case("eps_ninf", (2, 4, 7, 8), 3, (4, 3, 3), (4, 1, 1), (0, 1, 1), eps=-INF, unshared=False, shared_region=(3,), seed=304))
    cases.append(mex_case("no_softmax", (2, 6, 6, 6), 4, (6, 1, 1), (6, 1, 1), softmax=False, unshared_region=(2,), seed=305))
    cases.append(mex_case("round_up", (2, 3, 9, 10), 3, (1, 2, 2), (1, 2, 2), round_down=False, oob=-0.5, unshared=False, shared_region=(2,), seed=306))
    cases.append(mex_case("oob_value", (1, 3, 7, 7), 2, (2, 3, 3), (1, 2, 2), (1, 1, 1), oob=2.5, softmax=True, seed=307))
    cases.append(mex_case("channel_regions", (2, 6, 5, 5), 3, (2, 1, 1), (1, 1, 1), softmax=True, unshared=False, shared_region=(2, 2, 3), seed=308))
    cases.append(mex_case("one_by_one_k1", (2, 5, 6, 6), 3, (1, 1, 1), (1, 1, 1), softmax=True, unshared_region=(1, 2, 2), seed=309))
    cases.append(mex_case("whole_image_stride", (2, 8, 4, 4), 10, (8, 4, 4), (-1, -1, -1), softmax=True, seed=310))
    cases.append(mex_case("wide_M_K", (2, 40, 6, 6), 70, (40, 1, 1), (40, 1, 1), softmax=True, unshared_region=(2,), seed=311, normalize=True))
    cases.append(mex_case("empty_batch", (0, 4, 6, 6), 3, (4, 1, 1), (4, 1, 1), softmax=True, seed=312))
    # mid-size patches (32 < K < 256) with many instances: the GEMM-tiled kernels, with regions, padding and remainders
    cases.append(mex_case("tiled_regions", (3, 48, 7, 7), 20, (48, 1, 1), (48, 1, 1), softmax=True, unshared_region=(1, 2, 3), seed=315, normalize=True))
    cases.append(mex_case("tiled_spatial", (2, 6, 13, 12), 33, (6, 3, 3), (6, 3, 3), eps=0.75, unshared=False, shared_region=(2,), seed=316))
    cases.append(mex_case("tiled_padded", (2, 5, 9, 9), 18, (5, 3, 3), (5, 3, 3), (0, 1, 1), eps=-1.25, oob=0.3, softmax=True, unshared_region=(2,), seed=317))
    # GEMM-sized layers (many instances): the tensor-core kernels
    cases.append(mex_case("tc_unshared", (3, 64, 8, 8), 96, (64, 1, 1), (64, 1, 1), softmax=True, unshared_region=(2,), seed=318, normalize=True))
    cases.append(mex_case("tc_remainders", (5, 56, 6, 6), 72, (56, 1, 1), (56, 1, 1), eps=0.5, unshared=False, shared_region=(-1,), seed=319))
    cases.append(mex_case("tc_spatial_padded", (2, 32, 9, 9), 50, (16, 2, 2), (16, 2, 2), (0, 1, 1), eps=-1.25, oob=0.3, softmax=True,
                          unshared_region=(2,), seed=320))
    cases.append(mex_case("tc_long_patches", (2, 128, 6, 6), 100, (128, 1, 1), (128, 1, 1), softmax=True, unshared_region=(2,), seed=321, normalize=True))
    cases.append(mex_case("tc_longer_patches", (3, 160, 4, 4), 56, (160, 1, 1), (160, 1, 1), softmax=True, eps=0.7, unshared_region=(2,), seed=322, normalize=True))
    # few instances over long patches (classifier-head shape): overlapping, padded blocks and disjoint blocks with a remainder
    cases.append(mex_case("head_overlap", (3, 16, 9, 9), 5, (16, 5, 5), (16, 2, 2), (0, 1, 1), softmax=True, unshared_region=(2,), seed=313))
    cases.append(mex_case("head_disjoint", (3, 16, 9, 9), 7, (16, 4, 4), (16, 4, 4), eps=2.0, unshared=False, shared_region=(1,), seed=314, normalize=True))
    return cases


MEX_SMALL = _mex_small()

MEX_CONFIGS = [
    mex_case("cfg2", (64, 32, 16, 16), 64, (32, 1, 1), (32, 1, 1), softmax=True, eps=1.0, unshared_region=(2,), seed=1, normalize=True),
    mex_case("cfg4_mex_sub", (2, 256, 32, 32), 256, (4, 2, 2), (4, 2, 2), eps=0.5, softmax=True, unshared=False, shared_region=(-1,), seed=3),
    mex_case("cfg5_mex2_sub", (4, 128, 16, 16), 256, (128, 1, 1), (128, 1, 1), softmax=True, unshared_region=(2,), seed=4, normalize=True),
    mex_case("cfg5_mex1_sub", (4, 64, 32, 32), 128, (64, 1, 1), (64, 1, 1), softmax=True, unshared_region=(2,), seed=5, normalize=True),
    mex_case("cfg5_mex3_sub", (4, 256, 8, 8), 512, (256, 1, 1), (256, 1, 1), softmax=True, unshared_region=(2,), seed=7, normalize=True),
    mex_case("cfg3_mex4_sub", (6, 256, 2, 2), 512, (256, 1, 1), (256, 1, 1), softmax=True, unshared_region=(2,), seed=8, normalize=True),
    mex_case("tc_many_tiles", (8, 48, 50, 50), 48, (48, 1, 1), (48, 1, 1), softmax=True, unshared=False, shared_region=(-1,), seed=6, normalize=True),
    mex_case("cfg5_head_sub", (4, 512, 4, 4), 10, (512, 4, 4), (1, 1, 1), softmax=True, seed=4, normalize=True),
]


# Layers whose unshared regions alternate along the width run on the pair-tile tensor-core kernels: instance and tap
# counts that are not multiples of the 16-wide chunks or of the tile widths, two-pixel-wide maps, several channel
# blocks, a negative epsilon and a position count that is not a multiple of a tile.
MEX_PAIR = [
    mex_case("pair_tails", (5, 70, 6, 10), 90, (70, 1, 1), (70, 1, 1), eps=0.7, softmax=True, unshared_region=(2,), seed=401, normalize=True),
    mex_case("pair_channel_blocks", (3, 96, 4, 6), 64, (48, 1, 1), (48, 1, 1), softmax=True, unshared_region=(2,), seed=402, normalize=True),
    mex_case("pair_two_wide", (9, 64, 3, 2), 130, (64, 1, 1), (64, 1, 1), softmax=False, unshared_region=(1, 1, 2), seed=403),
    mex_case("pair_eps_neg", (4, 52, 8, 8), 60, (52, 1, 1), (52, 1, 1), eps=-1.5, softmax=True, unshared_region=(2,), seed=404),
    mex_case("pair_short_patches", (6, 24, 8, 12), 80, (24, 1, 1), (24, 1, 1), softmax=True, unshared_region=(2,), seed=405, normalize=True),
    mex_case("pair_long_patches", (3, 300, 4, 4), 150, (300, 1, 1), (300, 1, 1), softmax=True, unshared_region=(2,), seed=406, normalize=True),
    # shapes whose offsets-gradient chunks are boxes of a tensor map: whole rows (two per chunk), runs inside a row,
    # ragged instance and tap tiles, a second tap tile of two channels, two instance groups, a batch that ends mid-way
    mex_case("pair_box_rows", (5, 40, 8, 16), 70, (40, 1, 1), (40, 1, 1), softmax=True, unshared_region=(2,), seed=407, normalize=True),
    mex_case("pair_box_runs", (3, 130, 4, 32), 200, (130, 1, 1), (130, 1, 1), eps=0.5, softmax=True, unshared_region=(2,), seed=408, normalize=True),
    mex_case("pair_box_groups", (2, 64, 16, 8), 300, (64, 1, 1), (64, 1, 1), softmax=False, unshared_region=(2,), seed=409),
]


# Short spatial blocks that tile the input rows (block width = stride, 2 or 4): the per-position maxima are taken from
# whole block rows.  A negative epsilon (minima), several channel blocks, a height that leaves a remainder, enough
# instances for the tensor-core kernels and too few for them.
MEX_ROWS = [
    mex_case("rows_w4_neg", (3, 6, 9, 12), 9, (3, 2, 4), (3, 2, 4), eps=-0.8, softmax=True, seed=323),
    mex_case("rows_w2_many", (2, 12, 6, 20), 40, (4, 3, 2), (4, 3, 2), eps=1.5, unshared=False, shared_region=(-1,), seed=324),
    mex_case("rows_w2_tc", (2, 16, 8, 16), 64, (4, 2, 2), (4, 2, 2), eps=0.5, softmax=True, unshared=False, shared_region=(-1,), seed=325),
]


# Few instances over whole-sample patches with one offsets region: the classifier-head kernels (several positions per
# CTA forward, both gradients from one read of x backward).  Tap counts off the tile sizes, 3 to 13 instances, several
# channel blocks, a negative epsilon, no softmax.
MEX_HEAD = [
    mex_case("head_taps_tail", (5, 37, 3, 3), 13, (37, 3, 3), (37, 3, 3), softmax=True, seed=411, normalize=True),
    mex_case("head_channel_blocks", (6, 96, 3, 3), 6, (48, 3, 3), (48, 3, 3), softmax=True, unshared=False, shared_region=(-1,), seed=412, normalize=True),
    mex_case("head_eps_neg", (9, 64, 2, 2), 3, (64, 2, 2), (64, 2, 2), eps=-0.8, softmax=False, seed=413),
    mex_case("head_long", (3, 300, 4, 4), 10, (300, 4, 4), (300, 4, 4), softmax=True, eps=2.0, seed=414, normalize=True),
    # aligned patches of at least 512 taps: slices of 1024 taps, groups of 16 positions (last group and last slice ragged)
    mex_case("head_wide_blocks", (19, 128, 4, 4), 16, (64, 4, 4), (64, 4, 4), softmax=True, unshared=False, shared_region=(-1,), seed=415, normalize=True),
    mex_case("head_wide_neg", (17, 40, 4, 4), 5, (40, 4, 4), (40, 4, 4), eps=-0.7, softmax=False, seed=416),
    mex_case("head_wide_m3", (33, 96, 4, 4), 3, (96, 4, 4), (96, 4, 4), softmax=True, eps=1.5, seed=417, normalize=True),
]


# ------------------------------------------------------------------------- acceptance rule
def rel_err(a, b):
    """max |a-b| over finite entries of b, relative to max |b| (0 for empty)."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    fin = np.isfinite(b)
    if not fin.any():
        return 0.0
    scale = max(float(np.abs(b[fin]).max()), 1e-30)
    return float(np.abs(a[fin] - b[fin]).max()) / scale


def assert_parity(ours, ref32, ref64=None, tol=1e-5, what=""):
    """Acceptance rule of the parity tests.

    1. NaN and +-inf masks must be identical to the float32 oracle's.
    2. On finite entries, max|ours - oracle32| <= tol * max|oracle32|  (tensor-scale relative error).
    3. Where the float32 oracle is itself farther than tol from the float64 oracle (long sequential
       float32 sums: parameter gradients), ours must instead be no farther from float64 than
       max(tol, the float32 oracle's own distance).
    """
    ours = np.asarray(ours)
    ref32 = np.asarray(ref32)
    assert ours.shape == ref32.shape, "%s: shape %s vs %s" % (what, ours.shape, ref32.shape)
    assert np.array_equal(np.isnan(ours), np.isnan(ref32)), "%s: NaN masks differ" % what
    assert np.array_equal(np.isposinf(ours), np.isposinf(ref32)), "%s: +inf masks differ" % what
    assert np.array_equal(np.isneginf(ours), np.isneginf(ref32)), "%s: -inf masks differ" % what
    e32 = rel_err(ours, ref32)
    if e32 <= tol:
        return e32
    if ref64 is not None:
        e_ours, e_ref = rel_err(ours, ref64), rel_err(ref32, ref64)
        assert e_ours <= max(tol, e_ref), "%s: rel err vs f64 oracle %.3g (f32 oracle itself: %.3g, vs f32 oracle: %.3g)" % (
            what, e_ours, e_ref, e32)
        return e_ours
    raise AssertionError("%s: rel err %.3g > %.3g" % (what, e32, tol))
