"""Unsupervised initialisation on the CUDA operators against the CPU restatement on explicit patches: the same seeds and
the same batches, step by step.  float64 shows that the two formulations are the same arithmetic; float32 carries the
stated tolerance (sums over all patches of a batch in float32, in a different order)."""
import numpy as np
import pytest
import torch

from oracle import unsupervised_oracle as uo
from simnets_tf_b200 import keras as layers
from simnets_tf_b200 import unsupervised as un
from simnets_tf_b200.simnet import SPECS, SimNet

pytestmark = pytest.mark.gpu

GEOMETRIES = [   # (batch, channels, h, w), blocks, strides, k
    ((4, 3, 12, 11), (3, 3), (1, 1), 8),
    ((3, 1, 14, 14), (2, 2), (2, 2), 32),
    ((2, 16, 6, 6), (1, 1), (1, 1), 5),
    ((6, 5, 13, 14), (4, 2), (2, 3), 64),
]
TOL = {torch.float64: 1e-9, torch.float32: 2e-4}


def _batches(rng, shape, n, k):
    """Images made of k noisy prototypes per patch position, so that clusters exist and responsibilities are not flat."""
    proto = rng.normal(size=(k,) + shape[1:])
    return [proto[rng.integers(0, k, shape[0])] + 0.3 * rng.normal(size=shape) for _ in range(n)]


def _close(got, want, tol, what, rows=None):
    got, want = got.double().cpu().numpy().reshape(want.shape), np.asarray(want)
    if rows is not None:
        got, want = got[rows], want[rows]
    err = np.abs(got - want).max() / max(np.abs(want).max(), 1e-30)
    assert err <= tol, "%s: %.3g > %.3g" % (what, err, tol)
    return err


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32], ids=["f64", "f32"])
@pytest.mark.parametrize("geo", GEOMETRIES, ids=lambda g: "x".join(map(str, g[0])) + "_b%dx%d_s%dx%d_k%d" % (g[1] + g[2] + (g[3],)))
def test_kmeans_steps_equal_the_restatement(geo, dtype):
    shape, blocks, strides, k = geo
    rng = np.random.default_rng(11)
    batches = _batches(rng, shape, 3, k)
    u = rng.random(k)
    km = un.KMeans(blocks, strides, k)
    first = torch.from_numpy(batches[0]).to("cuda", dtype)
    km.init(first, uniforms=u)
    p0 = uo.extract_patches(first.double().cpu().numpy(), blocks, strides)
    centres, _ = uo.kmeans_pp_seed(p0, k, u)
    _close(km.centres, centres, 0.0 if dtype == torch.float64 else 1e-7, "seeds")      # the same patches are picked
    counts = np.zeros(k)
    for i, b in enumerate(batches):
        x = torch.from_numpy(b).to("cuda", dtype)
        km.update(x)
        centres, counts, _ = uo.kmeans_step(centres, counts, uo.extract_patches(x.double().cpu().numpy(), blocks, strides))
        assert np.array_equal(km.counts.cpu().numpy(), counts), "assignment counts differ at step %d" % i
        _close(km.centres, centres, TOL[dtype], "centres after step %d" % i)


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32], ids=["f64", "f32"])
@pytest.mark.parametrize("geo", GEOMETRIES, ids=lambda g: "x".join(map(str, g[0])) + "_b%dx%d_s%dx%d_k%d" % (g[1] + g[2] + (g[3],)))
def test_gmm_steps_equal_the_restatement(geo, dtype):
    shape, blocks, strides, k = geo
    rng = np.random.default_rng(12)
    batches = _batches(rng, shape, 3, k)
    gm = un.DiagonalGMM(blocks, strides, k)
    first = torch.from_numpy(batches[0]).to("cuda", dtype)
    p0 = uo.extract_patches(first.double().cpu().numpy(), blocks, strides)
    picks = rng.integers(0, len(p0), k)
    gm.init(first, picks=picks)
    means, covs = uo.gmm_seed(p0, picks)
    _close(gm.means, means, 1e-7, "seed means")
    _close(gm.covs, covs, TOL[dtype], "seed covariances")
    for i, b in enumerate(batches):
        x = torch.from_numpy(b).to("cuda", dtype)
        gm.update(x)
        before = means
        means, covs, r = uo.gmm_step(means, covs, uo.extract_patches(x.double().cpu().numpy(), blocks, strides))
        # a component whose whole mass is a rounding error of the softmax is not comparable between precisions: those that
        # hold a visible share are compared, those with none at all must have stayed where they were
        mass = r.sum(0)
        held, none = mass > (1e-280 if dtype == torch.float64 else 1e-4), mass == 0
        assert held.sum() >= 2
        _close(gm.means, means, TOL[dtype] * (1 if dtype == torch.float64 else 5), "means after step %d" % i, held)
        _close(gm.covs, covs, TOL[dtype] * (1 if dtype == torch.float64 else 5), "covariances after step %d" % i, held)
        if none.any():
            _close(gm.means, before, 0.0, "means of unclaimed components", none)
            _close(gm.covs, np.full_like(covs, un.MIN_VAR), 1e-6, "covariances of unclaimed components", none)
        # carry the library's state over so that one ill-conditioned component does not separate the two runs for good
        means, covs = (a.double().cpu().numpy().reshape(k, -1) for a in (gm.means, gm.covs))
    t, w = gm.parameters()
    _close(w, np.sqrt(covs), 1e-6, "weights")


@pytest.mark.parametrize("kind", ["kmeans", "gmm"])
def test_network_layer_is_initialised_from_its_own_input(kind):
    """cfg3's Similarity layer (2x2 blocks at stride 2, padded, NaN outside): the patches that count are the VALID ones
    whatever the layer's padding, and the layer ends up holding what the restatement computes from the same batches."""
    spec = SPECS["cfg3"]
    net = SimNet(spec, seed=3)
    rng = np.random.default_rng(13)
    data = (rng.normal(size=(24,) + tuple(spec["input_shape"])) * np.linspace(0.5, 2.0, 24)[:, None, None, None]).astype(np.float32)
    sim = net.stages[0]
    layers.perform_unsupervised_init(net, kind=kind, data=data, batch_size=8, seed=5)
    blocks, strides, k = sim.blocks, sim.strides, sim.num_instances
    ref_rng = np.random.RandomState(5)
    batches = [uo.extract_patches(data[i:i + 8].astype(np.float64), blocks, strides) for i in range(0, 24, 8)]
    if kind == "kmeans":
        centres, _ = uo.kmeans_pp_seed(batches[0], k, ref_rng.random_sample(k))
        counts = np.zeros(k)
        for p in batches:
            centres, counts, _ = uo.kmeans_step(centres, counts, p)
        _close(sim.templates.detach(), centres, 2e-4, "templates")
        assert bool((sim.sweights == 1).all())
    else:
        means, covs = uo.gmm_seed(batches[0], ref_rng.randint(0, len(batches[0]), size=k))
        for p in batches:
            means, covs, _ = uo.gmm_step(means, covs, p)
        _close(sim.templates.detach(), means, 1e-3, "templates")
        _close(sim.sweights.detach(), np.sqrt(covs), 1e-3, "weights")
    y = net(torch.from_numpy(data[:4]).cuda())
    assert y.shape == (4, spec["classes"]) and bool(torch.isfinite(y).all())


def test_sequence_of_layers_and_channels_last():
    """A plain list of layers: the second Similarity layer is initialised from what the first one produces, and a
    channels_last layer takes [n, h, w, c] data."""
    rng = np.random.default_rng(14)
    a = layers.Similarity(num_instances=6, blocks=[3, 3], strides=[1, 1], padding='VALID', channels_last=True)
    b = layers.Similarity(num_instances=4, blocks=[2, 2], strides=[2, 2], padding='VALID', channels_last=True)
    data = rng.normal(size=(8, 9, 9, 2)).astype(np.float32)
    layers.perform_unsupervised_init([a, b], kind='kmeans', data=lambda: iter([data[:4], data[4:]]), seed=1)
    assert a.templates.shape == (6, 2, 3, 3) and b.templates.shape == (4, 6, 2, 2)
    mid = a(torch.from_numpy(data).cuda()).detach().permute(0, 3, 1, 2).double().cpu().numpy()
    centres, _ = uo.kmeans_pp_seed(uo.extract_patches(mid[:4], [2, 2], [2, 2]), 4, np.random.RandomState(1).random_sample(4))
    counts = np.zeros(4)
    for lo in (0, 4):
        centres, counts, _ = uo.kmeans_step(centres, counts, uo.extract_patches(mid[lo:lo + 4], [2, 2], [2, 2]))
    _close(b.templates.detach(), centres, 2e-4, "second layer's templates")
    with pytest.raises(ValueError, match="defined for Similarity layers"):
        layers.perform_unsupervised_init([a, b], layers=[torch.nn.Identity()], data=data, batch_size=4)
