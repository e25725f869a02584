"""Unsupervised initialisation without a GPU: the CPU restatement against textbook properties (it has no golden vectors to
be pinned to: the reference delegates this path to tf.contrib.factorization and tests none of it), and the estimators'
host logic (seeding, the per-batch update, the all-reduce of the statistics over two gloo ranks) with the patch statistics
stood in for by that restatement."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import unsupervised_oracle as uo
from simnets_tf_b200 import unsupervised as un


def _blobs(rng, k, n, shape, spread=0.05):
    """n images whose every patch is one of k well separated constant-plus-noise patterns."""
    levels = np.linspace(-2.0, 2.0, k)
    which = rng.integers(0, k, size=n)
    x = levels[which][:, None, None, None] + spread * rng.normal(size=(n,) + shape)
    return x.astype(np.float64), which, levels


def test_patches_are_the_unfolded_windows():
    rng = np.random.default_rng(0)
    x = rng.normal(size=(2, 3, 7, 6))
    for blocks, strides in (((3, 3), (1, 1)), ((2, 3), (2, 1)), ((1, 1), (1, 1)), ((3, 2), (3, 2))):
        p = uo.extract_patches(x, blocks, strides)
        want = torch.nn.functional.unfold(torch.from_numpy(x), kernel_size=blocks, stride=strides)     # [b, c*bh*bw, L]
        assert np.array_equal(p, want.permute(0, 2, 1).reshape(-1, p.shape[1]).numpy())


def test_kmeans_restatement_recovers_separated_blobs_and_keeps_running_means():
    rng = np.random.default_rng(1)
    x, _, levels = _blobs(rng, 4, 64, (1, 3, 3))
    p = uo.extract_patches(x, (3, 3), (1, 1))
    centres, picks = uo.kmeans_pp_seed(p, 4, rng.random(4))
    assert len(set(np.round(centres.mean(1)).tolist())) == 4          # D^2 sampling lands one seed in every blob
    counts = np.zeros(4)
    seen = [[] for _ in range(4)]
    for lo in range(0, len(p), 16):
        centres, counts, a = uo.kmeans_step(centres, counts, p[lo:lo + 16])
        for c in range(4):
            seen[c].append(p[lo:lo + 16][a == c])
    assert counts.sum() == len(p)
    for c in range(4):
        np.testing.assert_allclose(centres[c], np.concatenate(seen[c]).mean(0), rtol=1e-10, atol=1e-12)   # the seed itself drops out
    assert np.allclose(np.sort(centres.mean(1)), levels, atol=0.05)


def test_gmm_restatement_never_lowers_the_likelihood_and_respects_the_floor():
    rng = np.random.default_rng(2)
    x, _, _ = _blobs(rng, 3, 48, (2, 2, 2), spread=0.2)
    p = uo.extract_patches(x, (2, 2), (1, 1))
    means, covs = uo.gmm_seed(p, rng.integers(0, len(p), 3), min_var=0.0)
    last = uo.gmm_mean_log_likelihood(means, covs, p)
    for _ in range(8):
        means, covs, r = uo.gmm_step(means, covs, p, min_var=0.0)
        np.testing.assert_allclose(r.sum(1), 1.0, rtol=1e-12)
        now = uo.gmm_mean_log_likelihood(means, covs, p)
        assert now >= last - 1e-9                                  # EM with no floor is monotone
        last = now
    _, floored, _ = uo.gmm_step(means, covs, p)
    assert (floored >= uo.MIN_VAR * 0.999).all()


@pytest.mark.parametrize("blocks,strides", [((3, 3), (1, 1)), ((2, 2), (2, 2)), ((1, 1), (1, 1))])
def test_estimators_on_stand_in_statistics_equal_the_restatement(blocks, strides):
    rng = np.random.default_rng(3)
    batches = [rng.normal(size=(3, 2, 6, 7)) for _ in range(3)]
    ops = uo.OraclePatchOps(blocks, strides)
    k = 5
    u = rng.random(k)
    km = un.KMeans(blocks, strides, k, ops=ops)
    km.init(torch.from_numpy(batches[0]), uniforms=u)
    centres, _ = uo.kmeans_pp_seed(uo.extract_patches(batches[0], blocks, strides), k, u)
    counts = np.zeros(k)
    for b in batches:
        km.update(torch.from_numpy(b))
        centres, counts, _ = uo.kmeans_step(centres, counts, uo.extract_patches(b, blocks, strides))
    np.testing.assert_allclose(km.centres.reshape(k, -1).numpy(), centres, rtol=1e-10, atol=1e-12)
    np.testing.assert_array_equal(km.counts.numpy(), counts)
    t, w = km.parameters()
    assert t.shape == (k, 2) + tuple(blocks) and bool((w == 1).all())

    picks = rng.integers(0, len(uo.extract_patches(batches[0], blocks, strides)), k)
    gm = un.DiagonalGMM(blocks, strides, k, ops=ops)
    gm.init(torch.from_numpy(batches[0]), picks=picks)
    means, covs = uo.gmm_seed(uo.extract_patches(batches[0], blocks, strides), picks)
    np.testing.assert_allclose(gm.covs.reshape(k, -1).numpy(), covs, rtol=1e-10)
    for b in batches:
        gm.update(torch.from_numpy(b))
        means, covs, _ = uo.gmm_step(means, covs, uo.extract_patches(b, blocks, strides))
    np.testing.assert_allclose(gm.means.reshape(k, -1).numpy(), means, rtol=1e-8, atol=1e-10)
    np.testing.assert_allclose(gm.covs.reshape(k, -1).numpy(), covs, rtol=1e-8, atol=1e-10)
    t, w = gm.parameters()
    np.testing.assert_allclose(w.reshape(k, -1).numpy(), np.sqrt(covs), rtol=1e-8)


def test_kind_and_input_are_checked():
    class L(object):
        blocks, strides, num_instances = [3, 3], [1, 1], 4
    with pytest.raises(ValueError, match='kind must be one of "kmeans" or "gmm"'):
        un.similarity_unsupervised_init("pca", L())
    est = un.similarity_unsupervised_init("kmeans", L(), ops=uo.OraclePatchOps([3, 3], [1, 1]))
    with pytest.raises(ValueError, match="at least one whole patch"):
        est.init(torch.zeros(1, 1, 2, 5))
    with pytest.raises(ValueError, match="batch size must be given"):
        un.perform_unsupervised_init([], data=np.zeros((4, 1, 3, 3)))


def test_library_statistics_refuse_cpu_tensors():
    ops = un.LibraryPatchOps([3, 3], [1, 1])
    x = torch.zeros(1, 1, 4, 4)
    with pytest.raises(RuntimeError, match="no CPU kernels"):
        ops.neg_scaled_sqdist(x, torch.zeros(2, 1, 3, 3), torch.ones(2, 1, 3, 3))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(4)
        first = rng.normal(size=(4, 2, 5, 5))
        batches = [rng.normal(size=(4, 2, 5, 5)) for _ in range(2)]
        ops = uo.OraclePatchOps((3, 3), (1, 1))
        u, picks = rng.random(3), rng.integers(0, 36, 3)
        res = []
        for group, lo, hi in ((dist.group.WORLD, 2 * rank, 2 * rank + 2), (None, 0, 4)):
            km = un.KMeans((3, 3), (1, 1), 3, ops=ops, group=group)
            gm = un.DiagonalGMM((3, 3), (1, 1), 3, ops=ops, group=group)
            km.init(torch.from_numpy(first), uniforms=u)
            gm.init(torch.from_numpy(first), picks=picks)
            for b in batches:
                km.update(torch.from_numpy(b[lo:hi]))
                gm.update(torch.from_numpy(b[lo:hi]))
            res.append(torch.cat([km.centres.flatten(), km.counts, gm.means.flatten(), gm.covs.flatten()]))
        if rank == 0:
            np.save(out, np.array([float((res[0] - res[1]).abs().max()), float(res[1].abs().max())]))
    finally:
        dist.destroy_process_group()


def test_statistics_summed_over_two_ranks_equal_the_unsharded_step(tmp_path):
    out = str(tmp_path / "r.npy")
    mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    err, scale = np.load(out)
    assert scale > 0 and err < 1e-12 * max(scale, 1.0)
