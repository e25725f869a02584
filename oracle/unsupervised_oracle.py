"""CPU restatement (numpy, float64 unless told otherwise) of the unsupervised initialisation of a Similarity layer: test
infrastructure, never imported by the product.

PARITY UNPINNED.  The reference (HUJI-Deep/simnets-tf python/simnets/unsupervised/kmeans.py:39-57, gmm.py:37-71) delegates
both estimators to `tf.contrib.factorization` of TensorFlow 1.x (no version is pinned anywhere in the reference's tree;
`tf.contrib` exists in 1.0-1.15 only), which is neither vendored there nor installable here, and the reference holds no
test or golden vector for this path.  What this file restates is therefore the published algorithms those calls name, over
explicitly extracted patches:

* patches: every `blocks` window at `strides` steps that lies wholly inside the image ('VALID', kmeans.py:43-45), here in
  (channel, row, column) order so that a centre reshapes straight into a template [channels, block_h, block_w] (the
  reference extracts (row, column, channel) and transposes afterwards, kmeans.py:51-53);
* k-means++ seeding (Arthur & Vassilvitskii 2007) driven by given uniform numbers, and the mini-batch k-means update with
  per-centre counts (Sculley 2010);
* one EM step of a diagonal Gaussian mixture with uniform mixing weights held fixed (params='mc'), the covariance taken
  about the new mean and a floor added to it.
"""
import numpy as np

MIN_VAR = 1e-3


def extract_patches(x, blocks, strides):
    """x [batch, channels, h, w] -> [batch * out_h * out_w, channels * block_h * block_w], patches in (batch, row, column)
    order, each flattened as (channel, block row, block column)."""
    b, c, h, w = x.shape
    oh, ow = (h - blocks[0]) // strides[0] + 1, (w - blocks[1]) // strides[1] + 1
    out = np.empty((b, oh, ow, c, blocks[0], blocks[1]), dtype=x.dtype)
    for i in range(oh):
        for j in range(ow):
            out[:, i, j] = x[:, :, i * strides[0]:i * strides[0] + blocks[0], j * strides[1]:j * strides[1] + blocks[1]]
    return out.reshape(b * oh * ow, c * blocks[0] * blocks[1])


def kmeans_pp_seed(patches, k, uniforms):
    """Seeds chosen by D^2 sampling: number c is the first patch whose running sum of nearest-seed distances exceeds
    uniforms[c] times the total."""
    n = len(patches)
    picks = [min(int(uniforms[0] * n), n - 1)]
    nearest = None
    for c in range(1, k):
        d = ((patches - patches[picks[-1]]) ** 2).sum(1)
        nearest = d if nearest is None else np.minimum(nearest, d)
        cum = np.cumsum(nearest.astype(np.float64))
        picks.append(n - 1 if cum[-1] <= 0 else min(int(np.searchsorted(cum, uniforms[c] * cum[-1], side="right")), n - 1))
    return patches[picks].copy(), picks


def kmeans_step(centres, counts, patches):
    """One mini-batch step; returns (centres, counts, assignment)."""
    d = ((patches[:, None, :] - centres[None, :, :]) ** 2).sum(2)
    a = d.argmin(1)
    centres, counts = centres.copy(), counts.copy()
    for c in range(len(centres)):
        mine = patches[a == c]
        if len(mine):
            counts[c] += len(mine)
            centres[c] += (mine.sum(0) - len(mine) * centres[c]) / counts[c]
    return centres, counts, a


def gmm_seed(patches, picks, min_var=MIN_VAR):
    means = patches[list(picks)].copy()
    var = patches.var(axis=0) + min_var
    return means, np.tile(var, (len(means), 1))


def gmm_log_joint(means, covs, patches):
    """log N(p; mu_c, diag cov_c) up to the constants shared by all components, [patches, k]."""
    d = ((patches[:, None, :] - means[None]) ** 2 / covs[None]).sum(2)
    return -0.5 * (d + np.log(covs).sum(1)[None])


def gmm_step(means, covs, patches, min_var=MIN_VAR):
    """One EM step; returns (means, covs, responsibilities).  A component that no patch of the batch claims at all (zero
    mass, where the textbook step divides zero by zero) keeps its mean and gets the floor as its covariance."""
    lj = gmm_log_joint(means, covs, patches)
    lj -= lj.max(1, keepdims=True)
    r = np.exp(lj)
    r /= r.sum(1, keepdims=True)
    mass = r.sum(0)[:, None]
    dead = mass[:, 0] <= np.finfo(patches.dtype).tiny
    safe = np.where(dead[:, None], 1.0, mass)
    new_means = r.T @ patches / safe
    new_covs = r.T @ (patches ** 2) / safe - new_means ** 2 + min_var
    new_means[dead], new_covs[dead] = means[dead], min_var
    return new_means, new_covs, r


def gmm_mean_log_likelihood(means, covs, patches):
    lj = gmm_log_joint(means, covs, patches) - 0.5 * patches.shape[1] * np.log(2 * np.pi) - np.log(len(means))
    m = lj.max(1, keepdims=True)
    return float((m[:, 0] + np.log(np.exp(lj - m).sum(1))).mean())


class OraclePatchOps(object):
    """The two patch statistics of simnets_tf_b200.unsupervised on explicit patches, as torch CPU tensors: lets the host
    logic of the estimators (and their all-reduce) run where no GPU is."""

    def __init__(self, blocks, strides):
        self.blocks, self.strides = list(blocks), list(strides)

    def _p(self, x):
        import torch
        p = extract_patches(x.numpy(), self.blocks, self.strides)
        oh = (x.shape[2] - self.blocks[0]) // self.strides[0] + 1
        return torch.from_numpy(p), oh, len(p) // (x.shape[0] * oh)

    def neg_scaled_sqdist(self, x, centres, scales):
        p, oh, ow = self._p(x)
        c, s = centres.reshape(len(centres), -1), scales.reshape(len(scales), -1)
        d = -(((p[:, None, :] - c[None]) ** 2) * s[None]).sum(2)
        return d.reshape(x.shape[0], oh, ow, len(c)).permute(0, 3, 1, 2).contiguous()

    def moments(self, x, centres, resp):
        p, oh, ow = self._p(x)
        c = centres.reshape(len(centres), -1)
        r = resp.permute(0, 2, 3, 1).reshape(-1, len(c))
        diff = p[:, None, :] - c[None]
        return ((r[:, :, None] * diff).sum(0).reshape(centres.shape), (r[:, :, None] * diff ** 2).sum(0).reshape(centres.shape))
