"""Unsupervised initialisation of a Similarity layer from data: its templates (and weights) become the cluster centres
(and spreads) of the layer's own input patches, found by mini-batch k-means or by EM on a diagonal Gaussian mixture.
Interface of HUJI-Deep/simnets-tf python/simnets/unsupervised/__init__.py:6-33 and python/simnets/keras.py:191-238.

The reference assembles both estimators from TensorFlow 1.x's `tf.contrib.factorization`, which is not part of its tree:
`KMeans(patches, k, use_mini_batch=True, initial_clusters='kmeans_plus_plus')` (unsupervised/kmeans.py:46) and
`gmm(patches, initial_clusters='random', random_seed=33, covariance_type='diag', params='mc')` (unsupervised/gmm.py:44-45)
over `tf.extract_image_patches(..., padding='VALID')` of the op's input.  What is kept here is what the reference itself
fixes: VALID patches with the op's blocks and strides whatever the op's own padding, one estimator step per batch, k-means
assigning `templates = centres, weights = 1` (kmeans.py:54-57) and the mixture assigning `templates = means,
weights = sqrt(diagonal covariances)` (gmm.py:66-71).  The estimators follow the published algorithms those calls name
(k-means++ seeding, Sculley's mini-batch k-means with per-centre counts, one full EM step per batch with uniform mixing
weights and a variance floor); the random draws of TensorFlow's own kernels are not reproducible outside it.

Patches are never written out.  Both estimators need two things per batch, and both are the Similarity operator itself:

* the squared distance of every patch to every centre, scaled per coordinate: the L2 Similarity forward pass,
  `-sum w (p - c)^2`;
* per centre, the sums `sum r (p - c)` and `sum r (p - c)^2` over the patches with responsibilities r: the L2 Similarity
  parameter gradients with `output_grad = r` and unit weights, `dT = 2 sum r (p - c)` and `dW = -sum r (p - c)^2`
  (include/utils/similarity_utils.hpp:88-90).

So a step is one forward and one parameter-gradient launch of the library plus element-wise work on [k, patch] tensors, and
the statistics of a data-parallel job are summed over ranks by one all-reduce before the centres move.
"""

import importlib

import numpy as np
import torch

_sim = importlib.import_module(__package__ + ".ops.similarity")     # the module: `ops.similarity` itself is the op function

MIN_VAR = 1e-3      # variance floor added to every diagonal covariance by an EM step


class LibraryPatchOps(object):
    """The two patch statistics on the CUDA operators.  Tensors must live on a CUDA device: there is no CPU route."""

    def __init__(self, blocks, strides, flags=0):
        self.attrs = dict(similarity_function='L2', blocks=list(blocks), strides=list(strides), padding=[0, 0],
                          normalization_term=False, ignore_nan_input=False, out_of_bounds_value=0.0)
        self.flags = flags

    def neg_scaled_sqdist(self, x, centres, scales):
        """[batch, k, out_h, out_w]: -sum_j scales[c, j] (patch[j] - centres[c, j])^2."""
        return _sim.similarity_forward(x, centres, scales, flags=self.flags, **self.attrs)

    def moments(self, x, centres, resp):
        """(sum r (p - c), sum r (p - c)^2), each shaped like `centres`, for resp [batch, k, out_h, out_w]."""
        dt, dw = _sim.similarity_parameters_grad(x, centres, torch.ones_like(centres), resp, flags=self.flags, **self.attrs)
        return dt.mul_(0.5), dw.neg_()


def _patch_grid(x, blocks, strides):
    return (x.shape[2] - blocks[0]) // strides[0] + 1, (x.shape[3] - blocks[1]) // strides[1] + 1


def _patch_at(x, blocks, strides, flat_index):
    """Patch number `flat_index` of the VALID grid in (batch, row, column) order, [channels, block_h, block_w]."""
    oh, ow = _patch_grid(x, blocks, strides)
    b, rem = divmod(int(flat_index), oh * ow)
    i, j = divmod(rem, ow)
    return x[b, :, i * strides[0]:i * strides[0] + blocks[0], j * strides[1]:j * strides[1] + blocks[1]]


def _all_reduce(group, *tensors):
    """Sum the statistics over the ranks of `group` (one collective over a flat buffer); nothing to do without one."""
    if group is None:
        return tensors
    import torch.distributed as dist
    flat = torch.cat([t.reshape(-1) for t in tensors])
    dist.all_reduce(flat, group=group)
    out, o = [], 0
    for t in tensors:
        out.append(flat[o:o + t.numel()].view_as(t))
        o += t.numel()
    return out


class _Estimator(object):
    def __init__(self, blocks, strides, num_instances, seed, ops=None, group=None):
        self.blocks, self.strides, self.k = list(blocks), list(strides), int(num_instances)
        self.ops = ops if ops is not None else LibraryPatchOps(blocks, strides)
        self.group = group
        self.rng = np.random.RandomState(seed)

    def _check(self, x):
        if x.dim() != 4 or x.shape[2] < self.blocks[0] or x.shape[3] < self.blocks[1]:
            raise ValueError("input must be [batch, channels, height, width] and hold at least one whole patch")
        return x.contiguous()


class KMeans(_Estimator):
    """Mini-batch k-means over the patches of each batch.

    init(batch): k-means++ seeding on the first batch: the first centre is a patch drawn uniformly, each further one a
    patch drawn with probability proportional to its squared distance to the nearest centre chosen so far.
    update(batch): every patch goes to its nearest centre; with n_c patches of this batch at centre c and N_c seen before,
    `c += (sum of those patches - n_c c) / (N_c + n_c)`, that is, every centre stays the mean of all patches ever assigned
    to it with their assignment-time weights (per-centre learning rate 1 / count)."""

    def __init__(self, blocks, strides, num_instances, seed=0, ops=None, group=None):
        super(KMeans, self).__init__(blocks, strides, num_instances, seed, ops, group)
        self.centres = None
        self.counts = None

    def init(self, x, uniforms=None):
        """`uniforms`: the k numbers in [0, 1) that pick the seeds (default: drawn from this object's seeded generator).
        With a process group every rank must pass the same batch here: seeding is not sharded."""
        x = self._check(x)
        oh, ow = _patch_grid(x, self.blocks, self.strides)
        n = x.shape[0] * oh * ow
        u = self.rng.random_sample(self.k) if uniforms is None else np.asarray(uniforms, dtype=np.float64)
        first = min(int(u[0] * n), n - 1)
        centres = [_patch_at(x, self.blocks, self.strides, first)]
        nearest = None
        for c in range(1, self.k):
            last = centres[-1].unsqueeze(0).contiguous()
            d = self.ops.neg_scaled_sqdist(x, last, torch.ones_like(last)).neg_().clamp_(min=0).reshape(-1)
            nearest = d if nearest is None else torch.minimum(nearest, d)
            cum = np.cumsum(nearest.double().cpu().numpy())
            pick = n - 1 if cum[-1] <= 0 else min(int(np.searchsorted(cum, u[c] * cum[-1], side="right")), n - 1)
            centres.append(_patch_at(x, self.blocks, self.strides, pick))
        self.centres = torch.stack(centres).contiguous()
        self.counts = torch.zeros(self.k, dtype=x.dtype, device=x.device)
        return self.centres

    def update(self, x):
        x = self._check(x)
        score = self.ops.neg_scaled_sqdist(x, self.centres, torch.ones_like(self.centres))
        onehot = torch.zeros_like(score).scatter_(1, score.argmax(dim=1, keepdim=True), 1.0)
        shift, _ = self.ops.moments(x, self.centres, onehot)            # sum over the centre's patches of (p - c)
        n, shift = _all_reduce(self.group, onehot.sum(dim=(0, 2, 3)), shift)
        self.counts = self.counts + n
        self.centres = self.centres + shift / self.counts.clamp(min=1).view(-1, 1, 1, 1)
        return self.centres

    def parameters(self):
        """(templates, weights) as the reference assigns them."""
        return self.centres, torch.ones_like(self.centres)


class DiagonalGMM(_Estimator):
    """EM on a mixture of k diagonal Gaussians with fixed uniform mixing weights; means and covariances are re-estimated.

    init(batch): the means are k patches of the first batch drawn uniformly, every covariance the per-coordinate variance
    of all patches of that batch plus the floor.
    update(batch): one full EM step on this batch from the current parameters: responsibilities
    `r ∝ exp(-1/2 sum ((p - mu)^2 / var + log var))`, then `mu' = sum r p / sum r` and
    `var' = sum r p^2 / sum r - mu'^2 + floor`.  A component that no patch of the batch claims at all (zero mass, where the
    textbook step divides zero by zero) keeps its mean and gets the floor as its covariance."""

    def __init__(self, blocks, strides, num_instances, seed=33, ops=None, group=None, min_var=MIN_VAR):
        super(DiagonalGMM, self).__init__(blocks, strides, num_instances, seed, ops, group)
        self.min_var = float(min_var)
        self.means = None
        self.covs = None

    def init(self, x, picks=None):
        """`picks`: the k patch numbers that become the means (default: drawn from this object's seeded generator).
        With a process group every rank must pass the same batch here: seeding is not sharded."""
        x = self._check(x)
        oh, ow = _patch_grid(x, self.blocks, self.strides)
        n = x.shape[0] * oh * ow
        picks = self.rng.randint(0, n, size=self.k) if picks is None else picks
        self.means = torch.stack([_patch_at(x, self.blocks, self.strides, p) for p in picks]).contiguous()
        # variance of the data in two passes (mean first, then squares about it: no cancellation in float32)
        ones = torch.ones((x.shape[0], 1, oh, ow), dtype=x.dtype, device=x.device)
        zero = torch.zeros_like(self.means[:1])
        total, _ = self.ops.moments(x, zero, ones)
        mean = total / n
        _, sq = self.ops.moments(x, mean.contiguous(), ones)
        self.covs = (sq / n + self.min_var).expand_as(self.means).contiguous()
        return self.means, self.covs

    def update(self, x):
        x = self._check(x)
        half_mahalanobis = self.ops.neg_scaled_sqdist(x, self.means, (1.0 / self.covs).contiguous())
        logdet = self.covs.log().sum(dim=(1, 2, 3))
        resp = torch.softmax(0.5 * (half_mahalanobis - logdet.view(1, -1, 1, 1)), dim=1)
        shift, sq = self.ops.moments(x, self.means, resp)
        mass, shift, sq = _all_reduce(self.group, resp.sum(dim=(0, 2, 3)), shift, sq)
        mass = mass.clamp(min=torch.finfo(x.dtype).tiny).view(-1, 1, 1, 1)
        step = shift / mass
        self.covs = (sq / mass - step * step + self.min_var).contiguous()     # second moment about the NEW mean
        self.means = (self.means + step).contiguous()
        return self.means, self.covs

    def parameters(self):
        """(templates, weights) as the reference assigns them: means and the square roots of the covariances."""
        return self.means, self.covs.sqrt()


def similarity_unsupervised_init(kind, layer, seed=None, ops=None, group=None):
    """The estimator for a `keras.Similarity` layer (or anything with `blocks`, `strides`, `num_instances`): an object with
    `init(batch)`, to be called once with the first batch, and `update(batch)`, to be called with every batch (the first
    one too), the counterparts of the reference's `(init_op, update_op)` pair; `assign_to(layer)` stores the result."""
    if kind == 'kmeans':
        est = KMeans(layer.blocks, layer.strides, layer.num_instances, 0 if seed is None else seed, ops, group)
    elif kind == 'gmm':
        est = DiagonalGMM(layer.blocks, layer.strides, layer.num_instances, 33 if seed is None else seed, ops, group)
    else:
        raise ValueError('kind must be one of "kmeans" or "gmm"')
    return est


def assign_to(layer, estimator):
    """Store the estimator's current (templates, weights) in the layer's variables."""
    templates, weights = estimator.parameters()
    with torch.no_grad():
        if layer.templates is None:
            layer.templates = torch.nn.Parameter(templates.clone())
            layer.sweights = torch.nn.Parameter(weights.clone())
        else:
            layer.templates.copy_(templates)
            layer.sweights.copy_(weights)


def _batches(data, batch_size):
    if callable(data):
        return data
    if batch_size is None:
        raise ValueError('data is nparray, so batch size must be given')

    def gen():
        for i in range(0, len(data), batch_size):
            yield data[i:i + batch_size]
    return gen


def _input_of(model, layer, x):
    """What reaches `layer` when `x` enters `model`: a SimNet-style module with a layer plan, or a sequence of modules."""
    plan = getattr(model, "_plan", None)
    if plan is not None:
        idx = next(i for i, (_, m) in enumerate(plan) if m is layer)
        return model.forward_range(x, 0, idx)
    for m in model:
        if m is layer:
            return x
        x = m(x)
    raise ValueError("layer is not part of the model")


def perform_unsupervised_init(model, kind='gmm', layers=[], data=None, batch_size=None, seed=None, group=None, device="cuda"):
    """Initialise the Similarity layers of `model` one after the other, front to back, each from the activations that reach
    it with the layers in front already initialised (python/simnets/keras.py:191-238).  `data`: an array [n, c, h, w] (then
    `batch_size` is required) or a callable returning an iterator over batches.  The reference's other branch (PCA filters
    for Keras `Conv2D` layers) has no counterpart: there are no convolution layers in this library."""
    from . import keras as _layers
    members = [m for _, m in model._plan if m is not None] if hasattr(model, "_plan") else list(model)
    layers = list(layers) if layers else [m for m in members if isinstance(m, _layers.Similarity)]
    gen = _batches(data, batch_size)
    for layer in layers:
        if not isinstance(layer, _layers.Similarity):
            raise ValueError("unsupervised initialisation is defined for Similarity layers, got %s" % type(layer).__name__)
        est = similarity_unsupervised_init(kind, layer, seed=seed, group=group)
        with torch.no_grad():
            for idx, batch in enumerate(gen()):
                x = _input_of(model, layer, torch.as_tensor(batch).to(device))
                if layer.channels_last:
                    x = x.permute(0, 3, 1, 2)
                if idx == 0:
                    est.init(x)
                est.update(x)
        assign_to(layer, est)
    return model
