"""The layer classes of simnets_tf_b200.keras, with the grid of the reference's own layer tests
(python/simnets/test/keras/__init__.py:12-140): attributes reach the op, output shapes, channels_last equivalence,
padding 'SAME' / 'VALID', the offsets shape created by build(), get_config keys, normalize_offsets on / off; and, as in
python/simnets/test/__init__.py:156-187,374-402, that the gradient wiring of the differentiable ops carries the attrs of
the forward op (checked by comparing autograd gradients with the grad entry points called with the same attrs)."""
import importlib

import numpy as np
import pytest
import torch

from simnets_tf_b200 import keras as layers

mex_ops = importlib.import_module("simnets_tf_b200.ops.mex")
sim_ops = importlib.import_module("simnets_tf_b200.ops.similarity")

pytestmark = pytest.mark.gpu


def _x(*shape, seed=0):
    return torch.from_numpy(np.random.default_rng(seed).normal(size=shape).astype(np.float32)).cuda()


# ---- Mex
def test_mex_attributes_reach_the_layer_and_its_config():
    l = layers.Mex(num_instances=10, padding='VALID', strides=[1, 2, 2], blocks=[1, 2, 3], epsilon=2.0, use_unshared_regions=False,
                   shared_offset_region=[2, 2], unshared_offset_region=[4, 4], softmax_mode=True, blocks_out_of_bounds_value=1.0,
                   blocks_round_down=False, normalize_offsets=True)
    # As in the reference's test, the layer is built and its shape inferred, not run: a two-entry region list passes the
    # dims helper (first entry for height and width) while the op's kernel accepts one or three entries only.
    shape = l.compute_output_shape((2, 3, 40, 40))
    assert l.padding == [0, 0, 0] and l.strides == [1, 2, 2] and l.blocks == [1, 2, 3]
    cfg = l.get_config()
    assert sorted(cfg) == sorted(['num_instances', 'padding', 'strides', 'blocks', 'epsilon', 'use_unshared_regions', 'shared_offset_region',
                                  'unshared_offset_region', 'softmax_mode', 'blocks_out_of_bounds_value', 'blocks_round_down',
                                  'normalize_offsets', 'offsets_initializer', 'channels_last'])
    assert cfg['num_instances'] == 10 and cfg['epsilon'] == 2.0 and cfg['use_unshared_regions'] is False
    assert cfg['shared_offset_region'] == [2, 2] and cfg['unshared_offset_region'] == [4, 4] and cfg['softmax_mode'] is True
    assert cfg['blocks_out_of_bounds_value'] == 1.0 and cfg['blocks_round_down'] is False and cfg['normalize_offsets'] is True
    # round-up output size: ceil((40 - 2) / 2) + 1, ceil((40 - 3) / 2) + 1
    assert tuple(shape) == (2, 30, 20, 20)
    assert tuple(l.offsets.shape) == (100, 10, 1, 2, 3)      # shared regions of 2x2 positions, all 3 channels: 10 * 10 * 1
    with pytest.raises(ValueError, match="1 or 3"):
        l(_x(2, 3, 40, 40))


@pytest.mark.parametrize("num_instances,padding,strides,blocks,input_shape,output_shape", [
    (10, [1, 0, 1], [1, 1, 1], [1, 2, 2], (3, 10, 13), (50, 9, 14)),
    (10, [2, 1, 1], [1, 3, 2], [1, 2, 2], (3, 10, 13), (70, 5, 8)),
    (2, [1, 1, 1], [1, 3, 2], [1, 2, 2], (1, 10, 13), (6, 5, 8)),
])
def test_mex_output_shapes(num_instances, padding, strides, blocks, input_shape, output_shape):
    l = layers.Mex(num_instances=num_instances, padding=padding, strides=strides, blocks=blocks, epsilon=2.0, use_unshared_regions=False,
                   shared_offset_region=[2, 2], unshared_offset_region=[4, 4], softmax_mode=True, blocks_out_of_bounds_value=1.0,
                   blocks_round_down=False, normalize_offsets=True)
    assert tuple(l.compute_output_shape((2,) + input_shape)[1:]) == output_shape


def test_mex_channels_last_equals_channels_first():
    kw = dict(num_instances=3, padding='VALID', strides=[1, 2, 2], blocks=[1, 1, 1], epsilon=1.0, use_unshared_regions=True,
              unshared_offset_region=[2], softmax_mode=True, offsets_initializer='ones')
    l1, l2 = layers.Mex(**kw), layers.Mex(channels_last=True, **kw)
    data = _x(1, 3, 10, 11)
    res1 = l1(data)
    res2 = l2(data.permute(0, 2, 3, 1).contiguous())
    assert torch.allclose(res1, res2.permute(0, 3, 1, 2), rtol=1e-6, atol=1e-6)


def test_mex_build_creates_offsets_of_the_helper_shape():
    l = layers.Mex(num_instances=7, blocks=[3, 2, 2], strides=[3, 2, 2], use_unshared_regions=True, unshared_offset_region=[2])
    l.build((4, 6, 9, 8), device="cuda")
    nreg = layers._mex_dims_helper([6, 9, 8], 7, blocks=[3, 2, 2], padding=[0, 0, 0], strides=[3, 2, 2], use_unshared_regions=True,
                                   unshared_offset_region=[2])
    assert tuple(l.offsets.shape) == (nreg, 7, 3, 2, 2) and nreg == 2 * 2 * 2
    # 'SAME' pads by half a block, -1 entries take the image dimension
    l = layers.Mex(num_instances=2, blocks=[-1, 3, 3], padding='SAME')
    l.build((1, 5, 8, 8), device="cuda")
    assert l.blocks == [5, 3, 3] and l.padding == [2, 1, 1]


def test_mex_normalize_offsets_on_and_off():
    x = _x(2, 6, 4, 4, seed=3)
    a = layers.Mex(num_instances=4, blocks=[6, 1, 1], strides=[6, 1, 1], softmax_mode=True, normalize_offsets=False)
    b = layers.Mex(num_instances=4, blocks=[6, 1, 1], strides=[6, 1, 1], softmax_mode=True, normalize_offsets=True)
    ya = a(x)
    b.build(tuple(x.shape), device="cuda")
    with torch.no_grad():
        b.offsets.copy_(a.offsets)
    yb = b(x)
    flat = a.offsets.reshape(a.offsets.shape[0] * 4, -1)
    lse = torch.logsumexp(flat.double(), dim=1).reshape(a.offsets.shape[0], 4)
    # subtracting a per-(region, instance) constant from the offsets subtracts it from the output
    reg = mex_ops._geometry(mex_ops._desc(x, 4, mex_ops._attrs(blocks=[6, 1, 1], strides=[6, 1, 1], softmax_mode=True)))
    assert reg.num_regions == a.offsets.shape[0]
    diff = (ya - yb).double()                                   # [B, 4 * Co, H, W]
    want = lse.mean(dim=0) if reg.num_regions == 1 else None
    if want is not None:
        assert torch.allclose(diff.mean(dim=(0, 2, 3)), want, rtol=1e-5, atol=1e-5)
    # gradient reaches the raw offsets through the normalisation: rows of d(offsets) sum to zero
    yb.sum().backward()
    rows = b.offsets.grad.reshape(b.offsets.shape[0] * 4, -1).sum(dim=1)
    assert float(rows.abs().max()) < 1e-3 * float(b.offsets.grad.abs().max()) + 1e-6


# ---- Similarity
def test_similarity_attributes_reach_the_layer_and_its_config():
    l = layers.Similarity(num_instances=5, similarity_function='L1', strides=[2, 3], blocks=[3, 2], padding='VALID', normalization_term=False,
                          normalization_term_fudge=1.0, ignore_nan_input=False, out_of_bounds_value=1.0)
    y = l(_x(2, 3, 40, 40))
    assert l.blocks == [3, 2] and l.strides == [2, 3] and l.padding == [0, 0]
    cfg = l.get_config()
    assert sorted(cfg) == sorted(['num_instances', 'similarity_function', 'strides', 'blocks', 'padding', 'normalization_term',
                                  'normalization_term_fudge', 'ignore_nan_input', 'out_of_bounds_value', 'templates_initializer',
                                  'weights_initializer', 'channels_last'])
    assert cfg['similarity_function'] == 'L1' and cfg['normalization_term_fudge'] == 1.0 and cfg['out_of_bounds_value'] == 1.0
    assert tuple(y.shape) == (2, 5, 19, 13)
    with pytest.raises(ValueError):
        layers.Similarity(num_instances=5, padding='FULL')


@pytest.mark.parametrize("num_instances,padding,strides,blocks,input_shape,output_shape", [
    (10, [0, 1], [1, 1], [2, 2], (3, 10, 13), (10, 9, 14)),
    (10, [1, 1], [3, 2], [2, 2], (3, 10, 13), (10, 4, 7)),
    (2, [1, 1], [3, 2], [2, 2], (1, 10, 13), (2, 4, 7)),
])
def test_similarity_output_shapes(num_instances, padding, strides, blocks, input_shape, output_shape):
    l = layers.Similarity(num_instances=num_instances, similarity_function='L1', strides=strides, blocks=blocks, padding=padding,
                          normalization_term=False, normalization_term_fudge=1.0, out_of_bounds_value=1.0)
    assert tuple(l.compute_output_shape((2,) + input_shape)[1:]) == output_shape


def test_similarity_padding_same_and_valid():
    x = _x(2, 3, 12, 12)
    same = layers.Similarity(num_instances=4, blocks=[3, 3], strides=[1, 1], padding='SAME')
    valid = layers.Similarity(num_instances=4, blocks=[3, 3], strides=[1, 1], padding='valid')
    assert same.padding == [1, 1] and valid.padding == [0, 0]
    assert tuple(same(x).shape) == (2, 4, 12, 12) and tuple(valid(x).shape) == (2, 4, 10, 10)


def test_similarity_channels_last_equals_channels_first():
    kw = dict(num_instances=3, padding='VALID', strides=[2, 2], blocks=[1, 1], templates_initializer='ones', weights_initializer='ones')
    l1, l2 = layers.Similarity(**kw), layers.Similarity(channels_last=True, **kw)
    data = _x(1, 3, 10, 11)
    res1 = l1(data)
    res2 = l2(data.permute(0, 2, 3, 1).contiguous())
    assert torch.allclose(res1, res2.permute(0, 3, 1, 2), rtol=1e-6, atol=1e-6)


# ---- gradient wiring carries the forward op's attrs
def test_similarity_autograd_uses_the_forward_attrs():
    attrs = dict(similarity_function='L1', blocks=[2, 3], strides=[2, 1], padding=[1, 0], out_of_bounds_value=0.5)
    x, t = _x(2, 3, 9, 8, seed=1).requires_grad_(True), _x(4, 3, 2, 3, seed=2).requires_grad_(True)
    w = (_x(4, 3, 2, 3, seed=3).abs() + 0.1).requires_grad_(True)
    y = sim_ops.similarity(x, t, w, **attrs)
    dy = _x(*y.shape, seed=4)
    y.backward(dy)
    full = sim_ops._attrs(**attrs)
    assert torch.equal(x.grad, sim_ops.similarity_input_grad(x.detach(), t.detach(), w.detach(), dy, **full))
    dt, dw = sim_ops.similarity_parameters_grad(x.detach(), t.detach(), w.detach(), dy, **full)
    assert torch.equal(t.grad, dt) and torch.equal(w.grad, dw)


def test_mex_autograd_uses_the_forward_attrs():
    attrs = dict(softmax_mode=True, padding=[0, 1, 1], strides=[2, 2, 1], blocks=[2, 3, 2], epsilon=0.5, blocks_out_of_bounds_value=0.25,
                 blocks_round_down=False, use_unshared_regions=False, shared_offset_region=[2])
    x = _x(2, 4, 7, 6, seed=5).requires_grad_(True)
    g = mex_ops._geometry(mex_ops._desc(x, 3, mex_ops._attrs(**attrs)))
    off = _x(g.num_regions, 3, 2, 3, 2, seed=6).requires_grad_(True)
    y = mex_ops.mex(x, off, 3, **attrs)
    dy = _x(*y.shape, seed=7)
    y.backward(dy)
    assert torch.allclose(x.grad, mex_ops.mex_input_grad(x.detach(), off.detach(), y.detach(), dy, 3, **attrs), rtol=1e-6, atol=1e-7)
    assert torch.allclose(off.grad, mex_ops.mex_offsets_grad(x.detach(), off.detach(), y.detach(), dy, 3, **attrs), rtol=1e-6, atol=1e-7)
