"""Host-side logic of the data-parallel path on CPU ranks (gloo, world size 2): batch sharding, the
flat gradient bucket and its all-reduce, and that shard gradients summed over ranks equal the
unsharded gradients.  The operators are stood in for by the CPU oracle: this test is about the
plumbing around them, which is identical on GPUs."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from simnets_tf_b200 import dp
from simnets_tf_b200.simnet import SPECS


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_shard_bounds_cover_batch_exactly():
    for gb, ws in ((2048, 8), (2048, 1), (10, 4), (3, 4), (0, 2)):
        spans = [dp.shard_bounds(gb, ws, r) for r in range(ws)]
        assert spans[0][0] == 0 and spans[-1][1] == gb
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert max(b - a for a, b in spans) - min(b - a for a, b in spans) <= 1


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle
        from oracle.simnet_cpu import CpuSimNet
        spec = SPECS["cfg3"]
        gb = 4
        rng = np.random.default_rng(3)
        x = rng.uniform(-0.5, 0.5, size=(gb,) + tuple(spec["input_shape"])).astype(np.float32)
        labels = rng.integers(0, 10, size=gb)
        net = CpuSimNet(spec, oracle.load("port"), seed=9)
        bucket = dp.GradBucket(net.parameters())
        lo, hi = dp.shard_bounds(gb, world, rank)
        bucket.zero()
        _, grads = net.step(x[lo:hi], labels[lo:hi], global_batch=gb)
        flat = torch.cat([torch.from_numpy(g).flatten() for g in grads])
        bucket.flat.copy_(flat)
        bucket.all_reduce()
        # a rank that stops before the collective is noticed on the host, not on a device
        if rank == 0:
            full = CpuSimNet(spec, oracle.load("port"), seed=9)
            _, want = full.step(x, labels, global_batch=gb)
            want = np.concatenate([g.flatten() for g in want])
            got = bucket.flat.numpy()
            err = np.abs(got - want).max() / np.abs(want).max()
            np.save(out, np.array([err, bucket.flat.numel()]))
    finally:
        dist.destroy_process_group()


def test_sharded_gradients_sum_to_unsharded(tmp_path, port):
    out = str(tmp_path / "result.npy")
    mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    err, n = np.load(out)
    assert n == 701696
    # float32 sums in a different order (two shard sums added vs one running sum): a few 1e-5 of the largest entry
    assert err < 2e-4


def test_bucket_views_alias_flat_storage():
    params = [torch.nn.Parameter(torch.randn(3, 4)), torch.nn.Parameter(torch.randn(5))]
    b = dp.GradBucket(params)
    (params[0].sum() * 2 + params[1].sum() * 3).backward()
    assert torch.equal(b.flat, torch.cat([torch.full((12,), 2.0), torch.full((5,), 3.0)]))
    assert b.all_reduce() is None         # no process group: nothing to do
    b.zero()
    assert float(b.flat.abs().sum()) == 0 and params[0].grad.data_ptr() == b.flat.data_ptr()
