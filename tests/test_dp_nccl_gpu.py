"""On real GPUs: (1) a step split in two pieces around the cut of dp.OverlappedStep (with and without CUDA graphs)
gives the gradients of the plain forward + backward; (2) with at least two GPUs, gradients of batch shards summed by
an NCCL all-reduce equal the gradients of the whole batch computed on one GPU.  The second test continues, across
ranks, the batch loops in which the reference sums parameter gradients (src/kernels/mex_grad_kernel_cpu.cpp:298-368,
similarity_grad_kernel_cpu.cpp:84-144); it skips on a single GPU."""
import os
import socket

import numpy as np
import pytest
import torch

from simnets_tf_b200 import dp
from simnets_tf_b200.simnet import SPECS, SimNet

pytestmark = pytest.mark.gpu


def _data(spec, n, seed=21):
    rng = np.random.default_rng(seed)
    x = rng.uniform(-0.5, 0.5, size=(n,) + tuple(spec["input_shape"])).astype(np.float32)
    return x, rng.integers(0, spec["classes"], size=n).astype(np.int64)


@pytest.mark.parametrize("graphs", [False, True])
def test_overlapped_step_equals_plain_backward(graphs):
    spec = SPECS["cfg5"]
    x, labels = _data(spec, 8)
    xd, ld = torch.from_numpy(x).cuda(), torch.from_numpy(labels).cuda()
    net = SimNet(spec, seed=4, device="cuda")
    bucket = dp.GradBucket(net.parameters())
    bucket.zero()
    loss = net.loss(xd, ld, 8)
    loss.backward()
    want, want_loss = bucket.flat.clone(), float(loss.detach())
    del loss                                 # (an autograd graph of the default stream kept alive would break the capture)
    step = dp.OverlappedStep(net, bucket, xd, ld, 8, graphs=graphs)
    assert 0 < step.cut < len(net._plan) and 0 < step.tail_begin < bucket.flat.numel()
    for _ in range(2):                       # a replay must not accumulate into the previous one
        got_loss = float(step.run().detach())
        torch.cuda.synchronize()
        assert abs(got_loss - want_loss) <= 1e-6 * max(1.0, abs(want_loss))
        scale = float(want.abs().max())
        assert float((bucket.flat - want).abs().max()) <= 1e-6 * scale


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank(rank, world, port, out):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        spec = SPECS["cfg5"]
        n = 16
        x, labels = _data(spec, n)
        xd, ld = torch.from_numpy(x).to(dev), torch.from_numpy(labels).to(dev)
        net = SimNet(spec, seed=4, device=dev)
        bucket = dp.GradBucket(net.parameters())
        lo, hi = dp.shard_bounds(n, world, rank)
        step = dp.OverlappedStep(net, bucket, xd[lo:hi].contiguous(), ld[lo:hi].contiguous(), n, graphs=False)
        step.run()                                                   # shard gradients, two overlapped all-reduces
        torch.cuda.synchronize()
        summed = bucket.flat.clone()
        if rank == 0:
            bucket.zero()
            net.loss(xd, ld, n).backward()
            worst, off = 0.0, 0
            for p in bucket.params:
                a, b = summed[off:off + p.numel()], bucket.flat[off:off + p.numel()]
                worst = max(worst, float((a - b).abs().max() / b.abs().max().clamp_min(1e-30)))
                off += p.numel()
            np.save(out, np.array([worst]))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_nccl_summed_shard_gradients_equal_one_gpu_gradients(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    import torch.multiprocessing as mp
    out = str(tmp_path / "err.npy")
    mp.spawn(_rank, args=(2, _free_port(), out), nprocs=2, join=True)
    assert float(np.load(out)[0]) <= 1e-4
