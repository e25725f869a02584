"""Data parallelism for the parameter gradients: the batch is split over ranks, parameters are
replicated, and the gradients of every template, weight and offsets tensor live in ONE flat float32
bucket that a single all-reduce sums over the ranks.

The reference has no distributed code at all; what it does have is the batch loop that sums parameter
gradients over samples (src/kernels/similarity_grad_kernel_cpu.cpp:84-144,
src/kernels/mex_grad_kernel_cpu.cpp:298-368).  Summing shard results over ranks continues that sum.
"""
import torch
import torch.distributed as dist


class GradBucket(object):
    """Flat gradient storage: each parameter's `.grad` is a view into `flat`, so autograd accumulates
    straight into the bucket and nothing is packed or copied before the collective."""

    def __init__(self, parameters):
        self.params = [p for p in parameters if p.requires_grad]
        if not self.params:
            raise ValueError("no trainable parameters")
        dev, dtype = self.params[0].device, self.params[0].dtype
        total = sum(p.numel() for p in self.params)
        self.flat = torch.zeros(total, dtype=dtype, device=dev)
        off = 0
        self.views = []
        for p in self.params:
            v = self.flat[off:off + p.numel()].view_as(p)
            p.grad = v
            self.views.append(v)
            off += p.numel()

    def zero(self):
        self.flat.zero_()
        for p, v in zip(self.params, self.views):   # re-attach in case an optimizer dropped .grad
            if p.grad is not v:
                p.grad = v

    def all_reduce(self, group=None, async_op=False):
        """Sum the bucket over all ranks (no-op without an initialised process group of size > 1)."""
        if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
            return None
        return dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=group, async_op=async_op)

    def nbytes(self):
        return self.flat.numel() * self.flat.element_size()


def shard_bounds(global_batch, world_size, rank):
    """[begin, end) of this rank's contiguous slice of the batch; sizes differ by at most one."""
    base, extra = divmod(int(global_batch), int(world_size))
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)
