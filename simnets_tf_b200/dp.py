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
            # the layer classes pass this on to the library, whose parameter-gradient kernels then add into the bucket
            # themselves (SIMNETS_FLAG_ACCUMULATE) instead of handing a tensor to autograd's accumulation
            p._simnets_grad_sink = v
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

    def offset_of(self, param):
        """Element offset of a parameter's gradient inside `flat`."""
        off = 0
        for p in self.params:
            if p is param:
                return off
            off += p.numel()
        raise KeyError("parameter is not in the bucket")

    def all_reduce_range(self, begin, end, group=None):
        """Sum flat[begin:end] over all ranks on the current stream (no-op without a process group of size > 1)."""
        if end <= begin or not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
            return None
        return dist.all_reduce(self.flat[begin:end], op=dist.ReduceOp.SUM, group=group)


class OverlappedStep(object):
    """One data-parallel forward + backward step whose gradient all-reduce overlaps the backward pass.

    The network is cut at `net.split_point()`: piece A = forward of everything, loss, backward of the layers behind the
    cut (their parameter gradients, the tail of the bucket, are then final); piece B = backward of the layers in front.
    Per step: A on the main stream; the tail's all-reduce on a second stream as soon as A is done; B on the main
    stream meanwhile; the head's all-reduce behind B; join.  With `graphs=True` A and B are two CUDA graphs captured
    once and replayed; the collectives are always enqueued eagerly, outside any capture (capture needs that no autograd
    graph built on another stream is still alive, e.g. through a loss tensor kept from an earlier step).  The reference has no
    distributed code; the sums continued here are its batch loops (src/kernels/mex_grad_kernel_cpu.cpp:298-368,
    similarity_grad_kernel_cpu.cpp:84-144)."""

    def __init__(self, net, bucket, x, labels, global_batch, graphs=True):
        import torch
        self.torch, self.net, self.bucket, self.x, self.labels, self.gb = torch, net, bucket, x, labels, global_batch
        self.cut = net.split_point()
        tail = net.parameters_from(self.cut) if self.cut > 0 else []
        self.tail_begin = bucket.offset_of(tail[0]) if tail else bucket.flat.numel()
        self.side = torch.cuda.Stream(device=x.device)
        self.done_a = torch.cuda.Event()
        self.graph_a = self.graph_b = None
        self.loss = None
        self._mid = self._mid_leaf = None
        if graphs:
            self._capture()

    # -- the two pieces, eager
    def _piece_a(self):
        net = self.net
        self.bucket.zero()
        end = len(net._plan)
        if self.cut > 0:
            self._mid = net.forward_range(self.x, 0, self.cut)
            self._mid_leaf = self._mid.detach().requires_grad_(True)
            logits = net.forward_range(self._mid_leaf, self.cut, end)
        else:
            logits = net.forward_range(self.x, 0, end)
        self.loss = net.loss_of_logits(logits, self.labels, self.gb)
        self.loss.backward()

    def _piece_b(self):
        if self.cut > 0:
            self._mid.backward(self._mid_leaf.grad)

    def _capture(self):
        torch = self.torch
        cap = torch.cuda.Stream(device=self.x.device)
        cap.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(cap):                 # warm-up on the capture stream, as graph capture requires
            for _ in range(2):
                self._piece_a()
                self._piece_b()
        torch.cuda.current_stream().wait_stream(cap)
        torch.cuda.synchronize()
        self.graph_a, self.graph_b = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph_a, stream=cap):
            self._piece_a()
        with torch.cuda.graph(self.graph_b, pool=self.graph_a.pool(), stream=cap):
            self._piece_b()
        torch.cuda.synchronize()

    def compute(self):
        """Both pieces without any collective (device-time measurements of the compute alone)."""
        if self.graph_a is not None:
            self.graph_a.replay()
            self.graph_b.replay()
        else:
            self._piece_a()
            self._piece_b()
        return self.loss

    def run(self):
        torch, main = self.torch, self.torch.cuda.current_stream()
        n = self.bucket.flat.numel()
        if self.graph_a is not None:
            self.graph_a.replay()
        else:
            self._piece_a()
        self.done_a.record(main)
        with torch.cuda.stream(self.side):
            self.side.wait_event(self.done_a)
            self.bucket.all_reduce_range(self.tail_begin, n)
        if self.graph_b is not None:
            self.graph_b.replay()
        else:
            self._piece_b()
        self.bucket.all_reduce_range(0, self.tail_begin)
        main.wait_stream(self.side)
        return self.loss


def shard_bounds(global_batch, world_size, rank):
    """[begin, end) of this rank's contiguous slice of the batch; sizes differ by at most one."""
    base, extra = divmod(int(global_batch), int(world_size))
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)
