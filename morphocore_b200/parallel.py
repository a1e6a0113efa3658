"""Data parallelism over the batch for training with the morphological layers.

Images are independent in the forward pass and in grad_input; only the parameter gradients (structuring
elements and alphas) are sums over the batch. Each rank (one process per GPU) runs the layers on its
contiguous slice of the global batch, and the parameter gradients, which autograd accumulates directly
into views of ONE flat buffer, are summed across ranks with a single all-reduce per step (NCCL over
NVLink on GPUs, gloo on CPU in the tests) and divided by the world size. The reference has no
multi-GPU code; this is the only collective the path needs.
"""
import torch
import torch.distributed as dist


def shard_range(global_batch: int, rank: int, world_size: int):
    """(start, count) of the contiguous slice of the batch owned by `rank`; the first
    global_batch % world_size ranks take one extra element."""
    if world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError(f"invalid rank {rank} for world size {world_size}")
    base, extra = divmod(global_batch, world_size)
    start = rank * base + min(rank, extra)
    return start, base + (1 if rank < extra else 0)


class GradBucket:
    """Flat gradient buffer shared by a list of parameters.

    Every parameter's .grad is a view into `flat`, so the backward kernels' results land in the buffer
    without a gather, `zero()` is one memset and `all_reduce()` is one collective.
    """

    def __init__(self, params, process_group=None):
        self.params = [p for p in params if p.requires_grad]
        if not self.params:
            raise ValueError("no trainable parameters")
        first = self.params[0]
        for p in self.params:
            if p.dtype != first.dtype or p.device != first.device:
                raise ValueError("all parameters of a bucket must share dtype and device")
        self.group = process_group
        self.flat = torch.zeros(sum(p.numel() for p in self.params), dtype=first.dtype, device=first.device)
        offset = 0
        for p in self.params:
            p.grad = self.flat[offset:offset + p.numel()].view_as(p)
            offset += p.numel()

    def zero(self):
        self.flat.zero_()

    def check_views(self):
        """Every parameter's .grad must still be its view into the flat buffer. optimizer.zero_grad() with
        torch's default set_to_none=True (or any code that rebinds p.grad) breaks the alias: the all-reduce would
        then sum a stale buffer while the optimizer steps on gradients no rank has shared."""
        offset = 0
        for n, p in enumerate(self.params):
            want = self.flat.data_ptr() + offset * self.flat.element_size()
            if p.grad is None or p.grad.data_ptr() != want or p.grad.numel() != p.numel():
                raise RuntimeError(
                    f"GradBucket: the gradient of parameter {n} is no longer a view of the flat buffer "
                    "(optimizer.zero_grad(set_to_none=True) or a rebound .grad); clear gradients with bucket.zero() "
                    "or zero_grad(set_to_none=False)")
            offset += p.numel()

    def world_size(self):
        return dist.get_world_size(self.group) if dist.is_available() and dist.is_initialized() else 1

    def all_reduce(self, average: bool = True):
        """Sum the buffer over the ranks (mean with `average`). Every rank must call it with a buffer of
        the same length; a mismatch is reported on the host before any collective runs."""
        self.check_views()
        world = self.world_size()
        if world == 1:
            return
        sizes = [None] * world
        if not getattr(self, "_checked", False):
            dist.all_gather_object(sizes, self.flat.numel(), group=self.group)
            if len(set(sizes)) != 1:
                raise RuntimeError(f"gradient buckets differ across ranks: {sizes}")
            self._checked = True
        dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=self.group)
        if average:
            self.flat.div_(world)
