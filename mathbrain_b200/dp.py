"""Data-parallel plumbing of the hot path: one process per GPU, batch sharded, one gradient exchange per step.

Samples are independent on this path (no cross-sample operation), so ranks never exchange activations; the only
collective is the sum of the parameter gradients and of the vocabulary-sized slot-embedding gradient
(`torch.distributed` all-reduce; NCCL over NVLink on GPUs, gloo in the CPU tests).
"""
import torch
import torch.distributed as dist


def shard_bounds(n_items, rank, world):
    """Contiguous, balanced split of n_items over `world` ranks: [lo, hi) of `rank`."""
    base, rem = divmod(n_items, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def balanced_shards(costs, world):
    """Split items with the given costs into `world` shards of equal size (len(costs) must divide evenly) whose
    total costs are as even as a greedy longest-first packing makes them: items sorted by cost, each handed to the
    least-loaded shard that still has room.  Deterministic; returns a list of `world` sorted index lists.

    On this path a sample costs T_b * K_b (time steps times listed slots), and a step ends when the slowest rank
    does, so the maximum shard cost is what the packing minimises."""
    costs = [float(c) for c in costs]
    n = len(costs)
    if world < 1 or n % world != 0:
        raise ValueError("balanced_shards: %d items do not split evenly over %d ranks" % (n, world))
    per = n // world
    load = [0.0] * world
    out = [[] for _ in range(world)]
    for i in sorted(range(n), key=lambda j: (-costs[j], j)):
        r = min((r for r in range(world) if len(out[r]) < per), key=lambda r: (load[r], r))
        out[r].append(i)
        load[r] += costs[i]
    return [sorted(o) for o in out]


def slot_embedding_grad(dE_list, unique_tensor, vocab, out=None):
    """Scatter-add per-sample slot gradients [B, K, D] (one tensor per layer / per K,V) into a [vocab, D] fp32
    buffer: what the embedding table receives from the listed slots.  Entries of `unique_tensor` < 0 are skipped."""
    D = dE_list[0].shape[-1]
    if out is None:
        out = torch.zeros(vocab, D, dtype=torch.float32, device=dE_list[0].device)
    else:
        out.zero_()
    # every tensor scatters through the same index: sum them first (fp32), then one masked scatter-add
    acc = dE_list[0].to(torch.float32, copy=True)
    for g in dE_list[1:]:
        acc = acc.add_(g)
    acc.mul_((unique_tensor >= 0).unsqueeze(-1))
    out.index_add_(0, unique_tensor.clamp_min(0).reshape(-1), acc.reshape(-1, D))
    return out


class GradBucket:
    """The gradients of a group of parameters (one layer's, say) laid out in ONE flat fp32 buffer: every p.grad is a
    view into it, so autograd accumulates straight into the bucket and the exchange needs neither a flatten copy nor
    a copy back.  all_reduce_async() hands the bucket to the process group as soon as the group's backward has been
    enqueued (the collective runs on the backend's own stream, behind the work already queued on the current stream)
    and returns at once; wait() makes the current stream wait for it."""

    def __init__(self, params, group=None):
        self.params = [p for p in params if p.requires_grad]
        n = sum(p.numel() for p in self.params)
        dev = self.params[0].device if self.params else None
        self.flat = torch.zeros(n, dtype=torch.float32, device=dev)
        self.group = group
        self.handle = None
        off = 0
        for p in self.params:
            p.grad = self.flat[off:off + p.numel()].view_as(p)
            off += p.numel()

    def zero(self):
        self.flat.zero_()

    def all_reduce_async(self):
        self.handle = dist.all_reduce(self.flat, group=self.group, async_op=True)
        return self.handle

    def wait(self):
        if self.handle is not None:
            self.handle.wait()
            self.handle = None


def allreduce_gradients(params, extra=(), group=None):
    """Sum the .grad of `params` (flattened into one bucket) and every tensor in `extra` over all ranks, in place."""
    grads = [p.grad for p in params if p.grad is not None]
    if grads:
        flat = torch.cat([g.reshape(-1).float() for g in grads])
        dist.all_reduce(flat, group=group)
        off = 0
        for g in grads:
            n = g.numel()
            g.copy_(flat[off:off + n].view_as(g))
            off += n
    for t in extra:
        dist.all_reduce(t, group=group)
