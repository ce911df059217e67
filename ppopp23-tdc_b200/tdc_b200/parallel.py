"""Batch-sharded inference over the GPUs of one box.

The path shards along batch only: images are independent and the Tucker ranks are too small
to split.  The reference has no multi-GPU code for this path; its skeleton runs one image on
one GPU (A100-evaluation/EndToEnd/resnet18-tk/src/main.cu:127-155).  Here every rank (one
process per GPU, torch.distributed) holds a replica of the weights, runs the identical forward
on its contiguous slice of the batch, and ONE collective at the end gathers the results
(all_gather of equal, padded slices; NCCL over NVLink on GPUs, gloo in the CPU tests).  No
collective and no remote access happens inside the forward.

Failure.  A rank can only leave between steps (none of its kernels or collectives in flight).  The others notice
at their next gather: the collective raises — at once when the peer's connection is gone, after the process
group's timeout when the peer is merely silent — and `gather_slices` turns that into `ShardError`, so a driver loop
catches one exception type, drops the step and decides whether to re-form the group with the ranks that are left.
Nothing waits without a limit as long as the process group was created with a timeout.
"""
import torch


class ShardError(RuntimeError):
    """The gather of a sharded step did not complete: a peer rank is gone or silent.  The local slice of the step is
    in `.local` (it was computed before the collective), so the caller may still use or re-send it."""

    def __init__(self, msg, local=None):
        super().__init__(msg)
        self.local = local


def shard_bounds(batch, world, rank):
    """[start, stop) of `rank`'s contiguous slice; the first `batch % world` ranks get one more."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("rank %d of world %d" % (rank, world))
    base, extra = divmod(batch, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_sizes(batch, world):
    return [shard_bounds(batch, world, r)[1] - shard_bounds(batch, world, r)[0] for r in range(world)]


def forward_sharded(forward, images, group=None, gather=True):
    """Runs `forward` on this rank's slice of `images` (the full batch, the same tensor on every
    rank) and returns the gathered result for the whole batch on every rank, or only the local
    slice when gather=False."""
    import torch.distributed as dist
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    a, b = shard_bounds(images.shape[0], world, rank)
    if b > a:
        local = forward(images[a:b])
    elif images.shape[0] and gather and world > 1:
        # fewer images than ranks: this rank owns none; it runs one image only to learn the
        # result's shape and contributes zero rows to the gather
        local = forward(images[:1])[:0]
    else:
        local = None
    if not gather or world == 1:
        return local
    return gather_slices(local, images.shape[0], group)


def gather_slices(local, batch, group=None, like=None):
    """all_gather of per-rank slices of unequal length: each rank pads its slice to the longest,
    one collective moves them, the padding is cut off and the slices are concatenated in rank
    order.  `like` gives dtype/device/trailing shape for a rank whose slice is empty."""
    import torch.distributed as dist
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    sizes = shard_sizes(batch, world)
    longest = max(sizes)
    ref = local if local is not None else like
    if ref is None:
        raise ValueError("a rank with an empty slice needs `like` to know the result's shape")
    pad = ref.new_zeros((longest,) + tuple(ref.shape[1:]))
    if local is not None and local.shape[0]:
        pad[: local.shape[0]] = local
    out = [torch.empty_like(pad) for _ in range(world)]
    try:
        dist.all_gather(out, pad, group=group)
    except (RuntimeError, dist.DistBackendError) as e:       # peer gone (connection closed) or silent (group timeout)
        raise ShardError("rank %d of %d: the gather of this step failed: %s" % (rank, world, str(e).splitlines()[0]), local) from e
    return torch.cat([o[:n] for o, n in zip(out, sizes)], dim=0)
