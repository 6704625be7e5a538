"""Sharding of independent sample streams over the ranks of one node.

Sample streams are independent given the context, so the sampling / log-density
path shards by streams with no collective inside the decode loop: every rank
prefills the (replicated) context locally, decodes its own slice of streams and
the per-stream results are gathered once at the end (NCCL on GPUs; the same code
runs over gloo on CPU tensors for testing).  The reference has no multi-GPU
code; this module is new functionality around the unchanged predictor API.
"""
from __future__ import annotations

from typing import Callable, Sequence, Tuple

import torch
import torch.distributed as dist


def shard_bounds(n_streams: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, even split; the first ``n_streams % world`` ranks hold one extra stream."""
    base, extra = divmod(n_streams, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def gather_streams(local: torch.Tensor, n_streams: int, group=None) -> torch.Tensor:
    """All-gather per-stream rows ``[n_local, ...]`` into ``[n_streams, ...]`` on every rank."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return local
    world = dist.get_world_size(group)
    sizes = [shard_bounds(n_streams, world, r) for r in range(world)]
    if n_streams % world == 0:
        out = local.new_empty((n_streams,) + tuple(local.shape[1:]))
        dist.all_gather_into_tensor(out, local.contiguous(), group=group)
        return out
    # uneven split: pad every shard to the largest one, gather, drop the padding
    most = max(hi - lo for lo, hi in sizes)
    padded = local.new_zeros((most,) + tuple(local.shape[1:]))
    padded[: local.shape[0]] = local
    out = local.new_empty((world * most,) + tuple(local.shape[1:]))
    dist.all_gather_into_tensor(out, padded, group=group)
    out = out.view((world, most) + tuple(local.shape[1:]))
    return torch.cat([out[r, : hi - lo] for r, (lo, hi) in enumerate(sizes)], dim=0)


def sharded_call(fn: Callable[..., Sequence[torch.Tensor]], stream_args: Sequence[torch.Tensor],
                 variates: Sequence[torch.Tensor] = (), group=None):
    """Run ``fn(*stream_args_shard, *variate_shards)`` on this rank's streams and gather.

    ``stream_args`` are full-job tensors with the stream axis first; ``variates`` have the
    stream axis SECOND (``[Nt, B, ...]``, the order random numbers are consumed in) and are
    drawn for the full job on every rank, so the result does not depend on the world size.
    ``fn`` returns per-stream tensors (stream axis first); the gathered tensors are returned.
    """
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    n = stream_args[0].shape[0]
    lo, hi = shard_bounds(n, world, rank)
    outs = fn(*[a[lo:hi] for a in stream_args], *[v[:, lo:hi] for v in variates])
    return tuple(gather_streams(o, n, group) for o in outs)
