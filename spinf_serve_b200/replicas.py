"""Bulk scoring over several GPUs of one node: independent replicas over a content-partitioned queue. The reference is single-GPU by
design ("Several GPUs: one process each, behind your own load balancer", docs/configuration.md:26-27 in the spinf-serve tree);
contents never interact (a job attends only inside its own slot of the stream, spinf_serve/scorer.py:174), so the data path needs
no collective: rank r scores contents r, r + world, r + 2 world, ... with its own full copy of the weights, and the per-content
results are gathered on the host at the end."""

import torch.distributed as dist


def shard_items(items, rank: int, world: int):
    """the score_grouped items of this rank: a static partition by position in the queue (contents are independent, so any
    partition gives the same scores; striding keeps long and short contents evenly spread)"""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside a world of {world}")
    return items[rank::world]


def gather_results(local: dict, group=None, dst: int = 0):
    """{key: scores} of every rank -> the merged dict on rank `dst` (None elsewhere). Host objects over the process group: pass a
    gloo group when the default group is NCCL."""
    if not dist.is_available() or not dist.is_initialized():
        return dict(local)
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    parts = [None] * world if rank == dst else None
    dist.gather_object(local, parts, dst=dst, group=group)
    if rank != dst:
        return None
    merged = {}
    for part in parts:
        for key, val in part.items():
            if key in merged:
                raise ValueError(f"content {key!r} was scored by two replicas")
            merged[key] = val
    return merged


def score_sharded(scorer, items, group=None):
    """every rank scores its shard with its own scorer (Scorer.score_grouped); -> merged results on rank 0, None elsewhere"""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    return gather_results(scorer.score_grouped(shard_items(items, rank, world)), group)
