"""Bulk scoring over several GPUs of one node: independent replicas over a content-partitioned queue. The reference is single-GPU by
design ("Several GPUs: one process each, behind your own load balancer", docs/configuration.md:26-27 in the spinf-serve tree);
contents never interact (a job attends only inside its own slot of the stream, spinf_serve/scorer.py:174), so the data path needs
no collective: every rank holds its own full copy of the weights and scores the contents it draws from a shared host-side queue
(ContentQueue; a static stride, shard_items, is kept for callers without a store), and the per-content results are gathered on
the host at the end."""

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


# ------------------------------------------------------------------------------------------------ the shared queue
class ContentQueue:
    """A queue of content chunks shared by the replicas of one node: chunk c = items[c * chunk : (c + 1) * chunk], and the next
    chunk to hand out is a counter in the process group's key-value store (a host-side TCP store; `add` is atomic). A replica
    asks for the next chunk whenever its packer wants more work, so a GPU that drew short contents simply comes back sooner:
    the partition follows the work, not a fixed stride. Nothing of this touches the GPUs or NCCL.

    store None: a process-local counter (one replica)."""

    def __init__(self, n_items: int, chunk: int, store=None, name: str = "spinf/queue"):
        if chunk < 1:
            raise ValueError("chunk must be at least 1")
        self.n_chunks = -(-n_items // chunk)
        self.n_items, self.chunk, self.store, self.name = n_items, chunk, store, name
        self.taken = []      # chunk ids this replica drew
        self._local = 0

    def _draw(self) -> int:
        if self.store is None:
            self._local += 1
            return self._local - 1
        return int(self.store.add(self.name, 1)) - 1

    def __iter__(self):
        while True:
            c = self._draw()
            if c >= self.n_chunks:
                return
            self.taken.append(c)
            yield c

    def items(self, items):
        """the score_grouped items of the chunks this replica draws, in drawing order (a generator: the scorer's packing thread
        pulls from it as it packs)"""
        for c in self:
            yield from items[c * self.chunk : (c + 1) * self.chunk]


def group_store():
    """the key-value store of the default process group (None without one)"""
    if not dist.is_available() or not dist.is_initialized():
        return None
    from torch.distributed import distributed_c10d

    return distributed_c10d._get_default_store()


def score_queued(scorer, items, chunk: int = 16, group=None, name: str = "spinf/queue", store=None):
    """every rank scores the chunks it draws from the shared queue with its own scorer -> (merged results on rank 0, None
    elsewhere; the ContentQueue, whose `taken` says what this rank drew). `name` must be new for every call on a store."""
    queue = ContentQueue(len(items), chunk, store if store is not None else group_store(), name)
    local = scorer.score_grouped(queue.items(items))
    return gather_results(local, group), queue
