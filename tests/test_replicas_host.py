"""The multi-GPU path is replicas over a content-partitioned queue with no collective on the data path; its host logic (sharding,
gathering per-content results) runs here as 2 gloo ranks on CPU with a stand-in scorer."""

import os

import numpy as np
import torch.distributed as dist
import torch.multiprocessing as mp

from spinf_serve_b200 import replicas


class FakeScorer:
    """scores depend on the content key only, as the real scorer's do (batch invariance)"""

    def score_grouped(self, items):
        return {key: [np.full(3, float(sum(key)) + i) for i in range(n)] for key, first, n in items}


def _items(n):
    return [((c, 7 * c), 0, 1 + c % 3) for c in range(n)]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        merged = replicas.score_sharded(FakeScorer(), _items(11))
        if rank == 0:
            out.put({k: [a.tolist() for a in v] for k, v in merged.items()})
        else:
            assert merged is None
    finally:
        dist.destroy_process_group()


def test_two_replicas_cover_the_queue_without_overlap():
    items = _items(11)
    shards = [replicas.shard_items(items, r, 2) for r in range(2)]
    assert sorted(shards[0] + shards[1]) == sorted(items) and not set(shards[0]) & set(shards[1])
    assert abs(len(shards[0]) - len(shards[1])) <= 1


def test_two_gloo_ranks_merge_to_the_single_process_result():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    merged = out.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    want = FakeScorer().score_grouped(_items(11))
    assert merged == {k: [a.tolist() for a in v] for k, v in want.items()}


def test_single_process_path_needs_no_process_group():
    assert replicas.score_sharded(FakeScorer(), _items(4)).keys() == FakeScorer().score_grouped(_items(4)).keys()


def _queue_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        merged, queue = replicas.score_queued(FakeScorer(), _items(53), chunk=4, name="spinf/test/q1")
        taken = [None] * world
        dist.all_gather_object(taken, queue.taken)
        if rank == 0:
            out.put(({k: [a.tolist() for a in v] for k, v in merged.items()}, taken))
        else:
            assert merged is None
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_draw_disjoint_chunks_from_the_shared_queue():
    """53 contents in chunks of 4 = 14 chunks: the two ranks' draws are disjoint and cover them all, and the merged result is the
    single-process result"""
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 31500 + os.getpid() % 2000
    procs = [ctx.Process(target=_queue_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    merged, taken = out.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(taken[0] + taken[1]) == list(range(14)) and not set(taken[0]) & set(taken[1])
    want = FakeScorer().score_grouped(_items(53))
    assert merged == {k: [a.tolist() for a in v] for k, v in want.items()}


def test_queue_without_a_store_hands_every_chunk_to_the_one_replica():
    q = replicas.ContentQueue(10, 3)
    items = _items(10)
    assert list(q.items(items)) == items and q.taken == [0, 1, 2, 3]
    merged, q2 = replicas.score_queued(FakeScorer(), items, chunk=3)
    assert merged.keys() == FakeScorer().score_grouped(items).keys() and q2.taken == [0, 1, 2, 3]
