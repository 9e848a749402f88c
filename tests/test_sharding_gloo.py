"""Batch sharding + logits gather on two CPU ranks (gloo): the host logic of the multi-GPU path."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import __graft_entry__ as entry


def test_shard_bounds_cover_the_batch(pkg):
    sb = pkg.sharding.shard_bounds
    for B in (0, 1, 7, 64, 1024, 1025):
        for W in (1, 2, 3, 8):
            spans = [sb(B, W, r) for r in range(W)]
            assert spans[0][0] == 0 and spans[-1][1] == B
            assert all(spans[i][1] == spans[i + 1][0] for i in range(W - 1))
            sizes = [e - s for s, e in spans]
            assert max(sizes) - min(sizes) <= 1
    assert sb(1024, 8, 3) == (384, 512)
    with pytest.raises(ValueError):
        sb(8, 2, 2)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, B: int, fail_rank: int, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    pkg = entry.import_package()
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        s, e = pkg.sharding.shard_bounds(B, world, rank)
        # "logits" of image i are [i, i+0.5, ...] so order and ownership are visible after the gather
        local = torch.arange(s, e, dtype=torch.float32)[:, None] + torch.tensor([0.0, 0.5, 0.25])
        if rank == fail_rank:
            local = local[:-1]          # a rank that lost a row must be caught before the collective
            try:
                pkg.sharding.gather_logits(local, B)
                q.put((rank, "no error"))
            except ValueError as err:
                q.put((rank, "ValueError"))
            return
        if fail_rank >= 0:
            q.put((rank, "skipped"))
            return
        full = pkg.sharding.gather_logits(local, B)
        want = torch.arange(B, dtype=torch.float32)[:, None] + torch.tensor([0.0, 0.5, 0.25])
        q.put((rank, bool(torch.equal(full, want))))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("B", [8, 7, 1])
def test_gather_logits_two_ranks(B):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, B, -1, q)) for r in range(2)]
    [p.start() for p in procs]
    res = dict(q.get(timeout=120) for _ in procs)
    [p.join(timeout=60) for p in procs]
    assert res == {0: True, 1: True}


def test_wrong_shard_size_is_rejected_on_the_host():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, 8, 1, q)) for r in range(2)]
    [p.start() for p in procs]
    res = dict(q.get(timeout=120) for _ in procs)
    [p.join(timeout=60) for p in procs]
    assert res == {0: "skipped", 1: "ValueError"}


def _gatherer_worker(rank: int, world: int, port: int, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    pkg = entry.import_package()
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, C = 8, 5
        g = pkg.sharding.LogitsGatherer(B, C, torch.float32, torch.device("cpu"))
        ok = True
        for step in range(3):                      # both staging rows and both result buffers get reused
            s, e = pkg.sharding.shard_bounds(B, world, rank)
            local = (torch.arange(s, e, dtype=torch.float32)[:, None] + 0.125 * torch.arange(C)) * (step + 1)
            g.submit(local)
            want = (torch.arange(B, dtype=torch.float32)[:, None] + 0.125 * torch.arange(C)) * (step + 1)
            ok = ok and bool(torch.equal(g.result(), want))
        try:
            g.submit(torch.zeros(3, C))            # a rank that arrives with the wrong shard fails on the host
            ok = False
        except ValueError:
            pass
        q.put((rank, ok))
    finally:
        dist.destroy_process_group()


def test_logits_gatherer_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gatherer_worker, args=(r, 2, port, q)) for r in range(2)]
    [p.start() for p in procs]
    res = dict(q.get(timeout=120) for _ in procs)
    [p.join(timeout=60) for p in procs]
    assert res == {0: True, 1: True}


def test_logits_gatherer_refuses_uneven_shards(pkg):
    with pytest.raises(RuntimeError):
        pkg.sharding.LogitsGatherer(8, 5, torch.float32, torch.device("cpu")).result()
