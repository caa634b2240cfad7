"""Row sharding and the id all-gather, on CPU with the gloo backend (world size 2 and 3).
The sampled ids come from a CPU stand-in so that only the exchange logic is under test."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from executorch_b200.sharded import ShardedSampler, shard_rows


def test_shard_rows_partitions_exactly():
    for rows in (0, 1, 7, 256, 32768, 1000):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_rows(rows, r, world) for r in range(world)]
            assert spans[0][0] == 0
            for (s0, c0), (s1, _) in zip(spans, spans[1:]):
                assert s0 + c0 == s1
            assert spans[-1][0] + spans[-1][1] == rows
            counts = [c for _, c in spans]
            assert max(counts) - min(counts) <= 1
    assert shard_rows(32768, 3, 8) == (12288, 4096)
    with pytest.raises(ValueError):
        shard_rows(10, 2, 2)


def _fake_local_sample(logits, states):
    # deterministic function of the row contents and the row's state: stands in for the kernel
    return (logits.to(torch.float64).sum(dim=1).to(torch.int64) * 31 + states) % 1000


def _worker(rank, world, port, total_rows, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(123)
        logits = torch.randint(0, 50, (total_rows, 16), generator=g).to(torch.float32)
        states = torch.arange(total_rows, dtype=torch.int64)
        sh = ShardedSampler(_fake_local_sample, total_rows)
        s, c = sh.start, sh.count
        out = sh.sample_rows(logits[s:s + c], states[s:s + c])
        want = _fake_local_sample(logits, states)
        q.put((rank, bool(torch.equal(out, want)), (s, c)))
        with pytest.raises(ValueError):
            sh.sample_rows(logits[: c + 1], states[: c + 1])
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,total_rows", [(2, 64), (2, 7), (3, 10)])
def test_all_ranks_end_with_all_ids(world, total_rows):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29000 + (os.getpid() % 500) + world * 7 + total_rows
    procs = [ctx.Process(target=_worker, args=(r, world, port, total_rows, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok, _ in results)
    spans = sorted(sp for _, _, sp in results)
    assert spans[0][0] == 0 and spans[-1][0] + spans[-1][1] == total_rows


def _late_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import time
    from executorch_b200.sharded import ExchangeTimeout
    total_rows = 8
    logits = torch.zeros((total_rows, 4))
    states = torch.arange(total_rows, dtype=torch.int64)
    if rank == 0:
        sh = ShardedSampler(_fake_local_sample, total_rows, deadline_s=1.5)
        t0 = time.time()
        try:
            sh.sample_rows(logits[sh.start:sh.start + sh.count], states[sh.start:sh.start + sh.count])
            q.put((rank, "returned", time.time() - t0))
        except ExchangeTimeout:
            q.put((rank, "timeout", time.time() - t0))
    else:
        # this rank never joins the exchange: it fails on the host, between steps
        time.sleep(4.0)
        q.put((rank, "absent", 0.0))
    # the process group is not usable after an abandoned collective: leave without the
    # collective teardown (once the result is on its way)
    q.close()
    q.join_thread()
    os._exit(0)


def test_a_rank_that_never_arrives_ends_the_exchange_with_an_error():
    """Failure detection on the host: rank 1 never calls the exchange; rank 0's deadline turns
    the wait into ExchangeTimeout instead of blocking."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29000 + (os.getpid() % 500) + 431
    procs = [ctx.Process(target=_late_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict((r, (what, dt)) for r, what, dt in (q.get(timeout=120) for _ in range(2)))
    for p in procs:
        p.join(timeout=60)
    assert results[0][0] == "timeout", results
    assert 1.0 <= results[0][1] < 4.0, results
    assert results[1][0] == "absent"
