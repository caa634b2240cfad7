"""Row sharding across the GPUs of one node, with real samplers: the id exchanges (NCCL
all-gather; ids stored into the peers' buffers by the kernel epilogue, synchronised by a
barrier behind the launch or by arrival marks inside it) must leave every
rank with the tokens a single GPU would produce. Runs only where at least two GPUs are
visible; ranks leave together, between steps."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import oracle
        from executorch_b200 import Sampler, seeds_to_states
        from executorch_b200 import workloads as W
        from executorch_b200.sharded import ShardedSampler

        vocab, total = 20000, 16 * world
        x = W.rows_numpy("c3", list(range(total)), vocab=vocab)
        seeds = np.arange(total, dtype=np.uint64) + 3
        want = oracle.Restatement().sample_rows(x, 0.7, 0.9, seeds, dtype="bf16", threads=2)
        s = Sampler(vocab, 0.7, 0.9, 0, device=dev)
        ok = True
        for mode in ("nccl", "p2p", "p2p-in-kernel"):
            scatter = {"nccl": None, "p2p": s.sample_rows_scatter, "p2p-in-kernel": s.sample_rows_exchange}[mode]
            sh = ShardedSampler(s.sample_rows, total, scatter=scatter, device=dev,
                                in_kernel_sync=mode == "p2p-in-kernel")
            lo, n = sh.start, sh.count
            t = torch.from_numpy(x[lo:lo + n].view(np.int16)).to(dev).view(torch.bfloat16)
            kept = []
            for k in range(4):
                # every step draws from other seeds, so a buffer that a faster rank overwrote
                # with its next step's ids would hold wrong tokens
                sk = seeds + np.uint64(1000 * k)
                wk = want if k == 0 else oracle.Restatement().sample_rows(x, 0.7, 0.9, sk, dtype="bf16", threads=2)
                ids = sh.sample_rows(t, seeds_to_states(sk[lo:lo + n], dev))
                if rank == world - 1 and mode != "nccl":
                    torch.cuda._sleep(20_000_000)  # a slow consumer: this rank reads its ids late
                kept.append((ids, wk))
                if mode != "nccl" and len(kept) == 2:
                    # the previous step's ids are still intact while the next step is in flight
                    # (the exchange rotates over three regions)
                    torch.cuda.synchronize()
                    ok = ok and np.array_equal(kept[0][0].cpu().numpy(), kept[0][1])
                    kept.pop(0)
                torch.cuda.synchronize()
                ok = ok and np.array_equal(ids.cpu().numpy(), wk)
            dist.barrier()
        ok = ok and s.status == 0  # no arrival wait ran out
        s.close()
        q.put((rank, ok))
    finally:
        dist.barrier()
        dist.destroy_process_group()


def test_sharded_sampling_matches_single_gpu_tokens():
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + os.getpid() % 300
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert all(ok for _, ok in results), results
