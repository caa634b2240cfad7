#!/usr/bin/env python
"""Benchmark of the token-sampling hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one pass of the sampler over one batch: configuration 3 of the baseline (256
rows x V=128256 bf16 Zipf-shaped logits, temperature 0.7, top-p 0.95, per-row xorshift seed
= row id) per GPU. With N > 1 (one process per GPU under torchrun) every rank samples its own
256 rows and the int64 ids are all-gathered (weak scaling). Prints ONE JSON line on rank 0.

  value      rows/s with the logits resident in HBM (device-timed, max over ranks)
  e2e        rows/s through the host-buffer entry of the C ABI: pinned host logits copied to
             the device, sampled, ids copied back, inside the timed region
  roofline   logits bytes read per launch / mean kernel time, against the measured HBM copy
             bandwidth of this pool (MEASURED_PEAKS.json) or the stated fallback
  cpu_baseline  the reference's own CPU sampler (compiled unmodified in oracle/_ref; the C
             restatement if that is absent) on this machine's host cores, N = 1 only
  parity     after the timed region one more step is run from known RNG states and its ids are
             compared with the CPU oracle (64 rows) and, for N > 1, with an all-gather of every
             rank's own ids: a mismatch makes the run fail
  other_configs  short device-timed runs of the other baseline shapes and modes (N = 1 only)

--impl reference times the reference's CPU sampler alone on the same batch.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "sampled_rows_per_s_topp_v128256_bf16"
WORKLOAD = "c3"
NBUF = 4  # rotating input buffers: 4 x 65.7 MB > 126 MB of L2
FALLBACK_HBM_GBS = 6650.0

PARITY_ROWS = 64
KERNEL_SOURCES = ["executorch_b200/csrc/sampler_kernels.cu", "executorch_b200/csrc/guided_sum.cuh",
                  "executorch_b200/csrc/cluster_topp.cuh", "executorch_b200/csrc/cluster_math.cuh",
                  "executorch_b200/csrc/exact_math.cuh", "executorch_b200/csrc/class_math.cuh",
                  "executorch_b200/csrc/value_class_tail.cuh"]


def kernel_source_hash():
    """Hash of the kernel sources (git blob hashes, concatenated and hashed again)."""
    import hashlib
    h = hashlib.sha1()
    for rel in KERNEL_SOURCES:
        with open(os.path.join(ROOT, rel), "rb") as f:
            data = f.read()
        h.update(hashlib.sha1(b"blob %d\0" % len(data) + data).hexdigest().encode())
    return h.hexdigest()


def dram_traffic(kernel: str):
    """DRAM bytes (read + write) of one launch of `kernel` on the benchmark batch, from the ncu
    capture recorded in profiles/traffic.json, and whether the kernel sources have changed since."""
    try:
        with open(os.path.join(ROOT, "profiles", "traffic.json")) as f:
            t = json.load(f)
        entry = t["kernels"][kernel]
        return int(entry["dram_bytes_per_launch"]), t.get("source_hash") != kernel_source_hash()
    except Exception:
        return None, True


def config_dict(gpus: int, greedy: bool, exchange: str, workload: str = WORKLOAD):
    """The `config` object; the same for both arms of the benchmark."""
    from executorch_b200 import workloads as W
    cfg = W.CONFIGS[workload]
    if workload == "c5":
        # strong scaling: the configuration's 32 768 rows are divided among the GPUs
        per = cfg.rows // gpus
        return {
            "workload": f"c5: {cfg.rows} rows x V={cfg.vocab} bf16 Zipf logits in all, T={cfg.temperature}, "
                        f"top-p {cfg.topp}, seed=row; rows divided evenly among the GPUs",
            "rows_per_gpu": per, "vocab": cfg.vocab, "global_rows": per * gpus,
            "l2": f"one input batch per GPU ({per * cfg.vocab * 2 / 1e9:.1f} GB > 126 MB L2)",
            "exchange": "none (ids stay on the GPU that sampled them)",
        }
    names = {"p2p": "ids stored into every peer's buffer by the kernel epilogue + symmetric-memory barrier on a "
                    "side stream",
             "p2p-in-kernel": "ids stored into every peer's buffer by the kernel epilogue + arrival marks and a "
                              "bounded wait at the end of the same launch",
             "nccl": "all_gather of int64 ids (NCCL)"}
    return {
        "workload": ("c3 second pass: 256 rows x V=128256 bf16 Zipf logits per GPU, T=0 (argmax)" if greedy
                     else "c3: 256 rows x V=128256 bf16 Zipf logits per GPU, T=0.7, top-p 0.95, seed=row"),
        "rows_per_gpu": cfg.rows, "vocab": cfg.vocab, "global_rows": cfg.rows * gpus,
        "l2": f"{NBUF} rotating input batches ({NBUF * cfg.rows * cfg.vocab * 2 / 1e6:.0f} MB > 126 MB L2)",
        "exchange": names[exchange] if gpus > 1 else "none",
    }


def hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.05)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            f = [x.strip() for x in s.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx = float(f[1])
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_reference_pass(x_host, cfg, seeds, threads, native=True):
    """One pass of the reference's CPU sampler over the batch. Returns (wall_s, kind, how).
    `native`: Sampler::sample<BFloat16> on the 16-bit logits (what sample_from_logits calls);
    otherwise Sampler::sample<float> on their exact upcast (the parity oracle's own path)."""
    import oracle
    timing = {}
    if oracle.Reference.available(stable=False):
        ref = oracle.Reference(stable=False)
        ref.sample_rows(x_host, cfg.temperature, cfg.topp, seeds, dtype=cfg.dtype, threads=threads,
                        native=native, timing=timing)
        return timing["wall_seconds"], "reference", (
            "Sampler::sample<BFloat16> of the unmodified sampler.cpp" if native
            else "Sampler::sample<float> of the unmodified sampler.cpp on the upcast logits")
    r = oracle.Restatement()
    r.sample_rows(x_host, cfg.temperature, cfg.topp, seeds, dtype=cfg.dtype, threads=threads, timing=timing)
    return timing["wall_seconds"], "port", "C restatement (float on upcast logits)"


def cpu_baseline(x_host, cfg, seeds, budget_cpu_s=15.0):
    threads = os.cpu_count() or 1
    rows = x_host.shape[0]
    wall, kind, how = cpu_reference_pass(x_host, cfg, seeds, threads)  # also warms the pages
    reps = int(max(1, min(200, budget_cpu_s / max(wall * threads, 1e-6))))
    t = 0.0
    for _ in range(reps):
        w, kind, how = cpu_reference_pass(x_host, cfg, seeds, threads)
        t += w
    return {"value": rows * reps / t, "unit": "rows/s", "cores": threads, "kind": kind,
            "sample": f"{reps} passes over the {rows}-row batch, one fresh Sampler per row, "
                      f"rows striped over {threads} threads; {how}"}


def run_reference(args, rank, world):
    """The reference arm: the reference's own CPU implementation on this box's host cores.
    Each step samples a slice of the 256-row batch, sized so that the K steps take about a
    minute and a half whatever K is (rows/s does not depend on the slice size)."""
    if rank != 0:
        return
    import numpy as np
    from executorch_b200 import workloads as W
    workload = args.workload
    cfg = W.CONFIGS[workload]
    rows = 256  # the batch a step draws its rows from (c3: the whole batch)
    # same distribution as the device-born benchmark rows; a 64-row host sample tiled to the
    # batch keeps generation short (the sampler's cost does not depend on which rows repeat)
    base = W.rows_numpy(workload, list(range(64)))
    x = np.ascontiguousarray(np.tile(base, (rows // 64, 1)))
    seeds = np.arange(rows, dtype=np.uint64)
    threads = os.cpu_count() or 1
    t_full, kind, how = cpu_reference_pass(x, cfg, seeds, threads)  # also warms the pages
    budget_s = 90.0
    per_step = int(rows * (budget_s / max(args.steps + args.warmup, 1)) / max(t_full, 1e-6))
    per_step = max(min(rows, per_step), min(rows, threads))
    xs, ss = x[:per_step], seeds[:per_step]
    for _ in range(args.warmup):
        cpu_reference_pass(xs, cfg, ss, threads)
    t = 0.0
    for _ in range(args.steps):
        w, kind, how = cpu_reference_pass(xs, cfg, ss, threads)
        t += w
    value = per_step * args.steps / t
    # for the record: the same sampler on the fp32 upcast (the oracle's path), and on one thread
    variants = {}
    for label, nat, thr in (("float_upcast_all_threads", False, threads), ("native_one_thread", True, 1),
                            ("float_upcast_one_thread", False, 1)):
        n = max(min(per_step, 4 * thr), 1)
        w, _, _ = cpu_reference_pass(x[:n], cfg, seeds[:n], thr, native=nat)
        variants[label] = {"rows_per_s": n / w, "threads": thr, "rows": n}
    line = {
        "impl": "reference",
        "metric": "sampled_rows_per_s_topp_v256000_bf16" if workload == "c5" else METRIC,
        "value": value, "unit": "rows/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t / args.steps,
        "higher_is_better": True, "scaling": "strong" if workload == "c5" else "weak", "vs_baseline": None,
        "dtype": "f32", "logits_dtype": "bf16", "data": "synthetic",
        "config": config_dict(args.gpus, False, args.exchange, workload),
        "cpu_baseline": {"value": value, "unit": "rows/s", "cores": threads, "kind": kind,
                         "sample": f"each step = {per_step} rows of the {rows}-row batch on {threads} threads; {how}",
                         "variants": variants},
        "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def other_configs(dev, peak, kernel_choice):
    """Short device-timed runs of the other baseline shapes and modes: mean launch time over a
    few launches (CUDA events on the launching stream), logits bytes / time, fraction of the
    HBM peak. Inputs rotate over buffers larger than L2 where the shape allows it."""
    import numpy as np
    import torch
    from executorch_b200 import Sampler, seeds_to_states
    from executorch_b200 import workloads as W

    out = {}

    def timed(name, rows, temperature, topp, label, reps=5, nbuf=2, single_calls=0):
        cfg = W.CONFIGS[name]
        bufs = [W.rows_torch(name, b * rows, rows, dev) for b in range(nbuf)]
        s = Sampler(cfg.vocab, temperature, topp, 0, device=dev)
        s.set_kernel_choice(kernel_choice)
        seeds = np.arange(rows, dtype=np.uint64)
        sts = [seeds_to_states(seeds, dev) for _ in range(reps + 2)]
        for i in range(2):
            s.sample_rows(bufs[i % nbuf], sts[i])
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(reps):
            s.sample_rows(bufs[i % nbuf], sts[2 + i])
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / reps
        nbytes = rows * cfg.vocab * W.BYTES[cfg.dtype]
        rec = {"rows": rows, "vocab": cfg.vocab, "logits_dtype": cfg.dtype, "temperature": temperature, "topp": topp,
               "kernel_ms": ms, "rows_per_s": rows / (ms * 1e-3), "gb_per_s": nbytes / (ms * 1e-3) / 1e9,
               "frac": nbytes / (ms * 1e-3) / 1e9 / peak}
        if single_calls:
            # the reference-shaped call: one row, token back on the host, every draw
            row = bufs[0][0]
            s.sample(row)
            t0 = time.perf_counter()
            for _ in range(single_calls):
                s.sample(row)
            rec["us_per_draw_sample_call"] = (time.perf_counter() - t0) / single_calls * 1e6
        s.close()
        del bufs
        torch.cuda.empty_cache()
        out[label] = rec

    timed("c1", 2048, 0.8, 0.9, "c1_topp_fp32_v32000")
    timed("c1", 2048, 0.8, 1.0, "c1_multinomial_fp32_v32000")
    timed("c2", 1, 0.7, 0.9, "c2_single_row_bf16_v128256", reps=50, nbuf=1, single_calls=50)
    timed("c3", 256, 0.0, 0.95, "c3_greedy_bf16_v128256", reps=20, nbuf=4)
    timed("c3", 256, 0.7, 1.0, "c3_multinomial_bf16_v128256", reps=10, nbuf=4)
    timed("c4", 512, 1.0, 0.9, "c4_topp_fp16_v151936", reps=2, nbuf=1)
    timed("c5", 2048, 0.8, 0.9, "c5_topp_bf16_v256000", reps=3, nbuf=1)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=20)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-other-configs", action="store_true")
    ap.add_argument("--kernel", type=int, default=0, choices=[0, 1, 2, 3],
                    help="kernel choice of the handle (0 = automatic; see etb200_sampler_set_kernel_choice)")
    ap.add_argument("--workload", default=WORKLOAD, choices=["c3", "c5"],
                    help="c3 (default): the headline batch, 256 rows per GPU, weak scaling. c5: 32768 rows x "
                         "V=256000 divided among the GPUs (16.8 GB in all), strong scaling, no id exchange")
    ap.add_argument("--greedy", action="store_true",
                    help="config 3's second pass instead of the headline: temperature 0 (argmax) on the same batch")
    ap.add_argument("--exchange", default="p2p", choices=["p2p", "p2p-in-kernel", "nccl"],
                    help="N > 1: ids stored into the peers' buffers by the kernel, ranks synchronised by a barrier "
                         "behind the launch (p2p) or by arrival marks inside it (p2p-in-kernel); or all-gathered (nccl)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import numpy as np
    import torch
    import torch.distributed as dist

    from executorch_b200 import Sampler, seeds_to_states
    from executorch_b200 import workloads as W

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the sampler has no CPU path")
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun for N > 1")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    workload = args.workload
    strong = workload == "c5"
    cfg = W.CONFIGS[workload]
    rows, vocab = (cfg.rows // world if strong else cfg.rows), cfg.vocab
    total_rows = rows * world
    warmup = max(args.warmup, 3)
    nbuf = 1 if strong else NBUF  # one c5 shard alone is far larger than L2
    if strong:
        args.greedy = False
        args.no_cpu_baseline = args.no_other_configs = True
        args.exchange = "nccl"  # unused: no exchange in this workload

    # inputs born in HBM: nbuf distinct batches for this rank (rows are a function of their id)
    bufs = [W.rows_torch(workload, (rank * nbuf + b) * rows, rows, dev) for b in range(nbuf)]
    seeds = np.arange(rank * rows, (rank + 1) * rows, dtype=np.uint64)
    states0 = seeds_to_states(seeds, dev)
    states = states0.clone()
    local_ids = torch.empty(rows, dtype=torch.int64, device=dev)
    all_ids = torch.empty(total_rows, dtype=torch.int64, device=dev) if world > 1 else local_ids
    sampler = Sampler(vocab, 0.0 if args.greedy else cfg.temperature, cfg.topp, 0, device=dev)
    sampler.set_kernel_choice(args.kernel)
    if args.greedy:
        args.no_cpu_baseline = True

    exchange, exchange_mode = None, (args.exchange if world > 1 else "none")
    if world > 1 and not strong and args.exchange in ("p2p", "p2p-in-kernel"):
        try:
            from executorch_b200.sharded import PeerIdExchange
            exchange = PeerIdExchange(total_rows, dev)
        except Exception:  # symmetric memory unavailable: use the collective
            exchange = None
        # every rank must take the same path
        flag = torch.tensor([1 if exchange is not None else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag) == 0:
            exchange, exchange_mode = None, "nccl"

    in_kernel_sync = exchange_mode == "p2p-in-kernel"

    def step(i, k_start=None, k_end=None):
        """One step: sample this rank's rows and make every rank hold all ids. Returns the buffer
        that will hold them (complete once the stream / the overlapped barrier has caught up)."""
        if exchange is not None:
            exchange.begin_step()
        if k_start is not None:
            k_start.record()
        if exchange is not None and in_kernel_sync:
            sampler.sample_rows_exchange(bufs[i % nbuf], states, exchange.dest_ptrs, exchange.mark_ptrs, rank,
                                         rank * rows, exchange.next_epoch())
            if k_end is not None:
                k_end.record()
            return exchange.finish(barrier=False)
        if exchange is not None:
            sampler.sample_rows_scatter(bufs[i % nbuf], states, exchange.dest_ptrs, rank * rows)
            if k_end is not None:
                k_end.record()
            # the barrier runs on a side stream: the next step's launch does not queue behind it
            return exchange.finish(overlap=True)[0]
        sampler.sample_rows(bufs[i % nbuf], states, out=local_ids)
        if k_end is not None:
            k_end.record()
        if world > 1 and not strong:
            dist.all_gather_into_tensor(all_ids, local_ids)
        return local_ids if strong else all_ids

    for i in range(warmup):
        states.copy_(states0)
        step(i)
    if exchange is not None:
        exchange.drain()
    torch.cuda.synchronize()

    # ---- device-timed region: K steps, inputs resident
    k_start = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    k_end = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = sampler.launch_count
    clocks = ClockSampler(local_rank)
    if rank == 0:
        clocks.start()
        time.sleep(0.3)  # nvidia-smi needs a moment before its first sample
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0.record()
    for i in range(args.steps):
        step(i, k_start[i], k_end[i])
    if exchange is not None:
        exchange.drain()  # every step's exchange is complete inside the timed region
    t1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    clock_info = clocks.stop() if rank == 0 else None
    launches = sampler.launch_count - launches0
    if exchange is not None and in_kernel_sync and sampler.status != 0:
        raise RuntimeError("an arrival wait of the in-kernel id exchange ran out: the ranks were not in step")
    elapsed_ms = t0.elapsed_time(t1)
    kernel_ms = statistics.mean(a.elapsed_time(b) for a, b in zip(k_start, k_end))
    if world > 1:
        tt = torch.tensor([elapsed_ms, kernel_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        elapsed_ms, kernel_ms = float(tt[0]), float(tt[1])
    value = total_rows * args.steps / (elapsed_ms * 1e-3)

    # ---- parity: one more step, from known states, checked outside the timed region
    import oracle
    vb = args.steps % nbuf
    states.copy_(states0)
    got_all = step(args.steps)
    if exchange is not None:
        exchange.drain()
    torch.cuda.synchronize()
    got_all = got_all.clone()
    mine = got_all[rank * rows:(rank + 1) * rows] if (world > 1 and not strong) else got_all
    exchange_verified = None
    if world > 1 and not strong:
        # every rank's own ids of the same step, gathered by NCCL: the exchange must agree
        ref_all = torch.empty(total_rows, dtype=torch.int64, device=dev)
        dist.all_gather_into_tensor(ref_all, mine.contiguous())
        okf = torch.tensor([1 if torch.equal(ref_all, got_all) else 0], device=dev)
        dist.all_reduce(okf, op=dist.ReduceOp.MIN)
        exchange_verified = bool(int(okf))
    parity_rows = parity_equal = 0
    if rank == 0:
        xh = bufs[vb][:PARITY_ROWS].cpu().view(torch.int16).numpy().view(np.uint16)
        sd = seeds[:PARITY_ROWS]
        want = oracle.Restatement().sample_rows(xh, 0.0 if args.greedy else cfg.temperature, cfg.topp, sd,
                                                dtype=cfg.dtype, threads=min(16, os.cpu_count() or 1))
        gh = mine[:PARITY_ROWS].cpu().numpy()
        parity_rows, parity_equal = PARITY_ROWS, int((gh == want).sum())

    # ---- end to end through the host-buffer entry of the C ABI (pinned host logits)
    e2e_rows = min(rows, 1024) if strong else rows  # c5: a slice (a whole shard is gigabytes per step)
    host_bufs = [bufs[b % nbuf][:e2e_rows].cpu().view(torch.int16).pin_memory().view(torch.bfloat16)
                 for b in range(2)]
    host_states = seeds[:e2e_rows].copy()
    for i in range(2):
        host_states[:] = seeds[:e2e_rows]
        sampler.sample_rows_host(host_bufs[i % 2], host_states)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0 = time.perf_counter()
    for i in range(args.e2e_steps):
        ids_host = sampler.sample_rows_host(host_bufs[i % 2], host_states)
    e_ms = (time.perf_counter() - e0) * 1e3
    if world > 1:
        tt = torch.tensor([e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e_ms = float(tt[0])
    e2e_value = e2e_rows * world * args.e2e_steps / (e_ms * 1e-3)
    h2d = e2e_rows * vocab * 2 + e2e_rows * 8
    d2h = e2e_rows * 8 + e2e_rows * 8
    assert ids_host.shape == (e2e_rows,)

    if rank == 0:
        peak, which = hbm_peak()
        algo_bytes = rows * (vocab * 2 + 8 + 16)  # logits once + id + rng state in/out
        achieved = algo_bytes / (kernel_ms * 1e-3) / 1e9
        kernel_name = "argmax_rows_kernel" if args.greedy else "sample_rows_kernel"
        traffic, stale = dram_traffic(kernel_name) if not strong else (None, False)
        line = {
            "metric": ("sampled_rows_per_s_topp_v256000_bf16" if strong else
                       "argmax_rows_per_s_v128256_bf16" if args.greedy else METRIC),
            "value": value, "unit": "rows/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True,
            "scaling": "strong" if strong else "weak", "vs_baseline": None, "dtype": "f32",
            "logits_dtype": "bf16",
            "data": "synthetic",
            "config": config_dict(world, args.greedy, exchange_mode if world > 1 else args.exchange, workload),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": traffic, "traffic_stale": stale,
                         "peak_source": f"of {which}", "kernel_ms": kernel_ms, "kernel": kernel_name,
                         "algorithmic_bytes_per_launch": algo_bytes},
            "parity": {"checked_rows": parity_rows, "equal": parity_equal, "exchange_verified": exchange_verified,
                       "against": "CPU oracle (C restatement of sampler.cpp) on the rows of one extra step"},
            "e2e": {"value": e2e_value, "unit": "rows/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e_ms / args.e2e_steps,
                    "rows_per_step_per_gpu": e2e_rows},
            "gpu_launches": int(launches),
            "clocks": clock_info,
        }
        if world == 1 and not args.no_cpu_baseline:
            x_host = host_bufs[0].view(torch.int16).numpy().view(np.uint16)
            line["cpu_baseline"] = cpu_baseline(x_host, cfg, seeds)
        if world == 1 and not args.no_other_configs and not args.greedy:
            del bufs, host_bufs
            torch.cuda.empty_cache()
            line["other_configs"] = other_configs(dev, peak, args.kernel)
        print(json.dumps(line), flush=True)
    sampler.close()
    if world > 1:
        dist.destroy_process_group()
    if parity_rows and parity_equal != parity_rows:
        raise SystemExit(f"parity check failed: {parity_equal} of {parity_rows} rows equal the oracle's tokens")
    if exchange_verified is False:
        raise SystemExit("the id exchange did not leave every rank with every rank's ids")


if __name__ == "__main__":
    main()
