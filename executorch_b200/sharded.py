"""Row-sharded sampling across the GPUs of one node: one process per GPU, rows split in
contiguous blocks, and one all-gather of the sampled int64 ids (8 bytes per row) as the
only exchange. The reference has no multi-device path; rows are independent, so sharding
changes no result: row r draws from state r whichever rank owns it."""
from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist


def shard_rows(rows: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous block of rows owned by ``rank``: (first_row, count). Blocks are equal
    when ``world`` divides ``rows``; otherwise the first ``rows % world`` ranks get one more."""
    if world < 1 or not (0 <= rank < world) or rows < 0:
        raise ValueError(f"bad shard request rows={rows} rank={rank} world={world}")
    base, extra = divmod(rows, world)
    start = rank * base + min(rank, extra)
    return start, base + (1 if rank < extra else 0)


class ExchangeTimeout(RuntimeError):
    """The id exchange did not complete within its deadline (a rank is missing or late)."""


class PeerIdExchange:
    """The id exchange without a collective call: int64 buffers of ``total_rows`` per rank in
    torch's symmetric memory (every rank can address every peer's copy over NVLink), plus 16
    arrival marks per rank. The sampling kernel's epilogue stores each id into all copies.

    A rank that has passed the synchronisation of step k may start step k + 1 while a slower
    peer still reads the ids of step k, so the buffers ROTATE: step k uses region k mod 3. The
    ids returned for step k stay valid until this rank launches step k + 3, provided its
    reader is enqueued on the sampling stream before the launch of step k + 1.

    Two ways to synchronise the ranks after the stores:

    * ``Sampler.sample_rows_scatter`` + ``finish()``: ``finish`` enqueues a symmetric-memory
      barrier after which this rank's copy holds the ids of all ranks. With
      ``finish(overlap=True)`` the barrier runs on a side stream, so that the next step's
      sampling launch does not queue behind it; the returned event marks its completion and
      ``begin_step`` makes a launch wait for the barrier two steps back, which is what frees
      the region it is about to overwrite.
    * ``Sampler.sample_rows_exchange`` with ``mark_ptrs`` and ``next_epoch()``: the last block
      of the launch marks its arrival at every rank and waits (with a limit) for theirs, so
      the launch itself ends with a complete buffer and ``finish(barrier=False)`` only
      returns it. The caller checks ``Sampler.status`` (2 = the wait ran out) before trusting
      the ids of a step.

    Ranks must be the GPUs of one node."""

    REGIONS = 3

    def __init__(self, total_rows: int, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.total_rows = total_rows
        # ids and arrival marks live in one symmetric allocation: [3 x total_rows ids | 16 marks]
        self.storage = symm_mem.empty(self.REGIONS * total_rows + 16, dtype=torch.int64, device=device)
        self.storage.zero_()
        self.handle = symm_mem.rendezvous(self.storage, self.group)
        self.base_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.mark_ptrs = [int(p) + 8 * self.REGIONS * total_rows for p in self.handle.buffer_ptrs]
        if len(self.base_ptrs) > 16:
            raise ValueError("at most 16 ranks can exchange ids through peer buffers")
        self.epoch = 0
        self.step = 0
        self.device = device
        self.side = torch.cuda.Stream(device=device)
        self.done = [None] * self.REGIONS  # completion events of the overlapped barriers
        torch.cuda.synchronize(device)
        self.handle.barrier(channel=0)  # every rank's marks are zero before anyone writes one
        torch.cuda.synchronize(device)

    @property
    def region(self) -> int:
        return self.step % self.REGIONS

    @property
    def dest_ptrs(self):
        """Addresses of every rank's buffer for the current step."""
        off = 8 * self.region * self.total_rows
        return [p + off for p in self.base_ptrs]

    @property
    def buffer(self) -> torch.Tensor:
        lo = self.region * self.total_rows
        return self.storage[lo:lo + self.total_rows]

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch

    def begin_step(self) -> None:
        """Before the sampling launch of a step: the region it writes was read by the peers two
        barriers ago at the latest."""
        ev = self.done[(self.step + 1) % self.REGIONS]  # the barrier of step - 2
        if ev is not None:
            torch.cuda.current_stream(self.device).wait_event(ev)

    def finish(self, barrier: bool = True, overlap: bool = False):
        """After the sampling launch of a step. Returns this rank's buffer for the step, and
        with ``overlap`` also the event a reader must wait for. Advances to the next region."""
        buf = self.buffer
        ev = None
        if barrier and overlap:
            main = torch.cuda.current_stream(self.device)
            launched = torch.cuda.Event()
            launched.record(main)
            with torch.cuda.stream(self.side):
                self.side.wait_event(launched)
                self.handle.barrier(channel=0)
                ev = torch.cuda.Event()
                ev.record(self.side)
            self.done[self.region] = ev
        elif barrier:
            # all ranks' stores are ordered before the barrier's release on each stream
            self.handle.barrier(channel=0)
            self.done[self.region] = None
        self.step += 1
        return (buf, ev) if overlap else buf

    def drain(self) -> None:
        """Makes the current stream wait for every overlapped barrier still in flight."""
        main = torch.cuda.current_stream(self.device)
        for ev in self.done:
            if ev is not None:
                main.wait_event(ev)


class ShardedSampler:
    """Samples this rank's rows with ``local_sample`` and gathers all ids on every rank.

    ``local_sample(logits, rng_states) -> int64 ids`` is normally ``Sampler.sample_rows``;
    tests inject a CPU stand-in to exercise the exchange with the gloo backend."""

    def __init__(self, local_sample: Callable[[torch.Tensor, torch.Tensor | None], torch.Tensor],
                 total_rows: int, group=None, scatter=None, device=None, in_kernel_sync: bool = False,
                 deadline_s: float | None = None):
        """``scatter(logits, rng_states, dest_ptrs, dest_offset)`` (normally
        ``Sampler.sample_rows_scatter``) selects the peer-buffer exchange instead of the
        all-gather; it needs equal shards and a CUDA ``device``. With ``in_kernel_sync`` the
        callable is ``Sampler.sample_rows_exchange`` and the ranks synchronise inside the
        sampling launch instead of through a barrier behind it. With ``deadline_s`` the
        all-gather is waited for at most that long and ``ExchangeTimeout`` is raised instead
        of blocking when a rank never arrives."""
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised")
        self.local_sample = local_sample
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.total_rows = total_rows
        self.start, self.count = shard_rows(total_rows, self.rank, self.world)
        self.even = total_rows % self.world == 0
        self.scatter = scatter
        self.in_kernel_sync = in_kernel_sync
        self.deadline_s = deadline_s
        self.exchange = None
        if scatter is not None:
            if not self.even:
                raise ValueError("the peer-buffer exchange needs equal shards")
            self.exchange = PeerIdExchange(total_rows, device, group)

    def _gather(self, out: torch.Tensor, part: torch.Tensor) -> None:
        if self.deadline_s is None:
            dist.all_gather_into_tensor(out, part, group=self.group)
            return
        import datetime

        work = dist.all_gather_into_tensor(out, part, group=self.group, async_op=True)
        try:
            done = work.wait(timeout=datetime.timedelta(seconds=self.deadline_s))
        except RuntimeError as exc:  # the backend's own way of reporting the timeout
            raise ExchangeTimeout(f"rank {self.rank}: id all-gather not complete after "
                                  f"{self.deadline_s} s: {exc}") from exc
        if done is False:
            raise ExchangeTimeout(f"rank {self.rank}: id all-gather not complete after {self.deadline_s} s")

    def sample_rows(self, local_logits: torch.Tensor, local_states: torch.Tensor | None,
                    out: torch.Tensor | None = None) -> torch.Tensor:
        if local_logits.shape[0] != self.count:
            raise ValueError(f"rank {self.rank} owns {self.count} rows, got {local_logits.shape[0]}")
        if self.exchange is not None:
            if self.in_kernel_sync:
                ex = self.exchange
                self.scatter(local_logits, local_states, ex.dest_ptrs, ex.mark_ptrs, ex.rank, self.start,
                             ex.next_epoch())
                return ex.finish(barrier=False)
            self.scatter(local_logits, local_states, self.exchange.dest_ptrs, self.start)
            return self.exchange.finish()
        ids = self.local_sample(local_logits, local_states)
        if out is None:
            out = torch.empty(self.total_rows, dtype=torch.int64, device=ids.device)
        if self.even:
            self._gather(out, ids)
        else:
            # ragged shards: pad to the largest block, gather, then drop the padding
            width = -(-self.total_rows // self.world)
            padded = torch.zeros(width, dtype=torch.int64, device=ids.device)
            padded[: self.count] = ids
            gathered = torch.empty(width * self.world, dtype=torch.int64, device=ids.device)
            self._gather(gathered, padded)
            for r in range(self.world):
                s, c = shard_rows(self.total_rows, r, self.world)
                out[s:s + c] = gathered[r * width: r * width + c]
        return out
