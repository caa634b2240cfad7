"""The bounded wait of the in-kernel id exchange, made to run out on ONE GPU: the launch is
told that two ranks exchange ids, both ranks' buffers and arrival marks live in this GPU's own
memory, and nobody ever writes rank 1's mark. Nothing faults or hangs: the wait gives up after
its time limit, the launch ends normally, the status word reads 2 and clears, rank 0's own ids
are right, and the next epoch -- with rank 1's mark written beforehand -- completes with
status 0."""
import time

import numpy as np
import pytest
import torch

import oracle
from executorch_b200 import Sampler, seeds_to_states
from executorch_b200 import workloads as W

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("temperature,topp", [(0.7, 0.9), (0.0, 0.9)])
def test_arrival_wait_runs_out_and_reports_status(cuda_device, temperature, topp):
    dev = cuda_device
    vocab, rows = 20000, 8
    x = W.rows_numpy("c3", list(range(rows)), vocab=vocab)
    seeds = np.arange(rows, dtype=np.uint64) + 11
    want = oracle.Restatement().sample_rows(x, temperature, topp, seeds, dtype="bf16", threads=2)
    t = torch.from_numpy(x.view(np.int16)).to(dev).view(torch.bfloat16)
    s = Sampler(vocab, temperature, topp, 0, device=dev)
    try:
        s.set_wait_limit(0.002)
        # two "ranks", both in this GPU's memory: [rank 0 ids | rank 1 ids], 16 marks each
        ids = torch.full((2, 2 * rows), -1, dtype=torch.int64, device=dev)
        marks = torch.zeros((2, 16), dtype=torch.int64, device=dev)
        dest = [ids[0].data_ptr(), ids[1].data_ptr()]
        mark_ptrs = [marks[0].data_ptr(), marks[1].data_ptr()]
        torch.cuda.synchronize(dev)
        t0 = time.time()
        s.sample_rows_exchange(t, seeds_to_states(seeds, dev), dest, mark_ptrs, 0, 0, 1)
        torch.cuda.synchronize(dev)  # returns: the wait is limited
        assert time.time() - t0 < 5.0
        assert s.status == 2          # rank 1 never arrived
        assert s.status == 0          # reading clears it
        got = ids.cpu().numpy()
        assert np.array_equal(got[0, :rows], want) and np.array_equal(got[1, :rows], want)
        assert (got[:, rows:] == -1).all()  # rank 1's ids: stale, as documented
        m = marks.cpu().numpy()
        assert m[0, 0] == 1 and m[1, 0] == 1 and m[0, 1] == 0
        # next epoch: "rank 1" has arrived (its mark is written before the launch)
        marks[0, 1] = 2
        torch.cuda.synchronize(dev)
        s.sample_rows_exchange(t, seeds_to_states(seeds, dev), dest, mark_ptrs, 0, 0, 2)
        torch.cuda.synchronize(dev)
        assert s.status == 0
        assert np.array_equal(ids.cpu().numpy()[0, :rows], want)
    finally:
        s.close()
