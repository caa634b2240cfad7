"""The allocation-free entry point, etb200_sample_rows_static, called through the C ABI.

Some hosts of this library are not allowed to allocate device memory once they are running
(a runtime with a pre-planned arena, a tenant with a fixed budget on a shared GPU, a loop
that cannot take cudaMalloc's implicit synchronisation). For them the library keeps the
sampling kernel's candidate lists in a fixed array inside the library image. This test
checks that the entry point gives exactly the tokens and RNG states of the handle-based
entry point, on two calls in a row (the second call finds the first call's leftovers in the
shared array), that it refuses a vocabulary whose lists cannot fit, and that it really
leaves the device's memory accounting untouched.

The file name sorts last on purpose: a run that stops at the first failure has then already
run every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from executorch_b200 import _lib
from executorch_b200 import workloads as W

pytestmark = pytest.mark.gpu


def _handle_based(lib, vocab, temperature, topp, logits, states, device_index):
    h = C.c_void_p()
    _lib.check(lib.etb200_sampler_create(vocab, temperature, topp, 0, device_index, C.byref(h)))
    out = torch.empty(logits.shape[0], dtype=torch.int64, device=logits.device)
    st = states.clone()
    _lib.check(lib.etb200_sampler_sample_rows(
        h, C.c_void_p(logits.data_ptr()), _lib.DTYPE_BFLOAT16, logits.shape[0], logits.stride(0),
        C.c_void_p(st.data_ptr()), C.c_void_p(out.data_ptr()),
        C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    torch.cuda.synchronize()
    lib.etb200_sampler_destroy(h)
    return out, st


def _static(lib, vocab, temperature, topp, logits, states):
    out = torch.empty(logits.shape[0], dtype=torch.int64, device=logits.device)
    st = states.clone()
    code = lib.etb200_sample_rows_static(
        vocab, temperature, topp, C.c_void_p(logits.data_ptr()), _lib.DTYPE_BFLOAT16,
        logits.shape[0], logits.stride(0), C.c_void_p(st.data_ptr()), C.c_void_p(out.data_ptr()),
        C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert code == _lib.OK, lib.etb200_static_last_error_message()
    torch.cuda.synchronize()
    return out, st


def test_static_scratch_entry_matches_handle_entry_twice_in_a_row(cuda_device):
    lib = _lib.load()
    torch.cuda.set_device(cuda_device)
    vocab, rows = 128256, 96  # more rows than the 32 blocks the array can serve at once
    x = W.rows_numpy("c3", list(range(rows)))
    logits = torch.from_numpy(x.view(np.int16)).to(cuda_device).view(torch.bfloat16)
    for call, (temperature, topp, seed0) in enumerate(((0.7, 0.95, 0), (0.9, 0.5, 1000))):
        seeds = (np.arange(rows, dtype=np.uint64) + np.uint64(seed0)).view(np.int64)
        states = torch.from_numpy(seeds.copy()).to(cuda_device)
        want_ids, want_states = _handle_based(lib, vocab, temperature, topp, logits, states, cuda_device.index)
        got_ids, got_states = _static(lib, vocab, temperature, topp, logits, states)
        # integer results: the bar is exact equality, as in the other parity tests
        assert torch.equal(got_ids, want_ids), (call, (got_ids != want_ids).nonzero()[:8])
        assert torch.equal(got_states, want_states), call
    # multinomial and greedy go through the same entry point (no scratch needed there)
    for temperature, topp in ((0.7, 1.0), (0.0, 0.9)):
        states = torch.arange(rows, dtype=torch.int64, device=cuda_device)
        want_ids, _ = _handle_based(lib, vocab, temperature, topp, logits, states, cuda_device.index)
        got_ids, _ = _static(lib, vocab, temperature, topp, logits, states)
        assert torch.equal(got_ids, want_ids), (temperature, topp)


def test_static_scratch_entry_refuses_what_cannot_fit_and_bad_arguments(cuda_device):
    lib = _lib.load()
    torch.cuda.set_device(cuda_device)
    dummy = torch.zeros(16, dtype=torch.bfloat16, device=cuda_device)
    ids = torch.zeros(1, dtype=torch.int64, device=cuda_device)
    st = torch.zeros(1, dtype=torch.int64, device=cuda_device)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    too_big = (64 << 20) // 16 + 1
    code = lib.etb200_sample_rows_static(too_big, 0.7, 0.9, C.c_void_p(dummy.data_ptr()), _lib.DTYPE_BFLOAT16,
                                         1, too_big, C.c_void_p(st.data_ptr()), C.c_void_p(ids.data_ptr()), stream)
    assert code == _lib.INVALID_ARGUMENT
    msg = lib.etb200_static_last_error_message().decode()
    assert "static array" in msg and "4194304" in msg
    code = lib.etb200_sample_rows_static(16, 0.7, 0.9, C.c_void_p(dummy.data_ptr()), _lib.DTYPE_BFLOAT16,
                                         1, 16, None, C.c_void_p(ids.data_ptr()), stream)
    assert code == _lib.INVALID_ARGUMENT  # no handle, so no state to fall back on
    code = lib.etb200_sample_rows_static(16, 0.7, 0.9, C.c_void_p(dummy.data_ptr()), 7,
                                         1, 16, C.c_void_p(st.data_ptr()), C.c_void_p(ids.data_ptr()), stream)
    assert code == _lib.NOT_SUPPORTED


def test_static_scratch_entry_allocates_nothing(cuda_device):
    """Free device memory, as the driver reports it, does not move across calls. Outputs are
    allocated once up front so that torch's own allocator stays out of the picture."""
    lib = _lib.load()
    torch.cuda.set_device(cuda_device)
    vocab, rows = 32000, 64
    x = W.rows_numpy("c3", list(range(rows)), vocab=vocab)
    logits = torch.from_numpy(x.view(np.int16)).to(cuda_device).view(torch.bfloat16)
    states = torch.arange(rows, dtype=torch.int64, device=cuda_device)
    out = torch.empty(rows, dtype=torch.int64, device=cuda_device)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def call():
        code = lib.etb200_sample_rows_static(
            vocab, 0.7, 0.9, C.c_void_p(logits.data_ptr()), _lib.DTYPE_BFLOAT16, rows, vocab,
            C.c_void_p(states.data_ptr()), C.c_void_p(out.data_ptr()), stream)
        assert code == _lib.OK, lib.etb200_static_last_error_message()
        torch.cuda.synchronize()

    call()  # first call on this device: symbol lookup (and the module load, if still pending)
    free0, _ = torch.cuda.mem_get_info(cuda_device)
    for _ in range(5):
        call()
    free1, _ = torch.cuda.mem_get_info(cuda_device)
    assert free1 == free0
