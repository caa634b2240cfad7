"""Python mirror of the reference's sampling interface, backed by the CUDA library.

``Sampler`` keeps the constructor and methods of ``executorch::extension::llm::Sampler``
(extension/llm/sampler/sampler.h:37-83) and adds the batched ``sample_rows``;
``sample_from_logits`` and ``logits_to_token`` mirror extension/llm/sampler/util.h:25-71.
Every call goes through the C ABI declared in include/etb200_sampler.h.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import _lib

K_TOPP = 0.9  # kTopp, sampler.h:29

_TORCH_DTYPES = {
    torch.float16: _lib.DTYPE_HALF,
    torch.float32: _lib.DTYPE_FLOAT,
    torch.bfloat16: _lib.DTYPE_BFLOAT16,
    torch.uint16: _lib.DTYPE_UINT16,
}


def _dtype_code(t: torch.Tensor) -> int:
    try:
        return _TORCH_DTYPES[t.dtype]
    except KeyError:
        # sample_from_logits aborts on other dtypes (util.h:30-34)
        raise _lib.SamplerError(_lib.NOT_SUPPORTED, f"unsupported logits dtype {t.dtype}") from None


def seeds_to_states(seeds, device) -> torch.Tensor:
    """Per-row xorshift64* states initialised from per-row seeds (uint64 bit patterns kept
    in an int64 tensor, which is what torch can index and copy)."""
    a = np.ascontiguousarray(np.asarray(seeds, dtype=np.uint64)).view(np.int64)
    return torch.from_numpy(a.copy()).to(device)


class Sampler:
    """``Sampler(vocab_size, temperature, topp, rng_seed)`` or ``Sampler(vocab_size,
    temperature)`` (top-p 0.9 and a wall-clock seed), as sampler.cpp:173-187."""

    def __init__(self, vocab_size: int, temperature: float, topp: float | None = None,
                 rng_seed: int | None = None, device: int | torch.device | None = None):
        self._h = C.c_void_p()
        lib = _lib.load()
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device: the B200 sampler has no CPU path")
        if device is None:
            device = torch.cuda.current_device()
        self.device = torch.device("cuda", device) if isinstance(device, int) else torch.device(device)
        self.vocab_size = int(vocab_size)
        idx = self.device.index if self.device.index is not None else torch.cuda.current_device()
        if (topp is None) != (rng_seed is None):
            raise TypeError("pass both topp and rng_seed (4-argument form) or neither (2-argument form)")
        if topp is None:
            _lib.check(lib.etb200_sampler_create_default(self.vocab_size, temperature, idx, C.byref(self._h)))
        else:
            _lib.check(lib.etb200_sampler_create(
                self.vocab_size, temperature, topp, C.c_uint64(rng_seed & (2**64 - 1)), idx, C.byref(self._h)))

    def close(self) -> None:
        if getattr(self, "_h", None) is not None and self._h.value:
            _lib.load().etb200_sampler_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- sampler.h:48-60
    def set_temperature(self, temperature: float) -> None:
        _lib.check(_lib.load().etb200_sampler_set_temperature(self._h, temperature))

    def set_topk(self, topk: int) -> None:
        _lib.check(_lib.load().etb200_sampler_set_topk(self._h, topk))

    def set_kernel_choice(self, choice: int) -> None:
        """0 (default): automatic; 1: one block per row; 2: a thread-block cluster per row where
        that applies; 3: one block per row with the estimate-guided sum. Same tokens from all."""
        _lib.check(_lib.load().etb200_sampler_set_kernel_choice(self._h, choice))

    @property
    def rng_state(self) -> int:
        out = C.c_uint64(0)
        _lib.check(_lib.load().etb200_sampler_get_rng_state(self._h, C.byref(out)))
        return int(out.value)

    @rng_state.setter
    def rng_state(self, value: int) -> None:
        _lib.check(_lib.load().etb200_sampler_set_rng_state(self._h, C.c_uint64(value & (2**64 - 1))))

    @property
    def last_retry_count(self) -> int:
        """Rows of the most recent sampling call that the fast kernel handed to the plain
        one-block-per-row kernel (synchronises)."""
        out = C.c_int32(0)
        _lib.check(_lib.load().etb200_sampler_last_retry_count(self._h, C.byref(out)))
        return int(out.value)

    @property
    def launch_count(self) -> int:
        out = C.c_uint64(0)
        _lib.check(_lib.load().etb200_sampler_launch_count(self._h, C.byref(out)))
        return int(out.value)

    def _stream(self) -> C.c_void_p:
        return C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def _check_rows(self, logits: torch.Tensor) -> None:
        if logits.dim() != 2:
            raise ValueError(f"expected [rows, vocab] logits, got shape {tuple(logits.shape)}")
        if logits.shape[1] != self.vocab_size:
            raise ValueError(f"last dimension {logits.shape[1]} != vocab_size {self.vocab_size}")
        if logits.stride(1) != 1:
            raise ValueError("logits rows must be contiguous (stride 1 in the vocab dimension)")

    def sample(self, logits: torch.Tensor) -> int:
        """``int32_t Sampler::sample(T* logits)`` on one row of device logits; uses and
        advances the sampler's own RNG state."""
        if logits.device.type != "cuda":
            raise ValueError("sample() takes device logits; use sample_rows_host for host memory")
        row = logits.reshape(-1)
        if row.numel() != self.vocab_size or row.stride(0) != 1:
            raise ValueError("sample() needs one contiguous row of vocab_size logits")
        out = C.c_int32(-1)
        _lib.check(_lib.load().etb200_sampler_sample(
            self._h, C.c_void_p(row.data_ptr()), _dtype_code(row), self._stream(), C.byref(out)))
        return int(out.value)

    def sample_rows(self, logits: torch.Tensor, rng_states: torch.Tensor | None = None,
                    out: torch.Tensor | None = None) -> torch.Tensor:
        """Samples every row of ``logits`` ([rows, vocab], device). ``rng_states`` is an int64
        device tensor of per-row xorshift64* states, advanced in place (not needed at
        temperature 0). Asynchronous on the current stream; returns int64 ids on device."""
        self._check_rows(logits)
        if logits.device != self.device:
            raise ValueError(f"logits on {logits.device}, sampler on {self.device}")
        rows = logits.shape[0]
        if out is None:
            out = torch.empty(rows, dtype=torch.int64, device=self.device)
        elif out.dtype != torch.int64 or out.numel() < rows or not out.is_contiguous():
            raise ValueError("out must be a contiguous int64 tensor with one element per row")
        states_ptr = C.c_void_p(0)
        if rng_states is not None:
            if (rng_states.dtype != torch.int64 or rng_states.numel() != rows
                    or not rng_states.is_contiguous() or rng_states.device != self.device):
                raise ValueError("rng_states must be a contiguous int64 device tensor, one per row")
            states_ptr = C.c_void_p(rng_states.data_ptr())
        _lib.check(_lib.load().etb200_sampler_sample_rows(
            self._h, C.c_void_p(logits.data_ptr()), _dtype_code(logits), rows, logits.stride(0),
            states_ptr, C.c_void_p(out.data_ptr()), self._stream()))
        return out

    def sample_rows_ex(self, logits: torch.Tensor, rng_states: torch.Tensor | None, *,
                       temperature: torch.Tensor | None = None, topp: torch.Tensor | None = None,
                       topk: torch.Tensor | None = None, scale: float = 1.0,
                       edit_ids: torch.Tensor | None = None, edit_bias: torch.Tensor | None = None,
                       edit_offsets: torch.Tensor | None = None,
                       out: torch.Tensor | None = None) -> torch.Tensor:
        """``sample_rows`` for a serving batch: per-row ``temperature`` / ``topp`` (float32) and
        ``topk`` (int32) device tensors replace the handle's settings (``SamplingConfig`` of
        ``LLMSession::decode_one``); ``edit_ids`` (int32) / ``edit_bias`` (float32, -inf masks)
        are added to the logits IN PLACE first -- for every row, or for the rows that
        ``edit_offsets`` (int64, rows + 1 entries) assigns them to -- and ``scale`` multiplies
        every logit as the kernel reads it: the mask, bias and multiply logit processors."""
        self._check_rows(logits)
        rows = logits.shape[0]
        if out is None:
            out = torch.empty(rows, dtype=torch.int64, device=self.device)
        opt = _lib.RowOptions()
        opt.scale = float(scale)

        def ptr(t, dtype, n, name):
            if t is None:
                return None
            if t.dtype != dtype or t.numel() != n or not t.is_contiguous() or t.device != self.device:
                raise ValueError(f"{name} must be a contiguous {dtype} device tensor with {n} entries")
            return t.data_ptr()

        opt.temperature_device = ptr(temperature, torch.float32, rows, "temperature")
        opt.topp_device = ptr(topp, torch.float32, rows, "topp")
        opt.topk_device = ptr(topk, torch.int32, rows, "topk")
        n_edits = 0 if edit_ids is None else edit_ids.numel()
        opt.n_edits = n_edits
        opt.edit_ids_device = ptr(edit_ids, torch.int32, n_edits, "edit_ids")
        opt.edit_bias_device = ptr(edit_bias, torch.float32, n_edits, "edit_bias")
        opt.edit_offsets_device = ptr(edit_offsets, torch.int64, rows + 1, "edit_offsets")
        states_ptr = C.c_void_p(0)
        if rng_states is not None:
            if (rng_states.dtype != torch.int64 or rng_states.numel() != rows
                    or not rng_states.is_contiguous() or rng_states.device != self.device):
                raise ValueError("rng_states must be a contiguous int64 device tensor, one per row")
            states_ptr = C.c_void_p(rng_states.data_ptr())
        _lib.check(_lib.load().etb200_sampler_sample_rows_ex(
            self._h, C.c_void_p(logits.data_ptr()), _dtype_code(logits), rows, logits.stride(0),
            states_ptr, C.c_void_p(out.data_ptr()), C.byref(opt), self._stream()))
        return out

    def sample_rows_scatter(self, logits: torch.Tensor, rng_states: torch.Tensor | None,
                            dest_ptrs, dest_offset: int) -> None:
        """Like ``sample_rows``, but the id of row r is stored into every int64 buffer of
        ``dest_ptrs`` (device addresses, this GPU's and its peers') at index ``dest_offset + r``.
        Asynchronous; the caller synchronises the ranks afterwards."""
        self._check_rows(logits)
        rows = logits.shape[0]
        states_ptr = C.c_void_p(0)
        if rng_states is not None:
            if (rng_states.dtype != torch.int64 or rng_states.numel() != rows
                    or not rng_states.is_contiguous() or rng_states.device != self.device):
                raise ValueError("rng_states must be a contiguous int64 device tensor, one per row")
            states_ptr = C.c_void_p(rng_states.data_ptr())
        arr = (C.c_void_p * len(dest_ptrs))(*[C.c_void_p(int(p)) for p in dest_ptrs])
        _lib.check(_lib.load().etb200_sampler_sample_rows_scatter(
            self._h, C.c_void_p(logits.data_ptr()), _dtype_code(logits), rows, logits.stride(0),
            states_ptr, arr, len(dest_ptrs), dest_offset, self._stream()))

    def sample_rows_exchange(self, logits: torch.Tensor, rng_states: torch.Tensor | None,
                             dest_ptrs, mark_ptrs, rank: int, dest_offset: int, epoch: int) -> None:
        """``sample_rows_scatter`` with the cross-GPU synchronisation inside the launch: when
        the launch has completed, the buffer ``dest_ptrs[rank]`` holds the ids of all ranks.
        ``mark_ptrs[p]`` is rank p's array of arrival marks; ``epoch`` grows by one per call on
        every rank. ``logits`` may have zero rows."""
        rows = logits.shape[0]
        if rows:
            self._check_rows(logits)
        states_ptr = C.c_void_p(0)
        if rng_states is not None and rows:
            if (rng_states.dtype != torch.int64 or rng_states.numel() != rows
                    or not rng_states.is_contiguous() or rng_states.device != self.device):
                raise ValueError("rng_states must be a contiguous int64 device tensor, one per row")
            states_ptr = C.c_void_p(rng_states.data_ptr())
        if len(dest_ptrs) != len(mark_ptrs):
            raise ValueError("one destination buffer and one mark array per rank")
        dst = (C.c_void_p * len(dest_ptrs))(*[C.c_void_p(int(p)) for p in dest_ptrs])
        marks = (C.c_void_p * len(mark_ptrs))(*[C.c_void_p(int(p)) for p in mark_ptrs])
        _lib.check(_lib.load().etb200_sampler_sample_rows_exchange(
            self._h, C.c_void_p(logits.data_ptr() if rows else 0), _dtype_code(logits), rows,
            logits.stride(0) if rows else 0, states_ptr, dst, marks, len(dest_ptrs), rank, dest_offset,
            epoch, self._stream()))

    def set_wait_limit(self, seconds: float) -> None:
        """Limit of the in-kernel wait of ``sample_rows_exchange`` for the other ranks."""
        _lib.check(_lib.load().etb200_sampler_set_wait_limit_ns(self._h, C.c_uint64(int(seconds * 1e9))))

    @property
    def status(self) -> int:
        """Reads and clears the device status word (synchronises): 0, 2 after an arrival wait of
        ``sample_rows_exchange`` ran out, 3 if the long-nucleus tail found its counts inconsistent
        for some row (not expected)."""
        v = C.c_int32(0)
        _lib.check(_lib.load().etb200_sampler_get_status(self._h, C.byref(v)))
        return int(v.value)

    def sample_rows_host(self, logits, rng_states: np.ndarray | None, dtype: str | None = None
                         ) -> np.ndarray:
        """Host-memory entry: ``logits`` is a [rows, vocab] CPU tensor or numpy array
        (uint16 payloads need ``dtype`` 'bf16', 'fp16' or 'u16'); ``rng_states`` a uint64 numpy
        array advanced in place. Copies in, samples, copies ids back, synchronises."""
        if isinstance(logits, torch.Tensor):
            code = _dtype_code(logits)
            if logits.dim() != 2 or logits.shape[1] != self.vocab_size or logits.stride(1) != 1:
                raise ValueError("expected contiguous [rows, vocab] host logits")
            ptr, rows, stride = logits.data_ptr(), logits.shape[0], logits.stride(0)
        else:
            a = logits
            if a.ndim != 2 or a.shape[1] != self.vocab_size or not a.flags.c_contiguous:
                raise ValueError("expected C-contiguous [rows, vocab] host logits")
            if a.dtype == np.float32:
                code = _lib.DTYPE_FLOAT
            elif a.dtype == np.float16:
                code = _lib.DTYPE_HALF
            elif a.dtype == np.uint16:
                code = {"bf16": _lib.DTYPE_BFLOAT16, "fp16": _lib.DTYPE_HALF, "u16": _lib.DTYPE_UINT16}[dtype or "bf16"]
            else:
                raise _lib.SamplerError(_lib.NOT_SUPPORTED, f"unsupported logits dtype {a.dtype}")
            ptr, rows, stride = a.ctypes.data, a.shape[0], a.shape[1]
        out = np.empty(rows, dtype=np.int64)
        sp = C.c_void_p(0)
        if rng_states is not None:
            if rng_states.dtype != np.uint64 or rng_states.shape != (rows,) or not rng_states.flags.c_contiguous:
                raise ValueError("rng_states must be a contiguous uint64 array, one per row")
            sp = C.c_void_p(rng_states.ctypes.data)
        _lib.check(_lib.load().etb200_sampler_sample_rows_host(
            self._h, C.c_void_p(ptr), code, rows, stride, sp, C.c_void_p(out.ctypes.data), self._stream()))
        return out


def sample_from_logits(logits_tensor: torch.Tensor, sampler: Sampler) -> int:
    """util.h:25-55: the vocabulary is the last dimension; a rank-3 [B, S, V] tensor is
    sampled at the last sequence position of batch 0."""
    vocab = logits_tensor.shape[-1]
    t = logits_tensor
    if t.dim() == 3:
        t = t[0, t.shape[1] - 1]
    else:
        t = t.reshape(-1)[:vocab]
    return sampler.sample(t)


def sample_all_from_logits(logits_tensor: torch.Tensor, sampler: Sampler,
                           rng_states: torch.Tensor | None = None) -> torch.Tensor:
    """Batched form of sample_from_logits: every batch row ([B, V], or the last position of
    each batch of [B, S, V]) is sampled; the reference reads batch 0 only (util.h:48-51)."""
    t = logits_tensor
    if t.dim() == 3:
        t = t[:, t.shape[1] - 1, :]
    elif t.dim() == 1:
        t = t[None, :]
    return sampler.sample_rows(t, rng_states)


def logits_to_token(logits_tensor: torch.Tensor, temperature: float = 0.0) -> int:
    """util.h:64-71: a temporary two-argument Sampler (top-p 0.9, wall-clock seed)."""
    s = Sampler(logits_tensor.shape[-1], temperature, device=logits_tensor.device)
    try:
        return sample_from_logits(logits_tensor, s)
    finally:
        s.close()
