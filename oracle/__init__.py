"""TEST INFRASTRUCTURE, not product code: ctypes bindings for the CPU oracles.

Two checkers live here, and only ``tests/``, ``__graft_entry__.smoke()`` and the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` may import this package:

* ``Restatement`` -- ``oracle/sampler_oracle.c``, a plain-C restatement of
  ``extension/llm/sampler/sampler.cpp`` (float instantiation, tie order pinned to
  "probability descending, index ascending").
* ``Reference`` -- the reference's own, unmodified ``sampler.cpp`` compiled by
  ``oracle/Makefile`` into ``oracle/_ref`` (``stable=False``: shipped ``std::sort`` tie
  order; ``stable=True``: the same source with ``std::stable_sort`` substituted by a
  forced include). Present only where the Makefile has been run against a reference
  checkout; the prebuilt libraries travel with the working tree.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

HALF, FLOAT, BFLOAT16, UINT16 = 5, 6, 15, 27  # ScalarType numbering of the reference

_NP_TO_CODE = {np.dtype(np.float32): FLOAT}


def build(reference: str | None = None) -> None:
    """Compile the C restatement, and the reference libraries when a checkout exists."""
    cmd = ["make", "-s", "-f", os.path.join(HERE, "Makefile"), "all"]
    if reference:
        cmd.append(f"REF={reference}")
    subprocess.run(cmd, check=True, cwd=HERE)


def dtype_code(arr: np.ndarray, dtype: str | None) -> int:
    """``dtype`` names what the uint16 payload means: 'bf16', 'fp16' or 'u16'."""
    if arr.dtype == np.float32:
        return FLOAT
    if arr.dtype == np.float16:
        return HALF
    if arr.dtype == np.uint16:
        return {"bf16": BFLOAT16, "fp16": HALF, "u16": UINT16}[dtype or "bf16"]
    raise TypeError(f"unsupported array dtype {arr.dtype}")


def _as_rows(logits: np.ndarray):
    a = np.ascontiguousarray(logits)
    if a.ndim == 1:
        a = a[None, :]
    assert a.ndim == 2
    return a


class Restatement:
    """The C restatement (``oracle/_build/liboracle_sampler.so``)."""

    def __init__(self):
        path = os.path.join(HERE, "_build", "liboracle_sampler.so")
        if not os.path.exists(path):
            build()
        self.lib = C.CDLL(path)
        L = self.lib
        L.oracle_random_f32.restype = C.c_float
        L.oracle_random_f32.argtypes = [C.POINTER(C.c_uint64)]
        L.oracle_random_u32.restype = C.c_uint32
        L.oracle_random_u32.argtypes = [C.POINTER(C.c_uint64)]
        L.oracle_sample_rows.restype = C.c_double
        L.oracle_sample_rows.argtypes = [
            C.c_void_p, C.c_int, C.c_int64, C.c_int32, C.c_int64, C.c_float, C.c_float,
            C.c_int32, C.c_void_p, C.c_void_p, C.c_int, C.POINTER(C.c_double)]
        L.oracle_sample_sequence_f32.restype = None
        L.oracle_sample_sequence_f32.argtypes = [
            C.c_void_p, C.c_int32, C.c_float, C.c_float, C.c_uint64, C.c_int64, C.c_void_p]
        L.oracle_row_details_f32.restype = None
        L.oracle_row_details_f32.argtypes = [
            C.c_void_p, C.c_int32, C.c_float, C.c_float, C.c_uint64, C.c_void_p,
            C.POINTER(C.c_float), C.POINTER(C.c_int32), C.POINTER(C.c_int32),
            C.POINTER(C.c_float), C.POINTER(C.c_int32)]
        L.oracle_bf16_to_f32.restype = C.c_float
        L.oracle_bf16_to_f32.argtypes = [C.c_uint16]
        L.oracle_f16_to_f32.restype = C.c_float
        L.oracle_f16_to_f32.argtypes = [C.c_uint16]

    def coins(self, seed: int, n: int):
        """First n coins and states of the xorshift64* generator started at ``seed``."""
        st = C.c_uint64(seed)
        out, states = [], []
        for _ in range(n):
            out.append(float(self.lib.oracle_random_f32(C.byref(st))))
            states.append(int(st.value))
        return out, states

    def sample_rows(self, logits, temperature, topp, seeds, dtype=None, topk=0,
                    threads=1, return_states=False, timing=None):
        a = _as_rows(logits)
        rows, vocab = a.shape
        code = dtype_code(a, dtype)
        states = np.ascontiguousarray(np.asarray(seeds, dtype=np.uint64).copy())
        assert states.shape == (rows,)
        out = np.empty(rows, dtype=np.int32)
        wall = C.c_double(0)
        cpu = self.lib.oracle_sample_rows(
            a.ctypes.data, code, rows, vocab, vocab, temperature, topp, topk,
            states.ctypes.data, out.ctypes.data, threads, C.byref(wall))
        if timing is not None:
            timing["cpu_seconds"] = cpu
            timing["wall_seconds"] = wall.value
        return (out, states) if return_states else out

    def sample_sequence(self, row_f32, temperature, topp, seed, ndraws):
        a = np.ascontiguousarray(row_f32, dtype=np.float32)
        out = np.empty(ndraws, dtype=np.int32)
        self.lib.oracle_sample_sequence_f32(
            a.ctypes.data, a.shape[0], temperature, topp, seed, ndraws, out.ctypes.data)
        return out

    def row_details(self, row_f32, temperature, topp, seed):
        a = np.ascontiguousarray(row_f32, dtype=np.float32)
        probs = np.empty_like(a)
        coin, cum = C.c_float(0), C.c_float(0)
        n0, last, tok = C.c_int32(0), C.c_int32(0), C.c_int32(0)
        self.lib.oracle_row_details_f32(
            a.ctypes.data, a.shape[0], temperature, topp, seed, probs.ctypes.data,
            C.byref(coin), C.byref(n0), C.byref(last), C.byref(cum), C.byref(tok))
        return dict(probs=probs, coin=coin.value, n0=n0.value, last_idx=last.value,
                    cum=cum.value, token=tok.value)


class Reference:
    """The reference's own sampler.cpp, compiled unmodified (``oracle/_ref``)."""

    def __init__(self, stable: bool = True):
        name = "libref_sampler_stable.so" if stable else "libref_sampler.so"
        path = os.path.join(HERE, "_ref", name)
        if not os.path.exists(path):
            raise FileNotFoundError(
                f"{path} is missing: run `make -f oracle/Makefile ref` where the reference "
                "checkout is available")
        self.lib = C.CDLL(path)
        L = self.lib
        L.ref_sample_rows.restype = C.c_double
        L.ref_sample_rows.argtypes = [
            C.c_void_p, C.c_int, C.c_int, C.c_int64, C.c_int32, C.c_int64, C.c_float,
            C.c_float, C.c_int32, C.c_void_p, C.c_void_p, C.c_int, C.POINTER(C.c_double)]
        L.ref_sample_sequence.restype = None
        L.ref_sample_sequence.argtypes = [
            C.c_void_p, C.c_int, C.c_int, C.c_int32, C.c_float, C.c_float, C.c_uint64,
            C.c_int64, C.c_void_p]

    @staticmethod
    def available(stable: bool = True) -> bool:
        name = "libref_sampler_stable.so" if stable else "libref_sampler.so"
        return os.path.exists(os.path.join(HERE, "_ref", name))

    def sample_rows(self, logits, temperature, topp, seeds, dtype=None, topk=0,
                    threads=1, native=False, timing=None):
        """``native=True`` runs the reference's own sample<Half>/sample<BFloat16>."""
        a = _as_rows(logits)
        rows, vocab = a.shape
        code = dtype_code(a, dtype)
        seeds = np.ascontiguousarray(np.asarray(seeds, dtype=np.uint64))
        out = np.empty(rows, dtype=np.int32)
        wall = C.c_double(0)
        cpu = self.lib.ref_sample_rows(
            a.ctypes.data, code, 1 if native else 0, rows, vocab, vocab, temperature,
            topp, topk, seeds.ctypes.data, out.ctypes.data, threads, C.byref(wall))
        if timing is not None:
            timing["cpu_seconds"] = cpu
            timing["wall_seconds"] = wall.value
        return out

    def sample_sequence(self, row, temperature, topp, seed, ndraws, dtype=None):
        a = np.ascontiguousarray(row)
        code = dtype_code(a, dtype)
        out = np.empty(ndraws, dtype=np.int32)
        self.lib.ref_sample_sequence(
            a.ctypes.data, code, 0, a.shape[0], temperature, topp, seed, ndraws,
            out.ctypes.data)
        return out
