"""Seeded synthetic logits with the shapes and value distributions of the five benchmark
configurations of the sampling path. No dataset is involved; every row is a function of
``(config, row)`` alone, so a row is the same bytes whichever GPU or rank generates it.

Two generators with the same distributions:

* ``rows_numpy``  -- host generator (numpy Philox keyed by config and row). Parity tests
  use it so that the CPU oracle and the GPU see identical bytes.
* ``rows_torch``  -- device generator for benchmarks whose inputs must be born in HBM
  (up to 16.8 GB); it draws from torch's CUDA Philox generator seeded per (config, shard).

16-bit rows are returned as raw ``uint16`` payloads (numpy) or ``bfloat16``/``float16``
tensors (torch).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


@dataclass(frozen=True)
class Config:
    name: str
    rows: int
    vocab: int
    dtype: str  # 'fp32' | 'bf16' | 'fp16'
    kind: str  # 'normal' | 'zipf' | 'stress'
    temperature: float
    topp: float
    slope: float = 0.0
    sigma: float = 1.0
    note: str = ""


CONFIGS = {
    # 10 000 single rows, V=32000 fp32, N(0, 3^2); run at T=0, (T=0.8, topp=1.0), (T=0.8, topp=0.9)
    "c1": Config("c1", 10_000, 32_000, "fp32", "normal", 0.8, 0.9, sigma=3.0),
    # one row, V=128256 bf16, Zipf profile, 100 000 sequential draws (latency case)
    "c2": Config("c2", 1, 128_256, "bf16", "zipf", 0.7, 0.9, slope=1.1, sigma=0.5),
    # 256 rows x V=128256 bf16, Zipf profile, T=0.7, topp=0.95; second pass argmax
    "c3": Config("c3", 256, 128_256, "bf16", "zipf", 0.7, 0.95, slope=1.1, sigma=0.5),
    # 4096 rows x V=151936 fp16: first half peaked, second half flat; T=1, topp=0.9
    "c4": Config("c4", 4096, 151_936, "fp16", "stress", 1.0, 0.9),
    # 32768 rows x V=256000 bf16, Zipf slope 1.0, sigma 0.7, T=0.8, topp=0.9
    "c5": Config("c5", 32_768, 256_000, "bf16", "zipf", 0.8, 0.9, slope=1.0, sigma=0.7),
}

_CONFIG_ID = {"c1": 1, "c2": 2, "c3": 3, "c4": 4, "c5": 5}

BYTES = {"fp32": 4, "bf16": 2, "fp16": 2}


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16, returned as uint16 payloads."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounding = ((u >> 16) & 1) + np.uint32(0x7FFF)
    return ((u + rounding) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def to_f32(rows: np.ndarray, dtype: str) -> np.ndarray:
    """Exact upcast of a generated row block to fp32."""
    if dtype == "fp32":
        return np.asarray(rows, dtype=np.float32)
    if dtype == "bf16":
        return bf16_bits_to_f32(rows)
    return rows.view(np.float16).astype(np.float32)


def _row_values(cfg: Config, cid: int, row: int, vocab: int) -> np.ndarray:
    g = np.random.Generator(np.random.Philox(key=[cid, row]))
    if cfg.kind == "normal":
        return (cfg.sigma * g.standard_normal(vocab, dtype=np.float32)).astype(np.float32)
    if cfg.kind == "zipf":
        rank = g.permutation(vocab)
        noise = g.standard_normal(vocab, dtype=np.float32)
        return (-cfg.slope * np.log(rank.astype(np.float32) + 1.0)
                + cfg.sigma * noise).astype(np.float32)
    # stress: the first half of the configuration's rows is peaked, the second half flat
    if row < cfg.rows // 2:
        v = g.standard_normal(vocab, dtype=np.float32)
        hot = g.choice(vocab, size=5, replace=False)
        v[hot[0]] = 12.0
        v[hot[1:]] = 8.0
        return v
    return (0.05 * g.standard_normal(vocab, dtype=np.float32)).astype(np.float32)


def rows_numpy(name: str, row_ids, vocab: int | None = None) -> np.ndarray:
    """Rows ``row_ids`` of configuration ``name``: fp32 array, or uint16 payloads for 16-bit
    dtypes. ``vocab`` overrides the vocabulary size (small parity cases)."""
    cfg = CONFIGS[name]
    cid = _CONFIG_ID[name]
    vocab = vocab or cfg.vocab
    out = []
    for r in row_ids:
        v = _row_values(cfg, cid, int(r), vocab)
        if cfg.dtype == "bf16":
            v = f32_to_bf16_bits(v)
        elif cfg.dtype == "fp16":
            v = v.astype(np.float16).view(np.uint16)
        out.append(v)
    return np.stack(out)


def rows_torch(name: str, row_start: int, rows: int, device, vocab: int | None = None,
               chunk: int = 1024):
    """``rows`` rows of configuration ``name`` generated on ``device`` (same distributions
    as ``rows_numpy``, different bytes). Generated in chunks to bound scratch memory."""
    import torch

    cfg = CONFIGS[name]
    cid = _CONFIG_ID[name]
    vocab = vocab or cfg.vocab
    tdtype = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}[cfg.dtype]
    out = torch.empty((rows, vocab), dtype=tdtype, device=device)
    gen = torch.Generator(device=device)
    for c0 in range(0, rows, chunk):
        n = min(chunk, rows - c0)
        gen.manual_seed((cid << 40) + row_start + c0)
        if cfg.kind == "normal":
            v = cfg.sigma * torch.randn((n, vocab), generator=gen, device=device)
        elif cfg.kind == "zipf":
            # a uniformly random permutation per row = the argsort of i.i.d. uniforms
            rank = torch.rand((n, vocab), generator=gen, device=device).argsort(dim=1)
            v = -cfg.slope * torch.log(rank.to(torch.float32) + 1.0)
            del rank
            v += cfg.sigma * torch.randn((n, vocab), generator=gen, device=device)
        else:
            v = torch.randn((n, vocab), generator=gen, device=device)
            ridx = torch.arange(row_start + c0, row_start + c0 + n, device=device)
            flat = ridx >= cfg.rows // 2
            v[flat] *= 0.05
            hot = torch.rand((n, vocab), generator=gen, device=device).topk(5, dim=1).indices
            peaked = ~flat
            vals = torch.tensor([12.0, 8.0, 8.0, 8.0, 8.0], device=device).expand(n, 5)
            pv = v[peaked]
            pv.scatter_(1, hot[peaked], vals[peaked])
            v[peaked] = pv
        out[c0:c0 + n] = v.to(tdtype)
        del v
    return out
