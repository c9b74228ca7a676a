"""Seeded synthetic inputs for the benchmark configurations (numpy side).

The Q4_0 / Q8_0 byte streams restate csrc/tlc_synth.cuh so that weights
generated on the host and on the device are identical; activations, norm
weights and embeddings are only ever generated here.

Distributions:
  Q4_0 block: d = f16(U[0.002, 0.02]), 16 bytes of packed nibbles ~ U{0..15}
  Q8_0 block: same d, 32 int8 ~ U{-127..127}
  activations: f16(N(0,1)); norm weights f16(1 + N(0, 0.02));
  embeddings f16(N(0,1) * 0.02); token ids ~ U[0, vocab)
"""
from __future__ import annotations

import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def mix64(z: np.ndarray) -> np.ndarray:
    """The finaliser of tlc_mix64 on uint64 arrays (wrap-around arithmetic)."""
    z = np.asarray(z, dtype=np.uint64)
    with np.errstate(over="ignore"):
        z = z + np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def tensor_id(name: str) -> int:
    """FNV-1a 64 of the tensor name: the id fed to the generator."""
    h = 0xCBF29CE484222325
    for b in name.encode():
        h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


def key(seed: int, tid: int) -> np.uint64:
    return mix64(mix64(np.uint64(seed)) ^ np.uint64(tid))


def _r(k: np.uint64, idx: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        return mix64(np.uint64(k) + idx.astype(np.uint64))


def _scale_bits(r: np.ndarray, scale_log2: int = 0) -> np.ndarray:
    v = (np.uint64(2000) + r % np.uint64(18001)).astype(np.float32)
    d = (v * np.float32(1e-6)).astype(np.float32)
    d = np.ldexp(d, scale_log2).astype(np.float32)  # exact power-of-two factor
    return d.astype(np.float16).view(np.uint16)


def q4_0_blocks(seed: int, tid: int, n_rows: int, n_cols: int, row0: int = 0, rows: int | None = None,
                scale_log2: int = 0) -> np.ndarray:
    """uint8 [rows, n_cols/32, 18]: the blocks of rows [row0, row0+rows) of the full tensor."""
    assert n_cols % 32 == 0
    rows = n_rows - row0 if rows is None else rows
    bpr = n_cols // 32
    b = (np.arange(rows * bpr, dtype=np.uint64) + np.uint64(row0 * bpr))
    k = key(seed, tid)
    with np.errstate(over="ignore"):
        d = _scale_bits(_r(k, np.uint64(3) * b), scale_log2)
        r1 = _r(k, np.uint64(3) * b + np.uint64(1))
        r2 = _r(k, np.uint64(3) * b + np.uint64(2))
    out = np.empty((rows * bpr, 18), np.uint8)
    out[:, 0:2] = d.astype("<u2").view(np.uint8).reshape(-1, 2)
    out[:, 2:10] = r1.astype("<u8").view(np.uint8).reshape(-1, 8)
    out[:, 10:18] = r2.astype("<u8").view(np.uint8).reshape(-1, 8)
    return out.reshape(rows, bpr, 18)


def q8_0_blocks(seed: int, tid: int, n_rows: int, n_cols: int, row0: int = 0, rows: int | None = None,
                scale_log2: int = 0) -> np.ndarray:
    """uint8 [rows, n_cols/32, 34]."""
    assert n_cols % 32 == 0
    rows = n_rows - row0 if rows is None else rows
    bpr = n_cols // 32
    b = (np.arange(rows * bpr, dtype=np.uint64) + np.uint64(row0 * bpr))
    k = key(seed, tid)
    out = np.empty((rows * bpr, 34), np.uint8)
    with np.errstate(over="ignore"):
        out[:, 0:2] = _scale_bits(_r(k, np.uint64(9) * b), scale_log2).astype("<u2").view(np.uint8).reshape(-1, 2)
        for j in range(8):
            r = _r(k, np.uint64(9) * b + np.uint64(1 + j))
            u = r.astype("<u8").view("<u2").reshape(-1, 4).astype(np.int64)
            out[:, 2 + 4 * j:6 + 4 * j] = (((u * 255) >> 16) - 127).astype(np.int8).view(np.uint8)
    return out.reshape(rows, bpr, 34)


def blocks(qtype: int, seed: int, tid: int, n_rows: int, n_cols: int, **kw) -> np.ndarray:
    if qtype == 2:
        return q4_0_blocks(seed, tid, n_rows, n_cols, **kw)
    if qtype == 8:
        return q8_0_blocks(seed, tid, n_rows, n_cols, **kw)
    raise ValueError(f"no synthetic generator for ggml type {qtype}")


def _uniform01(k: np.uint64, idx: np.ndarray) -> np.ndarray:
    return ((_r(k, idx) >> np.uint64(11)).astype(np.float64) + 0.5) / float(1 << 53)


def normal(seed: int, tid: int, shape, mean: float = 0.0, std: float = 1.0) -> np.ndarray:
    """float64 N(mean, std) by Box-Muller over the counter-based uniforms."""
    n = int(np.prod(shape))
    i = np.arange(n, dtype=np.uint64)
    k = key(seed, tid)
    with np.errstate(over="ignore"):
        u1 = _uniform01(k, np.uint64(2) * i)
        u2 = _uniform01(k, np.uint64(2) * i + np.uint64(1))
    z = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)
    return (mean + std * z).reshape(shape)


def activations(seed: int, name: str, shape) -> np.ndarray:
    return normal(seed, tensor_id(name), shape).astype(np.float16)


def norm_weight(seed: int, name: str, d: int) -> np.ndarray:
    return normal(seed, tensor_id(name), (d,), 1.0, 0.02).astype(np.float16)


def embedding_table(seed: int, name: str, vocab: int, d: int) -> np.ndarray:
    return normal(seed, tensor_id(name), (vocab, d), 0.0, 0.02).astype(np.float16)


def token_ids(seed: int, name: str, n: int, vocab: int) -> np.ndarray:
    k = key(seed, tensor_id(name))
    return (_r(k, np.arange(n, dtype=np.uint64)) % np.uint64(vocab)).astype(np.int32)
