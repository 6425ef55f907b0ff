"""Seeded synthetic GGUF blocks and activations (host side, numpy).

Counter-based: every 64-bit word is splitmix64(mix(seed) + index), so any
slice of a tensor can be generated independently and the device-side fill
kernels (csrc/fill.cu) produce the same bytes for the integer fields.

Distributions (the benchmark's workload definition):
  Q4_K block (144 B): d, dmin = fp16(|N(0,1)| * 2e-3); the 12 packed scale/min
      bytes and the 128 nibble bytes are uniform random bytes (which makes the
      sixteen 6-bit scales/mins uniform on 0..63 and the nibbles uniform 0..15).
  Q6_K block (210 B): ql[128], qh[64] uniform bytes; scales int8 uniform
      -32..31; d = fp16(|N(0,1)| * 1e-3).
  activations: fp32 N(0,1).
Block layouts: reference src/kernels.cu:20-32.
"""
from __future__ import annotations

import numpy as np

Q4K_BLOCK = 144
Q6K_BLOCK = 210
QK_K = 256

_GOLD = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)


def _mix(z: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = (z + _GOLD).astype(np.uint64)
        z = (z ^ (z >> np.uint64(30))) * _M1
        z = (z ^ (z >> np.uint64(27))) * _M2
        return z ^ (z >> np.uint64(31))


def words(seed: int, start: int, count: int) -> np.ndarray:
    """count 64-bit words of stream `seed`, beginning at word index `start`."""
    base = _mix(np.array([seed], dtype=np.uint64))[0]
    with np.errstate(over="ignore"):
        idx = np.arange(start, start + count, dtype=np.uint64) + base
    return _mix(idx)


def normals(seed: int, start: int, count: int) -> np.ndarray:
    """count N(0,1) float64 samples (Box-Muller; one 64-bit word per sample)."""
    w = words(seed ^ 0x5EEDFACE, start, count)
    u1 = ((w >> np.uint64(32)).astype(np.float64) + 1.0) * (1.0 / 4294967296.0)
    u2 = (w & np.uint64(0xFFFFFFFF)).astype(np.float64) * (1.0 / 4294967296.0)
    return np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)


def normal_f32(seed: int, n: int, scale: float = 1.0) -> np.ndarray:
    return (normals(seed, 0, n) * scale).astype(np.float32)


def normal_f16(seed: int, n: int, scale: float = 1.0) -> np.ndarray:
    return (normals(seed, 0, n) * scale).astype(np.float32).astype(np.float16)


def q4k_blocks(seed: int, n_blocks: int, first_block: int = 0) -> np.ndarray:
    """uint8 [n_blocks, 144]."""
    w = words(seed, first_block * 18, n_blocks * 18)
    blk = w.view(np.uint8).reshape(n_blocks, Q4K_BLOCK).copy()
    z = np.abs(normals(seed ^ 0xD0D0, first_block * 2, n_blocks * 2)) * 2e-3
    dd = z.astype(np.float32).astype(np.float16).view(np.uint16).reshape(n_blocks, 2)
    blk[:, 0:4] = dd.view(np.uint8).reshape(n_blocks, 4)
    return blk


def q6k_blocks(seed: int, n_blocks: int, first_block: int = 0) -> np.ndarray:
    """uint8 [n_blocks, 210]."""
    w = words(seed, first_block * 27, n_blocks * 27)
    blk = w.view(np.uint8).reshape(n_blocks, 216)[:, :Q6K_BLOCK].copy()
    blk[:, 192:208] = ((blk[:, 192:208] & 63).astype(np.int16) - 32).astype(np.int8).view(np.uint8)
    z = np.abs(normals(seed ^ 0xD0D0, first_block, n_blocks)) * 1e-3
    blk[:, 208:210] = z.astype(np.float32).astype(np.float16).view(np.uint8).reshape(n_blocks, 2)
    return blk


def q4k_matrix(seed: int, n_rows: int, n_cols: int) -> np.ndarray:
    """Row-major Q4_K tensor bytes, flat uint8 (rows contiguous, ceil(n_cols/256) blocks per row)."""
    bpr = (n_cols + QK_K - 1) // QK_K
    return q4k_blocks(seed, n_rows * bpr).reshape(-1)


def q6k_matrix(seed: int, n_rows: int, n_cols: int) -> np.ndarray:
    bpr = (n_cols + QK_K - 1) // QK_K
    return q6k_blocks(seed, n_rows * bpr).reshape(-1)


def q4k_row_bytes(n_cols: int) -> int:
    return (n_cols + QK_K - 1) // QK_K * Q4K_BLOCK


def q6k_row_bytes(n_cols: int) -> int:
    return (n_cols + QK_K - 1) // QK_K * Q6K_BLOCK


def expert_sizes(H: int, EFF: int, down_type: int = 14) -> tuple[int, int, int]:
    """(gate_sz, up_sz, down_sz) of one expert blob [gate][up][down]
    (reference src/forward.c:1127-1136)."""
    g = EFF * q4k_row_bytes(H)
    d = H * (q6k_row_bytes(EFF) if down_type == 14 else q4k_row_bytes(EFF))
    return g, g, d


def expert_blob(seed: int, H: int, EFF: int, down_type: int = 14) -> np.ndarray:
    g, u, d = expert_sizes(H, EFF, down_type)
    gate = q4k_matrix(seed * 3 + 0, EFF, H)
    up = q4k_matrix(seed * 3 + 1, EFF, H)
    down = q6k_matrix(seed * 3 + 2, H, EFF) if down_type == 14 else q4k_matrix(seed * 3 + 2, H, EFF)
    return np.concatenate([gate, up, down])


# ---- other GGUF block types (test inputs for the reference's Q8_0 / Q5_K / Q3_K matvecs) ----
Q8_0_BLOCK, Q5K_BLOCK, Q3K_BLOCK = 34, 176, 110


def q8_0_blocks(seed: int, n_blocks: int) -> np.ndarray:
    """uint8 [n_blocks, 34]: d = fp16(|N(0,1)| * 2e-3), 32 int8 weights uniform."""
    w = words(seed, 0, n_blocks * 5)
    blk = w.view(np.uint8).reshape(n_blocks, 40)[:, :Q8_0_BLOCK].copy()
    z = np.abs(normals(seed ^ 0xD0D0, 0, n_blocks)) * 2e-3
    blk[:, 0:2] = z.astype(np.float32).astype(np.float16).view(np.uint8).reshape(n_blocks, 2)
    return blk


def q5k_blocks(seed: int, n_blocks: int) -> np.ndarray:
    """uint8 [n_blocks, 176]: Q4_K's header and scale packing, 32 bytes of fifth bits, 128 bytes of nibbles."""
    w = words(seed, 0, n_blocks * 22)
    blk = w.view(np.uint8).reshape(n_blocks, Q5K_BLOCK).copy()
    z = np.abs(normals(seed ^ 0xD0D0, 0, n_blocks * 2)) * 2e-3
    blk[:, 0:4] = z.astype(np.float32).astype(np.float16).view(np.uint8).reshape(n_blocks, 4)
    return blk


def q3k_blocks(seed: int, n_blocks: int) -> np.ndarray:
    """uint8 [n_blocks, 110]: hmask 32, qs 64, scales 12, d = fp16(|N(0,1)| * 2e-3)."""
    w = words(seed, 0, n_blocks * 14)
    blk = w.view(np.uint8).reshape(n_blocks, 112)[:, :Q3K_BLOCK].copy()
    z = np.abs(normals(seed ^ 0xD0D0, 0, n_blocks)) * 2e-3
    blk[:, 108:110] = z.astype(np.float32).astype(np.float16).view(np.uint8).reshape(n_blocks, 2)
    return blk


TYPE_BLOCK = {0: (1, 4), 8: (32, Q8_0_BLOCK), 11: (QK_K, Q3K_BLOCK), 12: (QK_K, Q4K_BLOCK), 13: (QK_K, Q5K_BLOCK),
              14: (QK_K, Q6K_BLOCK)}  # GGUF type id -> (weights per block, bytes per block)


def typed_matrix(type_id: int, seed: int, n_rows: int, n_cols: int) -> np.ndarray:
    """Row-major tensor bytes of GGUF type 8 (Q8_0), 11 (Q3_K), 12 (Q4_K), 13 (Q5_K) or 14 (Q6_K)."""
    per = 32 if type_id == 8 else QK_K
    n = n_rows * ((n_cols + per - 1) // per)
    gen = {8: q8_0_blocks, 11: q3k_blocks, 12: q4k_blocks, 13: q5k_blocks, 14: q6k_blocks}[type_id]
    return gen(seed, n).reshape(-1)
