"""Seeded synthetic inputs for benchmarks and examples: N(0, sigma) values stored as bf16.

The reference has no random-number generator in its Tensor API (inputs are made on the host and
fed with `from_slice` / `from_raw_bytes`, tensor/src/data.rs:23-139), so inputs are drawn with numpy
and rounded to bf16 (top 16 bits of the f32, round to nearest even: dtype/src/lib.rs:300) here.
Plain numpy; nothing in this module computes on behalf of a kernel.
"""
from __future__ import annotations

import numpy as np


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """f32 -> bf16 bit patterns (uint16), round to nearest even; NaN stays NaN."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)
    nan = (u & np.uint32(0x7FFFFFFF)) > np.uint32(0x7F800000)
    if nan.any():
        r[nan] = ((u[nan] >> np.uint32(16)) | np.uint32(0x40)).astype(np.uint16)
    return r


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def normal_bf16_bits(rng: np.random.Generator, shape, sigma: float = 1.0) -> np.ndarray:
    """N(0, sigma) drawn as f32 from `rng`, rounded to bf16 bit patterns."""
    return f32_to_bf16_bits(rng.standard_normal(size=shape, dtype=np.float32) * np.float32(sigma))


def fill_normal_bf16(dev, buf, n: int, sigma: float, seed: int, chunk: int = 1 << 24, keep_host: bool = False, tile: bool = False):
    """Fills the first n bf16 elements of device buffer `buf` with N(0, sigma) drawn from `seed`, chunk by
    chunk (the host never holds more than one chunk unless keep_host).  With tile=True one chunk is drawn
    and repeated -- enough for timing runs whose results nobody checks.  Returns the host copy or None."""
    rng = np.random.default_rng(seed)
    host = np.empty(n, dtype=np.uint16) if keep_host else None
    off, first = 0, None
    while off < n:
        m = min(chunk, n - off)
        if tile and first is not None:
            bits = first[:m]
        else:
            bits = normal_bf16_bits(rng, m, sigma)
            if tile:
                first = bits
        buf.view(off * 2, m * 2).copyin(bits)
        if host is not None:
            host[off:off + m] = bits
        off += m
    dev.sync()
    return host


# ---------------------------------------------------------------------------------------------------------
# Chunk-seeded tensors: every chunk of a tensor has its own generator, seeded by (seed, chunk index), so that a
# process can draw exactly the part it owns -- and any other part later, to check what arrived there -- without
# drawing the rest.
# ---------------------------------------------------------------------------------------------------------
def normal_chunk_bf16(seed: int, index: int, shape, sigma: float = 1.0) -> np.ndarray:
    """Chunk `index` of the tensor drawn from `seed`: N(0, sigma) as bf16 bit patterns of the given shape."""
    return normal_bf16_bits(np.random.default_rng([int(seed), int(index)]), shape, sigma)


ROW_CHUNK = 64          # rows per chunk of a row-chunked matrix
COL_PANEL = 128         # columns per panel of a column-panelled matrix


def matrix_rows_bf16(seed: int, K: int, row0: int, nrows: int, sigma: float = 1.0) -> np.ndarray:
    """Rows [row0, row0 + nrows) of a row-chunked [M, K] matrix (chunks of ROW_CHUNK rows)."""
    out = np.empty((nrows, K), np.uint16)
    r = row0
    while r < row0 + nrows:
        c = r // ROW_CHUNK
        chunk = normal_chunk_bf16(seed, c, (ROW_CHUNK, K), sigma)
        lo, hi = r - c * ROW_CHUNK, min(ROW_CHUNK, row0 + nrows - c * ROW_CHUNK)
        out[r - row0:r - row0 + hi - lo] = chunk[lo:hi]
        r += hi - lo
    return out


def matrix_panels_bf16(seed: int, K: int, col0: int, ncols: int, sigma: float = 1.0) -> np.ndarray:
    """Columns [col0, col0 + ncols) of a column-panelled [K, N] matrix (panels of COL_PANEL columns), as a
    contiguous [K, ncols] array.  col0 and ncols are multiples of COL_PANEL."""
    assert col0 % COL_PANEL == 0 and ncols % COL_PANEL == 0
    out = np.empty((K, ncols), np.uint16)
    for j in range(ncols // COL_PANEL):
        out[:, j * COL_PANEL:(j + 1) * COL_PANEL] = normal_chunk_bf16(seed, col0 // COL_PANEL + j, (K, COL_PANEL), sigma)
    return out


def head_slice_bf16(seed: int, H: int, b: int, h: int, S: int, D: int, sigma: float = 1.0) -> np.ndarray:
    """The [S, D] slice of (batch b, head h) of a [B, H, S, D] tensor chunked per (batch, head)."""
    return normal_chunk_bf16(seed, b * H + h, (S, D), sigma)
