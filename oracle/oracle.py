"""CPU oracle for morok's dense hot path -- TEST INFRASTRUCTURE ONLY.

Loads ``libmorok_oracle.so`` (the C restatement in ``morok_oracle.c``) through ctypes and adds
(1) an independent numpy mirror of every function, used only to cross-check the C code, (2) the
seeded input generators both the oracle and the GPU path consume, and (3) the decoder layer of
the headline configs composed from the C functions in the order the reference's Tensor API
implies.

Nothing in the shipped package imports this module.  Only tests, the smoke check and the
benchmark's CPU-baseline / reference arm may.

Parity status: pinned against the reference's own known-answer tests for f32 matmul, rms_norm,
rotary embedding and causal attention; "parity unpinned" for bf16 GEMM, bf16 attention at
scale, GQA and the decoder layer (the reference has no numeric tests there).
"""
from __future__ import annotations

import ctypes as C
import math
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build(native: bool = False) -> str:
    """Compile the C oracle with the committed Makefile; returns the library path."""
    target = "native" if native else "all"
    subprocess.run(["make", "-s", "-C", _HERE, target], check=True)
    return os.path.join(_HERE, "libmorok_oracle_native.so" if native else "libmorok_oracle.so")


def lib(native: bool = False) -> C.CDLL:
    """Load (building if needed) the oracle library."""
    global _LIB
    if native:
        return _bind(C.CDLL(build(native=True)))
    if _LIB is None:
        path = os.path.join(_HERE, "libmorok_oracle.so")
        if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(os.path.join(_HERE, "morok_oracle.c")):
            build()
        _LIB = _bind(C.CDLL(path))
    return _LIB


def _bind(l: C.CDLL) -> C.CDLL:
    p, i64, f32, i32, sz = C.c_void_p, C.c_int64, C.c_float, C.c_int, C.c_size_t
    l.orc_matmul_f32.argtypes = [p, p, p, i64, i64, i64, i64, i64, i64, i32]
    l.orc_matmul_f32.restype = i32
    l.orc_matmul_bf16.argtypes = [p, p, p, p, i64, i64, i64, i32]
    l.orc_matmul_bf16.restype = i32
    l.orc_sdpa_f32.argtypes = [p, p, p, p, p, i64, i64, i64, i64, i64, i64, i64, f32, i32, p, f32]
    l.orc_sdpa_f32.restype = i32
    l.orc_sdpa_f32_offset.argtypes = [p, p, p, p, p, i64, i64, i64, i64, i64, i64, i64, f32, i32, i64, p, f32]
    l.orc_sdpa_f32_offset.restype = i32
    l.orc_rms_norm_f32.argtypes = [p, p, p, i64, i64, f32]
    l.orc_rms_norm_f32.restype = None
    l.orc_rope_f32.argtypes = [p, p, p, p, i64, i64, i64, i64, i32]
    l.orc_rope_f32.restype = None
    for name in ("orc_sigmoid_f32", "orc_silu_f32"):
        getattr(l, name).argtypes = [p, p, sz]
        getattr(l, name).restype = None
    for name in ("orc_swiglu_f32", "orc_add_f32"):
        getattr(l, name).argtypes = [p, p, p, sz]
        getattr(l, name).restype = None
    l.orc_bf16_to_f32.argtypes = [p, p, sz]
    l.orc_f32_to_bf16.argtypes = [p, p, sz]
    l.orc_round_bf16_inplace.argtypes = [p, sz]
    l.orc_f8_to_f32.argtypes = [p, p, sz, i32]
    l.orc_f32_to_f8.argtypes = [p, p, sz, i32]
    l.orc_thread_count.argtypes = [i64, i64, i32]
    l.orc_thread_count.restype = i32
    l.orc_max_threads.restype = i32
    l.orc_set_threads.argtypes = [i32]
    l.orc_set_threads.restype = i32
    return l


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f32c(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


# ---------------------------------------------------------------------------------------------
# bf16 helpers (bf16 values travel as uint16 bit patterns)
# ---------------------------------------------------------------------------------------------
def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bit patterns (uint16)."""
    x = _f32c(x)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().orc_f32_to_bf16(_ptr(x), _ptr(out), x.size)
    return out


def bf16_to_f32(b: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(b, dtype=np.uint16)
    return (b.astype(np.uint32) << 16).view(np.float32)


def round_bf16(x: np.ndarray) -> np.ndarray:
    """f32 -> bf16 -> f32."""
    return bf16_to_f32(f32_to_bf16(x))


def np_f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """numpy mirror of the RNE rounding (cross-check for the C helper)."""
    u = _f32c(x).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r[nan] = ((u[nan] >> 16) | 0x40).astype(np.uint16)
    return r


# ---------------------------------------------------------------------------------------------
# 8-bit floats (values travel as uint8 bit patterns; kind "e4m3" or "e5m2")
# ---------------------------------------------------------------------------------------------
def f32_to_f8(x: np.ndarray, kind: str = "e4m3") -> np.ndarray:
    """f32 -> 8-bit float codes: round to nearest even, saturating to the largest finite value."""
    x = _f32c(x)
    out = np.empty(x.shape, dtype=np.uint8)
    lib().orc_f32_to_f8(_ptr(x), _ptr(out), x.size, int(kind == "e5m2"))
    return out


def f8_to_f32(b: np.ndarray, kind: str = "e4m3") -> np.ndarray:
    b = np.ascontiguousarray(b, dtype=np.uint8)
    out = np.empty(b.shape, dtype=np.float32)
    lib().orc_f8_to_f32(_ptr(b), _ptr(out), b.size, int(kind == "e5m2"))
    return out


def np_f8_table(kind: str = "e4m3") -> np.ndarray:
    """All 256 codes decoded with plain arithmetic (cross-check for the C helper)."""
    codes = np.arange(256)
    sign = np.where(codes >> 7, -1.0, 1.0)
    if kind == "e5m2":
        e, m = (codes >> 2) & 31, codes & 3
        v = np.where(e == 0, m * 2.0 ** -16, (1 + m / 4.0) * 2.0 ** (e.astype(np.float64) - 15))
        v = np.where(e == 31, np.where(m == 0, np.inf, np.nan), v)
    else:
        e, m = (codes >> 3) & 15, codes & 7
        v = np.where(e == 0, m * 2.0 ** -9, (1 + m / 8.0) * 2.0 ** (e.astype(np.float64) - 7))
        v = np.where((e == 15) & (m == 7), np.nan, v)
    return (sign * v).astype(np.float32)


def np_f32_to_f8(x: np.ndarray, kind: str = "e4m3") -> np.ndarray:
    """numpy mirror of the encoder: nearest finite code by search, ties to the even code."""
    max_code = 0x7B if kind == "e5m2" else 0x7E
    tab = np_f8_table(kind)[: max_code + 1].astype(np.float64)
    x = _f32c(x)
    a = np.abs(x.astype(np.float64))
    lo = np.clip(np.searchsorted(tab, a, side="right") - 1, 0, max_code - 1)
    dl, dh = a - tab[lo], tab[lo + 1] - a
    code = np.where(dl < dh, lo, np.where(dh < dl, lo + 1, np.where(lo & 1, lo + 1, lo)))
    code = np.where(a >= tab[max_code], max_code, code)
    out = (code | np.where(np.signbit(x), 0x80, 0)).astype(np.uint8)
    out[np.isnan(x)] = 0x7F
    return out


# ---------------------------------------------------------------------------------------------
# C oracle wrappers
# ---------------------------------------------------------------------------------------------
def matmul_f32(a: np.ndarray, b: np.ndarray, nthreads: int = 0, native: bool = False) -> np.ndarray:
    """C = A @ B in f32 (tensor/src/matmul.rs:82-110).  1-D operands follow the reference's rules:
    [K]@[K,N] -> [N], [M,K]@[K] -> [M], [K]@[K] -> scalar."""
    a, b = _f32c(a), _f32c(b)
    a2 = a.reshape(1, -1) if a.ndim == 1 else a
    b2 = b.reshape(-1, 1) if b.ndim == 1 else b
    if a2.ndim > 2 or b2.ndim > 2:
        lead = np.broadcast_shapes(a2.shape[:-2], b2.shape[:-2])
        ab = np.broadcast_to(a2, lead + a2.shape[-2:]).reshape((-1,) + a2.shape[-2:])
        bb = np.broadcast_to(b2, lead + b2.shape[-2:]).reshape((-1,) + b2.shape[-2:])
        out = np.stack([matmul_f32(x, y, nthreads, native) for x, y in zip(ab, bb)])
        return out.reshape(lead + out.shape[-2:])
    (m, k), (k2, n) = a2.shape, b2.shape
    if k != k2:
        raise ValueError(f"dot shape mismatch: {a.shape} vs {b.shape}")
    c = np.empty((m, n), dtype=np.float32)
    r = lib(native).orc_matmul_f32(_ptr(a2), _ptr(b2), _ptr(c), m, n, k, k, n, n, nthreads)
    if r < 0:
        raise RuntimeError(f"orc_matmul_f32 failed: {r}")
    if a.ndim == 1 and b.ndim == 1:
        return c.reshape(())
    if a.ndim == 1:
        return c.reshape(n)
    if b.ndim == 1:
        return c.reshape(m)
    return c


def matmul_bf16(a_bits: np.ndarray, b_bits: np.ndarray, nthreads: int = 0):
    """bf16 storage evaluated in f32; returns (f32 result, bf16-rounded result bits)."""
    a_bits = np.ascontiguousarray(a_bits, dtype=np.uint16)
    b_bits = np.ascontiguousarray(b_bits, dtype=np.uint16)
    (m, k), (k2, n) = a_bits.shape, b_bits.shape
    assert k == k2
    c = np.empty((m, n), dtype=np.float32)
    cb = np.empty((m, n), dtype=np.uint16)
    r = lib().orc_matmul_bf16(_ptr(a_bits), _ptr(b_bits), _ptr(c), _ptr(cb), m, n, k, nthreads)
    if r < 0:
        raise RuntimeError(f"orc_matmul_bf16 failed: {r}")
    return c, cb


def sdpa_f32(q, k, v, scale=None, causal=False, mask=None, softcap=0.0, return_lse=False, causal_offset=0):
    """scaled_dot_product_attention in f32 (tensor/src/transformer.rs:78-137).
    q [B,H,Sq,D], k [B,Hkv,Sk,D], v [B,Hkv,Sk,Dv].  causal keeps col <= row + causal_offset
    (0: tril(0) of the Tensor method; past_seq_len: onnx/src/registry/transformer.rs:155-162)."""
    q, k, v = _f32c(q), _f32c(k), _f32c(v)
    B, H, Sq, D = q.shape
    _, Hkv, Sk, _ = k.shape
    Dv = v.shape[-1]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    o = np.empty((B, H, Sq, Dv), dtype=np.float32)
    lse = np.empty((B, H, Sq), dtype=np.float32) if return_lse else None
    m = None if mask is None else _f32c(mask)
    r = lib().orc_sdpa_f32_offset(_ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(lse), B, H, Hkv, Sq, Sk, D, Dv,
                                  float(scale), int(bool(causal)), int(causal_offset), _ptr(m), float(softcap or 0.0))
    if r != 0:
        raise RuntimeError(f"orc_sdpa_f32 failed: {r}")
    return (o, lse) if return_lse else o


def rms_norm_f32(x, eps=1e-5, gain=None):
    x = _f32c(x)
    cols = x.shape[-1]
    y = np.empty_like(x)
    g = None if gain is None else _f32c(gain)
    lib().orc_rms_norm_f32(_ptr(x), _ptr(g), _ptr(y), x.size // cols, cols, float(eps))
    return y


def rope_f32(x, cos, sin, interleaved=False, row_div=1):
    """x [..., D]; cos/sin [rows_cs, D/2]; flattened row r of x uses table row (r // row_div) % rows_cs."""
    x, cos, sin = _f32c(x), _f32c(cos), _f32c(sin)
    d = x.shape[-1]
    cos2, sin2 = cos.reshape(-1, d // 2), sin.reshape(-1, d // 2)
    y = np.empty_like(x)
    lib().orc_rope_f32(_ptr(x), _ptr(cos2), _ptr(sin2), _ptr(y), x.size // d, d, cos2.shape[0], row_div,
                       int(bool(interleaved)))
    return y


def silu_f32(x):
    x = _f32c(x)
    y = np.empty_like(x)
    lib().orc_silu_f32(_ptr(x), _ptr(y), x.size)
    return y


def sigmoid_f32(x):
    x = _f32c(x)
    y = np.empty_like(x)
    lib().orc_sigmoid_f32(_ptr(x), _ptr(y), x.size)
    return y


def swiglu_f32(gate, up):
    gate, up = _f32c(gate), _f32c(up)
    y = np.empty_like(gate)
    lib().orc_swiglu_f32(_ptr(gate), _ptr(up), _ptr(y), gate.size)
    return y


# ---------------------------------------------------------------------------------------------
# numpy mirror (independent restatement; cross-checks the C oracle, float64 where it helps)
# ---------------------------------------------------------------------------------------------
def np_matmul(a, b):
    return np.matmul(np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64))


def np_sdpa(q, k, v, scale=None, causal=False, mask=None, softcap=0.0, causal_offset=0):
    q, k, v = (np.asarray(t, dtype=np.float64) for t in (q, k, v))
    B, H, Sq, D = q.shape
    Hkv, Sk = k.shape[1], k.shape[2]
    if Hkv != H:  # unsqueeze(2).expand.reshape == repeat-interleave (onnx/src/registry/transformer.rs:80-103)
        k = np.repeat(k, H // Hkv, axis=1)
        v = np.repeat(v, H // Hkv, axis=1)
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    s = np.einsum("bhqd,bhkd->bhqk", q, k) * scale
    if causal:
        keep = np.arange(Sq)[:, None] + causal_offset >= np.arange(Sk)[None, :]
        s = np.where(keep, s, -np.inf)
    if mask is not None:
        s = s + np.asarray(mask, dtype=np.float64)
    if softcap and softcap > 0:
        s = np.tanh(s / softcap) * softcap
    s = s - s.max(axis=-1, keepdims=True)
    p = np.exp(s)
    p = p / p.sum(axis=-1, keepdims=True)
    return np.einsum("bhqk,bhkd->bhqd", p, v)


def np_rms_norm(x, eps=1e-5, gain=None):
    x = np.asarray(x, dtype=np.float64)
    y = x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)
    return y if gain is None else y * np.asarray(gain, dtype=np.float64)


def np_rope(x, cos, sin, interleaved=False):
    x = np.asarray(x, dtype=np.float64)
    if interleaved:
        x1, x2 = x[..., 0::2], x[..., 1::2]
    else:
        h = x.shape[-1] // 2
        x1, x2 = x[..., :h], x[..., h:]
    re = x1 * cos - x2 * sin
    im = x1 * sin + x2 * cos
    if interleaved:
        return np.stack([re, im], axis=-1).reshape(x.shape)
    return np.concatenate([re, im], axis=-1)


def np_silu(x):
    x = np.asarray(x, dtype=np.float64)
    return x / (1.0 + np.exp2(-x / math.log(2.0)))


# ---------------------------------------------------------------------------------------------
# Seeded inputs.  One numpy Generator per config, tensors drawn in the order listed; the GPU
# path must consume these same bytes.
# ---------------------------------------------------------------------------------------------
def uniform_f32(rng, shape):
    return rng.uniform(-1.0, 1.0, size=shape).astype(np.float32)


def normal_bf16(rng, shape, sigma=1.0):
    """N(0, sigma) -> f32 -> bf16 bit patterns."""
    return f32_to_bf16((rng.standard_normal(size=shape, dtype=np.float32) * np.float32(sigma)))


def rope_tables(seq: int, head_dim: int, theta: float = 10000.0):
    """cos/sin [seq, head_dim/2]: inv_freq_i = theta^(-2i/head_dim), angle = pos * inv_freq_i."""
    i = np.arange(head_dim // 2, dtype=np.float64)
    inv = theta ** (-2.0 * i / head_dim)
    ang = np.arange(seq, dtype=np.float64)[:, None] * inv[None, :]
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


def decoder_layer_weights(rng, hidden, n_q, n_kv, head_dim, ffn, sigma=0.02):
    """bf16 weights stored [in, out] row-major, drawn in this order."""
    shapes = {
        "wq": (hidden, n_q * head_dim), "wk": (hidden, n_kv * head_dim), "wv": (hidden, n_kv * head_dim),
        "wo": (n_q * head_dim, hidden), "wgate": (hidden, ffn), "wup": (hidden, ffn), "wdown": (ffn, hidden),
    }
    return {k: normal_bf16(rng, s, sigma) for k, s in shapes.items()}


def decoder_layer_f32(x_bits, w, batch, seq, n_q, n_kv, head_dim, eps=1e-5, theta=10000.0, g1=None, g2=None,
                      round_boundaries=False):
    """Pre-norm Llama-style block composed from the reference's own pieces in the order its Tensor
    API implies (rms_norm: tensor/src/nn/norm.rs:92-110; matmul: tensor/src/matmul.rs:82-110;
    apply_rotary_emb split-half: tensor/src/transformer.rs:32-69; GQA expansion:
    onnx/src/registry/transformer.rs:80-103; attention: tensor/src/transformer.rs:78-137; silu:
    tensor/src/activation.rs:309-318).  Evaluated in f32 on bf16-rounded x and weights.

    round_boundaries selects where intermediate results pass through bf16:
      False       nowhere (the pure-f32 oracle the headline tolerance is stated against);
      True/"ops"  after every op, as the dtypes of the reference's bf16 graph dictate (matmul casts its f32 sum back
                  to bf16, tensor/src/reduce.rs:673-691, before a residual add or the gate sees it);
      "kernels"   only where a kernel of the fused schedule stores a result: the residual add of `h + a @ Wo` /
                  `h + ff @ Wdown` and the gate `silu(x @ Wgate) * (x @ Wup)` consume the f32 sums of their matmuls,
                  which is what a kernel that keeps those ops together (the reference counts them as one kernel,
                  tensor/src/test/unit/fusion.rs:21-33,58-67) has in its registers."""
    mode = {False: "none", True: "ops", None: "none"}.get(round_boundaries, round_boundaries)
    if mode not in ("none", "ops", "kernels"):
        raise ValueError(f"round_boundaries: {round_boundaries!r}")
    rb = (lambda t: t) if mode == "none" else (lambda t: round_bf16(t))          # a stored result
    rb_op = (lambda t: round_bf16(t)) if mode == "ops" else (lambda t: t)        # a result that a fused kernel keeps in f32
    hidden = x_bits.shape[-1]
    T = batch * seq
    h = bf16_to_f32(x_bits).reshape(T, hidden)
    W = {k: bf16_to_f32(v) for k, v in w.items()}
    cos, sin = rope_tables(seq, head_dim, theta)

    n1 = rb(rms_norm_f32(h, eps, g1))
    q = rb(matmul_f32(n1, W["wq"])).reshape(batch, seq, n_q, head_dim)
    k = rb(matmul_f32(n1, W["wk"])).reshape(batch, seq, n_kv, head_dim)
    v = rb(matmul_f32(n1, W["wv"])).reshape(batch, seq, n_kv, head_dim)
    q = rb(rope_f32(q, cos, sin, False, row_div=n_q))
    k = rb(rope_f32(k, cos, sin, False, row_div=n_kv))
    qh, kh, vh = (np.ascontiguousarray(t.transpose(0, 2, 1, 3)) for t in (q, k, v))
    a = rb(sdpa_f32(qh, kh, vh, causal=True))
    a = np.ascontiguousarray(a.transpose(0, 2, 1, 3)).reshape(T, n_q * head_dim)
    h = rb(h + rb_op(matmul_f32(a, W["wo"])))
    n2 = rb(rms_norm_f32(h, eps, g2))
    ff = rb(swiglu_f32(rb_op(matmul_f32(n2, W["wgate"])), rb_op(matmul_f32(n2, W["wup"]))))
    out = rb(h + rb_op(matmul_f32(ff, W["wdown"])))
    return out.reshape(batch, seq, hidden)
