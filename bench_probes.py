"""Small single-kernel workloads for profiler captures and quick timings:  python bench.py --probe NAME [args]

A profiler capture wants one kernel, a few launches and a few GB on the device at most; these probes are the
commands the summaries under profiles/ were made with.

    gemm [M K N] [--f16] [--nt]        bf16 tensor-core GEMM (default 4096 4096 8192; inputs exceed L2)
    attn [B H S D] [--noncausal]       causal attention forward (default 2 16 4096 128)
    attn_mask [B H S D] [--softcap X] [--zero-mask]  the same with a per-batch padding mask (and a softcap)
    skinny [rows N K]                  few-row GEMM against `linear` weights [N, K]
    decode [batch kv_len]              decode attention: one query row per sequence against a long cache
    layer [batch seq hidden q_heads kv_heads ffn] [--plan]     one decoder layer through the Tensor API
    decode_layer [batch cache]         one decode step of that layer (per-kernel times, eager vs plan replay)
"""
from __future__ import annotations

import sys
import time

import numpy as np

import morok_b200 as mk
from morok_b200 import Tensor, synth


def _ints(args, n, default):
    skip = {i + 1 for i, a in enumerate(args) if a == "--softcap"}      # the value of an option is not a dimension
    vals = [int(a) for i, a in enumerate(args) if not a.startswith("--") and i not in skip]
    return tuple(vals) if len(vals) == n else default


def _timed(dev, fn, warm=3, n=20, stream=None):
    for _ in range(warm):
        fn()
    e0, e1 = mk.Event(dev), mk.Event(dev)
    e0.record(stream)
    for _ in range(n):
        fn()
    e1.record(stream)
    dev.sync()
    assert dev.kernel_status(stream) == 0
    return e0.elapsed_ms(e1) / n


def gemm(args):
    M, K, N = _ints(args, 3, (4096, 4096, 8192))
    dt = mk.MK_F16 if "--f16" in args else mk.MK_BF16
    nt = "--nt" in args
    dev = mk.Device(0)
    rng = np.random.default_rng(0)
    conv = (lambda x: x.astype(np.float16)) if dt == mk.MK_F16 else synth.f32_to_bf16_bits
    a = dev.from_numpy(conv(rng.standard_normal((M, K), dtype=np.float32)))
    b = dev.from_numpy(conv(rng.standard_normal((N, K) if nt else (K, N), dtype=np.float32) * np.float32(0.02)))
    c = dev.alloc(M * N * 2)
    ms = _timed(dev, lambda: dev.gemm(a, b, c, M, N, K, dt, trans_b=nt))
    print(f"gemm {M} x {K} x {N}{' [N,K] weights' if nt else ''}: {ms * 1e3:.1f} us, {2.0 * M * N * K / ms / 1e9:.1f} TFLOP/s")


def attn(args, masked=False):
    B, H, S, D = _ints(args, 4, (2, 16, 4096, 128))
    causal = "--noncausal" not in args
    softcap = float(args[args.index("--softcap") + 1]) if "--softcap" in args else 0.0
    dev = mk.Device(0)
    rng = np.random.default_rng(0)
    q, k, v = (dev.from_numpy(synth.normal_bf16_bits(rng, (B, H, S, D))) for _ in range(3))
    o = dev.alloc(B * H * S * D * 2)
    kw = {}
    if masked:       # a padding mask per batch element: the last keys of each sequence are hidden
        m = np.zeros((B, 1, 1, S), np.float32)
        if "--zero-mask" not in args:      # (--zero-mask: a mask that changes nothing -- the cost of asking)
            for b in range(B):
                m[b, :, :, S - 64 * (b + 1):] = -np.inf
        kw = dict(mask=dev.from_numpy(m), mask_strides=(S, 0, 0))
    ms = _timed(dev, lambda: dev.sdpa(q, k, v, o, B, H, H, S, S, D, dtype=mk.MK_BF16, causal=causal, softcap=softcap, **kw))
    flops = (2.0 if causal else 4.0) * B * H * S * S * D
    print(f"attention B={B} H={H} S={S} D={D} causal={causal}{' masked' if masked else ''}{f' softcap {softcap}' if softcap else ''}: "
          f"{ms * 1e3:.1f} us, {flops / ms / 1e9:.1f} TFLOP/s")


def skinny(args):
    M, N, K = _ints(args, 3, (16, 14336, 4096))
    dev = mk.Device(0)
    rng = np.random.default_rng(0)
    a = dev.from_numpy(rng.integers(0x3C00, 0x3C80, size=M * K, dtype=np.uint16))
    w = dev.from_numpy(rng.integers(0x3C00, 0x3C80, size=N * K, dtype=np.uint16))
    y = dev.alloc(M * N * 2)
    ms = _timed(dev, lambda: dev.gemm(a, w, y, M, N, K, mk.MK_BF16, trans_b=True), warm=3, n=1)
    print(f"linear {M} x {N} x {K}: {ms * 1e3:.1f} us, {N * K * 2 / ms / 1e6:.0f} GB/s of weights")


def decode(args):
    B, Sk = _ints(args, 2, (16, 8192))
    H, Hkv, D = 32, 8, 128
    dev = mk.Device(0)
    rng = np.random.default_rng(0)
    q = dev.from_numpy(rng.integers(0x3C00, 0x4000, (B, H, 1, D), dtype=np.uint16))
    k = dev.from_numpy(rng.integers(0, 0x4000, (B, Hkv, Sk, D), dtype=np.uint16))
    v = dev.from_numpy(rng.integers(0, 0x4000, (B, Hkv, Sk, D), dtype=np.uint16))
    o = dev.alloc(B * H * D * 2)
    ms = _timed(dev, lambda: dev.sdpa(q, k, v, o, B, H, Hkv, 1, Sk, D, dtype=mk.MK_BF16, causal=True, causal_offset=Sk - 1), warm=3, n=1)
    print(f"decode B={B} Hq/Hkv={H}/{Hkv} Sk={Sk} D={D}: {ms * 1e3:.1f} us, {2 * B * Hkv * Sk * D * 2 / ms / 1e6:.0f} GB/s of K+V")


def layer(args):
    """One pre-norm Llama decoder layer through the lazy Tensor API, timed on the device.  Default: the decoder-layer
    configuration of the headline set (batch 8 x seq 2048, hidden 4096, 32 query / 8 kv heads of 128, FFN 14336)."""
    use_plan = "--plan" in args
    batch, seq, hidden, n_q, n_kv, ffn = _ints(args, 6, (8, 2048, 4096, 32, 8, 14336))
    hd = hidden // n_q
    dev = mk.Device(0)
    rng = np.random.default_rng(0)
    T = lambda shape, sigma: Tensor.from_ndarray(dev, synth.normal_bf16_bits(rng, shape, sigma))   # noqa: E731
    x = T((batch * seq, hidden), 1.0)
    W = {"wq": T((hidden, n_q * hd), 0.02), "wk": T((hidden, n_kv * hd), 0.02), "wv": T((hidden, n_kv * hd), 0.02),
         "wo": T((n_q * hd, hidden), 0.02), "wgate": T((hidden, ffn), 0.02), "wup": T((hidden, ffn), 0.02), "wdown": T((ffn, hidden), 0.02)}
    inv = 1.0 / (10000.0 ** (np.arange(0, hd, 2, dtype=np.float64) / hd))
    ang = np.arange(seq, dtype=np.float64)[:, None] * inv[None, :]
    cos = Tensor.from_ndarray(dev, np.cos(ang).astype(np.float32).reshape(1, seq, 1, hd // 2))
    sin = Tensor.from_ndarray(dev, np.sin(ang).astype(np.float32).reshape(1, seq, 1, hd // 2))

    def graph():
        n1 = x.rms_norm(-1, 1e-5).cast(mk.MK_BF16)
        q = n1.matmul(W["wq"]).try_reshape((batch, seq, n_q, hd)).apply_rotary_emb(cos, sin, False).try_permute((0, 2, 1, 3))
        k = n1.matmul(W["wk"]).try_reshape((batch, seq, n_kv, hd)).apply_rotary_emb(cos, sin, False).try_permute((0, 2, 1, 3))
        v = n1.matmul(W["wv"]).try_reshape((batch, seq, n_kv, hd)).try_permute((0, 2, 1, 3))
        a = q.scaled_dot_product_attention(k, v, is_causal=True).try_permute((0, 2, 1, 3)).try_reshape((batch * seq, n_q * hd))
        h = x.try_add(a.matmul(W["wo"]))
        n2 = h.rms_norm(-1, 1e-5).cast(mk.MK_BF16)
        return h.try_add(n2.matmul(W["wgate"]).silu().try_mul(n2.matmul(W["wup"])).matmul(W["wdown"]))

    tokens = batch * seq
    flops = 2 * tokens * hidden * (n_q * hd + 2 * n_kv * hd + n_q * hd + 3 * ffn) + 4 * batch * n_q * seq * seq * hd // 2
    if use_plan:
        plan = graph().compile()
        run = plan.launch
        launches = plan.kernel_count()
    else:
        out = graph().realize()
        launches = out.last_launches()
        run = lambda: graph().realize()   # noqa: E731
    for _ in range(3):
        run()
    dev.sync()
    n = 10
    e0, e1 = mk.Event(dev), mk.Event(dev)
    t0 = time.perf_counter()
    e0.record()
    for _ in range(n):
        run()
    e1.record()
    dev.sync()
    wall = (time.perf_counter() - t0) / n * 1e3
    ms = e0.elapsed_ms(e1) / n
    assert dev.kernel_status() == 0
    print(f"decoder layer batch {batch} seq {seq} hidden {hidden} heads {n_q}/{n_kv} ffn {ffn}{' (plan replay)' if use_plan else ''}: "
          f"{ms:.3f} ms on the device, {wall:.3f} ms wall, {flops / ms / 1e9:.1f} TFLOP/s, {launches} kernels")


def decode_layer(args):
    """One decode step of a Llama-8B-shaped decoder layer through the Tensor API (16 sequences, one new token each, 8192
    cached keys, `linear` weights [out, in]): per-kernel device times of one eager realisation, then eager vs plan replay."""
    batch, cache = _ints(args, 2, (16, 8192))
    n_q, n_kv, hd, hidden, ffn = 32, 8, 128, 4096, 14336
    dev = mk.Device(0)
    rng = np.random.default_rng(0)

    def bf16(shape, lo=0x3C00, hi=0x3C80, signs=False):
        bits = rng.integers(lo, hi, shape, dtype=np.uint16)
        if signs:
            bits ^= rng.integers(0, 2, shape, dtype=np.uint16) << np.uint16(15)
        return Tensor.from_ndarray(dev, bits)

    h_in = bf16((batch, hidden), signs=True)
    # weights around +-0.02 (bf16 exponent 0x3C8..0x3CA), stored [out, in]
    shapes = dict(wq=(n_q * hd, hidden), wo=(hidden, n_q * hd), wgate=(ffn, hidden), wup=(ffn, hidden), wdown=(hidden, ffn))
    W = {k: bf16(s, 0x3C80, 0x3CA0, signs=True) for k, s in shapes.items()}
    Kc, Vc = bf16((batch, n_kv, cache, hd), signs=True), bf16((batch, n_kv, cache, hd), signs=True)
    inv = 10000.0 ** (-np.arange(0, hd, 2, dtype=np.float64) / hd)
    cos = Tensor.from_ndarray(dev, np.cos(cache * inv).astype(np.float32).reshape(1, 1, 1, hd // 2))
    sin = Tensor.from_ndarray(dev, np.sin(cache * inv).astype(np.float32).reshape(1, 1, 1, hd // 2))

    def graph():
        n1 = h_in.rms_norm(-1, 1e-5).cast(mk.MK_BF16)
        q = n1.linear(W["wq"]).try_reshape((batch, 1, n_q, hd)).apply_rotary_emb(cos, sin, False).try_permute((0, 2, 1, 3))
        a = q.scaled_dot_product_attention(Kc, Vc).try_permute((0, 2, 1, 3)).try_reshape((batch, n_q * hd))
        h = h_in.try_add(a.linear(W["wo"]))
        n2 = h.rms_norm(-1, 1e-5).cast(mk.MK_BF16)
        return h.try_add(n2.linear(W["wgate"]).silu().try_mul(n2.linear(W["wup"])).linear(W["wdown"]))

    for _ in range(3):
        graph().realize()
    dev.sync()
    for name, ms in graph().realize_profiled():
        print(f"  {name:24s} {ms * 1e3:7.1f} us")
    n = 50
    t0 = time.perf_counter()
    for _ in range(n):
        graph().realize()
    dev.sync()
    eager = (time.perf_counter() - t0) / n * 1e6
    plan = graph().compile()
    for _ in range(3):
        plan.launch()
    dev.sync()
    t0 = time.perf_counter()
    for _ in range(n):
        plan.launch()
    dev.sync()
    replay = (time.perf_counter() - t0) / n * 1e6
    nbytes = (2 * hidden * n_q * hd + 3 * hidden * ffn) * 2 + 2 * batch * n_kv * cache * hd * 2
    assert dev.kernel_status() == 0
    print(f"decode step, batch {batch}, cache {cache}: eager {eager:.1f} us, plan replay {replay:.1f} us "
          f"({nbytes / replay / 1e3:.0f} GB/s of weights + cache), {plan.kernel_count()} kernels")


PROBES = {"gemm": gemm, "attn": attn, "attn_mask": lambda a: attn(a, masked=True), "skinny": skinny, "decode": decode,
          "layer": layer, "decode_layer": decode_layer}


def main(argv):
    if not argv or argv[0] not in PROBES:
        print(__doc__)
        raise SystemExit(2)
    if mk.device_count() == 0:
        raise SystemExit("bench_probes: no CUDA device -- the library has no CPU fallback")
    PROBES[argv[0]](argv[1:])


if __name__ == "__main__":
    main(sys.argv[1:])
