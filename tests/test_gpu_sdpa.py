"""Attention forward through mk_sdpa_fwd of the C ABI against the CPU oracle."""
import numpy as np
import pytest

import morok_b200 as mk
from morok_b200 import _ffi
from oracle import oracle as orc
from gpu_util import assert_close, dev, to_f32, to_storage  # noqa: F401

pytestmark = pytest.mark.gpu
ST = {mk.MK_F32: np.float32, mk.MK_BF16: np.uint16, mk.MK_F16: np.float16}


def run_sdpa(dev, q, k, v, dt, scale=0.0, causal=False, softcap=0.0, mask=None, want_lse=False, causal_offset=0):
    B, H, Sq, D = q.shape
    Hkv, Sk, Dv = k.shape[1], k.shape[2], v.shape[3]
    Q, K, V = (dev.from_numpy(to_storage(t, dt)) for t in (q, k, v))
    O = dev.alloc(B * H * Sq * Dv * mk.dtype_size(dt))
    Mb = dev.from_numpy(mask.astype(np.float32)) if mask is not None else None
    L = dev.alloc(B * H * Sq * 4) if want_lse else None
    dev.sdpa(Q, K, V, O, B, H, Hkv, Sq, Sk, D, Dv, dtype=dt, scale=scale, causal=causal, softcap=softcap, mask=Mb, lse=L,
             causal_offset=causal_offset)
    assert dev.kernel_status() == 0
    o = to_f32(O.copyout(ST[dt], (B, H, Sq, Dv)), dt)
    lse = L.copyout(np.float32, (B, H, Sq)) if want_lse else None
    for b in (Q, K, V, O):
        b.free()
    return (o, lse) if want_lse else o


def test_known_answers(dev, golden):
    for case in golden["sdpa"]:
        q, k, v = (np.array(case[n], np.float32)[None, None] for n in ("q", "k", "v"))
        o = run_sdpa(dev, q, k, v, mk.MK_F32, causal=case["causal"], softcap=case["softcap"])
        assert o.shape == (1, 1, q.shape[2], v.shape[3])
        if "expected_row0" in case:
            assert np.max(np.abs(o[0, 0, 0] - np.array(case["expected_row0"]))) < case["abs_tol"]
        if case.get("finite"):
            assert np.all(np.isfinite(o))
        assert_close(o, orc.sdpa_f32(q, k, v, causal=case["causal"], softcap=case["softcap"]), mk.MK_F32, case["name"])


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("dt", [mk.MK_F32, mk.MK_BF16])
def test_general_path_gqa_mask_softcap_ragged(dev, causal, dt):
    rng = np.random.default_rng(7)
    B, H, Hkv, Sq, Sk, D, Dv = 2, 4, 2, 13, 29, 16, 24
    q, k, v = (to_f32(to_storage(rng.standard_normal(s, dtype=np.float32), dt), dt)
               for s in ((B, H, Sq, D), (B, Hkv, Sk, D), (B, Hkv, Sk, Dv)))
    mask = rng.standard_normal((Sq, Sk), dtype=np.float32) * 0.5
    for kw in ({}, {"mask": mask}, {"softcap": 2.0}, {"scale": 0.3, "mask": mask, "softcap": 5.0}):
        o, lse = run_sdpa(dev, q, k, v, dt, causal=causal, want_lse=True, **kw)
        ro, rl = orc.sdpa_f32(q, k, v, causal=causal, return_lse=True, scale=kw.get("scale"), mask=kw.get("mask"),
                              softcap=kw.get("softcap", 0.0))
        assert_close(o, ro, dt, f"sdpa {kw}")
        assert np.allclose(lse, rl, atol=1e-4, rtol=1e-4)


def test_sk_zero_and_empty(dev):
    q = np.ones((1, 2, 3, 8), np.float32)
    k = np.zeros((1, 2, 0, 8), np.float32)
    o = run_sdpa(dev, q, k, k, mk.MK_F32)
    assert o.shape == (1, 2, 3, 8) and np.all(o == 0)


TC_CASES = [
    # B, Hq, Hkv, Sq, Sk, causal
    (1, 1, 1, 128, 128, False), (1, 1, 1, 128, 128, True), (1, 2, 2, 256, 256, True), (2, 4, 2, 384, 384, True),
    (1, 2, 1, 200, 200, True), (1, 2, 2, 130, 333, False), (1, 1, 1, 100, 260, True), (1, 3, 3, 512, 512, False),
    (1, 1, 1, 1024, 1024, True),
]


@pytest.mark.parametrize("case", TC_CASES)
@pytest.mark.parametrize("dt", [mk.MK_BF16, mk.MK_F16])
@pytest.mark.parametrize("D", [128, 64])
def test_tensor_core_head_sizes_vs_oracle(dev, case, dt, D):
    B, H, Hkv, Sq, Sk, causal = case
    rng = np.random.default_rng(Sq * 3 + Sk + H)
    q, k, v = (to_f32(to_storage(rng.standard_normal(s, dtype=np.float32), dt), dt)
               for s in ((B, H, Sq, D), (B, Hkv, Sk, D), (B, Hkv, Sk, D)))
    o, lse = run_sdpa(dev, q, k, v, dt, causal=causal, want_lse=True)
    ro, rl = orc.sdpa_f32(q, k, v, causal=causal, return_lse=True)
    assert_close(o, ro, dt, f"{case}")
    assert np.allclose(lse, rl, atol=2e-3, rtol=1e-3)
    if causal:   # row 0 attends only to key 0 (tensor/src/test/unit/transformer.rs:103-116)
        assert_close(o[:, :, 0], np.repeat(v, H // Hkv, axis=1)[:, :, 0], dt, "row 0 == V[0]")


@pytest.mark.parametrize("S", [256, 4096])
def test_strided_bshd_layout(dev, S):
    """Q/K/V stored [B,S,H,D] (the projection output layout) are read in place through strides, and O is written in that
    layout too -- by each thread's own stores for the short sequence, through the staging tile and tile stores for the
    long one."""
    B, H, Hkv, D = (2, 4, 2, 128) if S == 256 else (1, 2, 1, 128)
    rng = np.random.default_rng(1)
    q = orc.round_bf16(rng.standard_normal((B, S, H, D), dtype=np.float32))
    k = orc.round_bf16(rng.standard_normal((B, S, Hkv, D), dtype=np.float32))
    v = orc.round_bf16(rng.standard_normal((B, S, Hkv, D), dtype=np.float32))
    Q, K, V = (dev.from_numpy(orc.f32_to_bf16(t)) for t in (q, k, v))
    O = dev.alloc(B * S * H * D * 2)
    dev.sdpa(Q, K, V, O, B, H, Hkv, S, S, D, dtype=mk.MK_BF16, causal=True,
             q_strides=(S * H * D, D, H * D), k_strides=(S * Hkv * D, D, Hkv * D), v_strides=(S * Hkv * D, D, Hkv * D),
             o_strides=(S * H * D, D, H * D))
    assert dev.kernel_status() == 0
    o = orc.bf16_to_f32(O.copyout(np.uint16, (B, S, H, D)))
    ref = orc.sdpa_f32(q.transpose(0, 2, 1, 3), k.transpose(0, 2, 1, 3), v.transpose(0, 2, 1, 3), causal=True)
    assert_close(o.transpose(0, 2, 1, 3), ref, mk.MK_BF16, "bshd layout")


def test_config3_shape_sampled_heads(dev):
    """B4 H32 S4096 D128 causal bf16: full-size run, two (batch, head) pairs checked against the
    oracle, plus size-independent checks on every head (row 0 == V[0]; constant V returns the constant)."""
    B, H, S, D = 4, 32, 4096, 128
    rng = np.random.default_rng(0)
    q_bits, k_bits, v_bits = (orc.normal_bf16(rng, (B, H, S, D)) for _ in range(3))
    Q, K, V = dev.from_numpy(q_bits), dev.from_numpy(k_bits), dev.from_numpy(v_bits)
    O = dev.alloc(B * H * S * D * 2)
    dev.sdpa(Q, K, V, O, B, H, H, S, S, D, dtype=mk.MK_BF16, causal=True)
    assert dev.kernel_status() == 0
    o = orc.bf16_to_f32(O.copyout(np.uint16, (B, H, S, D)))
    assert np.all(np.isfinite(o))
    assert_close(o[:, :, 0], orc.bf16_to_f32(v_bits[:, :, 0]), mk.MK_BF16, "row 0 == V[0]")
    for (b, h) in ((0, 0), (3, 31)):
        ref = orc.sdpa_f32(*(orc.bf16_to_f32(t[b:b + 1, h:h + 1]) for t in (q_bits, k_bits, v_bits)), causal=True)
        assert_close(o[b:b + 1, h:h + 1], ref, mk.MK_BF16, f"config 3 head ({b},{h})")
        # late causal rows average thousands of values: |O| ~ 0.03 there, so the absolute term of the bar is loose;
        # the relative rms error over the head is the sharper check
        rel_rms = float(np.sqrt(np.mean((o[b, h] - ref[0, 0]) ** 2)) / np.sqrt(np.mean(ref ** 2)))
        assert rel_rms < 1e-2, f"config 3 head ({b},{h}): relative rms error {rel_rms:.3e}"
    ones = dev.from_numpy(orc.f32_to_bf16(np.full((B, H, S, D), 0.5, np.float32)))
    dev.sdpa(Q, K, ones, O, B, H, H, S, S, D, dtype=mk.MK_BF16, causal=True)
    assert dev.kernel_status() == 0
    o2 = orc.bf16_to_f32(O.copyout(np.uint16, (B, H, S, D)))
    assert np.max(np.abs(o2 - 0.5)) < 1e-2


def test_config5_shape_sampled_heads_lse_and_rms(dev):
    """The sharded sweep's attention on one GPU: B8 H64 S8192 D128 causal bf16.  Four (batch, head) pairs against the
    oracle (output element-wise and by relative rms, log-sum-exp), plus row 0 == V[0] and finiteness on every head."""
    B, H, S, D = 8, 64, 8192, 128
    rng = np.random.default_rng(5)
    q_bits, k_bits, v_bits = (orc.normal_bf16(rng, (B, H, S, D)) for _ in range(3))
    Q, K, V = dev.from_numpy(q_bits), dev.from_numpy(k_bits), dev.from_numpy(v_bits)
    O, L = dev.alloc(B * H * S * D * 2), dev.alloc(B * H * S * 4)
    _ffi.check(dev.lib.mk_memset_async(dev.h, O.ptr, 0xFF, B * H * S * D * 2, None))
    before = dev.launch_count()
    dev.sdpa(Q, K, V, O, B, H, H, S, S, D, dtype=mk.MK_BF16, causal=True, lse=L)
    assert dev.kernel_status() == 0
    assert dev.launch_count() - before == 1
    o_bits = O.copyout(np.uint16, (B, H, S, D))
    assert not np.any(o_bits == 0xFFFF), "some output element was never written"
    lse = L.copyout(np.float32, (B, H, S))
    assert_close(orc.bf16_to_f32(o_bits[:, :, 0]), orc.bf16_to_f32(v_bits[:, :, 0]), mk.MK_BF16, "row 0 == V[0]")
    for (b, h) in ((0, 0), (3, 17), (5, 40), (7, 63)):
        ref, ref_lse = orc.sdpa_f32(*(orc.bf16_to_f32(t[b:b + 1, h:h + 1]) for t in (q_bits, k_bits, v_bits)), causal=True, return_lse=True)
        got = orc.bf16_to_f32(o_bits[b:b + 1, h:h + 1])
        assert np.all(np.isfinite(got))
        assert_close(got, ref, mk.MK_BF16, f"config 5 head ({b},{h})")
        rel_rms = float(np.sqrt(np.mean((got - ref) ** 2)) / np.sqrt(np.mean(ref ** 2)))
        assert rel_rms < 1e-2, f"config 5 head ({b},{h}): relative rms error {rel_rms:.3e}"
        assert np.max(np.abs(lse[b, h] - ref_lse[0, 0])) < 2e-3, f"config 5 head ({b},{h}): log-sum-exp off by {np.max(np.abs(lse[b, h] - ref_lse[0, 0])):.3e}"
    for x in (Q, K, V, O, L):
        x.free()
    dev.trim()


@pytest.mark.parametrize("case", [
    # dtype, B, Hq, Hkv, Sq, Sk, D, offset
    (mk.MK_BF16, 1, 4, 2, 128, 384, 128, 256),     # tensor-core kernel: a chunk of new rows behind a cache of 256 keys
    (mk.MK_BF16, 2, 2, 2, 200, 333, 128, 133),     # ragged
    (mk.MK_F16, 1, 2, 1, 256, 256, 128, 17),
    (mk.MK_F32, 1, 2, 2, 5, 40, 64, 35),           # general kernel
    (mk.MK_F32, 1, 1, 1, 6, 9, 32, -2),            # negative offset: the first rows see nothing and come out NaN
])
def test_causal_offset_vs_oracle(dev, case):
    dt, B, H, Hkv, Sq, Sk, D, off = case
    rng = np.random.default_rng(Sq + Sk + off)
    q, k, v = (to_f32(to_storage(rng.standard_normal(s, dtype=np.float32), dt), dt)
               for s in ((B, H, Sq, D), (B, Hkv, Sk, D), (B, Hkv, Sk, D)))
    o = run_sdpa(dev, q, k, v, dt, causal=True, causal_offset=off)
    ro = orc.sdpa_f32(q, k, v, causal=True, causal_offset=off)
    dead = np.isnan(ro)
    assert np.array_equal(np.isnan(o), dead)
    if off < 0:
        assert dead[:, :, : -off].all() and not dead[:, :, -off:].any()
    assert_close(np.where(dead, 0, o), np.where(dead, 0, ro), dt, f"{case}")


# ---------------------------------------------------------------------------------------------
# A few query rows against a long key/value stream (decoding with a cache, or a short chunk of new
# tokens: onnx/src/registry/transformer.rs:145-162 concatenates past_key and masks with
# tril(past_seq_len)).  (Hq / Hkv) * Sq <= 16 rows take the split-key kernel.
# ---------------------------------------------------------------------------------------------
DECODE_CASES = [
    # dtype, B, Hq, Hkv, Sq, Sk, D, causal
    (mk.MK_BF16, 1, 32, 8, 1, 8192, 128, True),      # one new token, 8 K keys: keys split across CTAs, then merged
    (mk.MK_BF16, 2, 8, 2, 1, 1000, 128, True),       # ragged last tile
    (mk.MK_BF16, 1, 8, 2, 3, 300, 128, True),        # three new rows: each sees one key more than the previous
    (mk.MK_F16, 3, 4, 4, 2, 77, 64, True),           # head size 64, no grouping
    (mk.MK_BF16, 1, 16, 1, 1, 4097, 64, False),      # 16 query heads on one kv head, not causal
    (mk.MK_F16, 64, 8, 8, 1, 130, 128, True),        # enough (batch, head) pairs that keys are not split
    (mk.MK_BF16, 1, 4, 4, 4, 5, 128, True),          # fewer keys than one tile
]


@pytest.mark.parametrize("case", DECODE_CASES)
def test_decode_rows_vs_oracle(dev, case):
    dt, B, H, Hkv, Sq, Sk, D, causal = case
    rng = np.random.default_rng(Sk + H + Sq)
    q, k, v = (to_f32(to_storage(rng.standard_normal(s, dtype=np.float32), dt), dt)
               for s in ((B, H, Sq, D), (B, Hkv, Sk, D), (B, Hkv, Sk, D)))
    off = Sk - Sq                                      # the new rows sit behind a cache of Sk - Sq keys
    before = dev.launch_count()
    o, lse = run_sdpa(dev, q, k, v, dt, causal=causal, causal_offset=off, want_lse=True)
    launched = dev.launch_count() - before
    assert launched in (1, 2)                          # the split-key kernel, plus its merge when keys were split
    if B * Hkv < 100 and Sk >= 512:                     # few (batch, kv head) pairs and a long stream: keys are split
        assert launched == 2
    ro, rl = orc.sdpa_f32(q, k, v, causal=causal, causal_offset=off, return_lse=True)
    assert_close(o, ro, dt, f"decode {case}")
    assert np.allclose(lse, rl, atol=2e-3, rtol=1e-3)


def test_decode_reads_a_bshd_cache_in_place(dev):
    """K/V cache stored [B, S, H, D] (as the projections write it) is read through strides."""
    B, S, H, Hkv, D = 2, 700, 8, 2, 128
    rng = np.random.default_rng(8)
    q = orc.round_bf16(rng.standard_normal((B, 1, H, D), dtype=np.float32))
    k = orc.round_bf16(rng.standard_normal((B, S, Hkv, D), dtype=np.float32))
    v = orc.round_bf16(rng.standard_normal((B, S, Hkv, D), dtype=np.float32))
    Q, K, V = (dev.from_numpy(orc.f32_to_bf16(t)) for t in (q, k, v))
    O = dev.alloc(B * H * D * 2)
    dev.sdpa(Q, K, V, O, B, H, Hkv, 1, S, D, dtype=mk.MK_BF16, causal=True, causal_offset=S - 1,
             q_strides=(H * D, D, H * D), k_strides=(S * Hkv * D, D, Hkv * D), v_strides=(S * Hkv * D, D, Hkv * D),
             o_strides=(H * D, D, H * D))
    assert dev.kernel_status() == 0
    o = orc.bf16_to_f32(O.copyout(np.uint16, (B, 1, H, D))).transpose(0, 2, 1, 3)
    ref = orc.sdpa_f32(q.transpose(0, 2, 1, 3), k.transpose(0, 2, 1, 3), v.transpose(0, 2, 1, 3))
    assert_close(o, ref, mk.MK_BF16, "decode over a [B,S,H,D] cache")


@pytest.mark.parametrize("D", [128, 64])
def test_head_sharded_delivery_by_tile_stores_into_stand_in_peers(dev, D):
    """The head-sharded form on one GPU: two more buffers of the same GPU stand in for the peers' O.  The kernel
    computes heads 2 .. 5 of 8 (GQA 2:1) and must deliver them, through its staging tile and one tile store per
    destination, into all three tensors without touching the other heads; ragged sequence length."""
    B, H, Hkv, S = 2, 8, 4, 600
    q0, nq, kv0, nkv = 2, 4, 1, 2
    rng = np.random.default_rng(D)
    q, k, v = orc.normal_bf16(rng, (B, H, S, D)), orc.normal_bf16(rng, (B, Hkv, S, D)), orc.normal_bf16(rng, (B, Hkv, S, D))
    Q, K, V = dev.from_numpy(q), dev.from_numpy(k), dev.from_numpy(v)
    outs = [dev.from_numpy(np.full((B, H, S, D), 0xFFFF, np.uint16)) for _ in range(3)]
    off = q0 * S * D * 2
    dev.sdpa(Q.view(off, (H - q0) * S * D * 2), K.view(kv0 * S * D * 2, (Hkv - kv0) * S * D * 2), V.view(kv0 * S * D * 2, (Hkv - kv0) * S * D * 2),
             outs[0], B, nq, nkv, S, S, D, dtype=mk.MK_BF16, causal=True,
             q_strides=(H * S * D, S * D, D), k_strides=(Hkv * S * D, S * D, D), v_strides=(Hkv * S * D, S * D, D),
             o_strides=(H * S * D, S * D, D), o_ptr=outs[0].ptr + off, peers=[o.ptr + off for o in outs[1:]])
    assert dev.kernel_status() == 0
    bf = orc.bf16_to_f32
    ref = orc.sdpa_f32(bf(q[:, q0:q0 + nq]), bf(k[:, kv0:kv0 + nkv]), bf(v[:, kv0:kv0 + nkv]), causal=True)
    first = None
    for o in outs:
        got = o.copyout(np.uint16, (B, H, S, D))
        assert np.all(got[:, :q0] == 0xFFFF) and np.all(got[:, q0 + nq:] == 0xFFFF), "heads of another rank were overwritten"
        assert_close(bf(got[:, q0:q0 + nq]), ref, mk.MK_BF16, "tile-store delivery of O")
        first = got if first is None else first
        assert np.array_equal(got, first), "the copies differ from each other"
    for x in [Q, K, V] + outs:
        x.free()


@pytest.mark.parametrize("S", [512, 384])
def test_tile_store_delivery_under_back_pressure_seven_stand_in_peers(dev, S):
    """Eight destinations per output tile (the local O and seven stand-ins for peers) and work items so short that
    the tile stores, not the arithmetic, set the pace: 1024 items of at most four key blocks on 148 CTAs, 0.5 GB of
    stores against 35 GFLOP.  Each use of the one staging tile then waits for the copy engine, with the softmax warps
    of both query tiles queueing behind it.  All eight copies must be identical, sampled heads must match the oracle,
    and no pipeline wait may give up.  S = 384: every second item has rows for one query tile only, so the other
    tile's warps sit items out and come back several uses of the staging tile later."""
    B, H, D = 16, 32, 128
    rng = np.random.default_rng(77)
    q, k, v = (orc.normal_bf16(rng, (B, H, S, D)) for _ in range(3))
    Q, K, V = dev.from_numpy(q), dev.from_numpy(k), dev.from_numpy(v)
    outs = [dev.from_numpy(np.full((B, H, S, D), 0xFFFF, np.uint16)) for _ in range(8)]
    for _ in range(3):        # the later launches start with the copy engine still busy
        dev.sdpa(Q, K, V, outs[0], B, H, H, S, S, D, dtype=mk.MK_BF16, causal=True, peers=[o.ptr for o in outs[1:]])
    dev.sync()
    assert dev.kernel_status() == 0
    bf = orc.bf16_to_f32
    first = outs[0].copyout(np.uint16, (B, H, S, D))
    assert not np.any(first == 0xFFFF), "part of the output was never written"
    for o in outs[1:]:
        assert np.array_equal(o.copyout(np.uint16, (B, H, S, D)), first), "the copies differ from each other"
    for b, h in ((0, 0), (5, 17), (15, 31), (9, 2)):
        ref = orc.sdpa_f32(bf(q[b:b + 1, h:h + 1]), bf(k[b:b + 1, h:h + 1]), bf(v[b:b + 1, h:h + 1]), causal=True)
        assert_close(bf(first[b:b + 1, h:h + 1]), ref, mk.MK_BF16, f"batch {b} head {h}")
    for x in [Q, K, V] + outs:
        x.free()


def oracle_sdpa_broadcast_mask(q, k, v, mask4, causal, softcap=0.0, scale=None):
    """The oracle takes one [Sq, Sk] mask; a mask that broadcasts over batch and head is applied pair by pair
    (bool masks become 0 / -inf first, tensor/src/transformer.rs:112-124)."""
    B, H, Sq, _ = q.shape
    Hkv, Sk = k.shape[1], k.shape[2]
    g = H // Hkv
    if mask4.dtype == np.bool_:
        mask4 = np.where(mask4, np.float32(0), np.float32(-np.inf))
    m = np.broadcast_to(mask4, (B, H, Sq, Sk))
    out = np.empty((B, H, Sq, v.shape[3]), np.float32)
    for b in range(B):
        for h in range(H):
            out[b, h] = orc.sdpa_f32(q[b:b + 1, h:h + 1], k[b:b + 1, h // g:h // g + 1], v[b:b + 1, h // g:h // g + 1], causal=causal,
                                     mask=np.ascontiguousarray(m[b, h]), softcap=softcap, scale=scale)[0, 0]
    return out


def mask_strides(shape4, Sk):
    """Element strides (batch, head, row) of a dense mask of shape [b, h, s, Sk] where b, h, s may be 1 (broadcast)."""
    b, h, s, _ = shape4
    return (0 if b == 1 else h * s * Sk, 0 if h == 1 else s * Sk, 0 if s == 1 else Sk)


@pytest.mark.parametrize("case", [
    # name, B, Hq, Hkv, Sq, Sk, D, mask shape (b, h, s), bool?, causal, softcap
    ("key padding per batch element, f32", 3, 4, 2, 384, 384, 128, (3, 1, 1), False, False, 0.0),
    ("key padding per batch element, bool, causal", 2, 4, 4, 300, 300, 128, (2, 1, 1), True, True, 0.0),
    ("one [Sq, Sk] mask for all heads", 1, 2, 1, 256, 320, 128, (1, 1, 256), False, False, 0.0),
    ("full [B, H, Sq, Sk] mask, ragged Sk (unaligned rows)", 2, 2, 2, 130, 203, 64, (2, 2, 130), False, True, 0.0),
    ("softcap only", 1, 4, 2, 256, 512, 128, None, False, False, 30.0),
    ("softcap under a causal rule: masked scores become -cap and take part", 1, 2, 2, 384, 384, 128, None, False, True, 20.0),
    ("bool mask and softcap, head size 64", 2, 2, 1, 200, 264, 64, (2, 1, 200), True, False, 15.0),
    # long key ranges: the scan for the first block a key-padding mask changes runs several rounds of eight blocks
    ("key padding late in a long ragged sequence", 2, 2, 2, 256, 1500, 128, (2, 1, 1), False, False, 0.0),
    ("bool key padding, long, causal, head size 64", 2, 2, 1, 1280, 1280, 64, (2, 1, 1), True, True, 0.0),
    ("key padding with a hole in the middle: plain blocks, a changed one, unchanged ones, the tail", 2, 2, 2, 200, 1408, 128, (2, 1, 1), False, False, 0.0),
    ("a key-padding mask that changes nothing", 1, 2, 2, 384, 1152, 128, (1, 1, 1), False, True, 0.0),
    ("softcap, causal, long and ragged: whole blocks above the diagonal", 1, 2, 1, 650, 650, 128, None, False, True, 25.0),
    ("softcap and key padding, causal, long", 2, 2, 2, 640, 640, 128, (2, 1, 1), True, True, 30.0),
])
def test_masks_and_softcap_run_on_the_tensor_core_kernel(dev, case):
    name, B, H, Hkv, Sq, Sk, D, mshape, is_bool, causal, cap = case
    rng = np.random.default_rng(len(name) + Sq)
    q, k, v = (orc.round_bf16(rng.standard_normal(s, dtype=np.float32)) for s in ((B, H, Sq, D), (B, Hkv, Sk, D), (B, Hkv, Sk, D)))
    mask4 = None
    if mshape is not None:
        shape4 = (mshape[0], mshape[1], mshape[2], Sk)
        if is_bool:
            mask4 = rng.random(shape4) > 0.3
            mask4[..., 0] = True                                 # key 0 stays visible: no row is masked out entirely
            if mshape[2] == 1:                                   # a padding mask: hide the tail of each sequence
                mask4[:] = True
                for b in range(shape4[0]):
                    mask4[b, ..., Sk - 17 * (b + 1):] = False
        else:
            mask4 = (rng.standard_normal(shape4) * 2).astype(np.float32)
            if mshape[2] == 1:
                mask4[:] = 0
                if "changes nothing" not in name:
                    for b in range(shape4[0]):
                        mask4[b, ..., Sk - 23 * (b + 1):] = -np.inf
                if "hole" in name:
                    mask4[..., 300:310] = -np.inf
                    mask4[1, ..., 700] = -1.5
    Q, K, V = (dev.from_numpy(orc.f32_to_bf16(t)) for t in (q, k, v))
    O = dev.alloc(B * H * Sq * D * 2)
    kw = {}
    if mask4 is not None:
        kw = dict(mask=dev.from_numpy(mask4), mask_strides=mask_strides(mask4.shape, Sk), mask_bool=is_bool)
    dev.profile_begin()
    dev.sdpa(Q, K, V, O, B, H, Hkv, Sq, Sk, D, dtype=mk.MK_BF16, causal=causal, softcap=cap, **kw)
    launched = [n for n, _ in dev.profile_end()]
    assert launched == [f"sdpa_tc_d{D}_general"], launched
    assert dev.kernel_status() == 0
    got = orc.bf16_to_f32(O.copyout(np.uint16, (B, H, Sq, D)))
    if mask4 is None:
        ref = orc.sdpa_f32(q, k, v, causal=causal, softcap=cap)
    else:
        ref = oracle_sdpa_broadcast_mask(q, k, v, mask4, causal, cap)
    assert_close(got, ref, mk.MK_BF16, name)


def test_tensor_api_takes_broadcast_and_bool_masks(dev):
    """`scaled_dot_product_attention(attn_mask=...)` with a bool key-padding mask [B, 1, 1, Sk] and with an additive
    [Sq, Sk] mask (tensor/src/transformer.rs:112-124), one kernel each."""
    from morok_b200 import Tensor
    B, H, S, D = 2, 4, 256, 128
    rng = np.random.default_rng(8)
    q, k, v = (orc.round_bf16(rng.standard_normal((B, H, S, D), dtype=np.float32)) for _ in range(3))
    T = lambda x: Tensor.from_ndarray(dev, orc.f32_to_bf16(x))      # noqa: E731
    pad = np.ones((B, 1, 1, S), np.bool_)
    pad[0, ..., 200:] = False
    pad[1, ..., 131:] = False
    out = T(q).scaled_dot_product_attention(T(k), T(v), attn_mask=Tensor.from_ndarray(dev, pad), is_causal=True).realize()
    assert out.last_launches() == 1
    assert_close(orc.bf16_to_f32(out.as_ndarray()), oracle_sdpa_broadcast_mask(q, k, v, pad, True), mk.MK_BF16, "bool padding mask")
    add = (rng.standard_normal((S, S)) * 3).astype(np.float32)
    out = T(q).scaled_dot_product_attention(T(k), T(v), attn_mask=Tensor.from_ndarray(dev, add)).realize()
    assert_close(orc.bf16_to_f32(out.as_ndarray()), orc.sdpa_f32(q, k, v, mask=add), mk.MK_BF16, "additive [Sq, Sk] mask")
    with pytest.raises(mk.MorokError):       # a mask that does not broadcast is refused when the graph is built
        T(q).scaled_dot_product_attention(T(k), T(v), attn_mask=Tensor.from_ndarray(dev, np.zeros((3, S, S), np.float32)))


@pytest.mark.parametrize("D", [32, 80, 96, 120])
@pytest.mark.parametrize("case", [(1, 2, 2, 256, 256, True), (2, 4, 2, 200, 333, False)])
def test_other_head_sizes_run_on_the_tensor_core_kernel(dev, case, D):
    """Head sizes between the two the kernel is built for (64, 128) run on the next larger one: the tile loads
    zero-fill the missing columns and the tile stores drop them.  The reference is generic in the head size
    (tensor/src/transformer.rs:88-96; scale 1 / sqrt(D) of the real D)."""
    B, H, Hkv, Sq, Sk, causal = case
    rng = np.random.default_rng(D + Sq)
    q, k, v = (orc.round_bf16(rng.standard_normal(s, dtype=np.float32)) for s in ((B, H, Sq, D), (B, Hkv, Sk, D), (B, Hkv, Sk, D)))
    Q, K, V = (dev.from_numpy(orc.f32_to_bf16(t)) for t in (q, k, v))
    O = dev.from_numpy(np.full((B, H, Sq, D), 0xFFFF, np.uint16))
    guard = dev.from_numpy(np.full(4096, 0xABCD, np.uint16))       # something right behind O that must stay untouched
    dev.profile_begin()
    dev.sdpa(Q, K, V, O, B, H, Hkv, Sq, Sk, D, dtype=mk.MK_BF16, causal=causal)
    launched = [n for n, _ in dev.profile_end()]
    assert launched == [f"sdpa_tc_d{64 if D <= 64 else 128}"], launched
    assert dev.kernel_status() == 0
    got_bits = O.copyout(np.uint16, (B, H, Sq, D))
    assert not np.any(got_bits == 0xFFFF)
    assert np.all(guard.copyout(np.uint16, (4096,)) == 0xABCD)
    assert_close(orc.bf16_to_f32(got_bits), orc.sdpa_f32(q, k, v, causal=causal), mk.MK_BF16, f"D={D} {case}")


@pytest.mark.parametrize("case", [
    # name, B, Hq, Hkv, Sq, Sk, causal, dtype, mask?, softcap
    ("causal, several key blocks and items", 2, 4, 2, 640, 640, True, mk.MK_BF16, False, 0.0),
    ("ragged, no causal rule, f16", 1, 3, 3, 200, 333, False, mk.MK_F16, False, 0.0),
    ("one query tile, many key blocks", 1, 2, 1, 100, 1500, False, mk.MK_BF16, False, 0.0),
    ("key-padding mask, causal", 2, 2, 2, 384, 384, True, mk.MK_BF16, True, 0.0),
    ("softcap", 1, 2, 2, 256, 384, True, mk.MK_BF16, False, 25.0),
])
def test_head_size_256_runs_on_the_tensor_core_kernel(dev, case):
    """256-wide heads: one query tile per CTA (O takes half of tensor memory), single-stage K / V.  The reference is
    generic in the head size (tensor/src/transformer.rs:88-96); LSE checked as well."""
    name, B, H, Hkv, Sq, Sk, causal, dt, masked, cap = case
    D = 256
    rng = np.random.default_rng(Sq + Sk)
    rnd = orc.round_bf16 if dt == mk.MK_BF16 else (lambda x: x.astype(np.float16).astype(np.float32))
    q, k, v = (rnd(rng.standard_normal(s, dtype=np.float32)) for s in ((B, H, Sq, D), (B, Hkv, Sk, D), (B, Hkv, Sk, D)))
    to_dev = (lambda t: dev.from_numpy(orc.f32_to_bf16(t))) if dt == mk.MK_BF16 else (lambda t: dev.from_numpy(t.astype(np.float16)))
    Q, K, V = (to_dev(t) for t in (q, k, v))
    O = dev.from_numpy(np.full((B, H, Sq, D), 0xFFFF, np.uint16))
    L = dev.alloc(B * H * Sq * 4)
    kw = {}
    mask4 = None
    if masked:
        mask4 = np.zeros((B, 1, 1, Sk), np.float32)
        for b in range(B):
            mask4[b, ..., Sk - 37 * (b + 1):] = -np.inf
        kw = dict(mask=dev.from_numpy(mask4), mask_strides=mask_strides(mask4.shape, Sk))
    dev.profile_begin()
    dev.sdpa(Q, K, V, O, B, H, Hkv, Sq, Sk, D, dtype=dt, causal=causal, softcap=cap, lse=L, **kw)
    launched = [n for n, _ in dev.profile_end()]
    assert launched == ["sdpa_tc_d256_general" if (masked or cap > 0) else "sdpa_tc_d256"], launched
    assert dev.kernel_status() == 0
    bits = O.copyout(np.uint16, (B, H, Sq, D))
    assert not np.any(bits == 0xFFFF)
    got = orc.bf16_to_f32(bits) if dt == mk.MK_BF16 else bits.view(np.float16).astype(np.float32)
    if mask4 is not None:
        ref = oracle_sdpa_broadcast_mask(q, k, v, mask4, causal, cap)
    else:
        ref, lse_ref = orc.sdpa_f32(q, k, v, causal=causal, softcap=cap, return_lse=True)
        lse = L.copyout(np.float32, (B, H, Sq))
        assert np.allclose(lse, lse_ref, rtol=2e-3, atol=2e-3), name
    assert_close(got, ref, dt, name)
