"""The lazy Tensor API on the GPU: the reference's own tests restated against it, kernel-count
contracts, and the decoder layer built through the API (C ABI underneath)."""
import os
import sys

import numpy as np
import pytest

import morok_b200 as mk
from morok_b200 import Tensor
from oracle import oracle as orc
from gpu_util import assert_close, dev  # noqa: F401

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
from make_golden import formula_operands  # noqa: E402

pytestmark = pytest.mark.gpu


def bf(dev, x):
    return Tensor.from_ndarray(dev, orc.f32_to_bf16(x))


def test_matmul_known_answers(dev, golden):
    for case in golden["matmul_small"]:
        a = Tensor.from_ndarray(dev, np.array(case["a"], np.float32).reshape(case["m"], case["k"]))
        b = Tensor.from_ndarray(dev, np.array(case["b"], np.float32).reshape(case["k"], case["n"]))
        c = a.matmul(b).realize()
        assert c.shape() == (case["m"], case["n"])
        assert np.max(np.abs(c.as_vec() - np.array(case["expected"]))) < case["abs_tol"], case["name"]
    for case in golden["matmul_1d"]:
        a = Tensor.from_ndarray(dev, np.array(case["a"], np.float32).reshape(case["a_shape"]))
        b = Tensor.from_ndarray(dev, np.array(case["b"], np.float32).reshape(case["b_shape"]))
        c = a.dot(b).realize()
        assert list(c.shape()) == case["out_shape"], case["name"]
        assert np.allclose(c.as_vec(), case["expected"], atol=case["abs_tol"])


def test_matmul_ladder_one_kernel_each(dev, golden):
    for case in golden["matmul_formula"]:
        a, b = formula_operands(case)
        c = Tensor.from_ndarray(dev, a).matmul(Tensor.from_ndarray(dev, b)).realize()
        assert c.last_launches() == 1            # matmul = 1 kernel (tensor/src/test/unit/fusion.rs:29-33)
        assert np.max(np.abs(c.as_ndarray() - a.astype(np.float64) @ b.astype(np.float64))) < case["abs_tol"], case["name"]


def test_transformer_known_answers(dev, golden):
    for case in golden["rms_norm"]:
        y = Tensor.from_ndarray(dev, np.array(case["x"], np.float32)).rms_norm(-1, case["eps"]).realize()
        assert np.max(np.abs(y.as_ndarray() - np.array(case["expected"]))) < case["abs_tol"]
    for case in golden["rope"]:
        x = Tensor.from_ndarray(dev, np.array(case["x"], np.float32).reshape(1, 1, 4))
        cos = Tensor.from_ndarray(dev, np.array(case["cos"], np.float32).reshape(1, 1, 2))
        sin = Tensor.from_ndarray(dev, np.array(case["sin"], np.float32).reshape(1, 1, 2))
        y = x.apply_rotary_emb(cos, sin, case["interleaved"]).realize()
        assert y.shape() == (1, 1, 4)
        assert np.max(np.abs(y.as_vec() - np.array(case["expected"]))) < case["abs_tol"], case["name"]
    for case in golden["sdpa"]:
        q, k, v = (Tensor.from_ndarray(dev, np.array(case[n], np.float32)[None, None]) for n in ("q", "k", "v"))
        o = q.scaled_dot_product_attention(k, v, is_causal=case["causal"], softcap=case["softcap"] or None).realize()
        assert o.last_launches() == 1            # one fused kernel instead of the reference's >= 5
        out = o.as_ndarray()
        if "expected_row0" in case:
            assert np.max(np.abs(out[0, 0, 0] - np.array(case["expected_row0"]))) < case["abs_tol"]
        if case.get("finite"):
            assert np.all(np.isfinite(out))


def test_linear_uses_transposed_weights_without_copy(dev):
    rng = np.random.default_rng(0)
    x = orc.round_bf16(rng.standard_normal((96, 128), dtype=np.float32))
    w = orc.round_bf16(rng.standard_normal((256, 128), dtype=np.float32) * np.float32(0.1))     # [out, in]
    y = bf(dev, x).linear(bf(dev, w)).realize()
    assert y.last_launches() == 1
    assert_close(orc.bf16_to_f32(y.as_ndarray()), orc.matmul_f32(x, w.T.copy()), mk.MK_BF16, "linear")


def test_fusions_keep_kernel_counts(dev):
    rng = np.random.default_rng(1)
    x = orc.round_bf16(rng.standard_normal((64, 128), dtype=np.float32))
    wg, wu = (orc.round_bf16(rng.standard_normal((128, 256), dtype=np.float32) * np.float32(0.1)) for _ in range(2))
    wd = orc.round_bf16(rng.standard_normal((256, 128), dtype=np.float32) * np.float32(0.1))
    X, Wg, Wu, Wd = bf(dev, x), bf(dev, wg), bf(dev, wu), bf(dev, wd)
    ff = X.matmul(Wg).silu().try_mul(X.matmul(Wu))
    out = X.try_add(ff.matmul(Wd)).realize()
    # gate and up products with the SwiGLU gate in the store of ONE GEMM kernel, then the down GEMM with the
    # residual add in its epilogue
    assert out.last_launches() == 2
    # a chain of bf16 ops: the oracle rounds to bf16 where the GPU stores bf16 (the per-op bar of
    # 2e-2 / 1e-2 is defined for one op on bf16-rounded inputs, not for compounded rounding)
    rb = orc.round_bf16
    ff_ref = rb(orc.swiglu_f32(orc.matmul_f32(x, wg), orc.matmul_f32(x, wu)))     # both products stay f32 until the gate is applied
    ref = x + orc.matmul_f32(ff_ref, wd)
    assert_close(orc.bf16_to_f32(out.as_ndarray()), ref, mk.MK_BF16, "ffn block")


@pytest.mark.parametrize("dtype", [mk.MK_F32, mk.MK_BF16])
def test_sigmoid_and_its_gate_fusions(dev, dtype):
    """sigmoid alone, x.sigmoid() * x (= silu) and sigmoid(g) * u: one kernel each
    (tensor/src/test/unit/fusion.rs:50-56)."""
    rng = np.random.default_rng(11)
    g = rng.standard_normal((37, 129), dtype=np.float32) * np.float32(3)
    u = rng.standard_normal((37, 129), dtype=np.float32)
    if dtype == mk.MK_BF16:
        g, u = orc.round_bf16(g), orc.round_bf16(u)
        mkt = lambda a: bf(dev, a)
        back = lambda t: orc.bf16_to_f32(t.as_ndarray())
    else:
        mkt = lambda a: Tensor.from_ndarray(dev, a)
        back = lambda t: t.as_ndarray()
    G, U = mkt(g), mkt(u)
    s = G.sigmoid().realize()
    assert s.last_launches() == 1
    assert_close(back(s), orc.sigmoid_f32(g), dtype, "sigmoid")
    for y in (G.sigmoid().try_mul(G), G.try_mul(G.sigmoid())):
        y.realize()
        assert y.last_launches() == 1
        assert_close(back(y), orc.silu_f32(g), dtype, "sigmoid(x) * x")
    y = G.sigmoid().try_mul(U).realize()
    assert y.last_launches() == 1
    assert_close(back(y), orc.sigmoid_f32(g) * u, dtype, "sigmoid gate")
    # a leaf plus a bias row (no product to fuse into): the broadcast add
    bias = rng.standard_normal((129,), dtype=np.float32)
    if dtype == mk.MK_BF16:
        bias = orc.round_bf16(bias)
    y = G.try_add(mkt(bias)).realize()
    assert y.last_launches() == 1
    assert_close(back(y), g + bias[None, :], dtype, "leaf + bias row")


def test_gate_block_of_two_products_is_one_kernel(dev):
    """`(x @ w1 + b1).sigmoid() * (x @ w2 + b2)` = 1 kernel (tensor/src/test/unit/fusion.rs:58-67), and the same
    block with silu, without biases, and with the operands of the product swapped."""
    rng = np.random.default_rng(12)
    x = orc.round_bf16(rng.standard_normal((48, 64), dtype=np.float32))
    w1, w2 = (orc.round_bf16(rng.standard_normal((64, 96), dtype=np.float32) * np.float32(0.2)) for _ in range(2))
    b1, b2 = (orc.round_bf16(rng.standard_normal((96,), dtype=np.float32)) for _ in range(2))
    X, W1, W2, B1, B2 = (bf(dev, t) for t in (x, w1, w2, b1, b2))
    g, u = orc.matmul_f32(x, w1), orc.matmul_f32(x, w2)
    back = lambda t: orc.bf16_to_f32(t.as_ndarray())
    cases = [
        (lambda: X.matmul(W1).try_add(B1).sigmoid().try_mul(X.matmul(W2).try_add(B2)), orc.sigmoid_f32(g + b1) * (u + b2), "sigmoid gate block"),
        (lambda: X.matmul(W2).try_add(B2).try_mul(X.matmul(W1).try_add(B1).sigmoid()), orc.sigmoid_f32(g + b1) * (u + b2), "swapped operands"),
        (lambda: X.matmul(W1).sigmoid().try_mul(X.matmul(W2)), orc.sigmoid_f32(g) * u, "sigmoid gate, no biases"),
        (lambda: X.matmul(W1).try_add(B1).silu().try_mul(X.matmul(W2)), orc.silu_f32(g + b1) * u, "silu gate with a gate bias"),
        (lambda: X.linear(bf(dev, np.ascontiguousarray(w1.T)), B1).sigmoid().try_mul(X.linear(bf(dev, np.ascontiguousarray(w2.T)), B2)),
         orc.sigmoid_f32(g + b1) * (u + b2), "two `linear`s with biases"),
    ]
    for build, ref, what in cases:
        y = build().realize()
        assert y.last_launches() == 1, what
        assert_close(back(y), ref, mk.MK_BF16, what)
    # the whole feed-forward of the reference's test: gate block, then the down projection with its bias = 2 kernels
    # (tensor/src/test/unit/fusion.rs:106-114)
    wd = orc.round_bf16(rng.standard_normal((96, 64), dtype=np.float32) * np.float32(0.2))
    bd = orc.round_bf16(rng.standard_normal((64,), dtype=np.float32))
    Wd, Bd = bf(dev, wd), bf(dev, bd)
    ff = X.matmul(W1).try_add(B1).sigmoid().try_mul(X.matmul(W2).try_add(B2))
    out = ff.matmul(Wd).try_add(Bd).realize()
    assert out.last_launches() == 2
    ff_ref = orc.round_bf16(orc.sigmoid_f32(g + b1) * (u + b2))
    assert_close(back(out), orc.matmul_f32(ff_ref, wd) + bd, mk.MK_BF16, "gate block + down projection")
    # f32 stays exact on the FMA kernels: two products with their biases, then the gate
    Xf, W1f, W2f, B1f, B2f = (Tensor.from_ndarray(dev, t) for t in (x, w1, w2, b1, b2))
    y = Xf.matmul(W1f).try_add(B1f).sigmoid().try_mul(Xf.matmul(W2f).try_add(B2f)).realize()
    assert y.last_launches() == 3
    assert_close(y.as_ndarray(), orc.sigmoid_f32(g + b1) * (u + b2), mk.MK_F32, "f32 gate block")


def test_batched_matmul_and_views(dev):
    rng = np.random.default_rng(2)
    a = rng.standard_normal((3, 17, 24), dtype=np.float32)
    b = rng.standard_normal((3, 24, 9), dtype=np.float32)
    c = Tensor.from_ndarray(dev, a).matmul(Tensor.from_ndarray(dev, b)).realize().as_ndarray()
    assert_close(c, np.stack([orc.matmul_f32(a[i], b[i]) for i in range(3)]), mk.MK_F32, "batched")
    p = Tensor.from_ndarray(dev, a).try_permute((1, 0, 2)).try_reshape((17, 72)).realize().as_ndarray()
    assert np.array_equal(p, a.transpose(1, 0, 2).reshape(17, 72))


def decoder_layer_api(dev, x_bits, w, batch, seq, n_q, n_kv, hd, eps=1e-5):
    """The op order the reference's Tensor API implies for a pre-norm Llama block."""
    hidden = x_bits.shape[-1]
    h = Tensor.from_ndarray(dev, x_bits.reshape(batch * seq, hidden))
    W = {k: Tensor.from_ndarray(dev, v) for k, v in w.items()}
    cos_np, sin_np = orc.rope_tables(seq, hd)
    cos = Tensor.from_ndarray(dev, cos_np.reshape(1, seq, 1, hd // 2))
    sin = Tensor.from_ndarray(dev, sin_np.reshape(1, seq, 1, hd // 2))
    n1 = h.rms_norm(-1, eps).cast(mk.MK_BF16)
    q = n1.matmul(W["wq"]).try_reshape((batch, seq, n_q, hd)).apply_rotary_emb(cos, sin, False).try_permute((0, 2, 1, 3))
    k = n1.matmul(W["wk"]).try_reshape((batch, seq, n_kv, hd)).apply_rotary_emb(cos, sin, False).try_permute((0, 2, 1, 3))
    v = n1.matmul(W["wv"]).try_reshape((batch, seq, n_kv, hd)).try_permute((0, 2, 1, 3))
    a = q.scaled_dot_product_attention(k, v, is_causal=True).try_permute((0, 2, 1, 3)).try_reshape((batch * seq, n_q * hd))
    h = h.try_add(a.matmul(W["wo"]))
    n2 = h.rms_norm(-1, eps).cast(mk.MK_BF16)
    ff = n2.matmul(W["wgate"]).silu().try_mul(n2.matmul(W["wup"]))
    return h.try_add(ff.matmul(W["wdown"]))


@pytest.mark.parametrize("cfg", [(2, 64, 4, 2, 128, 512, 768), (1, 300, 8, 2, 128, 1024, 1408)])
def test_decoder_layer_through_api(dev, cfg):
    batch, seq, n_q, n_kv, hd, hidden, ffn = cfg
    assert n_q * hd == hidden
    rng = np.random.default_rng(0)
    x = orc.normal_bf16(rng, (batch, seq, hidden), 1.0)
    w = orc.decoder_layer_weights(rng, hidden, n_q, n_kv, hd, ffn, sigma=0.02)
    out = decoder_layer_api(dev, x, w, batch, seq, n_q, n_kv, hd).realize()
    assert dev.kernel_status() == 0
    got = orc.bf16_to_f32(out.as_ndarray()).reshape(batch, seq, hidden)
    ref = orc.decoder_layer_f32(x, w, batch, seq, n_q, n_kv, hd)
    assert_close(got, ref, mk.MK_BF16, f"decoder layer {cfg}")
    # 2 norms (cast fused) + 6 GEMMs (2 with fused residual, 1 computing gate and up with the SwiGLU gate in its
    # store) + 2 RoPE + attention, and no transposition copies: attention reads [B,S,H,D] in place and stores
    # [B,S,H,D] directly
    assert out.last_launches() == 11


def test_config4_full_size_layer_causal_prefix_vs_oracle(dev):
    """The full decoder-layer configuration (batch 8 x seq 2048, hidden 4096, 32 q / 8 kv heads,
    head 128, FFN 14336) through the Tensor API.  Every op of the layer is per-token except causal
    attention, which only looks backwards, so the first P tokens of a batch element depend on
    nothing else: the oracle evaluates those prefixes and must match the same rows of the full run."""
    batch, seq, n_q, n_kv, hd, hidden, ffn = 8, 2048, 32, 8, 128, 4096, 14336
    rng = np.random.default_rng(0)
    x = orc.normal_bf16(rng, (batch, seq, hidden), 1.0)
    w = orc.decoder_layer_weights(rng, hidden, n_q, n_kv, hd, ffn, sigma=0.02)
    out = decoder_layer_api(dev, x, w, batch, seq, n_q, n_kv, hd).realize()
    assert dev.kernel_status() == 0
    assert out.last_launches() == 11
    got = orc.bf16_to_f32(out.as_ndarray()).reshape(batch, seq, hidden)
    assert np.all(np.isfinite(got))
    # The chain as a whole.  Eleven bf16 results in a row, the last one a sum of 14336 products of rounded activations: a
    # difference in the last bit of one intermediate moves later roundings, and two evaluations that differ anywhere
    # upstream end ~1e-2 (absolute, rms) apart at the output.  That holds between CPU evaluations as well -- the oracle
    # rounded after every op (what the dtypes of the reference's bf16 graph dictate, tensor/src/reduce.rs:673-691) and
    # the oracle rounded only where a fused kernel stores differ beyond 2e-2 rel + 1e-2 abs on ~4 % of the elements -- so
    # the element-wise bar is applied kernel by kernel on identical inputs (next test) and the chain is bounded in
    # relative rms: against the pure-f32 oracle it must be no further than the reference's own bf16 arithmetic is.
    for b, prefix in ((0, 160), (7, 96)):
        xs = x[b:b + 1, :prefix]
        g = got[b:b + 1, :prefix]
        ref = orc.decoder_layer_f32(xs, w, 1, prefix, n_q, n_kv, hd)
        ref_o = orc.decoder_layer_f32(xs, w, 1, prefix, n_q, n_kv, hd, round_boundaries="ops")
        ref_k = orc.decoder_layer_f32(xs, w, 1, prefix, n_q, n_kv, hd, round_boundaries="kernels")
        scale = float(np.sqrt(np.mean(ref ** 2)))

        def rms_rel(a, r):
            return float(np.sqrt(np.mean((a - r) ** 2))) / scale

        def outside(a, r):
            return float(np.mean(np.abs(a - r) > 1e-2 + 2e-2 * np.abs(r)))
        d_f32, d_ops, d_k, ops_f32 = rms_rel(g, ref), rms_rel(g, ref_o), rms_rel(g, ref_k), rms_rel(ref_o, ref)
        max_norm = float(np.abs(g - ref).max() / np.abs(ref).max())
        print(f"config 4 batch element {b}: rms rel vs pure-f32 oracle {d_f32:.3e} (normalised max {max_norm:.3e}), vs per-op bf16 "
              f"oracle {d_ops:.3e}, vs kernel-boundary oracle {d_k:.3e}; per-op bf16 oracle vs pure-f32 oracle {ops_f32:.3e}; fraction "
              f"outside the element-wise bar: GPU vs per-op oracle {outside(g, ref_o):.3f}, kernel-boundary oracle vs per-op oracle "
              f"{outside(ref_k, ref_o):.3f}")
        assert d_f32 < 1e-2 and max_norm < 2e-2, f"config 4, batch element {b}: rms rel {d_f32:.3e}, normalised max {max_norm:.3e}"
        assert d_f32 <= ops_f32 * 1.05 + 1e-4, f"further from the f32 oracle ({d_f32:.3e}) than the reference's own bf16 graph is ({ops_f32:.3e})"
        assert d_ops < 1e-2 and d_k < 1e-2
        # ... and no further from the reference's bf16 arithmetic than an equally valid CPU evaluation is
        assert outside(g, ref_o) <= outside(ref_k, ref_o) * 1.25 + 5e-3
    # batch elements are independent: identical inputs give identical outputs
    x2 = x.copy()
    x2[3] = x2[5]
    out2 = decoder_layer_api(dev, x2, w, batch, seq, n_q, n_kv, hd).realize()
    o2 = out2.as_ndarray().reshape(batch, seq, hidden)
    assert np.array_equal(o2[3], o2[5])
    assert np.array_equal(o2[0], out.as_ndarray().reshape(batch, seq, hidden)[0])


def test_config4_full_size_every_kernel_elementwise_on_identical_inputs(dev):
    """Config 4 at full size, kernel by kernel: every intermediate the layer's eleven kernels store is read back, and each
    kernel's output is compared element-wise (2e-2 relative + 1e-2 absolute) with the oracle's evaluation of THAT op on the
    inputs the kernel itself consumed (f32 arithmetic, one rounding to bf16 where the kernel stores).  Sampled token
    prefixes of two batch elements; attention over the prefix's causal window."""
    batch, seq, n_q, n_kv, hd, hidden, ffn = 8, 2048, 32, 8, 128, 4096, 14336
    rng = np.random.default_rng(0)
    x = orc.normal_bf16(rng, (batch, seq, hidden), 1.0)
    w = orc.decoder_layer_weights(rng, hidden, n_q, n_kv, hd, ffn, sigma=0.02)
    h0 = Tensor.from_ndarray(dev, x.reshape(batch * seq, hidden))
    W = {k: Tensor.from_ndarray(dev, v) for k, v in w.items()}
    cos_np, sin_np = orc.rope_tables(seq, hd)
    cos = Tensor.from_ndarray(dev, cos_np.reshape(1, seq, 1, hd // 2))
    sin = Tensor.from_ndarray(dev, sin_np.reshape(1, seq, 1, hd // 2))
    launches = 0

    def stored(t):          # one kernel per stage: realize it and keep its output
        nonlocal launches
        t.realize()
        launches += t.last_launches()
        return t

    n1 = stored(h0.rms_norm(-1, 1e-5).cast(mk.MK_BF16))
    q_pre, k_pre, v_pre = (stored(n1.matmul(W[n])) for n in ("wq", "wk", "wv"))
    q = stored(q_pre.try_reshape((batch, seq, n_q, hd)).apply_rotary_emb(cos, sin, False))
    k = stored(k_pre.try_reshape((batch, seq, n_kv, hd)).apply_rotary_emb(cos, sin, False))
    v = v_pre.try_reshape((batch, seq, n_kv, hd))
    a = stored(q.try_permute((0, 2, 1, 3)).scaled_dot_product_attention(k.try_permute((0, 2, 1, 3)), v.try_permute((0, 2, 1, 3)), is_causal=True)
               .try_permute((0, 2, 1, 3)).try_reshape((batch * seq, n_q * hd)))
    h = stored(h0.try_add(a.matmul(W["wo"])))
    n2 = stored(h.rms_norm(-1, 1e-5).cast(mk.MK_BF16))
    ff = stored(n2.matmul(W["wgate"]).silu().try_mul(n2.matmul(W["wup"])))
    out = stored(h.try_add(ff.matmul(W["wdown"])))
    assert dev.kernel_status() == 0
    assert launches == 11
    bf, rb = orc.bf16_to_f32, orc.round_bf16
    G = {name: t.as_ndarray() for name, t in dict(n1=n1, q_pre=q_pre, k_pre=k_pre, v=v_pre, q=q, k=k, a=a, h=h, n2=n2, ff=ff, out=out).items()}
    Wf = {name: bf(v) for name, v in w.items()}
    xf = bf(x).reshape(batch * seq, hidden)
    for b, prefix in ((0, 160), (7, 96)):
        r = slice(b * seq, b * seq + prefix)         # token rows of this prefix
        tok = lambda name: bf(G[name].reshape(batch * seq, -1)[r])      # noqa: E731
        checks = {
            "rms_norm 1": (tok("n1"), rb(orc.rms_norm_f32(xf[r], 1e-5))),
            "q projection": (tok("q_pre"), rb(orc.matmul_f32(tok("n1"), Wf["wq"]))),
            "k projection": (tok("k_pre"), rb(orc.matmul_f32(tok("n1"), Wf["wk"]))),
            "v projection": (tok("v"), rb(orc.matmul_f32(tok("n1"), Wf["wv"]))),
            "rope q": (tok("q"), rb(orc.rope_f32(tok("q_pre").reshape(1, prefix, n_q, hd), cos_np[:prefix], sin_np[:prefix], False, row_div=n_q)).reshape(prefix, -1)),
            "rope k": (tok("k"), rb(orc.rope_f32(tok("k_pre").reshape(1, prefix, n_kv, hd), cos_np[:prefix], sin_np[:prefix], False, row_div=n_kv)).reshape(prefix, -1)),
            "residual 1 (o projection + x)": (tok("h"), rb(xf[r] + orc.matmul_f32(tok("a"), Wf["wo"]))),
            "rms_norm 2": (tok("n2"), rb(orc.rms_norm_f32(tok("h"), 1e-5))),
            "gated feed-forward": (tok("ff"), rb(orc.swiglu_f32(orc.matmul_f32(tok("n2"), Wf["wgate"]), orc.matmul_f32(tok("n2"), Wf["wup"])))),
            "residual 2 (down projection + h)": (tok("out"), rb(tok("h") + orc.matmul_f32(tok("ff"), Wf["wdown"]))),
        }
        qh, kh, vh = (np.ascontiguousarray(tok(n).reshape(1, prefix, -1, hd).transpose(0, 2, 1, 3)) for n in ("q", "k", "v"))
        att = rb(orc.sdpa_f32(qh, kh, vh, causal=True))
        checks["attention"] = (tok("a"), np.ascontiguousarray(att.transpose(0, 2, 1, 3)).reshape(prefix, -1))
        for name, (got_k, want) in checks.items():
            assert_close(got_k, want, mk.MK_BF16, f"config 4, batch element {b}, kernel '{name}'")


def test_plan_replay_matches_eager_bit_for_bit(dev):
    """Prepare once, execute many (runtime/src/execution_plan.rs:88-106, 168-181): the decoder layer is
    recorded into a plan; replaying it gives the bits of the eager realisation, also after the input
    tensor has been overwritten in place, with one launch call per replay."""
    batch, seq, n_q, n_kv, hd, hidden, ffn = 2, 128, 4, 2, 128, 512, 768
    rng = np.random.default_rng(4)
    x1 = orc.normal_bf16(rng, (batch, seq, hidden), 1.0)
    x2 = orc.normal_bf16(rng, (batch, seq, hidden), 1.0)
    w = orc.decoder_layer_weights(rng, hidden, n_q, n_kv, hd, ffn, sigma=0.02)
    eager1 = decoder_layer_api(dev, x1, w, batch, seq, n_q, n_kv, hd).realize().as_ndarray()
    eager2 = decoder_layer_api(dev, x2, w, batch, seq, n_q, n_kv, hd).realize().as_ndarray()
    assert not np.array_equal(eager1, eager2)

    # the same graph, built on an input tensor we keep a handle to
    h_in = Tensor.from_ndarray(dev, x1.reshape(batch * seq, hidden))
    W = {k: Tensor.from_ndarray(dev, v) for k, v in w.items()}
    cos_np, sin_np = orc.rope_tables(seq, hd)
    cos = Tensor.from_ndarray(dev, cos_np.reshape(1, seq, 1, hd // 2))
    sin = Tensor.from_ndarray(dev, sin_np.reshape(1, seq, 1, hd // 2))
    n1 = h_in.rms_norm(-1, 1e-5).cast(mk.MK_BF16)
    q = n1.matmul(W["wq"]).try_reshape((batch, seq, n_q, hd)).apply_rotary_emb(cos, sin, False).try_permute((0, 2, 1, 3))
    k = n1.matmul(W["wk"]).try_reshape((batch, seq, n_kv, hd)).apply_rotary_emb(cos, sin, False).try_permute((0, 2, 1, 3))
    v = n1.matmul(W["wv"]).try_reshape((batch, seq, n_kv, hd)).try_permute((0, 2, 1, 3))
    a = q.scaled_dot_product_attention(k, v, is_causal=True).try_permute((0, 2, 1, 3)).try_reshape((batch * seq, n_q * hd))
    h = h_in.try_add(a.matmul(W["wo"]))
    n2 = h.rms_norm(-1, 1e-5).cast(mk.MK_BF16)
    out = h.try_add(n2.matmul(W["wgate"]).silu().try_mul(n2.matmul(W["wup"])).matmul(W["wdown"]))

    before = dev.launch_count()
    plan = out.compile()
    assert dev.launch_count() == before            # recording runs nothing
    assert plan.kernel_count() == 11 and out.last_launches() == 11
    plan.launch()
    assert dev.launch_count() == before + 11
    assert dev.kernel_status() == 0
    assert np.array_equal(out.as_ndarray(), eager1)
    h_in.write(x2.reshape(batch * seq, hidden))
    plan.launch().launch()                          # replays are idempotent on unchanged inputs
    assert dev.kernel_status() == 0
    assert np.array_equal(out.as_ndarray(), eager2)
    # a realized tensor has nothing left to record
    with pytest.raises(mk.MorokError):
        out.compile()
    plan.free()


def test_linear_bias_and_gemm_method(dev):
    """`linear` with a bias is one kernel (bias added in the GEMM's store); `gemm` composes
    alpha * A @ B + beta * C like the reference (tensor/src/matmul.rs:112-133, 161-187)."""
    rng = np.random.default_rng(6)
    x = orc.round_bf16(rng.standard_normal((96, 128), dtype=np.float32))
    w = orc.round_bf16(rng.standard_normal((256, 128), dtype=np.float32) * np.float32(0.1))     # [out, in]
    bias = orc.round_bf16(rng.standard_normal((256,), dtype=np.float32))
    y = bf(dev, x).linear(bf(dev, w), bf(dev, bias)).realize()
    assert y.last_launches() == 1
    assert_close(orc.bf16_to_f32(y.as_ndarray()), orc.matmul_f32(x, w.T.copy()) + bias[None, :], mk.MK_BF16, "linear + bias")

    a = rng.standard_normal((40, 24), dtype=np.float32)
    b = rng.standard_normal((24, 56), dtype=np.float32)
    c = rng.standard_normal((40, 56), dtype=np.float32)
    A, B, Cc = (Tensor.from_ndarray(dev, t) for t in (a, b, c))
    g = A.gemm(B, alpha=0.5, beta=2.0, c=Cc).realize().as_ndarray()
    assert_close(g, np.float32(0.5) * orc.matmul_f32(a, b) + np.float32(2.0) * c, mk.MK_F32, "gemm alpha beta")
    At, Bt = Tensor.from_ndarray(dev, a.T.copy()), Tensor.from_ndarray(dev, b.T.copy())
    g2 = At.gemm(Bt, trans_a=True, trans_b=True, c=Cc).realize()
    assert_close(g2.as_ndarray(), orc.matmul_f32(a, b) + c, mk.MK_F32, "gemm trans_a trans_b + C")


def test_plan_with_two_launch_kernels(dev):
    """A decoding step -- a few rows through a K-split GEMM, then a few query rows against a long key
    stream -- recorded as a plan: both paths take scratch memory while the plan is being recorded, and the
    replay must equal the eager run bit for bit."""
    rng = np.random.default_rng(12)
    rows, hidden, heads, kv_heads, hd, keys = 8, 4096, 32, 8, 128, 2048
    x = orc.normal_bf16(rng, (rows, hidden), 1.0)
    w = orc.normal_bf16(rng, (hidden, heads * hd), 0.02)
    k = orc.normal_bf16(rng, (rows, kv_heads, keys, hd), 1.0)
    v = orc.normal_bf16(rng, (rows, kv_heads, keys, hd), 1.0)

    def graph(X, W, K, V):
        q = X.matmul(W).try_reshape((rows, 1, heads, hd)).try_permute((0, 2, 1, 3))       # [rows, heads, 1, hd]
        return q.scaled_dot_product_attention(K, V)

    T = lambda a: Tensor.from_ndarray(dev, a)      # noqa: E731
    eager = graph(T(x), T(w), T(k), T(v)).realize()
    assert eager.last_launches() == 4                  # split GEMM + merge, split attention + merge
    out = graph(T(x), T(w), T(k), T(v))
    plan = out.compile()
    assert plan.kernel_count() == 4
    plan.launch()
    assert dev.kernel_status() == 0
    assert np.array_equal(out.as_ndarray(), eager.as_ndarray())
    ref = orc.sdpa_f32(orc.round_bf16(orc.matmul_f32(orc.bf16_to_f32(x), orc.bf16_to_f32(w))).reshape(rows, 1, heads, hd).transpose(0, 2, 1, 3),
                       orc.bf16_to_f32(k), orc.bf16_to_f32(v))
    assert_close(orc.bf16_to_f32(out.as_ndarray()), ref, mk.MK_BF16, "decode step")
    plan.free()
