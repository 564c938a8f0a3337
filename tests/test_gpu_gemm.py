"""GEMM parity on the GPU, through mk_gemm of the C ABI, against the CPU oracle."""
import os
import sys

import numpy as np
import pytest

import morok_b200 as mk
from morok_b200 import _ffi
from oracle import oracle as orc
from gpu_util import NP_OF, assert_close, dev, to_f32, to_storage  # noqa: F401

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
from make_golden import formula_operands  # noqa: E402

pytestmark = pytest.mark.gpu


def run_gemm(dev, a_f32, b_f32, dt_in, dt_out, trans_b=False, add_f32=None):
    """a [M,K], b [K,N] given as f32 values; storage conversion happens here.  Returns f32 result."""
    M, K = a_f32.shape
    N = b_f32.shape[1]
    a_s = to_storage(a_f32, dt_in)
    b_s = to_storage(np.ascontiguousarray(b_f32.T) if trans_b else b_f32, dt_in)
    A, B = dev.from_numpy(a_s), dev.from_numpy(b_s)
    Cb = dev.alloc(max(M * N, 1) * mk.dtype_size(dt_out))
    D = dev.from_numpy(to_storage(add_f32, dt_out)) if add_f32 is not None else None
    dev.gemm(A, B, Cb, M, N, K, dt_in, dt_out, trans_b=trans_b, add=D)
    assert dev.kernel_status() == 0
    out = Cb.copyout(np.float32 if dt_out == mk.MK_F32 else (np.uint16 if dt_out == mk.MK_BF16 else np.float16), (M, N)) \
        if M * N else np.zeros((M, N), np.float32)
    for b in (A, B, Cb) + ((D,) if D else ()):
        b.free()
    return to_f32(out, dt_out)


def test_f32_known_answers(dev, golden):
    for case in golden["matmul_small"]:
        a = np.array(case["a"], np.float32).reshape(case["m"], case["k"])
        b = np.array(case["b"], np.float32).reshape(case["k"], case["n"])
        c = run_gemm(dev, a, b, mk.MK_F32, mk.MK_F32)
        assert np.max(np.abs(c.ravel() - np.array(case["expected"]))) < case["abs_tol"], case["name"]


def test_f32_formula_ladder_bit_exact_with_oracle(dev, golden):
    for case in golden["matmul_formula"]:
        a, b = formula_operands(case)
        c = run_gemm(dev, a, b, mk.MK_F32, mk.MK_F32)
        ref64 = a.astype(np.float64) @ b.astype(np.float64)
        assert np.max(np.abs(c - ref64)) < case["abs_tol"], case["name"]
        orc_c = orc.matmul_f32(a, b)
        assert_close(c, orc_c, mk.MK_F32, case["name"])
        # same fmaf chain in the same order on both sides -> identical bits
        assert np.array_equal(c, orc_c), f"{case['name']}: {(c != orc_c).sum()} elements differ in the last bits"


def test_f32_config1_uniform_seed0(dev):
    rng = np.random.default_rng(0)
    a, b = orc.uniform_f32(rng, (1024, 1024)), orc.uniform_f32(rng, (1024, 1024))
    c = run_gemm(dev, a, b, mk.MK_F32, mk.MK_F32)
    ref = orc.matmul_f32(a, b)
    assert_close(c, ref, mk.MK_F32, "config 1")
    assert np.array_equal(c, ref)


@pytest.mark.parametrize("shape", [(1, 1, 1), (1, 17, 1), (17, 1, 33), (129, 65, 31), (5, 0, 4), (0, 3, 4), (3, 7, 0),
                                   (130, 257, 131)])
def test_f32_edge_shapes(dev, shape):
    m, k, n = shape
    rng = np.random.default_rng(3)
    a, b = orc.uniform_f32(rng, (m, k)), orc.uniform_f32(rng, (k, n))
    c = run_gemm(dev, a, b, mk.MK_F32, mk.MK_F32)
    assert_close(c, orc.matmul_f32(a, b), mk.MK_F32, str(shape))


TC_SHAPES = [(128, 64, 256), (128, 128, 256), (128, 256, 512), (256, 512, 512), (384, 192, 768),
             (300, 200, 520), (1, 8, 8), (127, 72, 264), (640, 1024, 1280)]


@pytest.mark.parametrize("shape", TC_SHAPES)
@pytest.mark.parametrize("dt", [mk.MK_BF16, mk.MK_F16])
def test_tensor_core_gemm_vs_oracle(dev, shape, dt):
    m, k, n = shape
    rng = np.random.default_rng(m * 7 + k * 3 + n)
    a = to_f32(to_storage(rng.standard_normal((m, k), dtype=np.float32), dt), dt)
    b = to_f32(to_storage(rng.standard_normal((k, n), dtype=np.float32) * np.float32(0.05), dt), dt)
    ref = orc.matmul_f32(a, b)
    got = run_gemm(dev, a, b, dt, dt)
    assert_close(got, ref, dt, f"{shape} dt={dt}")
    # f32 output exposes the accumulator itself: products are exact, only the summation order differs
    got32 = run_gemm(dev, a, b, dt, mk.MK_F32)
    assert_close(got32, ref, mk.MK_F32, f"{shape} dt={dt} f32 out")


@pytest.mark.parametrize("shape", [(128, 64, 256), (300, 200, 520), (256, 512, 512), (64, 136, 40)])
def test_tensor_core_gemm_transposed_weights(dev, shape):
    """`linear` stores weights [out, in] (tensor/src/matmul.rs:161-177): trans_b = 1."""
    m, k, n = shape
    rng = np.random.default_rng(11)
    a = orc.round_bf16(rng.standard_normal((m, k), dtype=np.float32))
    b = orc.round_bf16(rng.standard_normal((k, n), dtype=np.float32) * np.float32(0.05))
    assert_close(run_gemm(dev, a, b, mk.MK_BF16, mk.MK_BF16, trans_b=True), orc.matmul_f32(a, b), mk.MK_BF16, str(shape))


@pytest.mark.parametrize("dt_in,dt_out", [(mk.MK_BF16, mk.MK_BF16), (mk.MK_BF16, mk.MK_F32), (mk.MK_F32, mk.MK_F32)])
def test_gemm_add_epilogue(dev, dt_in, dt_out):
    m, k, n = 200, 136, 264
    rng = np.random.default_rng(5)
    a = to_f32(to_storage(rng.standard_normal((m, k), dtype=np.float32), dt_in), dt_in)
    b = to_f32(to_storage(rng.standard_normal((k, n), dtype=np.float32) * np.float32(0.1), dt_in), dt_in)
    d = to_f32(to_storage(rng.standard_normal((m, n), dtype=np.float32), dt_out), dt_out)
    got = run_gemm(dev, a, b, dt_in, dt_out, add_f32=d)
    assert_close(got, orc.matmul_f32(a, b) + d, dt_out, "add epilogue")


@pytest.mark.parametrize("shape", [(33, 17, 9), (64, 20, 130), (5, 3, 2)])
def test_bf16_shapes_without_16_byte_rows_use_fma_kernel(dev, shape):
    m, k, n = shape
    rng = np.random.default_rng(9)
    a = orc.round_bf16(rng.standard_normal((m, k), dtype=np.float32))
    b = orc.round_bf16(rng.standard_normal((k, n), dtype=np.float32))
    assert_close(run_gemm(dev, a, b, mk.MK_BF16, mk.MK_BF16), orc.matmul_f32(a, b), mk.MK_BF16, str(shape))


def test_bf16_k_zero_gives_zeros(dev):
    c = run_gemm(dev, np.zeros((4, 0), np.float32), np.zeros((0, 8), np.float32), mk.MK_BF16, mk.MK_BF16)
    assert c.shape == (4, 8) and np.all(c == 0)


def test_bf16_batched_broadcast(dev):
    """Batched matmul with a broadcast right operand (stride_b = 0)."""
    bsz, m, k, n = 3, 128, 64, 256
    rng = np.random.default_rng(2)
    a = orc.round_bf16(rng.standard_normal((bsz, m, k), dtype=np.float32))
    b = orc.round_bf16(rng.standard_normal((k, n), dtype=np.float32) * np.float32(0.1))
    A, B = dev.from_numpy(orc.f32_to_bf16(a)), dev.from_numpy(orc.f32_to_bf16(b))
    Cb = dev.alloc(bsz * m * n * 2)
    dev.gemm(A, B, Cb, m, n, k, mk.MK_BF16, batch=bsz, stride_a=m * k, stride_b=0, stride_c=m * n)
    assert dev.kernel_status() == 0
    got = orc.bf16_to_f32(Cb.copyout(np.uint16, (bsz, m, n)))
    for i in range(bsz):
        assert_close(got[i], orc.matmul_f32(a[i], b), mk.MK_BF16, f"batch {i}")
    for x in (A, B, Cb):
        x.free()


def test_config2_full_size_sampled_rows_and_linearity(dev):
    """bf16 M=8192 K=4096 N=14336: compare sampled rows with the oracle, and check the
    size-independent property C(A1+A2) = C(A1) + C(A2) on rows whose sums are exact in bf16."""
    M, K, N = 8192, 4096, 14336
    rng = np.random.default_rng(0)
    a_bits = orc.normal_bf16(rng, (M, K), 1.0)
    b_bits = orc.normal_bf16(rng, (K, N), 0.02)
    A, B = dev.from_numpy(a_bits), dev.from_numpy(b_bits)
    Cb = dev.alloc(M * N * 2)
    fill_poison(dev, Cb, M * N * 2)
    dev.gemm(A, B, Cb, M, N, K, mk.MK_BF16)
    assert dev.kernel_status() == 0
    c = Cb.copyout(np.uint16, (M, N))
    rows = np.array([0, 1, 127, 128, 129, 255, 256, 4095, 4096, 8063, 8064, 8190, 8191] + list(rng.integers(0, M, 21)))
    ref = orc.matmul_f32(orc.bf16_to_f32(a_bits[rows]), orc.bf16_to_f32(b_bits))
    assert_close(orc.bf16_to_f32(c[rows]), ref, mk.MK_BF16, "config 2 sampled rows")
    # every tile was written: C was filled with 0xFFFF (a NaN pattern) before the launch and no element kept it
    assert not np.any(c == 0xFFFF)
    # column checksum: sum over all rows of C equals (sum over rows of A) @ B within accumulated rounding
    colsum, ref_colsum = column_checksums(c, a_bits, b_bits)
    assert np.max(np.abs(colsum - ref_colsum)) < 0.02 * np.sqrt(M) + 2e-2 * np.max(np.abs(ref_colsum))
    for x in (A, B, Cb):
        x.free()


def fill_poison(dev, buf, nbytes):
    """0xFF in every byte of the buffer: a bf16 NaN pattern that no finished output element keeps."""
    _ffi.check(dev.lib.mk_memset_async(dev.h, buf.ptr, 0xFF, nbytes, None))
    dev.sync()


def column_checksums(c_bits, a_bits, b_bits, block=1024):
    """(sum over rows of C, (sum over rows of A) @ B), both in float64, evaluated block-wise to bound host memory."""
    M, N = c_bits.shape
    colsum = np.zeros(N, np.float64)
    for r in range(0, M, block):
        colsum += orc.bf16_to_f32(c_bits[r:r + block]).astype(np.float64).sum(axis=0)
    a_sum = np.zeros(a_bits.shape[1], np.float64)
    for r in range(0, M, block):
        a_sum += orc.bf16_to_f32(a_bits[r:r + block]).astype(np.float64).sum(axis=0)
    ref = np.zeros(N, np.float64)
    for k in range(0, a_bits.shape[1], block):
        ref += a_sum[k:k + block] @ orc.bf16_to_f32(b_bits[k:k + block]).astype(np.float64)
    return colsum, ref


def test_config5_full_size_sampled_rows_tile_seams_and_checksum(dev):
    """The sharded sweep's GEMM on one GPU: bf16 M=16384 K=8192 N=28672 (f32 accumulate, bf16 out).  32+ rows --
    first and last rows of 256-row tiles, the seams between tiles, random rows -- against the oracle; every
    element overwritten (0xFFFF poison); column checksum over the whole matrix."""
    M, K, N = 16384, 8192, 28672
    rng = np.random.default_rng(5)
    a_bits = orc.normal_bf16(rng, (M, K), 1.0)
    b_bits = orc.normal_bf16(rng, (K, N), 0.02)
    A, B = dev.from_numpy(a_bits), dev.from_numpy(b_bits)
    Cb = dev.alloc(M * N * 2)
    fill_poison(dev, Cb, M * N * 2)
    before = dev.launch_count()
    dev.gemm(A, B, Cb, M, N, K, mk.MK_BF16)
    assert dev.kernel_status() == 0
    assert dev.launch_count() - before == 1
    c = Cb.copyout(np.uint16, (M, N))
    seams = [0, 1, 127, 128, 255, 256, 257, 511, 512, 8191, 8192, 8447, 8448, 16127, 16128, 16255, 16256, 16382, 16383]
    rows = np.array(seams + list(rng.integers(0, M, 16)))
    assert len(rows) >= 32
    ref = orc.matmul_f32(orc.bf16_to_f32(a_bits[rows]), orc.bf16_to_f32(b_bits))
    got = orc.bf16_to_f32(c[rows])
    assert_close(got, ref, mk.MK_BF16, "config 5 GEMM sampled rows")
    rel_rms = float(np.sqrt(np.mean((got - ref) ** 2)) / np.sqrt(np.mean(ref ** 2)))
    assert rel_rms < 5e-3, f"relative rms error {rel_rms:.3e}"
    assert not np.any(c == 0xFFFF), "some output element was never written"
    colsum, ref_colsum = column_checksums(c, a_bits, b_bits)
    assert np.max(np.abs(colsum - ref_colsum)) < 0.03 * np.sqrt(M) + 2e-2 * np.max(np.abs(ref_colsum))
    for x in (A, B, Cb):
        x.free()
    dev.trim()


# ---------------------------------------------------------------------------------------------
# 8-bit float inputs (storage types dtype/src/lib.rs:142-143, accumulated in f32:
# tensor/src/reduce.rs:113).  Products of two 8-bit floats are exact in f32, so the FMA kernel is
# bit-identical with the oracle's fmaf chain; the tensor-core kernel (weights [N, K]) only differs
# in the order of the f32 additions.
# ---------------------------------------------------------------------------------------------
F8 = [mk.MK_F8E4M3, mk.MK_F8E5M2]


@pytest.mark.parametrize("dt", F8)
def test_fp8_fma_kernel_bit_exact(dev, dt):
    rng = np.random.default_rng(11)
    a = to_f32(to_storage(rng.standard_normal((70, 200), dtype=np.float32), dt), dt)
    b = to_f32(to_storage(rng.standard_normal((200, 90), dtype=np.float32), dt), dt)
    c = run_gemm(dev, a, b, dt, mk.MK_F32)                     # [K, N] weights: the FMA kernel
    assert np.array_equal(c, orc.matmul_f32(a, b))


@pytest.mark.parametrize("dt", F8)
@pytest.mark.parametrize("shape", [(128, 256, 256), (256, 512, 512), (300, 200 + 56, 520), (640, 1024, 1280), (100, 4096, 384)])
@pytest.mark.parametrize("dt_out", [mk.MK_F32, mk.MK_BF16])
def test_fp8_tensor_core_vs_oracle(dev, dt, shape, dt_out):
    M, K, N = shape
    rng = np.random.default_rng(M + K + N)
    a = to_f32(to_storage(rng.standard_normal((M, K), dtype=np.float32), dt), dt)
    b = to_f32(to_storage(rng.standard_normal((K, N), dtype=np.float32) * np.float32(0.25), dt), dt)
    before = dev.launch_count()
    c = run_gemm(dev, a, b, dt, dt_out, trans_b=True)           # `linear` form: tensor cores
    assert dev.launch_count() - before in (1, 2)     # one tensor-core kernel, plus the merge when K was split
    assert_close(c, orc.matmul_f32(a, b), dt_out, f"fp8 {shape}")


@pytest.mark.parametrize("dt", F8)
@pytest.mark.parametrize("shape", [(128, 256, 256), (300, 256, 528), (640, 1024, 1280), (2048, 384, 2560), (100, 4096, 384)])
def test_fp8_kn_weights_on_tensor_cores(dev, dt, shape):
    """[K, N] weights (morok's matmul layout) with 8-bit inputs: an MN-major tensor-core operand, rows of 128 elements
    along N.  The reference's table for 8-bit inputs has no layout restriction (schedule/src/optimizer/renderer.rs:482-491)."""
    M, K, N = shape
    rng = np.random.default_rng(M + K + N + 1)
    a = to_f32(to_storage(rng.standard_normal((M, K), dtype=np.float32), dt), dt)
    b = to_f32(to_storage(rng.standard_normal((K, N), dtype=np.float32) * np.float32(0.25), dt), dt)
    A, B = dev.from_numpy(to_storage(a, dt)), dev.from_numpy(to_storage(b, dt))
    Cb = dev.alloc(M * N * 4)
    dev.profile_begin()
    dev.gemm(A, B, Cb, M, N, K, dt, mk.MK_F32)
    launched = [n for n, _ in dev.profile_end()]
    assert launched[0] in ("gemm_tc_f8", "gemm_tc_pair_f8", "gemm_tc_ksplit"), launched
    assert dev.kernel_status() == 0
    assert_close(Cb.copyout(np.float32, (M, N)), orc.matmul_f32(a, b), mk.MK_F32, f"fp8 [K,N] {shape}")
    for x in (A, B, Cb):
        x.free()


def test_fp8_linear_scaling_is_exact(dev):
    """Scaling an operand by a power of two scales every product exactly: the result scales exactly too."""
    rng = np.random.default_rng(5)
    a = to_f32(to_storage(rng.standard_normal((256, 512), dtype=np.float32), mk.MK_F8E4M3), mk.MK_F8E4M3)
    b = to_f32(to_storage(rng.standard_normal((512, 256), dtype=np.float32), mk.MK_F8E4M3), mk.MK_F8E4M3)
    c1 = run_gemm(dev, a, b, mk.MK_F8E4M3, mk.MK_F32, trans_b=True)
    c2 = run_gemm(dev, a * np.float32(4), b * np.float32(2), mk.MK_F8E4M3, mk.MK_F32, trans_b=True)   # scaling up stays representable
    assert np.array_equal(c2, c1 * np.float32(8))


# ---------------------------------------------------------------------------------------------
# alpha * A B + beta * C (Tensor::gemm, tensor/src/matmul.rs:112-133) and the bias of `linear`
# (161-187) in the store of the GEMM kernel
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dt_in,dt_out,shape", [
    (mk.MK_BF16, mk.MK_BF16, (300, 200, 520)),      # tensor cores, staged coalesced epilogue
    (mk.MK_BF16, mk.MK_F32, (130, 64, 100)),        # tensor cores, element-wise stores (ldc * 4 not a multiple of 16)
    (mk.MK_F16, mk.MK_F16, (64, 96, 72)),           # one CTA
    (mk.MK_F32, mk.MK_F32, (70, 33, 45)),           # FMA kernel
])
def test_scaled_and_bias_epilogues(dev, dt_in, dt_out, shape):
    M, K, N = shape
    rng = np.random.default_rng(M + N)
    a = to_f32(to_storage(rng.standard_normal((M, K), dtype=np.float32), dt_in), dt_in)
    b = to_f32(to_storage(rng.standard_normal((K, N), dtype=np.float32) * np.float32(0.3), dt_in), dt_in)
    c = to_f32(to_storage(rng.standard_normal((M, N), dtype=np.float32), dt_out), dt_out)
    bias = to_f32(to_storage(rng.standard_normal((N,), dtype=np.float32), dt_out), dt_out)
    ab = orc.matmul_f32(a, b)
    A, B = dev.from_numpy(to_storage(a, dt_in)), dev.from_numpy(to_storage(b, dt_in))
    Cd, Bias = dev.from_numpy(to_storage(c, dt_out)), dev.from_numpy(to_storage(bias, dt_out))
    Y = dev.alloc(M * N * mk.dtype_size(dt_out))

    def result():
        assert dev.kernel_status() == 0
        return to_f32(Y.copyout(NP_OF[dt_out], (M, N)), dt_out)

    dev.gemm(A, B, Y, M, N, K, dt_in, dt_out, add=Cd, alpha=0.5, beta=-2.0)
    assert_close(result(), np.float32(0.5) * ab - np.float32(2.0) * c, dt_out, "alpha A B + beta C")
    dev.gemm(A, B, Y, M, N, K, dt_in, dt_out, alpha=3.0)
    assert_close(result(), np.float32(3.0) * ab, dt_out, "alpha A B")
    dev.gemm(A, B, Y, M, N, K, dt_in, dt_out, bias=Bias)
    assert_close(result(), ab + bias[None, :], dt_out, "A B + bias")
    dev.gemm(A, B, Y, M, N, K, dt_in, dt_out, bias=Bias, alpha=2.0, beta=0.25)
    assert_close(result(), np.float32(2.0) * ab + np.float32(0.25) * bias[None, :], dt_out, "alpha A B + beta bias")
    # flags off: alpha / beta fields are ignored
    d_plain = run_gemm(dev, a, b, dt_in, dt_out, add_f32=c)
    assert_close(d_plain, ab + c, dt_out, "A B + C")


@pytest.mark.parametrize("dt", [mk.MK_BF16, mk.MK_F16])
@pytest.mark.parametrize("shape,trans_b", [((256, 512, 512), False), ((300, 200, 520), False), ((64, 128, 200), True), ((640, 1024, 1280), True)])
def test_gated_pair_of_products_in_one_kernel(dev, dt, shape, trans_b):
    """C = silu(A B) * (A B2): the gated feed-forward `x.matmul(wg).silu() * x.matmul(wu)`, one kernel with two
    reduces in the reference (tensor/src/test/unit/fusion.rs:58-67, 106-114)."""
    M, K, N = shape
    rng = np.random.default_rng(M + N)
    a = to_f32(to_storage(rng.standard_normal((M, K), dtype=np.float32), dt), dt)
    b = to_f32(to_storage(rng.standard_normal((K, N), dtype=np.float32) * np.float32(0.1), dt), dt)
    b2 = to_f32(to_storage(rng.standard_normal((K, N), dtype=np.float32) * np.float32(0.1), dt), dt)
    lay = (lambda w: np.ascontiguousarray(w.T)) if trans_b else (lambda w: w)
    A, B, B2 = dev.from_numpy(to_storage(a, dt)), dev.from_numpy(to_storage(lay(b), dt)), dev.from_numpy(to_storage(lay(b2), dt))
    Y = dev.alloc(M * N * 2)
    before = dev.launch_count()
    dev.gemm(A, B, Y, M, N, K, dt, dt, trans_b=trans_b, swiglu_with=B2)
    assert dev.kernel_status() == 0 and dev.launch_count() == before + 1
    y = to_f32(Y.copyout(NP_OF[dt], (M, N)), dt)
    assert_close(y, orc.swiglu_f32(orc.matmul_f32(a, b), orc.matmul_f32(a, b2)), dt, f"gated {shape}")


@pytest.mark.parametrize("dt", [mk.MK_BF16, mk.MK_F16])
@pytest.mark.parametrize("gate", ["sigmoid", "silu"])
@pytest.mark.parametrize("shape,trans_b", [((256, 512, 512), False), ((300, 200, 520), False), ((64, 128, 200), True)])
def test_gate_block_with_biases_in_one_kernel(dev, dt, gate, shape, trans_b):
    """C = act(A B + b1) * (A B2 + b2): with act = sigmoid the reference's gate block
    `(x @ w1 + b1).sigmoid() * (x @ w2 + b2)`, one kernel there (tensor/src/test/unit/fusion.rs:58-67)."""
    M, K, N = shape
    rng = np.random.default_rng(M + N + 1)
    a = to_f32(to_storage(rng.standard_normal((M, K), dtype=np.float32), dt), dt)
    b = to_f32(to_storage(rng.standard_normal((K, N), dtype=np.float32) * np.float32(0.1), dt), dt)
    b2 = to_f32(to_storage(rng.standard_normal((K, N), dtype=np.float32) * np.float32(0.1), dt), dt)
    bias1, bias2 = (to_f32(to_storage(rng.standard_normal((N,), dtype=np.float32), dt), dt) for _ in range(2))
    lay = (lambda w: np.ascontiguousarray(w.T)) if trans_b else (lambda w: w)
    A, B, B2 = dev.from_numpy(to_storage(a, dt)), dev.from_numpy(to_storage(lay(b), dt)), dev.from_numpy(to_storage(lay(b2), dt))
    D1, D2 = dev.from_numpy(to_storage(bias1, dt)), dev.from_numpy(to_storage(bias2, dt))
    Y = dev.alloc(M * N * 2)
    act = orc.sigmoid_f32 if gate == "sigmoid" else orc.silu_f32
    g, u = orc.matmul_f32(a, b), orc.matmul_f32(a, b2)
    for gb, ub, what in [(D1, D2, "both biases"), (D1, None, "gate bias"), (None, D2, "up bias"), (None, None, "no bias")]:
        before = dev.launch_count()
        dev.gemm(A, B, Y, M, N, K, dt, dt, trans_b=trans_b, swiglu_with=B2, gate=gate, gate_bias=gb, up_bias=ub)
        assert dev.kernel_status() == 0 and dev.launch_count() == before + 1
        y = to_f32(Y.copyout(NP_OF[dt], (M, N)), dt)
        ref = act(g + (bias1[None, :] if gb is not None else np.float32(0))) * (u + (bias2[None, :] if ub is not None else np.float32(0)))
        assert_close(y, ref, dt, f"{gate} gate block {shape} {what}")


def test_gated_pair_needs_the_tensor_core_path(dev):
    a = dev.from_numpy(np.ones((4, 8), np.float32))
    b = dev.from_numpy(np.ones((8, 4), np.float32))
    y = dev.alloc(64)
    with pytest.raises(mk.MorokError) as e:
        dev.gemm(a, b, y, 4, 4, 8, mk.MK_F32, mk.MK_F32, swiglu_with=b)
    assert e.value.status == mk._ffi.MK_ERR_UNSUPPORTED


# ---------------------------------------------------------------------------------------------
# Few rows, long K (decoding): K is cut into ranges so that every SM streams weights; partial tiles
# are summed by a second kernel that also applies the epilogue.
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("M", [1, 8, 128])
@pytest.mark.parametrize("K,N,trans_b", [(4096, 4096, True), (4096, 1000, False), (8192 + 64, 520, True)])
@pytest.mark.parametrize("dt_in,dt_out", [(mk.MK_BF16, mk.MK_BF16), (mk.MK_F16, mk.MK_F32), (mk.MK_F8E4M3, mk.MK_BF16)])
def test_split_k_for_few_rows(dev, M, K, N, trans_b, dt_in, dt_out):
    if dt_in == mk.MK_F8E4M3 and not trans_b and N % 16:
        pytest.skip("[K, N] rows of 1000 one-byte elements are not 16-byte aligned: that shape runs on the FMA kernel")
    rng = np.random.default_rng(M + K + N)
    a = to_f32(to_storage(rng.standard_normal((M, K), dtype=np.float32), dt_in), dt_in)
    b = to_f32(to_storage(rng.standard_normal((K, N), dtype=np.float32) * np.float32(0.05), dt_in), dt_in)
    c = to_f32(to_storage(rng.standard_normal((M, N), dtype=np.float32), dt_out), dt_out)
    bias = to_f32(to_storage(rng.standard_normal((N,), dtype=np.float32), dt_out), dt_out)
    ab = orc.matmul_f32(a, b)
    A = dev.from_numpy(to_storage(a, dt_in))
    B = dev.from_numpy(to_storage(np.ascontiguousarray(b.T) if trans_b else b, dt_in))
    Cd, Bias = dev.from_numpy(to_storage(c, dt_out)), dev.from_numpy(to_storage(bias, dt_out))
    Y = dev.alloc(M * N * mk.dtype_size(dt_out))

    def result():
        assert dev.kernel_status() == 0
        return to_f32(Y.copyout(NP_OF[dt_out], (M, N)), dt_out)

    before = dev.launch_count()
    dev.gemm(A, B, Y, M, N, K, dt_in, dt_out, trans_b=trans_b)
    few_rows = M <= 16 and trans_b and dt_in != mk.MK_F8E4M3      # the weight-streaming kernel takes these in one launch
    assert dev.launch_count() == before + (1 if few_rows else 2)  # else: the split kernel and its merge
    assert_close(result(), ab, dt_out, "split-K")
    dev.gemm(A, B, Y, M, N, K, dt_in, dt_out, trans_b=trans_b, add=Cd, alpha=0.5, beta=2.0)
    assert_close(result(), np.float32(0.5) * ab + np.float32(2.0) * c, dt_out, "split-K alpha beta")
    dev.gemm(A, B, Y, M, N, K, dt_in, dt_out, trans_b=trans_b, bias=Bias)
    assert_close(result(), ab + bias[None, :], dt_out, "split-K bias")


@pytest.mark.parametrize("forced", [dict(pair=0, group_m=3), dict(pair=1, group_m=1), dict(pair=0, group_m=64, splits=1),
                                    dict(splits=5), dict(pair=1, splits=7)])
def test_every_tuning_record_keeps_results_correct(dev, forced):
    """A tuning record only changes the schedule: whatever a file holds, the product stays the oracle's."""
    rng = np.random.default_rng(77)
    for (M, N, K) in [(300, 520, 1088), (48, 1024, 2048)]:
        a = orc.round_bf16(rng.standard_normal((M, K), dtype=np.float32))
        b = orc.round_bf16(rng.standard_normal((K, N), dtype=np.float32) * np.float32(0.05))
        A, B = dev.from_numpy(orc.f32_to_bf16(a)), dev.from_numpy(orc.f32_to_bf16(b))
        Y = dev.alloc(M * N * 2)
        prob = (A, B, Y, M, N, K, mk.MK_BF16)
        dev.gemm_tuning_set(forced, *prob)
        try:
            dev.gemm(*prob)
            assert dev.kernel_status() == 0
            assert_close(orc.bf16_to_f32(Y.copyout(np.uint16, (M, N))), orc.matmul_f32(a, b), mk.MK_BF16, f"tuned {forced} {M}x{N}x{K}")
        finally:
            dev.gemm_tuning_set(None, *prob)


def test_autotune_times_candidates_and_keeps_the_fastest(dev, tmp_path):
    """mk_gemm_autotune: the search-and-cache step of the reference's optimiser
    (schedule/src/optimizer/beam.rs:223-291, 485-524) over this GEMM's schedule choices."""
    rng = np.random.default_rng(78)
    try:
        for (M, N, K, trans_b) in [(16, 4096, 4096, False), (1024, 2048, 1024, False)]:
            a = orc.round_bf16(rng.standard_normal((M, K), dtype=np.float32))
            b = orc.round_bf16(rng.standard_normal((K, N), dtype=np.float32) * np.float32(0.05))
            A = dev.from_numpy(orc.f32_to_bf16(a))
            B = dev.from_numpy(orc.f32_to_bf16(np.ascontiguousarray(b.T) if trans_b else b))
            Y = dev.alloc(M * N * 2)
            prob = (A, B, Y, M, N, K, mk.MK_BF16)
            t = dev.gemm_autotune(*prob, trans_b=trans_b, iters=5)
            assert t["candidates"] >= 5 and 0.0 < t["best_ms"] <= t["default_ms"]
            assert dev.gemm_tuning_get(*prob, trans_b=trans_b) == t          # recorded for later calls
            dev.gemm(*prob, trans_b=trans_b)
            assert dev.kernel_status() == 0
            assert_close(orc.bf16_to_f32(Y.copyout(np.uint16, (M, N))), orc.matmul_f32(a, b), mk.MK_BF16, "after autotune")
        path = str(tmp_path / "b200.tuning")
        dev.tuning_save(path)
        dev.tuning_clear()
        assert dev.tuning_load(path) == 2
        # an in-place residual would change its own input on every trial: refused
        with pytest.raises(mk.MorokError) as e:
            dev.gemm_autotune(A, B, Y, M, N, K, mk.MK_BF16, add=Y)
        assert e.value.status == _ffi.MK_ERR_INVALID and "overlaps" in str(e.value)
        # at most 16 rows against [N, K] weights run on the weight-streaming kernel: no schedule choices
        with pytest.raises(mk.MorokError) as e:
            dev.gemm_autotune(A, B, Y, 16, 1024, 1024, mk.MK_BF16, trans_b=True)
        assert e.value.status == _ffi.MK_ERR_UNSUPPORTED
        # exact f32 runs on the FMA kernel: nothing to tune
        F = dev.from_numpy(rng.standard_normal((64, 64), dtype=np.float32))
        G = dev.alloc(64 * 64 * 4)
        with pytest.raises(mk.MorokError) as e:
            dev.gemm_autotune(F, F, G, 64, 64, 64, mk.MK_F32)
        assert e.value.status == _ffi.MK_ERR_UNSUPPORTED
    finally:
        dev.tuning_clear()


# ---------------------------------------------------------------------------------------------
# At most 16 rows against `linear` weights [N, K]: the weight-streaming kernel (one launch, HBM bound).
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dt_in,dt_out", [(mk.MK_BF16, mk.MK_BF16), (mk.MK_F16, mk.MK_F16), (mk.MK_BF16, mk.MK_F32)])
@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (16, 1000, 520), (5, 40, 8), (16, 1192, 2104), (7, 8, 4096), (16, 14336, 264)])
def test_few_rows_stream_the_weights_once(dev, M, N, K, dt_in, dt_out):
    rng = np.random.default_rng(M * 7 + N + K)
    a = to_f32(to_storage(rng.standard_normal((M, K), dtype=np.float32), dt_in), dt_in)
    w = to_f32(to_storage(rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.05), dt_in), dt_in)
    c = to_f32(to_storage(rng.standard_normal((M, N), dtype=np.float32), dt_out), dt_out)
    bias = to_f32(to_storage(rng.standard_normal((N,), dtype=np.float32), dt_out), dt_out)
    ab = orc.matmul_f32(a, np.ascontiguousarray(w.T))
    A, W = dev.from_numpy(to_storage(a, dt_in)), dev.from_numpy(to_storage(w, dt_in))
    Cd, Bias = dev.from_numpy(to_storage(c, dt_out)), dev.from_numpy(to_storage(bias, dt_out))
    Y = dev.alloc(M * N * mk.dtype_size(dt_out))

    def result():
        assert dev.kernel_status() == 0
        return to_f32(Y.copyout(NP_OF[dt_out], (M, N)), dt_out)

    dev.profile_begin()
    dev.gemm(A, W, Y, M, N, K, dt_in, dt_out, trans_b=True)
    assert [n for n, _ in dev.profile_end()] == ["gemm_skinny"]
    assert_close(result(), ab, dt_out, "few rows")
    dev.gemm(A, W, Y, M, N, K, dt_in, dt_out, trans_b=True, add=Cd)
    assert_close(result(), ab + c, dt_out, "few rows + residual")
    dev.gemm(A, W, Y, M, N, K, dt_in, dt_out, trans_b=True, bias=Bias, alpha=0.5, beta=2.0)
    assert_close(result(), np.float32(0.5) * ab + np.float32(2.0) * bias[None, :], dt_out, "few rows alpha beta bias")
    # in place: the residual is the output buffer itself
    Y.copyin(to_storage(c, dt_out))
    dev.gemm(A, W, Y, M, N, K, dt_in, dt_out, trans_b=True, add=Y)
    assert_close(result(), ab + c, dt_out, "few rows in-place residual")
    if dt_out != mk.MK_F32:
        w2 = to_f32(to_storage(rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.05), dt_in), dt_in)
        W2 = dev.from_numpy(to_storage(w2, dt_in))
        u = orc.matmul_f32(a, np.ascontiguousarray(w2.T))
        dev.profile_begin()
        dev.gemm(A, W, Y, M, N, K, dt_in, dt_out, trans_b=True, swiglu_with=W2)
        small = 2 * N * K * 2 <= (40 << 20) or (N >= 1024 and K >= 1024)     # else the tensor-core kernels are faster
        assert [n for n, _ in dev.profile_end()] == (["gemm_skinny_gated"] if small else ["gemm_tc_pair_gated"])
        assert_close(result(), orc.swiglu_f32(ab, u), dt_out, "few rows gated")
        dev.gemm(A, W, Y, M, N, K, dt_in, dt_out, trans_b=True, swiglu_with=W2, gate="sigmoid", gate_bias=Bias, up_bias=Bias)
        assert_close(result(), orc.sigmoid_f32(ab + bias[None, :]) * (u + bias[None, :]), dt_out, "few rows sigmoid gate block")


def test_few_rows_with_strided_operands_and_batches(dev):
    """Row pitches larger than the rows (views into wider buffers) and a batch of problems."""
    rng = np.random.default_rng(5)
    M, N, K, lda, ldw, ldc, batch = 4, 72, 264, 272, 280, 80, 3
    a = orc.round_bf16(rng.standard_normal((batch, M, lda), dtype=np.float32))
    w = orc.round_bf16(rng.standard_normal((batch, N, ldw), dtype=np.float32) * np.float32(0.1))
    A, W = dev.from_numpy(orc.f32_to_bf16(a)), dev.from_numpy(orc.f32_to_bf16(w))
    Y = dev.from_numpy(np.full((batch, M, ldc), 0x7FC0, np.uint16))          # NaN patterns: untouched padding stays NaN
    dev.gemm(A, W, Y, M, N, K, mk.MK_BF16, trans_b=True, lda=lda, ldb=ldw, ldc=ldc, batch=batch,
             stride_a=M * lda, stride_b=N * ldw, stride_c=M * ldc)
    assert dev.kernel_status() == 0
    y = orc.bf16_to_f32(Y.copyout(np.uint16, (batch, M, ldc)))
    for i in range(batch):
        assert_close(y[i, :, :N], orc.matmul_f32(a[i, :, :K], np.ascontiguousarray(w[i, :, :K].T)), mk.MK_BF16, f"batch {i}")
    assert np.all(np.isnan(y[:, :, N:]))


def test_sharded_delivery_by_tile_stores_into_stand_in_peers(dev):
    """The N-sharded form on one GPU: two more buffers of the same GPU stand in for the peers' C.  The CTA-pair kernel
    must deliver every tile of its column block into all three matrices (tile stores: 32 x 64 boxes, rows and columns
    ragged against them) and leave the other columns untouched."""
    M, K, N, col0, ncols = 2040, 320, 5128, 2568, 2560          # this "rank" owns columns 2568 .. 5127 of a [M, 5128] matrix
    rng = np.random.default_rng(21)
    a, b = orc.normal_bf16(rng, (M, K), 1.0), orc.normal_bf16(rng, (K, N), 0.05)
    A, B = dev.from_numpy(a), dev.from_numpy(b)
    outs = [dev.from_numpy(np.full((M, N), 0xFFFF, np.uint16)) for _ in range(3)]
    dev.profile_begin()
    dev.gemm(A, B.view(col0 * 2, K * N * 2 - col0 * 2), outs[0], M, ncols, K, mk.MK_BF16, ldb=N, ldc=N,
             c_ptr=outs[0].ptr + col0 * 2, peers=[o.ptr + col0 * 2 for o in outs[1:]])
    launched = [name for name, _ in dev.profile_end()]
    assert launched == ["gemm_tc_pair_deliver"], launched
    assert dev.kernel_status() == 0
    ref = orc.matmul_f32(orc.bf16_to_f32(a), orc.bf16_to_f32(b[:, col0:]))
    first = None
    for o in outs:
        c = o.copyout(np.uint16, (M, N))
        assert np.all(c[:, :col0] == 0xFFFF), "columns of another rank were overwritten"
        assert not np.any(c[:, col0:] == 0xFFFF)
        assert_close(orc.bf16_to_f32(c[:, col0:]), ref, mk.MK_BF16, "tile-store delivery")
        first = c if first is None else first
        assert np.array_equal(c, first), "the copies differ from each other"
    for x in [A, B] + outs:
        x.free()


def test_tile_store_delivery_under_back_pressure_seven_stand_in_peers(dev):
    """Eight destinations per tile and a K so short that the tile stores set the pace (0.27 GB of stores against
    4 GFLOP): every epilogue warp queues behind the copy engine for its staging blocks, launch after launch.  All
    eight copies must be identical and match the oracle; no pipeline wait may give up."""
    M, K, N = 4096, 128, 4096
    rng = np.random.default_rng(33)
    a, b = orc.normal_bf16(rng, (M, K), 1.0), orc.normal_bf16(rng, (K, N), 0.05)
    A, B = dev.from_numpy(a), dev.from_numpy(b)
    outs = [dev.from_numpy(np.full((M, N), 0xFFFF, np.uint16)) for _ in range(8)]
    dev.profile_begin()
    for _ in range(3):
        dev.gemm(A, B, outs[0], M, N, K, mk.MK_BF16, peers=[o.ptr for o in outs[1:]])
    launched = [name for name, _ in dev.profile_end()]
    assert launched == ["gemm_tc_pair_deliver"] * 3, launched
    dev.sync()
    assert dev.kernel_status() == 0
    first = outs[0].copyout(np.uint16, (M, N))
    assert not np.any(first == 0xFFFF)
    rows = np.r_[0:64, 2000:2064, M - 64:M]
    assert_close(orc.bf16_to_f32(first[rows]), orc.matmul_f32(orc.bf16_to_f32(a[rows]), orc.bf16_to_f32(b)), mk.MK_BF16, "sampled rows")
    for o in outs[1:]:
        assert np.array_equal(o.copyout(np.uint16, (M, N)), first), "the copies differ from each other"
    for x in [A, B] + outs:
        x.free()

