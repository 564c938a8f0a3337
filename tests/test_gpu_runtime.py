"""Runtime half of the boundary on a real device, through the C ABI: module load + launch with the
reference's argument convention (buffers in PARAM-slot order, then i64 values:
runtime/src/dispatch.rs:45-83), streams and events with bounded waits (device/src/sync.rs:248-306),
copies, the LRU allocator on real HBM (device/src/test/unit/buffer.rs checks reuse by pointer
identity), and the copy-engine all-gather."""
import ctypes as C

import numpy as np
import pytest

import morok_b200 as mk
from morok_b200 import _ffi
from oracle import oracle as orc
from gpu_util import assert_close, dev  # noqa: F401

pytestmark = pytest.mark.gpu

# nvcc -ptx of:
#   extern "C" __global__ void axpy_i64(float* y, const float* x, long long n, long long a) {
#       long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
#       if (i < n) y[i] = (float)a * x[i] + y[i];
#   }
AXPY_PTX = r"""
.version 8.8
.target sm_100a
.address_size 64
.visible .entry axpy_i64(
	.param .u64 .ptr .align 1 axpy_i64_param_0,
	.param .u64 .ptr .align 1 axpy_i64_param_1,
	.param .u64 axpy_i64_param_2,
	.param .u64 axpy_i64_param_3
)
{
	.reg .pred 	%p<2>;
	.reg .b32 	%r<4>;
	.reg .f32 	%f<5>;
	.reg .b64 	%rd<13>;
	ld.param.u64 	%rd2, [axpy_i64_param_0];
	ld.param.u64 	%rd3, [axpy_i64_param_1];
	ld.param.u64 	%rd5, [axpy_i64_param_2];
	ld.param.u64 	%rd4, [axpy_i64_param_3];
	mov.u32 	%r1, %ctaid.x;
	mov.u32 	%r2, %ntid.x;
	mul.wide.u32 	%rd6, %r1, %r2;
	mov.u32 	%r3, %tid.x;
	cvt.u64.u32 	%rd7, %r3;
	add.s64 	%rd1, %rd6, %rd7;
	setp.ge.s64 	%p1, %rd1, %rd5;
	@%p1 bra 	$L__BB0_2;
	cvta.to.global.u64 	%rd8, %rd3;
	cvta.to.global.u64 	%rd9, %rd2;
	cvt.rn.f32.s64 	%f1, %rd4;
	shl.b64 	%rd10, %rd1, 2;
	add.s64 	%rd11, %rd8, %rd10;
	ld.global.f32 	%f2, [%rd11];
	add.s64 	%rd12, %rd9, %rd10;
	ld.global.f32 	%f3, [%rd12];
	fma.rn.f32 	%f4, %f2, %f1, %f3;
	st.global.f32 	[%rd12], %f4;
$L__BB0_2:
	ret;
}
"""


def test_module_load_and_launch_buffers_then_values(dev):
    lib = dev.lib
    img = AXPY_PTX.encode()
    mod, fn = C.c_void_p(), C.c_void_p()
    _ffi.check(lib.mk_module_load(dev.h, img, len(img), C.byref(mod)))
    _ffi.check(lib.mk_get_function(mod, b"axpy_i64", C.byref(fn)))
    n = 1000
    x, y = np.arange(n, dtype=np.float32), np.ones(n, dtype=np.float32)
    X, Y = dev.from_numpy(x), dev.from_numpy(y)
    # Program::execute order: buffer pointers first, then the i64 values, each passed by address
    args = [C.c_void_p(Y.ptr), C.c_void_p(X.ptr), C.c_int64(n), C.c_int64(3)]
    argv = (C.c_void_p * len(args))(*[C.cast(C.pointer(a), C.c_void_p) for a in args])
    before = dev.launch_count()
    grid, block = (C.c_uint32 * 3)((n + 127) // 128, 1, 1), (C.c_uint32 * 3)(128, 1, 1)
    _ffi.check(lib.mk_launch(fn, grid, block, 0, None, argv))
    assert np.array_equal(Y.copyout(np.float32, (n,)), 3 * x + 1)
    assert dev.launch_count() == before + 1
    missing = C.c_void_p()
    assert lib.mk_get_function(mod, b"no_such_kernel", C.byref(missing)) == _ffi.MK_ERR_CUDA
    zero = (C.c_uint32 * 3)(0, 1, 1)
    assert lib.mk_launch(fn, zero, block, 0, None, argv) == _ffi.MK_ERR_INVALID
    bad = C.c_void_p()
    assert lib.mk_module_load(dev.h, b"this is not ptx", 15, C.byref(bad)) == _ffi.MK_ERR_CUDA
    _ffi.check(lib.mk_module_unload(mod))
    assert dev.kernel_status() == 0          # the context is still healthy after the failed loads


def test_streams_events_and_bounded_waits(dev):
    s1, s2 = mk.Stream(dev), mk.Stream(dev)
    e0, e1, never = mk.Event(dev), mk.Event(dev), mk.Event(dev)
    n = 1 << 22
    a = dev.from_numpy(np.ones(n, np.float32))
    b, c = dev.alloc(n * 4), dev.alloc(n * 4)
    e0.record(s1)
    for _ in range(20):
        dev.add(a, a, b, n, mk.MK_F32, stream=s1)
    e1.record(s1)
    _ffi.check(dev.lib.mk_stream_wait_event(s2.h, e1.h))       # s2 continues only after s1's work
    dev.add(b, a, c, n, mk.MK_F32, stream=s2)
    s2.sync()
    assert np.all(c.copyout(np.float32, (n,), stream=s2) == 3.0)
    e1.wait(timeout_ms=5000)
    assert e0.elapsed_ms(e1) > 0
    with pytest.raises(mk.MorokError) as err:                  # waiting on an event nobody recorded is an error, not a hang
        never.wait(timeout_ms=10)
    assert err.value.status == _ffi.MK_ERR_INVALID
    assert s1.raw() != s2.raw() and s1.raw() != 0
    for x in (e0, e1, never):
        x.close()
    s1.close(); s2.close()


def test_lru_allocator_on_hbm_and_copies(dev):
    dev.trim()
    s0 = dev.stats()
    b = dev.alloc(3 << 20)
    assert not b.is_allocated                                   # lazy
    p1 = b.ptr
    b.free()
    b2 = dev.alloc(3 << 20)
    assert b2.ptr == p1                                         # reuse by pointer identity
    s1 = dev.stats()
    assert s1["cache_hits"] == s0["cache_hits"] + 1 and s1["device_allocs"] == s0["device_allocs"] + 1
    dev.inject_oom(1)                                           # host-injected OOM: flush + retry, no real exhaustion
    big = dev.alloc(5 << 20)
    assert big.ptr != 0 and dev.stats()["oom_flushes"] == s0["oom_flushes"] + 1
    # copies: d2d, view copy, pinned host round trip
    x = np.random.default_rng(0).integers(0, 255, 3 << 20, dtype=np.uint8)
    b2.copyin(x)
    d = dev.alloc(3 << 20)
    d.copy_from(b2)
    assert np.array_equal(d.copyout(np.uint8, x.shape), x)
    assert np.array_equal(d.view(4096, 8192).copyout(np.uint8, (8192,)), x[4096:4096 + 8192])
    host = C.c_void_p()
    _ffi.check(dev.lib.mk_host_alloc(1 << 20, C.byref(host)))
    _ffi.check(dev.lib.mk_memcpy_async(dev.h, host, d.ptr, 1 << 20, 1, None))
    dev.sync()
    assert np.array_equal(np.ctypeslib.as_array(C.cast(host, C.POINTER(C.c_uint8)), shape=(1 << 20,)), x[:1 << 20])
    _ffi.check(dev.lib.mk_host_free(host))
    with pytest.raises(mk.MorokError) as err:
        d.copyin(x[:100])
    assert err.value.status == _ffi.MK_ERR_SIZE_MISMATCH
    for buf in (b2, big, d):
        buf.free()


def test_all_gather_push_contiguous_and_strided(dev):
    """The copy-engine all-gather over (here: local) destination buffers."""
    world, shard = 4, 1000
    dst = [dev.from_numpy(np.zeros(world * shard, np.float32)) for _ in range(3)]
    ptrs = (C.c_void_p * 3)(*[d.ptr for d in dst])
    for r in range(world):
        src = dev.from_numpy(np.full(shard, r + 1, np.float32))
        _ffi.check(dev.lib.mk_all_gather_push(dev.h, None, src.ptr, shard * 4, ptrs, 3, r * shard * 4))
    dev.sync()
    want = np.repeat(np.arange(1, world + 1, dtype=np.float32), shard)
    for d in dst:
        assert np.array_equal(d.copyout(np.float32, (world * shard,)), want)
    # column shards of a row-major [rows, world*cols] matrix
    rows, cols = 37, 24
    full = [dev.from_numpy(np.zeros((rows, world * cols), np.float32)) for _ in range(2)]
    fptrs = (C.c_void_p * 2)(*[d.ptr for d in full])
    for r in range(world):
        blk = np.full((rows, cols), 10 * (r + 1), np.float32) + np.arange(cols, dtype=np.float32)
        src = dev.from_numpy(blk)
        _ffi.check(dev.lib.mk_all_gather_push_2d(dev.h, None, src.ptr, cols * 4, cols * 4, rows, fptrs, 2, r * cols * 4,
                                                 world * cols * 4))
    dev.sync()
    got = full[1].copyout(np.float32, (rows, world * cols))
    for r in range(world):
        assert np.array_equal(got[:, r * cols:(r + 1) * cols], 10 * (r + 1) + np.tile(np.arange(cols, dtype=np.float32), (rows, 1)))


def test_bounded_wait_runs_out_and_context_survives(dev):
    """Failure detection without a fault: a barrier wait that nothing satisfies gives up after its
    limit, the kernel returns, the host reads MK_ERR_KERNEL with the recorded code, the error word is
    cleared, and the same context then runs a tensor-core GEMM correctly."""
    import time
    assert dev.kernel_status() == 0
    t0 = time.perf_counter()
    dev.selftest_bounded_wait(50)
    elapsed = time.perf_counter() - t0
    assert 0.04 < elapsed < 1.5, elapsed         # the limit was honoured: neither skipped nor unbounded
    with pytest.raises(mk.MorokError) as ei:
        dev.kernel_status()
    assert ei.value.status == _ffi.MK_ERR_KERNEL and "0x901" in str(ei.value)
    assert dev.kernel_status() == 0              # read-and-clear
    with pytest.raises(mk.MorokError) as ei:     # limits outside 1..1000 ms are refused on the host
        dev.selftest_bounded_wait(5000)
    assert ei.value.status == _ffi.MK_ERR_INVALID
    rng = np.random.default_rng(3)
    a = orc.normal_bf16(rng, (256, 512), 1.0)
    b = orc.normal_bf16(rng, (512, 384), 1.0)
    A, B, Cb = dev.from_numpy(a), dev.from_numpy(b), dev.alloc(256 * 384 * 2)
    dev.gemm(A, B, Cb, 256, 384, 512, mk.MK_BF16)
    assert dev.kernel_status() == 0
    got = orc.bf16_to_f32(Cb.copyout(np.uint16, (256, 384)))
    assert_close(got, orc.matmul_f32(orc.bf16_to_f32(a), orc.bf16_to_f32(b)), mk.MK_BF16, "gemm after a timed-out wait")


def test_profile_lists_kernels_in_launch_order(dev):
    """Per-kernel device times, the counterpart of ExecutionPlan::execute_profiled
    (runtime/src/execution_plan.rs:200-221)."""
    rng = np.random.default_rng(21)
    M, N, K = 256, 512, 1024
    a = orc.round_bf16(rng.standard_normal((M, K), dtype=np.float32))
    b = orc.round_bf16(rng.standard_normal((K, N), dtype=np.float32) * np.float32(0.05))
    A, B = dev.from_numpy(orc.f32_to_bf16(a)), dev.from_numpy(orc.f32_to_bf16(b))
    Y, Z, R = (dev.alloc(M * N * 2) for _ in range(3))
    other = mk.Stream(dev)
    dev.profile_begin()
    with pytest.raises(mk.MorokError) as e:              # one profile per thread
        dev.profile_begin()
    assert e.value.status == _ffi.MK_ERR_INVALID
    dev.gemm(A, B, Y, M, N, K, mk.MK_BF16)
    dev.add(Y, Y, Z, M * N, mk.MK_BF16)
    dev.add(Y, Y, Z, M * N, mk.MK_BF16, stream=other)    # another stream: not part of this profile
    dev.rms_norm(Z, R, M, N, 1e-5, mk.MK_BF16)
    prof = dev.profile_end()
    other.sync()
    names = [n for n, _ in prof]
    assert len(prof) == 3 and names[0].startswith("gemm_tc") and names[1:] == ["add", "rms_norm"], prof
    assert all(0.0 < ms < 50.0 for _, ms in prof), prof
    assert dev.kernel_status() == 0
    assert_close(orc.bf16_to_f32(Y.copyout(np.uint16, (M, N))), orc.matmul_f32(a, b), mk.MK_BF16, "profiled gemm")
    # through the Tensor API: the feed-forward block is the gated pair GEMM and the down GEMM
    x = orc.round_bf16(rng.standard_normal((128, 256), dtype=np.float32))
    wg, wu = (orc.round_bf16(rng.standard_normal((256, 512), dtype=np.float32) * np.float32(0.1)) for _ in range(2))
    wd = orc.round_bf16(rng.standard_normal((512, 256), dtype=np.float32) * np.float32(0.1))
    T = lambda v: mk.Tensor.from_ndarray(dev, orc.f32_to_bf16(v))
    X = T(x)
    out = X.try_add(X.matmul(T(wg)).silu().try_mul(X.matmul(T(wu))).matmul(T(wd)))
    prof = out.realize_profiled()
    assert len(prof) == out.last_launches() == 2, prof
    assert prof[0][0] == "gemm_tc_pair_gated" and prof[1][0].startswith("gemm_tc"), prof
    other.close()


def test_threads_with_their_own_streams_share_one_device(dev):
    """Handles are usable from any thread, one stream is one ordered queue, and kernels that work in two
    launches keep their scratch per stream: four threads run K-split GEMMs and key-split decode attention
    at the same time and every result still matches the oracle."""
    import threading
    M, K, N = 16, 4096, 4096
    B_, H, Hkv, Sk, D = 2, 8, 2, 2048, 128
    jobs = []
    for t in range(4):
        rng = np.random.default_rng(100 + t)
        a = orc.round_bf16(rng.standard_normal((M, K), dtype=np.float32))
        w = orc.round_bf16(rng.standard_normal((K, N), dtype=np.float32) * np.float32(0.05))
        q, k, v = (orc.round_bf16(rng.standard_normal(s, dtype=np.float32)) for s in ((B_, H, 1, D), (B_, Hkv, Sk, D), (B_, Hkv, Sk, D)))
        jobs.append(dict(a=a, w=w, q=q, k=k, v=v, c_ref=orc.matmul_f32(a, w), o_ref=orc.sdpa_f32(q, k, v)))
    errors = []

    def worker(job):
        try:
            s = mk.Stream(dev)
            A, W, Q, Kc, Vc = (dev.from_numpy(orc.f32_to_bf16(job[n]), stream=s) for n in ("a", "w", "q", "k", "v"))
            Cb, Ob = dev.alloc(M * N * 2), dev.alloc(B_ * H * D * 2)
            for _ in range(6):
                before = dev.launch_count()
                dev.gemm(A, W, Cb, M, N, K, mk.MK_BF16, stream=s)
                dev.sdpa(Q, Kc, Vc, Ob, B_, H, Hkv, 1, Sk, D, dtype=mk.MK_BF16, stream=s)
                assert dev.launch_count() - before >= 4          # both ops took their two-launch form
            c = orc.bf16_to_f32(Cb.copyout(np.uint16, (M, N), stream=s))
            o = orc.bf16_to_f32(Ob.copyout(np.uint16, (B_, H, 1, D), stream=s))
            assert dev.kernel_status(s) == 0
            assert_close(c, job["c_ref"], mk.MK_BF16, "threaded split-K GEMM")
            assert_close(o, job["o_ref"], mk.MK_BF16, "threaded decode attention")
            s.close()
        except Exception as ex:     # noqa: BLE001
            errors.append(ex)

    threads = [threading.Thread(target=worker, args=(j,)) for j in jobs]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors


def test_attention_claim_counters_are_per_stream_and_per_plan(dev):
    """The persistent attention kernel claims work items from a counter.  A recorded plan keeps its counter for
    life and every stream has its own, so a plan replaying on one stream while hundreds of eager attention calls
    run on another never consume each other's claims: both outputs still match the oracle."""
    from morok_b200 import Tensor
    B, H, S, D = 1, 8, 1024, 128
    rng = np.random.default_rng(77)
    q1, k1, v1 = (orc.normal_bf16(rng, (B, H, S, D)) for _ in range(3))
    q2, k2, v2 = (orc.normal_bf16(rng, (B, H, S, D)) for _ in range(3))
    bf = orc.bf16_to_f32
    ref1 = orc.sdpa_f32(bf(q1), bf(k1), bf(v1), causal=True)
    ref2 = orc.sdpa_f32(bf(q2), bf(k2), bf(v2), causal=True)
    plan = Tensor.from_ndarray(dev, q1).scaled_dot_product_attention(Tensor.from_ndarray(dev, k1), Tensor.from_ndarray(dev, v1),
                                                                       is_causal=True).compile()
    Q2, K2, V2 = dev.from_numpy(q2), dev.from_numpy(k2), dev.from_numpy(v2)
    O2 = dev.alloc(B * H * S * D * 2)
    s_plan = mk.Stream(dev)
    for i in range(300):                    # more launches than there are counter slots
        plan.launch(s_plan)
        dev.sdpa(Q2, K2, V2, O2, B, H, H, S, S, D, dtype=mk.MK_BF16, causal=True)
    assert dev.kernel_status(s_plan) == 0
    assert dev.kernel_status() == 0
    assert_close(bf(plan.result.as_ndarray()), ref1, mk.MK_BF16, "attention replayed from a plan beside eager launches")
    assert_close(bf(O2.copyout(np.uint16, (B, H, S, D))), ref2, mk.MK_BF16, "eager attention beside a replaying plan")
    plan.free()
    s_plan.close()


def test_cached_block_is_not_reused_under_a_running_kernel(dev):
    """Reuse out of the allocator cache is ordered after the work that was in flight when the block was freed:
    A is freed while GEMMs that read it are still queued on stream 1, the next allocation of that size gets the
    same block back and is overwritten through stream 2 -- and the GEMM result is still that of the old contents."""
    M, K, N = 4096, 4096, 4096
    rng = np.random.default_rng(3)
    a = orc.normal_bf16(rng, (M, K), 1.0)
    b = orc.normal_bf16(rng, (K, N), 0.02)
    dev.trim()
    s1, s2 = mk.Stream(dev), mk.Stream(dev)
    A, Bw, Cb = dev.from_numpy(a), dev.from_numpy(b), dev.alloc(M * N * 2)
    dev.sync()
    a_ptr = A.ptr
    for _ in range(40):                         # tens of milliseconds of queued work that reads A
        dev.gemm(A, Bw, Cb, M, N, K, mk.MK_BF16, stream=s1)
    A.free()                                    # no sync: the allocator has to order the reuse itself
    X = dev.alloc(M * K * 2)
    assert X.ptr == a_ptr                       # the same block, straight from the cache
    X.copyin(np.full((M, K), 0x7FC0, np.uint16), stream=s2)      # NaNs over the old A, on another stream
    s1.sync()
    s2.sync()
    assert dev.kernel_status(s1) == 0
    rows = np.array([0, 1, 2047, 4095])
    got = orc.bf16_to_f32(Cb.copyout(np.uint16, (M, N))[rows])
    ref = orc.matmul_f32(orc.bf16_to_f32(a[rows]), orc.bf16_to_f32(b))
    assert_close(got, ref, mk.MK_BF16, "GEMM whose input block was freed and reused while it was queued")
    for x in (X, Bw, Cb):
        x.free()
    s1.close()
    s2.close()


def test_recorded_tensor_holds_no_data_until_its_plan_has_run(dev):
    from morok_b200 import Tensor
    rng = np.random.default_rng(5)
    a_bits, b_bits = orc.normal_bf16(rng, (64, 64), 1.0), orc.normal_bf16(rng, (64, 64), 1.0)
    a, b = Tensor.from_ndarray(dev, a_bits), Tensor.from_ndarray(dev, b_bits)
    c = a.matmul(b)
    plan = c.compile()
    with pytest.raises(mk.MorokError) as e:     # recorded, never launched: nothing to read yet
        c.as_ndarray()
    assert e.value.status == _ffi.MK_ERR_NOT_ALLOCATED
    with pytest.raises(mk.MorokError) as e:     # ... and nothing an eager graph could consume
        c.matmul(b).realize()
    assert e.value.status == _ffi.MK_ERR_NOT_ALLOCATED
    # the plan keeps the leaf buffers it reads: dropping the input tensors and recycling memory of their size
    # must not reach the plan's data
    del a, b
    junk = [dev.from_numpy(np.full((64, 64), 0x7FC0, np.uint16)) for _ in range(4)]
    plan.launch()
    dev.sync()
    assert dev.kernel_status() == 0
    got = orc.bf16_to_f32(c.as_ndarray())
    assert_close(got, orc.matmul_f32(orc.bf16_to_f32(a_bits), orc.bf16_to_f32(b_bits)), mk.MK_BF16, "plan replay after its inputs were dropped")
    for j in junk:
        j.free()
    plan.free()
