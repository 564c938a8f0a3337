"""mk_gemm_static: the GEMM entry point for callers that must not allocate device memory.

Some users of this library run inside a memory budget they do not own -- an inference server or a
framework allocator has already reserved the GPU, so a cudaMalloc from library code may fail, and
cudaMalloc / cudaFree stall every stream of the device.  mk_gemm_static runs the tensor-core GEMM
with its scratch (the kernel error words) in a fixed array inside the library, so it needs neither
an mk_device nor any allocation.  The test drives it through the C ABI with caller-owned buffers and
checks that it produces exactly what mk_gemm produces, twice in a row (the array is shared between
calls and keeps the previous call's contents).

This file sorts last on purpose: a run that stops at the first failure has then already run every
other test.
"""
import ctypes as C

import numpy as np
import pytest

import morok_b200 as mk
from morok_b200 import _ffi
from oracle import oracle as orc
from gpu_util import dev  # noqa: F401

pytestmark = pytest.mark.gpu


def desc_for(a, b, c, M, N, K, batch=1, trans_b=False, add=None, dtype_in=None, dtype_out=None, bias=None, alpha=None, beta=None):
    d = _ffi.GemmDesc()
    d.dtype_in = mk.MK_BF16 if dtype_in is None else dtype_in
    d.dtype_out = d.dtype_in if dtype_out is None else dtype_out
    d.M, d.N, d.K = M, N, K
    d.A, d.lda, d.B, d.ldb, d.C, d.ldc = a.ptr, K, b.ptr, (K if trans_b else N), c.ptr, N
    d.trans_b, d.batch = int(trans_b), batch
    d.stride_a, d.stride_b, d.stride_c = M * K, 0, M * N
    if add is not None:
        d.epilogue, d.D = _ffi.MK_EPI_ADD, add.ptr
    if bias is not None:
        d.epilogue, d.D = _ffi.MK_EPI_ADD_ROW, bias.ptr
    if alpha is not None:
        d.flags, d.alpha, d.beta = _ffi.MK_GEMM_SCALED, alpha, beta
    return d


def free_device_memory(dev) -> int:
    free, total = C.c_size_t(), C.c_size_t()
    _ffi.check(dev.lib.mk_mem_info(dev.h, C.byref(free), C.byref(total)))
    return free.value


def test_static_gemm_matches_mk_gemm_on_two_calls_in_a_row(dev):
    lib = dev.lib
    ordinal = dev.info().ordinal
    rng = np.random.default_rng(0)
    # batch, M, N, K, trans_b; the third case is large enough for the CTA-pair kernel (80 tiles of 256 x 256)
    cases = [(3, 200, 264, 136, False), (2, 384, 512, 320, True), (1, 2048, 2560, 256, False)]
    # everything the calls need is allocated up front, by the caller
    bufs = []
    for batch, M, N, K, tb in cases:
        a = orc.normal_bf16(rng, (batch, M, K), 1.0)
        b = orc.normal_bf16(rng, (N, K) if tb else (K, N), 0.05)
        resid = orc.normal_bf16(rng, (batch, M, N), 1.0)
        A, B, R = dev.from_numpy(a), dev.from_numpy(b), dev.from_numpy(resid)
        C_ref, C_new = dev.alloc(batch * M * N * 2), dev.from_numpy(np.full((batch, M, N), 0xFFFF, np.uint16))
        for x in (A, B, R, C_ref, C_new):
            x.ptr
        bufs.append((A, B, R, C_ref, C_new, a, b, resid))
    dev.sync()
    # one warm call per kernel variant: the driver loads a kernel's image on its first launch
    for (batch, M, N, K, tb), (A, B, R, C_ref, C_new, *_rest) in zip(cases, bufs):
        _ffi.check(lib.mk_gemm_static(ordinal, None, C.byref(desc_for(A, B, C_new, M, N, K, batch, tb, add=R)), None))
        _ffi.check(lib.mk_gemm(dev.h, None, C.byref(desc_for(A, B, C_ref, M, N, K, batch, tb, add=R))))
    dev.sync()
    assert dev.kernel_status() == 0
    allocs_before = dev.stats()["device_allocs"]
    free_before = free_device_memory(dev)

    for (batch, M, N, K, tb), (A, B, R, C_ref, C_new, a, b, resid) in zip(cases, bufs):
        d_ref = desc_for(A, B, C_ref, M, N, K, batch, tb, add=R)
        _ffi.check(lib.mk_gemm(dev.h, None, C.byref(d_ref)))
        assert dev.kernel_status() == 0
        C_new.copyin(np.full((batch, M, N), 0xFFFF, np.uint16))
        d_new = desc_for(A, B, C_new, M, N, K, batch, tb, add=R)
        err = C.c_uint32(123)
        _ffi.check(lib.mk_gemm_static(ordinal, None, C.byref(d_new), C.byref(err)))
        assert err.value == 0
        ref = C_ref.copyout(np.uint16, (batch, M, N))
        new = C_new.copyout(np.uint16, (batch, M, N))
        assert np.array_equal(new, ref), "the static-scratch entry point and mk_gemm disagree"
        # and both agree with the oracle within the bf16 bar
        bf = orc.bf16_to_f32
        w = bf(b).T if tb else bf(b)
        for i in range(batch):
            want = orc.matmul_f32(bf(a[i]), np.ascontiguousarray(w)) + bf(resid[i])
            assert np.all(np.abs(bf(new[i]) - want) <= 1e-2 + 2e-2 * np.abs(want))
    # Nothing was allocated along the way: the library's own allocator saw no request, and the device's free
    # memory (which a direct cudaMalloc inside the entry point would lower) is what it was.
    assert dev.stats()["device_allocs"] == allocs_before
    assert free_device_memory(dev) == free_before

    # asynchronous form (no error pointer), then the status query
    (batch, M, N, K, tb), (A, B, R, C_ref, C_new, *_rest) = cases[0], bufs[0]
    C_new.copyin(np.zeros((batch, M, N), np.uint16))
    _ffi.check(lib.mk_gemm_static(ordinal, None, C.byref(desc_for(A, B, C_new, M, N, K, batch, tb, add=R)), None))
    err = C.c_uint32(55)
    _ffi.check(lib.mk_gemm_static_status(ordinal, None, batch, C.byref(err)))
    assert err.value == 0
    assert np.array_equal(C_new.copyout(np.uint16, (batch, M, N)), C_ref.copyout(np.uint16, (batch, M, N)))
    assert free_device_memory(dev) == free_before


@pytest.mark.parametrize("case", [
    # dtype_in, dtype_out, M, N, K, trans_b, epilogue
    (mk.MK_F16, mk.MK_F16, 200, 264, 136, True, "bias_scaled"),      # f16, bias row, alpha / beta
    (mk.MK_BF16, mk.MK_F32, 130, 72, 200, False, "none"),            # f32 output exposes the accumulator
    (mk.MK_BF16, mk.MK_BF16, 257, 520, 72, False, "add"),            # M, N, K off the tile sizes
])
def test_static_gemm_other_dtypes_and_epilogues_match_mk_gemm(dev, case):
    dt_in, dt_out, M, N, K, tb, epi = case
    lib, ordinal = dev.lib, dev.info().ordinal
    rng = np.random.default_rng(M + N + K)
    conv = (lambda x: orc.f32_to_bf16(x)) if dt_in == mk.MK_BF16 else (lambda x: x.astype(np.float16))
    a = conv(rng.standard_normal((M, K), dtype=np.float32))
    b = conv(rng.standard_normal((N, K) if tb else (K, N), dtype=np.float32) * np.float32(0.1))
    es = 4 if dt_out == mk.MK_F32 else 2
    A, B = dev.from_numpy(a), dev.from_numpy(b)
    C_ref, C_new = dev.alloc(M * N * es), dev.alloc(M * N * es)
    kw = {}
    extra = None
    if epi == "bias_scaled":
        extra = dev.from_numpy(rng.standard_normal(N, dtype=np.float32).astype(np.float16))
        kw = dict(bias=extra, alpha=0.5, beta=2.0)
    elif epi == "add":
        extra = dev.from_numpy(orc.normal_bf16(rng, (M, N), 1.0))
        kw = dict(add=extra)
    d = desc_for(A, B, C_ref, M, N, K, 1, tb, dtype_in=dt_in, dtype_out=dt_out, **kw)
    _ffi.check(lib.mk_gemm(dev.h, None, C.byref(d)))
    assert dev.kernel_status() == 0
    d = desc_for(A, B, C_new, M, N, K, 1, tb, dtype_in=dt_in, dtype_out=dt_out, **kw)
    err = C.c_uint32(1)
    _ffi.check(lib.mk_gemm_static(ordinal, None, C.byref(d), C.byref(err)))
    assert err.value == 0
    npdt = np.float32 if dt_out == mk.MK_F32 else np.uint16
    assert np.array_equal(C_new.copyout(npdt, (M, N)), C_ref.copyout(npdt, (M, N)))
    for x in (A, B, C_ref, C_new, extra):
        if x is not None:
            x.free()


def test_static_gemm_rejects_what_it_cannot_take(dev):
    lib = dev.lib
    a = dev.alloc(1 << 16)
    a.ptr
    d = desc_for(a, a, a, 16, 16, 16, batch=_ffi.MK_STATIC_GEMM_MAX_BATCH + 1)
    assert lib.mk_gemm_static(0, None, C.byref(d), None) == _ffi.MK_ERR_INVALID
    assert b"exceeds the static scratch" in lib.mk_last_error()
    d = desc_for(a, a, a, 16, 20, 12)                 # rows of 12 / 20 elements are not 16-byte multiples
    assert lib.mk_gemm_static(0, None, C.byref(d), None) == _ffi.MK_ERR_UNSUPPORTED
    d = desc_for(a, a, a, 16, 16, 16)
    d.dtype_in = mk.MK_F32
    assert lib.mk_gemm_static(0, None, C.byref(d), None) == _ffi.MK_ERR_INVALID
    assert lib.mk_gemm_static(99, None, C.byref(d), None) == _ffi.MK_ERR_INVALID
    # the descriptor rules of mk_gemm hold here too: a null peer pointer and unknown flag bits are refused on the host
    d = desc_for(a, a, a, 16, 16, 16)
    d.n_peers = 1
    assert lib.mk_gemm_static(0, None, C.byref(d), None) == _ffi.MK_ERR_INVALID
    assert b"peer_C[0] is null" in lib.mk_last_error()
    d = desc_for(a, a, a, 16, 16, 16)
    d.flags = 0x80
    assert lib.mk_gemm_static(0, None, C.byref(d), None) == _ffi.MK_ERR_INVALID
    d = desc_for(a, a, a, 16, 16, 16)
    d.flags = _ffi.MK_GEMM_GATE_SIGMOID               # belongs to the gated epilogue, which this entry point does not offer
    assert lib.mk_gemm_static(0, None, C.byref(d), None) == _ffi.MK_ERR_INVALID
    err = C.c_uint32()
    assert lib.mk_gemm_static_status(0, None, _ffi.MK_STATIC_GEMM_MAX_BATCH + 1, C.byref(err)) == _ffi.MK_ERR_INVALID
