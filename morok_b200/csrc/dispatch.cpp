// Argument validation and kernel selection for the compute entry points.
#include <cmath>

#include "mk_internal.h"

using namespace mk;

namespace mk {
// The descriptor rules every GEMM entry point shares (mk_gemm and mk_gemm_static): dtypes, dimensions,
// leading dimensions, epilogue and flag combinations, peers.  Normalises batch <= 0 to 1.  *nothing_to_do is
// set for M == 0 or N == 0 (no output elements), which skips the pointer checks.
mk_status validate_gemm_desc(mk_gemm_desc& d, const char* who, bool* nothing_to_do) {
    *nothing_to_do = false;
    MK_REQUIRE((dtype_valid(d.dtype_in) || dtype_is_fp8(d.dtype_in)) && dtype_valid(d.dtype_out),
               "%s: unsupported dtype (%d -> %d): inputs f32 / bf16 / f16 / 8-bit float, output f32 / bf16 / f16", who, d.dtype_in, d.dtype_out);
    MK_REQUIRE(d.M >= 0 && d.N >= 0 && d.K >= 0, "%s: negative dimension (M=%lld N=%lld K=%lld)", who, (long long)d.M,
               (long long)d.N, (long long)d.K);
    if (d.batch <= 0) d.batch = 1;
    if (d.M == 0 || d.N == 0) {
        *nothing_to_do = true;
        return MK_OK;
    }
    MK_REQUIRE(d.C, "%s: null C", who);
    MK_REQUIRE(d.K == 0 || (d.A && d.B), "%s: null A or B", who);
    MK_REQUIRE(d.lda >= d.K, "%s: lda %lld < K %lld", who, (long long)d.lda, (long long)d.K);
    MK_REQUIRE(d.ldb >= (d.trans_b ? d.K : d.N), "%s: ldb %lld too small", who, (long long)d.ldb);
    MK_REQUIRE(d.ldc >= d.N, "%s: ldc %lld < N %lld", who, (long long)d.ldc, (long long)d.N);
    MK_REQUIRE(d.epilogue >= MK_EPI_NONE && d.epilogue <= MK_EPI_SWIGLU, "%s: unknown epilogue %d", who, d.epilogue);
    MK_REQUIRE(d.epilogue == MK_EPI_NONE || d.epilogue == MK_EPI_SWIGLU || d.D, "%s: the epilogue needs D", who);
    MK_REQUIRE(d.epilogue != MK_EPI_SWIGLU || (d.B2 && d.K > 0 && d.n_peers == 0 && !(d.flags & MK_GEMM_SCALED)),
               "%s: MK_EPI_SWIGLU needs B2 and K > 0, and takes neither peers nor alpha / beta", who);
    MK_REQUIRE((d.flags & ~(uint32_t)(MK_GEMM_SCALED | MK_GEMM_GATE_SIGMOID)) == 0, "%s: unknown flags 0x%x", who, d.flags);
    MK_REQUIRE(!(d.flags & MK_GEMM_GATE_SIGMOID) || d.epilogue == MK_EPI_SWIGLU, "%s: MK_GEMM_GATE_SIGMOID belongs to MK_EPI_SWIGLU", who);
    MK_REQUIRE(d.n_peers >= 0 && d.n_peers <= MK_MAX_PEERS, "%s: n_peers %d out of range", who, d.n_peers);
    for (int i = 0; i < d.n_peers; ++i) MK_REQUIRE(d.peer_C[i], "%s: peer_C[%d] is null", who, i);
    return MK_OK;
}
}  // namespace mk

extern "C" {

mk_status mk_gemm(mk_device* dev, mk_stream* s, const mk_gemm_desc* desc) {
    MK_REQUIRE(dev && desc, "mk_gemm: null argument");
    mk_gemm_desc d = *desc;
    bool nothing_to_do = false;
    mk_status vs = validate_gemm_desc(d, "mk_gemm", &nothing_to_do);
    if (vs != MK_OK) return vs;
    if (nothing_to_do) return MK_OK;
    if (dev->mock) return fail(MK_ERR_CUDA, "mk_gemm: no CUDA device (mock devices run no kernels)");
    MK_CUDA(cudaSetDevice(dev->ordinal));
    bool handled = false;
    mk_status st = gemm_skinny(dev, raw(s), d, &handled);      // at most 16 rows against [N, K] weights: stream the weights once
    if (st != MK_OK) return st;
    if (handled) return MK_OK;
    st = gemm_sm100(dev, raw(s), d, &handled);
    if (st != MK_OK) return st;
    if (handled) return MK_OK;
    if (d.epilogue == MK_EPI_SWIGLU)
        return fail(MK_ERR_UNSUPPORTED, "mk_gemm: MK_EPI_SWIGLU runs on the tensor-core kernel only (16-bit inputs and outputs, 16-byte aligned rows)");
    return gemm_simt(dev, raw(s), d);
}

mk_status mk_sdpa_fwd(mk_device* dev, mk_stream* s, const mk_sdpa_desc* desc) {
    MK_REQUIRE(dev && desc, "mk_sdpa_fwd: null argument");
    const mk_sdpa_desc& d = *desc;
    MK_REQUIRE(dtype_valid(d.dtype), "mk_sdpa_fwd: unknown dtype %d", d.dtype);
    MK_REQUIRE(d.B >= 0 && d.Hq >= 0 && d.Sq >= 0 && d.Sk >= 0 && d.D > 0 && d.Dv > 0, "mk_sdpa_fwd: bad shape");
    MK_REQUIRE(d.Hkv > 0 && d.Hq % d.Hkv == 0, "mk_sdpa_fwd: Hq %d is not a multiple of Hkv %d", d.Hq, d.Hkv);
    MK_REQUIRE(d.n_peers >= 0 && d.n_peers <= MK_MAX_PEERS, "mk_sdpa_fwd: n_peers %d out of range", d.n_peers);
    if (d.B == 0 || d.Hq == 0 || d.Sq == 0) return MK_OK;
    MK_REQUIRE(d.Q && d.O && (d.Sk == 0 || (d.K && d.V)), "mk_sdpa_fwd: null tensor");
    for (int i = 0; i < d.n_peers; ++i) MK_REQUIRE(d.peer_O[i], "mk_sdpa_fwd: peer_O[%d] is null", i);
    MK_REQUIRE(d.mask_kind >= MK_MASK_SQ_SK && d.mask_kind <= MK_MASK_BOOL, "mk_sdpa_fwd: unknown mask_kind %d", d.mask_kind);
    MK_REQUIRE(!d.mask || (d.mask_strides[0] >= 0 && d.mask_strides[1] >= 0 && d.mask_strides[2] >= 0), "mk_sdpa_fwd: negative mask stride");
    const float scale = d.scale > 0.0f ? d.scale : 1.0f / std::sqrt((float)d.D);
    if (dev->mock) return fail(MK_ERR_CUDA, "mk_sdpa_fwd: no CUDA device (mock devices run no kernels)");
    MK_CUDA(cudaSetDevice(dev->ordinal));
    bool handled = false;
    // a few query rows against a long key stream: the HBM-bound split-key kernel
    mk_status st = sdpa_decode(dev, raw(s), d, scale, &handled);
    if (st != MK_OK) return st;
    if (handled) return MK_OK;
    st = sdpa_sm100(dev, raw(s), d, scale, &handled);
    if (st != MK_OK) return st;
    if (handled) return MK_OK;
    return sdpa_simt(dev, raw(s), d, scale);
}

mk_status mk_launch_count(mk_device* dev, uint64_t* launches) {
    MK_REQUIRE(dev && launches, "mk_launch_count: null argument");
    *launches = dev->launches.load();
    return MK_OK;
}

}  // extern "C"
