// General attention forward on the FMA pipes: any dtype (f32 / bf16 / f16), any head size up to
// 512, additive mask, softcap, ragged Sq / Sk.  One warp owns one query row and walks the keys
// 32 at a time with an online softmax, so the [Sq, Sk] score matrix of the reference's
// formulation (tensor/src/transformer.rs:78-137 materialises it) never exists in memory.
// Serves every case the tensor-core kernel does not take; statistics and accumulation are f32.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math_constants.h>

#include "mk_internal.h"

namespace mk {
namespace {

template <typename T>
__device__ __forceinline__ float ldf(const T* p, int64_t i);
template <>
__device__ __forceinline__ float ldf<float>(const float* p, int64_t i) { return p[i]; }
template <>
__device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }
template <>
__device__ __forceinline__ float ldf<__half>(const __half* p, int64_t i) { return __half2float(p[i]); }

template <typename T>
__device__ __forceinline__ T cvt(float v);
template <>
__device__ __forceinline__ float cvt<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 cvt<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half cvt<__half>(float v) { return __float2half_rn(v); }

constexpr int MAX_D = 512;
constexpr int WARPS = 4;

struct SimtSdpa {
    mk_sdpa_desc d;
    float scale;
};

template <typename T>
__global__ void __launch_bounds__(WARPS * 32) sdpa_simt_kernel(const SimtSdpa P) {
    const mk_sdpa_desc& d = P.d;
    __shared__ float sq[WARPS][MAX_D];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t rows = (int64_t)d.B * d.Hq * d.Sq;
    const int group = d.Hq / d.Hkv;
    constexpr int OPL = MAX_D / 32;  // output columns per lane

    for (int64_t row = (int64_t)blockIdx.x * WARPS + warp; row < rows; row += (int64_t)gridDim.x * WARPS) {
        const int i = (int)(row % d.Sq);
        const int h = (int)((row / d.Sq) % d.Hq);
        const int b = (int)(row / ((int64_t)d.Sq * d.Hq));
        const int hk = h / group;
        const T* q = (const T*)d.Q + b * d.q_strides[0] + h * d.q_strides[1] + i * d.q_strides[2];
        const T* kb = (const T*)d.K + b * d.k_strides[0] + hk * d.k_strides[1];
        const T* vb = (const T*)d.V + b * d.v_strides[0] + hk * d.v_strides[1];
        const int64_t o_off = b * d.o_strides[0] + h * d.o_strides[1] + i * d.o_strides[2];
        // this row's mask values (tensor/src/transformer.rs:112-124): additive f32, or bool where false adds -inf
        const int64_t m_off = d.mask_kind == MK_MASK_SQ_SK ? (int64_t)i * d.Sk
                                                           : b * d.mask_strides[0] + h * d.mask_strides[1] + i * d.mask_strides[2];
        const float* mask_f = (d.mask && d.mask_kind != MK_MASK_BOOL) ? (const float*)d.mask + m_off : nullptr;
        const unsigned char* mask_b = (d.mask && d.mask_kind == MK_MASK_BOOL) ? (const unsigned char*)d.mask + m_off : nullptr;

        __syncwarp();
        for (int x = lane; x < d.D; x += 32) sq[warp][x] = ldf<T>(q, x);
        __syncwarp();

        float m = -CUDART_INF_F, l = 0.0f;
        float o[OPL];
#pragma unroll
        for (int c = 0; c < OPL; ++c) o[c] = 0.0f;

        // Causal rows never look past column i + causal_offset (keep col <= row + offset).  With a softcap
        // the reference applies tanh AFTER masking (tensor/src/transformer.rs:103-132), which turns
        // the masked -inf into -softcap; those columns then take part, so they are not skipped.
        const bool skip_masked = d.causal && !(d.softcap > 0.0f);
        const int64_t last_col = (int64_t)i + d.causal_offset;          // last visible column under the causal rule
        const int k_end = skip_masked ? (int)max((int64_t)0, min((int64_t)d.Sk, last_col + 1)) : d.Sk;
        for (int j0 = 0; j0 < k_end; j0 += 32) {
            const int j = j0 + lane;
            float s = -CUDART_INF_F;
            if (j < k_end) {
                const T* kr = kb + (int64_t)j * d.k_strides[2];
                float acc = 0.0f;
                for (int x = 0; x < d.D; ++x) acc = fmaf(sq[warp][x], ldf<T>(kr, x), acc);
                s = acc * P.scale;
                if (d.causal && j > last_col) s = -CUDART_INF_F;
                if (mask_f) s += mask_f[j];
                if (mask_b && !mask_b[j]) s = -CUDART_INF_F;
                if (d.softcap > 0.0f) s = tanhf(s / d.softcap) * d.softcap;
            }
            float mx = s;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
            const float m_new = fmaxf(m, mx);
            // A block whose every score is -inf leaves the running state untouched.
            if (m_new == -CUDART_INF_F) continue;
            const float alpha = (m == -CUDART_INF_F) ? 0.0f : expf(m - m_new);
            const float p = (j < k_end) ? expf(s - m_new) : 0.0f;
            float ps = p;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, off);
            l = l * alpha + ps;
            m = m_new;
#pragma unroll
            for (int c = 0; c < OPL; ++c) o[c] *= alpha;
            const int cnt = min(32, k_end - j0);
            for (int jj = 0; jj < cnt; ++jj) {
                const float pj = __shfl_sync(0xffffffffu, p, jj);
                const T* vr = vb + (int64_t)(j0 + jj) * d.v_strides[2];
#pragma unroll
                for (int c = 0; c < OPL; ++c) {
                    const int x = lane + 32 * c;
                    if (x < d.Dv) o[c] = fmaf(pj, ldf<T>(vr, x), o[c]);
                }
            }
        }
        // Sk == 0 yields zeros (an empty P V product); a row whose scores are all -inf yields NaN,
        // as exp(-inf - (-inf)) does in the reference's softmax.
        const float inv = (d.Sk == 0) ? 0.0f : (l > 0.0f ? 1.0f / l : CUDART_NAN_F);
#pragma unroll
        for (int c = 0; c < OPL; ++c) {
            const int x = lane + 32 * c;
            if (x < d.Dv) {
                const T val = cvt<T>(o[c] * inv);
                ((T*)d.O)[o_off + x] = val;
                for (int pq = 0; pq < d.n_peers; ++pq) ((T*)d.peer_O[pq])[o_off + x] = val;
            }
        }
        if (d.lse && lane == 0) d.lse[row] = (l > 0.0f) ? m + logf(l) : -CUDART_INF_F;
    }
}

}  // namespace

mk_status sdpa_simt(mk_device* dev, cudaStream_t st, const mk_sdpa_desc& d, float scale) {
    if (d.D > MAX_D || d.Dv > MAX_D)
        return fail(MK_ERR_UNSUPPORTED, "mk_sdpa_fwd: head size %d / %d exceeds %d", d.D, d.Dv, MAX_D);
    SimtSdpa P{d, scale};
    const int64_t rows = (int64_t)d.B * d.Hq * d.Sq;
    const int64_t want = (rows + WARPS - 1) / WARPS;
    const int64_t cap = (int64_t)dev->prop.multiProcessorCount * 16;
    const int grid = (int)(want < cap ? want : cap);
    if (d.dtype == MK_F32) sdpa_simt_kernel<float><<<grid, WARPS * 32, 0, st>>>(P);
    else if (d.dtype == MK_BF16) sdpa_simt_kernel<__nv_bfloat16><<<grid, WARPS * 32, 0, st>>>(P);
    else sdpa_simt_kernel<__half><<<grid, WARPS * 32, 0, st>>>(P);
    MK_CUDA(cudaGetLastError());
    note_launch(dev, st, "sdpa_simt");
    return MK_OK;
}

}  // namespace mk
