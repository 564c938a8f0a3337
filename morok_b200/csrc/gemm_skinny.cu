// GEMM for at most 16 rows against `linear` weights [N, K] (decoding: one new token per sequence).
// The work is reading the weights once -- 2 * M flop per 2 bytes -- so this kernel is built to keep HBM
// busy, not the tensor pipe: tcgen05's minimum M of 64 (128 here) would spend tensor memory, a K-split and
// a merge launch on a problem whose arithmetic fits one warp-level `mma.sync.m16n8k16` per 8 weight rows.
// The reference has no separate path: `linear` (tensor/src/matmul.rs:161-187) is the same generated
// kernel whatever M is.
//
//   grid   one persistent CTA per SM; the N / 8 blocks of 8 weight rows are dealt out as contiguous
//          ranges, so CTAs differ by at most one block (no wave quantisation, no second launch); a range is
//          walked in evenly sized groups of up to 4 blocks, (group, 256-k chunk) by (group, chunk)
//   load   one producer warp issues, per chunk, four 64-k TMA boxes of A (16 rows, from L2: every CTA reads
//          the same ones) and four 32-row boxes of the weights (from HBM; the group's blocks first) into
//          128-byte-swizzled stages of an 8-deep ring and signals a `full` mbarrier; the ring runs across
//          group boundaries, so it never drains.  (A first version filled the ring with cp.async from all
//          threads: it kept too few bytes in flight per SM and stopped at 2.5-3.0 TB/s.)
//   math   16 consumer warps = 4 blocks x 4 k quarters, one 64-k box each: A fragments and weight rows via
//          ldmatrix at the swizzled addresses (W[n][k] is the "col" operand of mma.sync as stored), one f32
//          accumulator per 16-k step so that no mma waits for another; the stage is released on an `empty`
//          mbarrier
//   store  the quarters' sums meet in shared memory through two more mbarrier pairs (no CTA-wide barrier
//          after start-up, every wait bounded); bias row / residual / alpha, beta as in the tensor-core
//          kernels, or with a second weight matrix the gated pair act(A W^T + b1) * (A W2^T + b2)
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>
#include <type_traits>

#include "mk_internal.h"
#include "ptx_sm100.cuh"

namespace mk {
namespace {

constexpr int BLOCKS = 4;                  // 8-row blocks of the weights per group
constexpr int KSPLIT = 4;                  // warps per block: each takes a quarter of every k chunk
constexpr int ROWS_A = 16;                 // the M of one mma
constexpr int KC = 256;                    // k per stage

struct SkinnyParams {
    const void *A, *W, *W2;
    void* C;
    const void *D, *D2;          // plain: residual (ldd = ldc) or bias row (ldd = 0); gated: bias rows of the two products
    int64_t M, N, K, lda, ldw, ldc, ldd;
    float alpha, beta;
    int scaled, gate_sigmoid, dtype_out;
    int row_blocks;              // ceil(N / 8)
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <bool BF16>
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if constexpr (BF16) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    } else {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
}

__device__ __forceinline__ float load_out(const void* p, int64_t i, int dt) {
    if (dt == MK_F32) return ((const float*)p)[i];
    if (dt == MK_BF16) return __bfloat162float(((const __nv_bfloat16*)p)[i]);
    return __half2float(((const __half*)p)[i]);
}
__device__ __forceinline__ void store_out(void* p, int64_t i, int dt, float v) {
    if (dt == MK_F32) ((float*)p)[i] = v;
    else if (dt == MK_BF16) ((__nv_bfloat16*)p)[i] = __float2bfloat16_rn(v);
    else ((__half*)p)[i] = __float2half_rn(v);
}

constexpr int CONSUMER_WARPS = BLOCKS * KSPLIT;          // 16
constexpr int THREADS = (CONSUMER_WARPS + 1) * 32;
constexpr int SUBS = KC / 64;                            // 64-k boxes per chunk = k quarters
static_assert(SUBS == KSPLIT, "one 64-k box per consumer warp and chunk");
constexpr int TA_BOX = ROWS_A * 128;                     // 2 KiB: 16 rows of 128 bytes
constexpr int TW_BOX = 8 * 128;                          // 1 KiB: one swizzle atom
constexpr int TA_BYTES = SUBS * TA_BOX;                  // 8 KiB
constexpr int TW_BYTES = SUBS * BLOCKS * TW_BOX;         // 16 KiB
constexpr int TRED_BYTES = 2 * (KSPLIT - 1) * BLOCKS * 32 * 8 * 4;   // two buffers of partial sums

template <bool DUAL>
struct Ring {
    static constexpr int STAGE_BYTES = TA_BYTES + (DUAL ? 2 : 1) * TW_BYTES;
    static constexpr int STAGES = DUAL ? 5 : 8;
    static constexpr int NUM_BARS = 2 * STAGES + 4;
    static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + TRED_BYTES + 256;
};

template <bool BF16, bool DUAL>
__global__ void __launch_bounds__(THREADS, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmW2,
                       const SkinnyParams p, KernelError* kerr) {
    using namespace ptx;
    using R = Ring<DUAL>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    float* red = reinterpret_cast<float*>(smem + R::STAGES * R::STAGE_BYTES);          // [2][KSPLIT - 1][BLOCKS][32 lanes][8]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + R::STAGES * R::STAGE_BYTES + TRED_BYTES);
    volatile uint32_t* abort_flag = reinterpret_cast<uint32_t*>(bars + R::NUM_BARS);
    const uint32_t bar_full = smem_u32(bars);                       // [STAGES] the chunk has landed
    const uint32_t bar_empty = smem_u32(bars + R::STAGES);          // [STAGES] all 16 consumer warps are done with it
    const uint32_t bar_rfull = smem_u32(bars + 2 * R::STAGES);      // [2] the 12 partial sums of a group are written
    const uint32_t bar_rempty = smem_u32(bars + 2 * R::STAGES + 2); // [2] the 4 finishing warps have read them
    const uint32_t smem_base = smem_u32(smem);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int i = 0; i < R::STAGES; ++i) {
            mbar_init(bar_full + 8 * i, 1);
            mbar_init(bar_empty + 8 * i, CONSUMER_WARPS);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar_rfull + 8 * i, (KSPLIT - 1) * BLOCKS);
            mbar_init(bar_rempty + 8 * i, BLOCKS);
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&tmA);
        prefetch_tensormap(&tmW);
        if (DUAL) prefetch_tensormap(&tmW2);
    }
    __syncthreads();

    // this CTA's contiguous range of 8-row blocks, cut evenly into groups of at most BLOCKS
    const int64_t blk_begin = (int64_t)blockIdx.x * p.row_blocks / gridDim.x;
    const int bt = (int)((int64_t)(blockIdx.x + 1) * p.row_blocks / gridDim.x - blk_begin);
    const int groups = (bt + BLOCKS - 1) / BLOCKS;
    const int nk = (int)((p.K + KC - 1) / KC);
    const int total = groups * nk;

    if (warp == CONSUMER_WARPS) {
        // producer: all lanes run the loop and the waits, one elected lane issues the copies
        const bool leader = elect_one_u32() != 0;
        int stage = 0, kc = 0, grp = 0, b0 = 0, b1 = bt / groups;
        int kcr = (int)(blockIdx.x % (unsigned)nk);     // CTAs walk K from different starting chunks
        uint32_t phase = 0;
        for (int it = 0; it < total; ++it) {
            if (!__all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, kerr, KERR_SKINNY_PRODUCER_WAIT, it))) break;
            if (leader) {
                const uint32_t full = bar_full + 8 * stage;
                const uint32_t sa = smem_base + stage * R::STAGE_BYTES, sw = sa + TA_BYTES;
                // One 32-row weight box per 64-k quarter whatever the group's size: a thread issues a TMA copy
                // every ~45 clocks, so 1 KiB boxes per block made the producer the bottleneck (3.2 TB/s).  Rows
                // past the group's blocks belong to the next group or CTA (or are zero past N); nobody reads them here.
                mbar_arrive_expect_tx(full, R::STAGE_BYTES);
                const int y0 = (int)(blk_begin + b0) * 8;
#pragma unroll
                for (int sb = 0; sb < SUBS; ++sb) {
                    const int x = kcr * KC + sb * 64;       // 128 bytes: a legal TMA start; past K the box is zero-filled
                    tma_load_2d(sa + sb * TA_BOX, &tmA, full, x, 0);
                    tma_load_2d(sw + sb * BLOCKS * TW_BOX, &tmW, full, x, y0);
                    if constexpr (DUAL) tma_load_2d(sw + TW_BYTES + sb * BLOCKS * TW_BOX, &tmW2, full, x, y0);
                }
            }
            if (++stage == R::STAGES) { stage = 0; phase ^= 1; }
            kcr = kcr + 1 == nk ? 0 : kcr + 1;
            if (++kc == nk) {
                kc = 0;
                ++grp;
                b0 = b1;
                b1 = (grp + 1) * bt / groups;
            }
        }
    } else {
        const int g = lane >> 2, t4 = lane & 3;
        const int wb = warp % BLOCKS, kh = warp / BLOCKS;
        constexpr int NACC = 4;                      // one accumulator per 16-k step of the warp's 64-k box
        float acc[NACC][4], acc2[DUAL ? NACC : 1][4];
#pragma unroll
        for (int j = 0; j < NACC; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                acc[j][e] = 0.f;
                if (DUAL) acc2[j][e] = 0.f;
            }
        // swizzled fragment addresses inside a stage: 16-byte piece c of row r sits at piece c ^ (r & 7)
        const int ar = lane & 15, wr = lane & 7;
        uint32_t a_addr[4], w_addr[2];
#pragma unroll
        for (int t = 0; t < 4; ++t) a_addr[t] = smem_base + kh * TA_BOX + ar * 128 + (((2 * t + (lane >> 4)) ^ (ar & 7)) << 4);
#pragma unroll
        for (int st = 0; st < 2; ++st) w_addr[st] = smem_base + TA_BYTES + (kh * BLOCKS + wb) * TW_BOX + wr * 128 + (((4 * st + (lane >> 3)) ^ wr) << 4);
        int stage = 0, kc = 0, grp = 0, b0 = 0, b1 = bt / groups;
        uint32_t phase = 0;
        for (int it = 0; it < total; ++it) {
            if (!__all_sync(0xffffffffu, mbar_wait(bar_full + 8 * stage, phase, abort_flag, kerr, KERR_SKINNY_CONSUMER_WAIT, it))) break;
            const bool active = wb < b1 - b0;        // warp-uniform
            if (active) {
                const uint32_t so = stage * R::STAGE_BYTES;
#pragma unroll
                for (int st = 0; st < 2; ++st) {
                    uint32_t a0[4], a1[4], b[4];
                    ldmatrix_x4(a_addr[2 * st] + so, a0);
                    ldmatrix_x4(a_addr[2 * st + 1] + so, a1);
                    ldmatrix_x4(w_addr[st] + so, b);
                    mma_16816<BF16>(acc[2 * st], a0, b[0], b[1]);
                    mma_16816<BF16>(acc[2 * st + 1], a1, b[2], b[3]);
                    if constexpr (DUAL) {
                        uint32_t b2[4];
                        ldmatrix_x4(w_addr[st] + so + TW_BYTES, b2);
                        mma_16816<BF16>(acc2[2 * st], a0, b2[0], b2[1]);
                        mma_16816<BF16>(acc2[2 * st + 1], a1, b2[2], b2[3]);
                    }
                }
            }
            // the mma instructions above could only issue once their fragments had arrived in registers:
            // the stage has been read
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + 8 * stage);
            if (++stage == R::STAGES) { stage = 0; phase ^= 1; }
            if (++kc < nk) continue;

            // the group's K loop is complete: the warps of k quarters 1-3 hand their sums over, quarter 0 finishes
            float sum[4], sum2[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                sum[e] = 0.f;
                sum2[e] = 0.f;
#pragma unroll
                for (int j = 0; j < NACC; ++j) {
                    sum[e] += acc[j][e];
                    acc[j][e] = 0.f;
                    if (DUAL) { sum2[e] += acc2[j][e]; acc2[j][e] = 0.f; }
                }
            }
            const int buf = grp & 1;
            const uint32_t use = (uint32_t)(grp >> 1) & 1u;      // parity of this buffer's current round
            float* rbuf = red + buf * ((KSPLIT - 1) * BLOCKS * 32 * 8);
            if (kh != 0) {
                if (!__all_sync(0xffffffffu, mbar_wait(bar_rempty + 8 * buf, use ^ 1, abort_flag, kerr, KERR_SKINNY_REDUCE_WAIT, grp))) break;
                float* r = rbuf + (((kh - 1) * BLOCKS + wb) * 32 + lane) * 8;
#pragma unroll
                for (int e = 0; e < 4; ++e) { r[e] = sum[e]; r[4 + e] = sum2[e]; }
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_rfull + 8 * buf);
            } else {
                if (!__all_sync(0xffffffffu, mbar_wait(bar_rfull + 8 * buf, use, abort_flag, kerr, KERR_SKINNY_REDUCE_WAIT, 1000000 + grp))) break;
#pragma unroll
                for (int q = 0; q < KSPLIT - 1; ++q) {
                    const float* r = rbuf + ((q * BLOCKS + wb) * 32 + lane) * 8;
#pragma unroll
                    for (int e = 0; e < 4; ++e) { sum[e] += r[e]; sum2[e] += r[4 + e]; }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_rempty + 8 * buf);
                if (active) {
                    const int64_t blk = blk_begin + b0 + wb;
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int64_t row = g + 8 * (e >> 1), col = blk * 8 + t4 * 2 + (e & 1);
                        if (row >= p.M || col >= p.N) continue;
                        float v = sum[e];
                        if constexpr (DUAL) {
                            float u = sum2[e];
                            if (p.D) v += load_out(p.D, col, p.dtype_out);
                            if (p.D2) u += load_out(p.D2, col, p.dtype_out);
                            const float sg = 1.0f / (1.0f + exp2f(v * -1.4426950408889634f));
                            v = (p.gate_sigmoid ? sg : v * sg) * u;
                        } else {
                            if (p.scaled) v *= p.alpha;
                            if (p.D) v = fmaf(p.beta, load_out(p.D, row * p.ldd + col, p.dtype_out), v);
                        }
                        store_out(p.C, row * p.ldc + col, p.dtype_out, v);
                    }
                }
            }
            kc = 0;
            ++grp;
            b0 = b1;
            b1 = (grp + 1) * bt / groups;
        }
    }
    // a wait that gave up: give the copies still in flight time to land before the CTA's shared memory is reused
    if (*abort_flag) __nanosleep(2000000);
    __syncthreads();
}

// MOROK_B200_GEMM_SKINNY: 0 = never, 1 = by the size rule below (default), 2 = whenever the problem qualifies.
int skinny_mode() {
    static int v = [] {
        const char* e = getenv("MOROK_B200_GEMM_SKINNY");
        return e ? atoi(e) : 1;
    }();
    return v;
}
// Measured against the K-split tensor-core path (16 rows, bf16, 50 back-to-back calls on one box, us):
//   4096 x 4096 12.4-14.6 vs 16.6 | 1024 x 4096 10.6 vs 18.5 | 6144 x 4096 14.7 vs 20.3 | 8192 x 4096 14.4 vs 20.5
//   14336 x 4096 26.7 vs 34.9 | 4096 x 14336 24.5 vs 37.0 | 2048 x 16384 20.6 vs 24.6 | 5120 x 13824 36.5 vs 41.0
//   gated pairs: 14336 x 4096 45.2 vs 63.7 | 4096 x 4096 12.1 vs 34.9 | 11008 x 4096 34.9 vs 59.7
// and it loses where rows are short or few: 65536 x 512 22.6 vs 21.5, 131072 x 256 32.9 vs 28.9, 512 x 65536
// (64 CTAs only) 67.7 vs 41.2.  Rule: small problems always (one launch), large ones when K >= 1024 and N >= 1024.
constexpr int64_t kSmallWeightBytes = 40ll << 20;
}  // namespace

// Runs the few-row kernel when the problem qualifies (with `dry_run` it only reports whether it would);
// otherwise leaves *handled = false.
mk_status gemm_skinny(mk_device* dev, cudaStream_t st, const mk_gemm_desc& d, bool* handled, bool dry_run) {
    *handled = false;
    if (skinny_mode() == 0 || dev->prop.major < 9) return MK_OK;      // TMA and mbarriers
    if (d.dtype_in != MK_BF16 && d.dtype_in != MK_F16) return MK_OK;
    if (!d.trans_b || d.M <= 0 || d.M > ROWS_A || d.N <= 0 || d.K <= 0 || d.n_peers != 0) return MK_OK;
    const bool dual = d.epilogue == MK_EPI_SWIGLU;
    if (dual && d.dtype_out == MK_F32) return MK_OK;
    if (skinny_mode() == 1 && d.N * d.K * 2 * (dual ? 2 : 1) > kSmallWeightBytes && (d.K < 1024 || d.N < 1024)) return MK_OK;
    // TMA wants 16-byte aligned bases and row pitches; K in whole 16-byte pieces keeps every box row aligned
    if ((reinterpret_cast<uintptr_t>(d.A) & 15) || (reinterpret_cast<uintptr_t>(d.B) & 15) || (dual && (reinterpret_cast<uintptr_t>(d.B2) & 15))) return MK_OK;
    if ((d.lda % 8) || (d.ldb % 8) || (d.K % 8) || (d.stride_a % 8) || (d.stride_b % 8)) return MK_OK;
    if (d.N > 0x3fffffffll || d.K > 0x3fffffffll) return MK_OK;
    if (dry_run) {
        *handled = true;
        return MK_OK;
    }

    const size_t es_out = dtype_size(d.dtype_out);
    for (int b = 0; b < d.batch; ++b) {
        SkinnyParams p{};
        p.A = (const char*)d.A + (size_t)b * d.stride_a * 2;
        p.W = (const char*)d.B + (size_t)b * d.stride_b * 2;
        p.W2 = dual ? (const char*)d.B2 + (size_t)b * d.stride_b * 2 : nullptr;
        p.C = (char*)d.C + (size_t)b * d.stride_c * es_out;
        if (dual) {
            p.D = d.D;
            p.D2 = d.D2;
        } else {
            p.D = d.epilogue == MK_EPI_ADD ? (const char*)d.D + (size_t)b * d.stride_c * es_out : d.epilogue == MK_EPI_ADD_ROW ? (const char*)d.D : nullptr;
        }
        p.M = d.M; p.N = d.N; p.K = d.K;
        p.lda = d.lda; p.ldw = d.ldb; p.ldc = d.ldc;
        p.ldd = d.epilogue == MK_EPI_ADD_ROW ? 0 : d.ldc;
        p.scaled = (d.flags & MK_GEMM_SCALED) ? 1 : 0;
        p.alpha = p.scaled ? d.alpha : 1.0f;
        p.beta = p.scaled ? d.beta : 1.0f;
        p.gate_sigmoid = (d.flags & MK_GEMM_GATE_SIGMOID) ? 1 : 0;
        p.dtype_out = d.dtype_out;
        p.row_blocks = (int)((d.N + 7) / 8);
        const int grid = std::min(dev->prop.multiProcessorCount, p.row_blocks);
        const bool bf = d.dtype_in == MK_BF16;
        alignas(64) CUtensorMap ta, tw, tw2;
        mk_status e1 = tma_encode_2d(&ta, d.dtype_in, p.A, (uint64_t)d.K, (uint64_t)d.M, (uint64_t)d.lda * 2, 64, ROWS_A);
        if (e1 == MK_OK) e1 = tma_encode_2d(&tw, d.dtype_in, p.W, (uint64_t)d.K, (uint64_t)d.N, (uint64_t)d.ldb * 2, 64, 8 * BLOCKS);
        tw2 = tw;
        if (e1 == MK_OK && dual) e1 = tma_encode_2d(&tw2, d.dtype_in, p.W2, (uint64_t)d.K, (uint64_t)d.N, (uint64_t)d.ldb * 2, 64, 8 * BLOCKS);
        if (e1 != MK_OK) return e1;
#define MK_SKINNY(BF, DUAL_)                                                                                                       \
    do {                                                                                                                           \
        auto kern = gemm_skinny_kernel<BF, DUAL_>;                                                                                 \
        MK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Ring<DUAL_>::SMEM_BYTES));                 \
        kern<<<grid, THREADS, Ring<DUAL_>::SMEM_BYTES, st>>>(ta, tw, tw2, p, stream_kerr(dev, st));                                           \
    } while (0)
        if (dual) { if (bf) MK_SKINNY(true, true); else MK_SKINNY(false, true); }
        else { if (bf) MK_SKINNY(true, false); else MK_SKINNY(false, false); }
#undef MK_SKINNY
        MK_CUDA(cudaGetLastError());
        note_launch(dev, st, dual ? "gemm_skinny_gated" : "gemm_skinny");
    }
    *handled = true;
    return MK_OK;
}

}  // namespace mk
