// bf16 / f16 / 8-bit float GEMM with f32 accumulation on Blackwell tensor cores (sm_100a).
//
// Replaces the kernel morok would generate for a matmul whose operands route to tensor cores
// (schedule/src/optimizer/tc.rs:126-168: bf16->f32 and f16->f32 accumulate; tc.rs:358-674 builds
// per-warp 16x8x16 fragments).  Here the whole GEMM is one persistent kernel:
//
//   warp 0  TMA producer   : global -> 128-byte-swizzled shared-memory tiles, STAGES-deep ring
//   warp 1  MMA issuer     : tcgen05.mma (128 x 256 x 16 per instruction) accumulating a 128 x 256
//                            f32 tile in tensor memory; the whole warp runs the loop, one elected
//                            lane is predicated on the instruction (descriptors in uniform registers)
//   warp 2  TMEM allocator : 512 columns = two accumulators, so that the epilogue of tile i
//                            overlaps the main loop of tile i+1
//   warps 4-7 epilogue     : tcgen05.ld -> alpha, + beta D (matrix or bias row), or the SwiGLU gate of a
//                            pair of products -> cast -> shared-memory staging -> 128-bit global
//                            stores in whole 256-byte row segments, to the local C and, for
//                            N-sharded runs, straight into every peer GPU's C.  The CTA-pair form delivers
//                            sharded 16-bit outputs differently: the epilogue warps write 32 x 64 blocks in
//                            tile-store layout and one lane issues a tile store per destination, so the copy
//                            engine moves the bytes while the next accumulator is drained
// For M > 128 the CTA-pair form below is used (two CTAs share each MMA, 256 x 256 tiles); for M <= 128
// and long K the tile's K range is cut into units so that every SM streams weights (see gemm_sm100()).
//
// A is row-major [M,K] (K-major operand).  B is row-major [K,N] -- morok's matmul layout, an
// MN-major operand read without any transpose pass -- or [N,K] for `linear` weights (K-major).
// Tiles past M / N / K are zero-filled by TMA on load and predicated on store.
// Every barrier wait is bounded (ptx::mbar_wait); a wait that gives up records a code in the
// device error word and the CTA drains and exits.
#include <algorithm>
#include <cstdlib>
#include <mutex>

#include "ptx_sm100.cuh"

namespace mk {
namespace {

using namespace ptx;

constexpr int BM = 128, BN = 256, BK = 64;     // BK in 16-bit elements: one 128-byte swizzled row (= 128 8-bit elements)
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;            // 16 KiB
constexpr int B_BYTES = BK * BN * 2;            // 32 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;  // 48 KiB
constexpr int TMEM_COLS = 512;                  // 2 accumulators x 256 f32 columns
constexpr int NUM_BARS = 2 * STAGES + 4;
constexpr int OUT_STAGE_BYTES = 4 * 32 * 256;   // per epilogue warp: 32 rows x 256 bytes of output
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + OUT_STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers + slots */;
constexpr int NUM_THREADS = 256;

struct TcParams {
    int64_t M, N, K;
    void* C;
    const void* D;
    int64_t ldc;
    int64_t ldd;          // row stride of D: ldc, or 0 when D is one row added to every row (a bias)
    float alpha, beta;    // C = alpha * acc + beta * D
    int scaled;           // alpha / beta differ from 1
    int splits;           // > 1: K is cut into `splits` ranges of kb_per_split k-blocks; unit u = (tile u / splits, range u % splits)
    int kb_per_split;     //      writes its f32 partial tile to row block (u % splits) of the workspace passed as C
    int dual;             // gated pair of products: accumulator columns 0-127 = A B (gate), 128-255 = A B2 (up); 128 output columns
    int gate_sigmoid;     //   the gate is sigmoid(g) instead of silu(g)
    const void* D2;       //   bias row of the second product (D is the bias row of the first), either may be null
    uint32_t idesc;       // 128 x 256 instruction (one CTA)
    uint32_t idesc2;      // 256 x 256 instruction (CTA pair)
    int tiles_m, tiles_n, group_m;
    int tiles_m2;         // 256-row tiles (CTA pair)
    int staged;   // C, peers and ldc allow 16-byte stores: use the shared-memory staged, coalesced epilogue
    int n_peers;
    void* peer_C[MK_MAX_PEERS];
    KernelError* kerr;
};

__device__ __forceinline__ void tile_coords(int t, const TcParams& p, int& tm, int& tn) {
    // Grouped raster: consecutive tiles walk group_m row-tiles for one column-tile, then the next
    // column-tile, so that the tiles in flight on the 148 SMs share A and B panels in L2.
    const int per_group = p.group_m * p.tiles_n;
    const int g = t / per_group;
    const int first_m = g * p.group_m;
    const int rows = min(p.group_m, p.tiles_m - first_m);
    const int r = t - g * per_group;
    tm = first_m + r % rows;
    tn = r / rows;
}

// 32 consecutive f32 accumulators of one output row (+ D) -> output elements packed in 32-bit words.
// The same raster over 256-row tiles (CTA-pair kernel).
__device__ __forceinline__ void tile_coords2(int t, const TcParams& p, int& tm, int& tn) {
    const int group = max(1, p.group_m / 2);
    const int per_group = group * p.tiles_n;
    const int g = t / per_group;
    const int first_m = g * group;
    const int rows = min(group, p.tiles_m2 - first_m);
    const int r = t - g * per_group;
    tm = first_m + r % rows;
    tn = r / rows;
}

template <int OUT>
__device__ __forceinline__ void convert_chunk(const TcParams& p, int64_t row, int64_t col, const uint32_t (&r)[32],
                                              uint32_t (&w)[(OUT == MK_F32) ? 32 : 16]) {
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
    if (p.scaled) {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] *= p.alpha;
    }
    const float beta = p.beta;
    if (p.D && row < p.M && col < p.N) {
        const int64_t off = row * p.ldd + col;
        const bool full = col + 32 <= p.N;
        if constexpr (OUT == MK_F32) {
            const float* Dp = (const float*)p.D + off;
            if (full) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float4 d = reinterpret_cast<const float4*>(Dp)[i];
                    v[4 * i] = fmaf(beta, d.x, v[4 * i]); v[4 * i + 1] = fmaf(beta, d.y, v[4 * i + 1]);
                    v[4 * i + 2] = fmaf(beta, d.z, v[4 * i + 2]); v[4 * i + 3] = fmaf(beta, d.w, v[4 * i + 3]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (col + i < p.N) v[i] = fmaf(beta, Dp[i], v[i]);
            }
        } else {
            using T = typename std::conditional<OUT == MK_BF16, __nv_bfloat16, __half>::type;
            using T2 = typename std::conditional<OUT == MK_BF16, __nv_bfloat162, __half2>::type;
            const T* Dp = (const T*)p.D + off;
            if (full) {
                uint4 dv[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) dv[i] = reinterpret_cast<const uint4*>(Dp)[i];
                const T2* d2 = reinterpret_cast<const T2*>(dv);
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    float2 f;
                    if constexpr (OUT == MK_BF16) f = __bfloat1622float2(d2[i]); else f = __half22float2(d2[i]);
                    v[2 * i] = fmaf(beta, f.x, v[2 * i]);
                    v[2 * i + 1] = fmaf(beta, f.y, v[2 * i + 1]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (col + i < p.N) {
                        if constexpr (OUT == MK_BF16) v[i] = fmaf(beta, __bfloat162float(Dp[i]), v[i]); else v[i] = fmaf(beta, __half2float(Dp[i]), v[i]);
                    }
            }
        }
    }
    if constexpr (OUT == MK_F32) {
#pragma unroll
        for (int i = 0; i < 32; ++i) w[i] = __float_as_uint(v[i]);
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            if constexpr (OUT == MK_BF16) {
                __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                w[i] = *reinterpret_cast<uint32_t*>(&h);
            } else {
                __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
                w[i] = *reinterpret_cast<uint32_t*>(&h);
            }
        }
    }
}

template <int OUT>
__device__ __forceinline__ void store_chunk(const TcParams& p, int64_t row, int64_t col, const uint32_t (&r)[32]) {
    // 32 consecutive f32 accumulators of one output row, starting at column `col`.
    if (row >= p.M || col >= p.N) return;
    const int64_t off = row * p.ldc + col, doff = row * p.ldd + col;
    const bool full = (col + 32 <= p.N);
    if constexpr (OUT == MK_F32) {
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
        if (p.scaled) {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] *= p.alpha;
        }
        const float* Dp = (const float*)p.D;
        const bool vec = full && ((reinterpret_cast<uintptr_t>((float*)p.C + off) & 15) == 0) && (p.ldc % 4 == 0);
        if (Dp) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (col + i < p.N) v[i] = fmaf(p.beta, Dp[doff + i], v[i]);
        }
        for (int q = -1; q < p.n_peers; ++q) {
            float* Cp = (float*)(q < 0 ? p.C : p.peer_C[q]) + off;
            if (vec) {
#pragma unroll
                for (int i = 0; i < 8; ++i) reinterpret_cast<float4*>(Cp)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (col + i < p.N) Cp[i] = v[i];
            }
        }
    } else {
        using T = typename std::conditional<OUT == MK_BF16, __nv_bfloat16, __half>::type;
        using T2 = typename std::conditional<OUT == MK_BF16, __nv_bfloat162, __half2>::type;
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
        if (p.scaled) {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] *= p.alpha;
        }
        const T* Dp = (const T*)p.D;
        const bool vec = full && ((reinterpret_cast<uintptr_t>((T*)p.C + off) & 15) == 0) && (p.ldc % 8 == 0);
        if (Dp) {
            if (vec && ((reinterpret_cast<uintptr_t>(Dp + doff) & 15) == 0)) {
                uint4 dv[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) dv[i] = reinterpret_cast<const uint4*>(Dp + doff)[i];
                const T2* d2 = reinterpret_cast<const T2*>(dv);
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    float2 f;
                    if constexpr (OUT == MK_BF16) f = __bfloat1622float2(d2[i]); else f = __half22float2(d2[i]);
                    v[2 * i] = fmaf(p.beta, f.x, v[2 * i]);
                    v[2 * i + 1] = fmaf(p.beta, f.y, v[2 * i + 1]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (col + i < p.N) {
                        if constexpr (OUT == MK_BF16) v[i] = fmaf(p.beta, __bfloat162float(Dp[doff + i]), v[i]);
                        else v[i] = fmaf(p.beta, __half2float(Dp[doff + i]), v[i]);
                    }
            }
        }
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            T2 h;
            if constexpr (OUT == MK_BF16) h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]); else h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
            packed[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        for (int q = -1; q < p.n_peers; ++q) {
            T* Cp = (T*)(q < 0 ? p.C : p.peer_C[q]) + off;
            if (vec) {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    reinterpret_cast<uint4*>(Cp)[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
            } else {
                const T* ph = reinterpret_cast<const T*>(packed);
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (col + i < p.N) Cp[i] = ph[i];
            }
        }
    }
}

// Adds a bias row (N elements of the output type, 16-byte aligned) to 32 accumulators of columns col .. col + 31.
template <int OUT>
__device__ __forceinline__ void add_bias_row(const void* bias, int64_t col, int64_t N, uint32_t (&acc)[32]) {
    using T = typename std::conditional<OUT == MK_BF16, __nv_bfloat16, __half>::type;
    using T2 = typename std::conditional<OUT == MK_BF16, __nv_bfloat162, __half2>::type;
    const T* b = (const T*)bias + col;
    if (col + 32 <= N) {      // col is a multiple of 32, so these are aligned 16-byte loads (every row reads the same 64 bytes)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(b) + i);
            const uint32_t ws[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const T2 h = *reinterpret_cast<const T2*>(&ws[j]);
                float2 f;
                if constexpr (OUT == MK_BF16) f = __bfloat1622float2(h); else f = __half22float2(h);
                acc[8 * i + 2 * j] = __float_as_uint(__uint_as_float(acc[8 * i + 2 * j]) + f.x);
                acc[8 * i + 2 * j + 1] = __float_as_uint(__uint_as_float(acc[8 * i + 2 * j + 1]) + f.y);
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            if (col + j < N) {
                float f;
                if constexpr (OUT == MK_BF16) f = __bfloat162float(b[j]); else f = __half2float(b[j]);
                acc[j] = __float_as_uint(__uint_as_float(acc[j]) + f);
            }
        }
    }
}

// 32 gate and 32 up accumulators of one row (columns col .. col + 31) -> act(gate + bias) * (up + bias2), rounded
// once, packed in 16 words.  sigmoid(x) = 1 / (1 + exp2(-x log2 e)) and silu(x) = x sigmoid(x), the formulas of
// the element-wise kernels (tensor/src/activation.rs:42-52, 309-318).
template <int OUT>
__device__ __forceinline__ void gated_chunk(const TcParams& p, int64_t col, uint32_t (&g)[32], uint32_t (&u)[32], uint32_t (&w)[16]) {
    static_assert(OUT != MK_F32, "the gated epilogue stores 16-bit outputs");
    if (p.D) add_bias_row<OUT>(p.D, col, p.N, g);
    if (p.D2) add_bias_row<OUT>(p.D2, col, p.N, u);
    const bool plain_sigmoid = p.gate_sigmoid != 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        float v[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const float a = __uint_as_float(g[2 * i + e]), b = __uint_as_float(u[2 * i + e]);
            const float sg = 1.0f / (1.0f + exp2f(a * -1.4426950408889634f));
            v[e] = (plain_sigmoid ? sg : a * sg) * b;
        }
        if constexpr (OUT == MK_BF16) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[0], v[1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        } else {
            __half2 h = __floats2half2_rn(v[0], v[1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
    }
}

__device__ __forceinline__ void arrive_tempty(uint32_t bar, bool remote) {
    if (remote) mbar_arrive_cluster(bar); else mbar_arrive(bar);
}

// Epilogue of one 128 x 256 accumulator: the calling warp (lane quarter q) drains its 32 rows from
// tensor memory at `taddr`, hands the accumulator back (arrival on `tempty_bar`, which may live in
// the pair's leader CTA) and writes the rows tile_row0 + 32 q .. + 31, columns col0 .. col0 + 255.
template <int OUT>
__device__ __forceinline__ void epilogue_tile(const TcParams& p, int64_t tile_row0, int64_t col0, uint32_t taddr, uint8_t* stage_out,
                                              int q, int lane, uint32_t tempty_bar, bool tempty_remote) {
    const int64_t row = tile_row0 + q * 32 + lane;
    if (p.staged) {
        // Coalesced path: each warp turns its 32 x 256 accumulator block into output elements
        // 256 bytes of a row at a time, parks them in shared memory (16-byte pieces XOR-swizzled
        // by row so that both directions are bank-conflict free) and writes them out with
        // half-warps covering 256 contiguous bytes of one row -- full 128-byte lines for the
        // local C and for the copies that travel to peer GPUs over NVLink.
        constexpr int ES = (OUT == MK_F32) ? 4 : 2;
        constexpr int PASS_COLS = 256 / ES;            // columns staged per pass
        constexpr int CHUNKS = PASS_COLS / 32;         // 32-column TMEM loads per pass
        constexpr int N16 = 32 * ES / 16;              // 16-byte pieces per 32 columns
        uint8_t* stage = stage_out + q * 8192;
        const int64_t row0 = tile_row0 + q * 32;
        const int passes = p.dual ? 1 : BN / PASS_COLS;   // gated: 128 output columns, one pass of 256 bytes per row
#pragma unroll 1
        for (int ps = 0; ps < passes; ++ps) {
            const int64_t pc0 = col0 + ps * PASS_COLS;
            if (pc0 >= p.N) break;  // warp-uniform
#pragma unroll
            for (int c = 0; c < CHUNKS; ++c) {
                uint32_t r[32];
                tmem_ld_32x32b_x32(taddr + ps * PASS_COLS + c * 32, r);
                tmem_wait_ld();
                uint32_t w[32 * ES / 4];
                if constexpr (OUT != MK_F32) {
                    if (p.dual) {
                        uint32_t u[32];
                        tmem_ld_32x32b_x32(taddr + 128 + c * 32, u);
                        tmem_wait_ld();
                        gated_chunk<OUT>(p, pc0 + c * 32, r, u, w);
                    } else {
                        convert_chunk<OUT>(p, row, pc0 + c * 32, r, w);
                    }
                } else {
                    convert_chunk<OUT>(p, row, pc0 + c * 32, r, w);
                }
#pragma unroll
                for (int i = 0; i < N16; ++i)
                    *reinterpret_cast<uint4*>(stage + lane * 256 + (((c * N16 + i) ^ (lane & 15)) << 4)) =
                        make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
            }
            if (ps == passes - 1 || pc0 + PASS_COLS >= p.N) {
                // last TMEM read of this tile: hand the accumulator back before the stores
                tc_fence_before();
                arrive_tempty(tempty_bar, tempty_remote);
            }
            __syncwarp();
            constexpr int EPC = 16 / ES;                // elements per 16-byte piece
#pragma unroll 4
            for (int it = 0; it < 16; ++it) {
                const int rr = it * 2 + (lane >> 4), ch = lane & 15;
                const int64_t grow = row0 + rr, gcol = pc0 + ch * EPC;
                if (grow >= p.M || gcol >= p.N) continue;
                const uint4 v = *reinterpret_cast<const uint4*>(stage + rr * 256 + ((ch ^ (rr & 15)) << 4));
                const int64_t off = (grow * p.ldc + gcol) * ES;
                if (gcol + EPC <= p.N) {
                    *reinterpret_cast<uint4*>((char*)p.C + off) = v;
                    for (int pq = 0; pq < p.n_peers; ++pq) *reinterpret_cast<uint4*>((char*)p.peer_C[pq] + off) = v;
                } else {
                    const int nrem = (int)(p.N - gcol);
                    const uint8_t* vb = reinterpret_cast<const uint8_t*>(&v);
                    for (int b = 0; b < nrem * ES; ++b) {
                        ((char*)p.C)[off + b] = vb[b];
                        for (int pq = 0; pq < p.n_peers; ++pq) ((char*)p.peer_C[pq])[off + b] = vb[b];
                    }
                }
            }
            __syncwarp();
        }
    } else {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
            if (col0 + c * 32 >= p.N) break;  // warp-uniform
            uint32_t r[32];
            tmem_ld_32x32b_x32(taddr + c * 32, r);
            tmem_wait_ld();
            store_chunk<OUT>(p, row, col0 + c * 32, r);
        }
        tc_fence_before();
        arrive_tempty(tempty_bar, tempty_remote);
    }
}

template <bool TRANS_B, int OUT, bool F8 = false>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const TcParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* stage_out = smem + STAGES * STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(stage_out + OUT_STAGE_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NUM_BARS);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const uint32_t bar_full = smem_u32(bars);                        // [STAGES] TMA landed
    const uint32_t bar_empty = smem_u32(bars + STAGES);              // [STAGES] MMAs done reading
    const uint32_t bar_tfull = smem_u32(bars + 2 * STAGES);          // [2] accumulator complete
    const uint32_t bar_tempty = smem_u32(bars + 2 * STAGES + 2);     // [2] accumulator drained

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (p.splits > 1) grid_launch_dependents();      // the merge kernel may become resident now; it waits for this grid to finish

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) {
            mbar_init(bar_full + 8 * i, 1);
            mbar_init(bar_empty + 8 * i, 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar_tfull + 8 * i, 1);
            mbar_init(bar_tempty + 8 * i, 128);
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&tmA);
        prefetch_tensormap(&tmB);
    }
    if (warp == 2) {
        tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    constexpr int BKE = F8 ? 2 * BK : BK;            // elements of K per 128-byte row of a stage
    constexpr int NB = F8 ? 128 : 64;                // elements of N per 128-byte row ([K, N] weights: an MN-major operand)
    constexpr int KSTEP = F8 ? 32 : 16;              // elements of K per MMA
    const int num_kb = (int)((p.K + BKE - 1) / BKE);
    const int splits = p.splits > 1 ? p.splits : 1;
    const int kbps = p.splits > 1 ? p.kb_per_split : num_kb;     // k-blocks per unit
    const int num_units = p.tiles_m * p.tiles_n * splits;
    const uint32_t smem_base = smem_u32(smem);

    if (warp == 0) {
        {   // warp-uniform like the issuer below: all lanes loop and wait, one elected lane issues the copies
            const bool leader = elect_one_u32() != 0;
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
                int tm, tn;
                tile_coords(u / splits, p, tm, tn);
                const int m0 = tm * BM, n0 = tn * BN;
                const int kb0 = (u % splits) * kbps, kb1 = min(num_kb, kb0 + kbps);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!__all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, p.kerr, KERR_GEMM_PRODUCER_WAIT, kb))) { ok = false; break; }
                    const uint32_t full = bar_full + 8 * stage;
                    const uint32_t sa = smem_base + stage * STAGE_BYTES, sb = sa + A_BYTES;
                    if (leader) {
                        mbar_arrive_expect_tx(full, STAGE_BYTES);
                        tma_load_2d(sa, &tmA, full, kb * BKE, m0);
                        if constexpr (TRANS_B) {
                            tma_load_2d(sb, &tmB, full, kb * BKE, n0);
                        } else {
                            // [K, N] weights: boxes of one 128-byte row along N (64 two-byte or 128 one-byte elements) x all k of the stage
#pragma unroll
                            for (int j = 0; j < BN / NB; ++j) tma_load_2d(sb + j * (BKE * 128), &tmB, full, n0 + j * NB, kb * BKE);
                        }
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // All 32 lanes run the loop and the waits, so that descriptors stay in uniform registers (what
        // tcgen05.mma reads); one elected lane is predicated on the instructions themselves.
        {
            const uint32_t leader = elect_one_u32();
            const uint32_t tm = __reduce_max_sync(0xffffffffu, tmem_base);
            const uint64_t adesc0 = smem_desc_sw128(smem_base, 16, 1024);
            const uint64_t bdesc0 = TRANS_B ? smem_desc_sw128(smem_base + A_BYTES, 16, 1024) : smem_desc_sw128(smem_base + A_BYTES, BKE * 128, 1024);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
                if (!__all_sync(0xffffffffu, mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag, p.kerr, KERR_GEMM_MMA_WAIT, 1000000))) break;
                tc_fence_after();
                const uint32_t d_tmem = tm + acc * BN;
                const int kb0 = (u % splits) * kbps, kb1 = min(num_kb, kb0 + kbps);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!__all_sync(0xffffffffu, mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.kerr, KERR_GEMM_MMA_WAIT, kb))) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t soff = (uint32_t)(stage * STAGE_BYTES) >> 4;
#pragma unroll
                    for (int ks = 0; ks < BK / 16; ++ks) {   // four 32-byte steps along K per stage, for 16- and 8-bit inputs alike
                        const uint64_t adesc = adesc0 + (soff + ((ks * 32) >> 4));
                        const uint64_t bdesc = bdesc0 + (soff + ((TRANS_B ? ks * 32 : ks * (KSTEP * 128)) >> 4));
                        if constexpr (F8) mma_f8_ss_lead(d_tmem, adesc, bdesc, p.idesc, ((kb - kb0) | ks) != 0 ? 1u : 0u, leader);
                        else mma_f16_ss_lead(d_tmem, adesc, bdesc, p.idesc, ((kb - kb0) | ks) != 0 ? 1u : 0u, leader);
                    }
                    mma_commit_lead(bar_empty + 8 * stage, leader);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                mma_commit_lead(bar_tfull + 8 * acc, leader);
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1;
            }
        }
    } else if (warp >= 4) {
        const int q = warp - 4;  // TMEM lane quarter == warp id % 4
        int acc = 0;
        uint32_t acc_phase = 0;
        TcParams pe = p;     // per-unit view of the output: a split unit writes its partial tile to its own block of rows
        for (int u = blockIdx.x; u < num_units; u += gridDim.x) {
            int tm, tn;
            tile_coords(u / splits, p, tm, tn);
            const bool ready = mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag, p.kerr, KERR_GEMM_EPILOGUE_WAIT, u);
            if (!__all_sync(0xffffffffu, ready)) break;
            tc_fence_after();
            if (splits > 1) pe.C = (char*)p.C + (int64_t)(u % splits) * p.M * p.ldc * (OUT == MK_F32 ? 4 : 2);
            epilogue_tile<OUT>(pe, (int64_t)tm * BM, (int64_t)tn * BN, tmem_base + (uint32_t(q * 32) << 16) + acc * BN, stage_out, q, lane,
                               bar_tempty + 8 * acc, false);
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1;
        }
    }

    // Teardown.  After an aborted wait give copies that are still in flight time to land before
    // the shared memory is released.
    if (*abort_flag) __nanosleep(2000000);
    tc_fence_before();
    __syncthreads();
    if (warp == 2) tmem_dealloc(tmem_base, TMEM_COLS);
}

// Tensor maps of the output as every destination sees it: [0] the local C, [1 ..] the peers' C (16-bit elements,
// box of 64 columns x 32 rows, 128-byte swizzle).
struct CStoreMaps {
    CUtensorMap m[1 + MK_MAX_PEERS];
};

// Epilogue of one 128 x 256 accumulator for N-sharded runs: the warp turns its 32 rows into 16-bit output, 64
// columns at a time, in the shared-memory layout of a 128-byte-swizzled tile store, and one lane hands each
// 32 x 64 block to the copy engine of the SM once per destination (local C and every peer's C over NVLink).
// The stores are asynchronous: the warp goes on draining while they travel, and only waits before it rewrites a
// block that may still be read (each of the four blocks of a tile is one bulk group, the four newest may be
// pending).  `stage` is this warp's 16 KiB (4 blocks of 32 rows x 128 bytes).
template <int OUT>
__device__ __forceinline__ void epilogue_tile_tma(const TcParams& p, const CStoreMaps& maps, int64_t tile_row0, int64_t col0, uint32_t taddr,
                                                  uint8_t* stage, int q, int lane, uint32_t tempty_bar, bool tempty_remote) {
    static_assert(OUT != MK_F32, "tile stores carry 16-bit outputs");
    const int64_t row0 = tile_row0 + q * 32;
    const int64_t row = row0 + lane;
    const int nslabs = (int)min((int64_t)(BN / 64), (p.N - col0 + 63) / 64);      // 64-column blocks of this tile inside N (>= 1)
#pragma unroll 1
    for (int sl = 0; sl < nslabs; ++sl) {
        uint8_t* blk = stage + sl * 4096;
        if (lane == 0) bulk_wait_group_read<3>();       // the store that last read this block (previous tile) is done with it
        __syncwarp();
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(taddr + sl * 64 + c * 32, r);
            tmem_wait_ld();
            uint32_t w[16];
            convert_chunk<OUT>(p, row, col0 + sl * 64 + c * 32, r, w);
#pragma unroll
            for (int i = 0; i < 4; ++i)
                *reinterpret_cast<uint4*>(blk + lane * 128 + (((c * 4 + i) ^ (lane & 7)) << 4)) = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
        }
        if (sl == nslabs - 1) {     // last read of this accumulator: hand it back before the stores are issued
            tc_fence_before();
            arrive_tempty(tempty_bar, tempty_remote);
        }
        fence_proxy_async_smem();   // this lane's shared-memory writes become visible to the copy engine
        __syncwarp();
        if (lane == 0) {
            if (row0 < p.M) {
                const uint32_t src = smem_u32(blk);
                const int x = (int)(col0 + sl * 64), y = (int)row0;
                for (int d = 0; d <= p.n_peers; ++d) tma_store_2d(&maps.m[d], src, x, y);
            }
            bulk_commit_group();
        }
    }
    // fewer than four blocks in this tile (ragged N): keep the group count per tile at four so that the wait above stays exact
    if (lane == 0)
        for (int sl = nslabs; sl < BN / 64; ++sl) bulk_commit_group();
}

// ---------------------------------------------------------------------------------------------------
// CTA-pair variant: two CTAs of a cluster (one per SM) share each MMA (cta_group::2).  The pair owns a
// 256 x 256 tile; CTA r loads rows r*128.. of A and columns r*128.. of B of every k-block (its own
// halves, plain TMA loads -- nothing is broadcast), the even CTA's issuing thread drives both tensor
// cores with M = 256 instructions, and each CTA drains the accumulator rows it holds.  Per MMA an SM
// reads 8 KiB of shared memory instead of 12, and its stage shrinks to 32 KiB, so the ring is 6 deep.
// Barriers: `full` lives in the leader and receives the byte counts of both CTAs' loads; `empty` and
// `tfull` exist in both CTAs and are signalled by two commits of the issuing thread (one per CTA);
// `tempty` lives in the leader and collects the arrivals of both epilogues.
// ---------------------------------------------------------------------------------------------------
constexpr int P_STAGES = 6;
constexpr int P_A_BYTES = BM * BK * 2;             // 16 KiB: this CTA's 128 rows of A
constexpr int P_B_BYTES = BK * (BN / 2) * 2;       // 16 KiB: this CTA's 128 columns of B
constexpr int P_STAGE_BYTES = P_A_BYTES + P_B_BYTES;

// Shared memory of the pair kernel: NSTG ring stages, the output staging, barriers.  With tile-store delivery
// (TMA_OUT) the staging holds a whole 128 x 256 tile of 16-bit output (64 KiB) and the ring is one stage shorter.
template <bool TMA_OUT>
struct PairCfg {
    static constexpr int NSTG = TMA_OUT ? P_STAGES - 1 : P_STAGES;
    static constexpr int OUT_BYTES = TMA_OUT ? 4 * 16384 : OUT_STAGE_BYTES;
    static constexpr int NUM_BARS = 2 * NSTG + 4;
    static constexpr int SMEM_BYTES = NSTG * P_STAGE_BYTES + OUT_BYTES + 1024 + 256;
};

template <bool TRANS_B, int OUT, bool F8 = false, bool TMA_OUT = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmB2,
                    const TcParams p, const __grid_constant__ CStoreMaps cmaps) {
    constexpr int P_STAGES = PairCfg<TMA_OUT>::NSTG, P_NUM_BARS = PairCfg<TMA_OUT>::NUM_BARS;     // shadow the file-level defaults
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* stage_out = smem + P_STAGES * P_STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(stage_out + PairCfg<TMA_OUT>::OUT_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + P_NUM_BARS);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const uint32_t bar_full = smem_u32(bars);                      // [P_STAGES] used in the leader only
    const uint32_t bar_empty = smem_u32(bars + P_STAGES);          // [P_STAGES] in both CTAs
    const uint32_t bar_tfull = smem_u32(bars + 2 * P_STAGES);      // [2] in both CTAs
    const uint32_t bar_tempty = smem_u32(bars + 2 * P_STAGES + 2); // [2] used in the leader only

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();       // 0 = leader (issues the MMAs), 1 = peer
    const uint32_t peer = rank ^ 1u;

    if (threadIdx.x == 0) {
        for (int i = 0; i < P_STAGES; ++i) {
            mbar_init(bar_full + 8 * i, 1);
            mbar_init(bar_empty + 8 * i, 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar_tfull + 8 * i, 1);
            mbar_init(bar_tempty + 8 * i, 256);    // 128 epilogue threads of each CTA
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&tmA);
        prefetch_tensormap(&tmB);
        prefetch_tensormap(&tmB2);
        if constexpr (TMA_OUT)
            for (int d = 0; d <= p.n_peers; ++d) prefetch_tensormap(&cmaps.m[d]);
    }
    if (warp == 2) {   // the same warp of both CTAs allocates the pair's tensor memory
        tmem_alloc_pair(smem_u32(tmem_slot), TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();        // both CTAs' barriers exist before anything signals across the pair
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    constexpr int BKE = F8 ? 2 * BK : BK;            // elements of K per 128-byte row of a stage
    constexpr int NB = F8 ? 128 : 64;                // elements of N per 128-byte row ([K, N] weights: an MN-major operand)
    constexpr int KSTEP = F8 ? 32 : 16;              // elements of K per MMA
    const int num_kb = (int)((p.K + BKE - 1) / BKE);
    const int num_tiles = p.tiles_m2 * p.tiles_n;   // 256 x 256 tiles, one per cluster and step
    const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
    const uint32_t smem_base = smem_u32(smem);

    if (warp == 0) {
        {   // warp-uniform like the issuer below: all lanes loop and wait, one elected lane issues the copies
            const bool leader = elect_one_u32() != 0;
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
                int tm, tn;
                tile_coords2(t, p, tm, tn);
                // gated pair of products: both CTAs take the same 128 columns, the leader from B, the peer from B2
                const int m0 = tm * (2 * BM) + (int)rank * BM, n0 = p.dual ? tn * (BN / 2) : tn * BN + (int)rank * (BN / 2);
                const CUtensorMap* tmBr = (p.dual && rank == 1) ? &tmB2 : &tmB;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!__all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, p.kerr, KERR_GEMM_PRODUCER_WAIT, kb))) { ok = false; break; }
                    const uint32_t full = bar_full + 8 * stage;
                    const uint32_t sa = smem_base + stage * P_STAGE_BYTES, sb = sa + P_A_BYTES;
                    if (leader) {
                        if (rank == 0) mbar_arrive_expect_tx(full, 2 * P_STAGE_BYTES);   // both CTAs' bytes land on the leader's barrier
                        tma_load_2d_pair(sa, &tmA, full, kb * BKE, m0);
                        if constexpr (TRANS_B) {
                            tma_load_2d_pair(sb, tmBr, full, kb * BKE, n0);
                        } else {
#pragma unroll
                            for (int j = 0; j < BN / 2 / NB; ++j) tma_load_2d_pair(sb + j * (BKE * 128), tmBr, full, n0 + j * NB, kb * BKE);
                        }
                    }
                    if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        if (rank == 0) {   // warp-uniform: all lanes loop and wait, one elected lane is predicated on the instructions
            const uint32_t leader = elect_one_u32();
            const uint32_t tm = __reduce_max_sync(0xffffffffu, tmem_base);
            const uint32_t peer_empty = map_to_cta(bar_empty, peer), peer_tfull = map_to_cta(bar_tfull, peer);
            const uint64_t adesc0 = smem_desc_sw128(smem_base, 16, 1024);
            const uint64_t bdesc0 = TRANS_B ? smem_desc_sw128(smem_base + P_A_BYTES, 16, 1024) : smem_desc_sw128(smem_base + P_A_BYTES, BKE * 128, 1024);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
                if (!__all_sync(0xffffffffu, mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag, p.kerr, KERR_GEMM_MMA_WAIT, 1000000))) break;
                tc_fence_after();
                const uint32_t d_tmem = tm + acc * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!__all_sync(0xffffffffu, mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.kerr, KERR_GEMM_MMA_WAIT, kb))) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t soff = (uint32_t)(stage * P_STAGE_BYTES) >> 4;
#pragma unroll
                    for (int ks = 0; ks < BK / 16; ++ks) {   // four 32-byte steps along K per stage, for 16- and 8-bit inputs alike
                        const uint64_t adesc = adesc0 + (soff + ((ks * 32) >> 4));
                        const uint64_t bdesc = bdesc0 + (soff + ((TRANS_B ? ks * 32 : ks * (KSTEP * 128)) >> 4));
                        if constexpr (F8) mma_f8_ss_pair_lead(d_tmem, adesc, bdesc, p.idesc2, (kb | ks) != 0 ? 1u : 0u, leader);
                        else mma_f16_ss_pair_lead(d_tmem, adesc, bdesc, p.idesc2, (kb | ks) != 0 ? 1u : 0u, leader);
                    }
                    mma_commit_pair_lead(bar_empty + 8 * stage, leader);      // stage free in the leader ...
                    mma_commit_pair_lead(peer_empty + 8 * stage, leader);     // ... and in the peer
                    if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                mma_commit_pair_lead(bar_tfull + 8 * acc, leader);
                mma_commit_pair_lead(peer_tfull + 8 * acc, leader);
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1;
            }
        }
    } else if (warp >= 4) {
        const int q = warp - 4;  // TMEM lane quarter == warp id % 4
        const uint32_t leader_tempty = map_to_cta(bar_tempty, 0);
        int acc = 0;
        uint32_t acc_phase = 0;
        for (int t = cluster_id; t < num_tiles; t += num_clusters) {
            int tm, tn;
            tile_coords2(t, p, tm, tn);
            const bool ready = mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag, p.kerr, KERR_GEMM_EPILOGUE_WAIT, t);
            if (!__all_sync(0xffffffffu, ready)) break;
            tc_fence_after();
            if constexpr (TMA_OUT)
                epilogue_tile_tma<OUT>(p, cmaps, (int64_t)tm * (2 * BM) + (int64_t)rank * BM, (int64_t)tn * BN,
                                       tmem_base + (uint32_t(q * 32) << 16) + acc * BN, stage_out + q * 16384, q, lane, leader_tempty + 8 * acc, true);
            else
                epilogue_tile<OUT>(p, (int64_t)tm * (2 * BM) + (int64_t)rank * BM, (int64_t)tn * (p.dual ? BN / 2 : BN),
                                   tmem_base + (uint32_t(q * 32) << 16) + acc * BN, stage_out, q, lane, leader_tempty + 8 * acc, true);
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1;
        }
        if constexpr (TMA_OUT) {
            if (lane == 0) bulk_wait_group<0>();     // every tile store of this warp has completed before the CTA may leave
            __syncwarp();
        }
    }

    // Teardown: neither CTA may leave while the other can still signal its barriers or read its
    // shared memory through an MMA.
    if (*abort_flag) __nanosleep(2000000);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 2) tmem_dealloc_pair(tmem_base, TMEM_COLS);
}

// Sums the f32 partial tiles of a K-split GEMM and applies what the epilogue would have: alpha, beta * D
// (a full matrix or one row), the cast.  One thread per four output columns.
struct MergeParams {
    const float* ws;      // [splits][M][ldw]
    void* C;
    const void* D;
    int64_t M, N, ldw, ldc, ldd;
    int splits;
    float alpha, beta;
};

template <int OUT>
__global__ void __launch_bounds__(256) gemm_split_merge_kernel(const MergeParams p) {
    grid_dependency_wait();       // the partial tiles of the preceding grid are complete and visible after this
    const int64_t quads = (p.N + 3) / 4;
    const int64_t total = p.M * quads;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = idx / quads, col = (idx - row * quads) * 4;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        const bool full = col + 4 <= p.N && (p.ldw % 4 == 0);
        for (int s = 0; s < p.splits; ++s) {
            const float* w = p.ws + ((int64_t)s * p.M + row) * p.ldw + col;
            if (full) {
                const float4 x = *reinterpret_cast<const float4*>(w);
                v[0] += x.x; v[1] += x.y; v[2] += x.z; v[3] += x.w;
            } else {
                for (int i = 0; i < 4; ++i)
                    if (col + i < p.N) v[i] += w[i];
            }
        }
        for (int i = 0; i < 4; ++i) {
            if (col + i >= p.N) break;
            float x = v[i] * p.alpha;
            const int64_t doff = row * p.ldd + col + i, coff = row * p.ldc + col + i;
            if constexpr (OUT == MK_F32) {
                if (p.D) x = fmaf(p.beta, ((const float*)p.D)[doff], x);
                ((float*)p.C)[coff] = x;
            } else if constexpr (OUT == MK_BF16) {
                if (p.D) x = fmaf(p.beta, __bfloat162float(((const __nv_bfloat16*)p.D)[doff]), x);
                ((__nv_bfloat16*)p.C)[coff] = __float2bfloat16_rn(x);
            } else {
                if (p.D) x = fmaf(p.beta, __half2float(((const __half*)p.D)[doff]), x);
                ((__half*)p.C)[coff] = __float2half_rn(x);
            }
        }
    }
}

typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

mk_status encode_2d(CUtensorMap* map, int dtype, const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                    uint32_t box_inner, uint32_t box_outer) {
    static PFN_encodeTiled encode = (PFN_encodeTiled)driver_entry("cuTensorMapEncodeTiled");
    if (!encode) return fail(MK_ERR_CUDA, "cuTensorMapEncodeTiled is unavailable (driver too old?)");
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {row_stride_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    const CUtensorMapDataType ty = dtype_is_fp8(dtype) ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                   : dtype == MK_BF16  ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                       : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUresult r = encode(map, ty, 2,
                        const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(MK_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
    return MK_OK;
}

// The coalesced epilogue writes 16-byte pieces: every destination row must start 16-byte aligned.
int staged_ok(const TcParams& p, size_t es) {
    if (getenv("MOROK_B200_GEMM_DIRECT_STORES")) return 0;
    if ((p.ldc * es) % 16) return 0;
    uintptr_t bits = reinterpret_cast<uintptr_t>(p.C) | reinterpret_cast<uintptr_t>(p.D);
    for (int q = 0; q < p.n_peers; ++q) bits |= reinterpret_cast<uintptr_t>(p.peer_C[q]);
    return (bits & 15) == 0;
}

// Row-tiles per raster group (tuning knob; MOROK_B200_GEMM_GROUP_M overrides the default).
int group_m_setting() {
    static int v = [] {
        const char* e = getenv("MOROK_B200_GEMM_GROUP_M");
        int x = e ? atoi(e) : 0;
        return x > 0 ? x : 32;
    }();
    return v;
}

template <bool TRANS_B, int OUT, bool F8 = false>
mk_status launch_tc(mk_device* dev, cudaStream_t st, const CUtensorMap& ta, const CUtensorMap& tb, const TcParams& p) {
    auto kern = gemm_tc_kernel<TRANS_B, OUT, F8>;
    MK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    const int tiles = p.tiles_m * p.tiles_n * (p.splits > 1 ? p.splits : 1);
    const int grid = tiles < dev->prop.multiProcessorCount ? tiles : dev->prop.multiProcessorCount;
    kern<<<grid, NUM_THREADS, SMEM_BYTES, st>>>(ta, tb, p);
    MK_CUDA(cudaGetLastError());
    note_launch(dev, st, F8 ? "gemm_tc_f8" : (p.splits > 1 ? "gemm_tc_ksplit" : "gemm_tc"));
    return MK_OK;
}

template <bool TRANS_B, int OUT, bool F8 = false>
mk_status launch_tc_pair(mk_device* dev, cudaStream_t st, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tb2, const TcParams& p) {
    auto kern = gemm_tc_pair_kernel<TRANS_B, OUT, F8, false>;
    MK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PairCfg<false>::SMEM_BYTES));
    const int tiles = p.tiles_m2 * p.tiles_n;
    const int clusters = tiles < dev->prop.multiProcessorCount / 2 ? tiles : dev->prop.multiProcessorCount / 2;
    static const CStoreMaps no_maps{};      // read by the tile-store variant only
    kern<<<2 * clusters, NUM_THREADS, PairCfg<false>::SMEM_BYTES, st>>>(ta, tb, tb2, p, no_maps);
    MK_CUDA(cudaGetLastError());
    note_launch(dev, st, p.dual ? "gemm_tc_pair_gated" : (F8 ? "gemm_tc_pair_f8" : "gemm_tc_pair"));
    return MK_OK;
}

// The same kernel with the epilogue that delivers finished tiles by tile stores (N-sharded runs, 16-bit output).
template <bool TRANS_B, int OUT>
mk_status launch_tc_pair_deliver(mk_device* dev, cudaStream_t st, const CUtensorMap& ta, const CUtensorMap& tb, const TcParams& p, const CStoreMaps& maps) {
    auto kern = gemm_tc_pair_kernel<TRANS_B, OUT, false, true>;
    constexpr int smem = PairCfg<true>::SMEM_BYTES;
    MK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    const int tiles = p.tiles_m2 * p.tiles_n;
    const int clusters = tiles < dev->prop.multiProcessorCount / 2 ? tiles : dev->prop.multiProcessorCount / 2;
    kern<<<2 * clusters, NUM_THREADS, smem, st>>>(ta, tb, tb, p, maps);
    MK_CUDA(cudaGetLastError());
    note_launch(dev, st, "gemm_tc_pair_deliver");
    return MK_OK;
}

// Peers receive their copies as tile stores issued from shared memory (MOROK_B200_PEER_TMA=0: as 16-byte stores of
// the epilogue warps, the older path).
bool peer_tma_enabled() {
    static int v = [] {
        const char* e = getenv("MOROK_B200_PEER_TMA");
        return e ? atoi(e) : 1;
    }();
    return v != 0;
}


// K ranges for few-row problems (MOROK_B200_GEMM_SPLITK=0/1 forces).
bool split_k_enabled() {
    static int v = [] {
        const char* e = getenv("MOROK_B200_GEMM_SPLITK");
        return e ? atoi(e) : 1;
    }();
    return v != 0;
}

// CTA pairs pay off once there are row tiles to pair and enough 256 x 256 tiles to give every SM pair one;
// below that the same number of SMs is busy either way and single CTAs measured 2-7 % faster
// (512 x 4096 x 4096, 1024 x 4096 x 4096).  MOROK_B200_GEMM_PAIR=0/1 forces.
bool use_pair(const mk_gemm_desc& d, int sms) {
    static int forced = [] {
        const char* e = getenv("MOROK_B200_GEMM_PAIR");
        return e ? atoi(e) : -1;
    }();
    if (forced >= 0) return forced != 0;
    const int64_t pair_tiles = ((d.M + 2 * BM - 1) / (2 * BM)) * ((d.N + BN - 1) / BN);
    return d.M > BM && pair_tiles >= sms / 2;
}

}  // namespace

// The 2-D tensor map builder for the other kernels of the library (128-byte swizzle, zero fill outside).
mk_status tma_encode_2d(void* map, int dtype, const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                        uint32_t box_inner, uint32_t box_outer) {
    return encode_2d(reinterpret_cast<CUtensorMap*>(map), dtype, base, inner, outer, row_stride_bytes, box_inner, box_outer);
}

// Runs the tensor-core kernel when the problem qualifies; otherwise leaves *handled = false and
// the caller uses the FMA kernel.
mk_status gemm_sm100(mk_device* dev, cudaStream_t st, const mk_gemm_desc& d, bool* handled) {
    *handled = false;
    if (dev->prop.major != 10) return MK_OK;
    const bool f8 = dtype_is_fp8(d.dtype_in);
    if (d.dtype_in != MK_BF16 && d.dtype_in != MK_F16 && !f8) return MK_OK;
    // 8-bit [K, N] weights are an MN-major operand like their 16-bit form: rows of 128 elements along N
    if (d.M <= 0 || d.N <= 0 || d.K <= 0) return MK_OK;
    // TMA needs 16-byte aligned bases and row pitches.
    const int64_t es_in = f8 ? 1 : 2, row_align = 16 / es_in;
    if ((reinterpret_cast<uintptr_t>(d.A) & 15) || (reinterpret_cast<uintptr_t>(d.B) & 15)) return MK_OK;
    if ((d.lda % row_align) || (d.ldb % row_align) || (d.stride_a % row_align) || (d.stride_b % row_align)) return MK_OK;
    if (d.M > 0x7fffff00ll || d.N > 0x7fffff00ll || d.K > 0x7fffff00ll) return MK_OK;
    const int64_t tiles_m = (d.M + BM - 1) / BM, tiles_n = (d.N + BN - 1) / BN;
    if (tiles_m * tiles_n > 0x7fffffffll) return MK_OK;
    const uint32_t bke = f8 ? 2 * BK : BK;   // elements in one 128-byte row of a stage
    const bool dual = d.epilogue == MK_EPI_SWIGLU;
    if (dual) {   // 16-bit output through the staged epilogue, B2 aligned like B
        if (d.dtype_out == MK_F32 || (reinterpret_cast<uintptr_t>(d.B2) & 15)) return MK_OK;
        if ((reinterpret_cast<uintptr_t>(d.D) & 15) || (reinterpret_cast<uintptr_t>(d.D2) & 15)) return MK_OK;    // bias rows are read 16 bytes at a time
        if ((d.ldc * 2) % 16 || (reinterpret_cast<uintptr_t>(d.C) & 15) || (d.stride_c * 2) % 16 || getenv("MOROK_B200_GEMM_DIRECT_STORES")) return MK_OK;
    }

    // a schedule found by mk_gemm_autotune for this problem replaces the built-in rules below where it applies
    mk_gemm_tuning tune{-1, 0, 0, 0, 0.0f, 0.0f};
    gemm_tuning_for(dev, d, &tune);

    const size_t es_out = dtype_size(d.dtype_out);
    for (int b = 0; b < d.batch; ++b) {
        const char* A = (const char*)d.A + (size_t)b * d.stride_a * es_in;
        const char* B = (const char*)d.B + (size_t)b * d.stride_b * es_in;
        alignas(64) CUtensorMap ta, tb;
        mk_status s1 = encode_2d(&ta, d.dtype_in, A, (uint64_t)d.K, (uint64_t)d.M, (uint64_t)d.lda * es_in, bke, BM);
        if (s1 != MK_OK) return s1;
        // the gated pair of products exists in the CTA-pair kernel only
        const bool pair = dual || ((tune.pair >= 0 && d.M > BM) ? tune.pair != 0 : use_pair(d, dev->prop.multiProcessorCount));
        // [N,K] weights: one box holds all the rows a CTA needs -- 256 for a single CTA, 128 in a pair
        if (d.trans_b) s1 = encode_2d(&tb, d.dtype_in, B, (uint64_t)d.K, (uint64_t)d.N, (uint64_t)d.ldb * es_in, bke, pair ? BN / 2 : BN);
        else s1 = encode_2d(&tb, d.dtype_in, B, (uint64_t)d.N, (uint64_t)d.K, (uint64_t)d.ldb * es_in, f8 ? 128 : 64, bke);
        if (s1 != MK_OK) return s1;
        alignas(64) CUtensorMap tb2 = tb;
        if (dual) {
            const char* B2 = (const char*)d.B2 + (size_t)b * d.stride_b * es_in;
            if (d.trans_b) s1 = encode_2d(&tb2, d.dtype_in, B2, (uint64_t)d.K, (uint64_t)d.N, (uint64_t)d.ldb * es_in, bke, BN / 2);
            else s1 = encode_2d(&tb2, d.dtype_in, B2, (uint64_t)d.N, (uint64_t)d.K, (uint64_t)d.ldb * es_in, f8 ? 128 : 64, bke);
            if (s1 != MK_OK) return s1;
        }

        TcParams p{};
        p.M = d.M; p.N = d.N; p.K = d.K;
        p.C = (char*)d.C + (size_t)b * d.stride_c * es_out;
        p.D = d.epilogue == MK_EPI_ADD ? (const char*)d.D + (size_t)b * d.stride_c * es_out
              : (d.epilogue == MK_EPI_ADD_ROW || dual) ? (const char*)d.D : nullptr;      // gated: the first product's bias row or null
        p.D2 = dual ? d.D2 : nullptr;
        p.gate_sigmoid = (dual && (d.flags & MK_GEMM_GATE_SIGMOID)) ? 1 : 0;
        p.ldc = d.ldc;
        p.ldd = d.epilogue == MK_EPI_ADD_ROW ? 0 : d.ldc;
        p.scaled = (d.flags & MK_GEMM_SCALED) ? 1 : 0;
        p.alpha = p.scaled ? d.alpha : 1.0f;
        p.beta = p.scaled ? d.beta : 1.0f;
        const uint32_t fmt = (d.dtype_in == MK_BF16 || d.dtype_in == MK_F8E5M2) ? 1u : 0u;   // bf16 / e5m2 = 1, f16 / e4m3 = 0
        p.idesc = idesc_f16(fmt, 0u, d.trans_b ? 0u : 1u, BM, BN);
        p.idesc2 = idesc_f16(fmt, 0u, d.trans_b ? 0u : 1u, 2 * BM, BN);
        p.tiles_m = (int)tiles_m;
        p.tiles_m2 = (int)((d.M + 2 * BM - 1) / (2 * BM));
        p.tiles_n = dual ? (int)((d.N + BN / 2 - 1) / (BN / 2)) : (int)tiles_n;
        p.dual = dual ? 1 : 0;
        p.group_m = tune.group_m > 0 ? tune.group_m : group_m_setting();
        p.n_peers = d.n_peers;
        for (int q = 0; q < d.n_peers; ++q) p.peer_C[q] = (char*)d.peer_C[q] + (size_t)b * d.stride_c * es_out;
        p.staged = staged_ok(p, es_out);
        p.kerr = stream_kerr(dev, st);

        // Few rows (decoding): one row of 128 x 256 tiles leaves most SMs idle while the work is streaming the
        // weights.  K is then cut into ranges, every (tile, range) unit writes an f32 partial tile to a
        // scratch block of the launching stream, and a small kernel sums the ranges and applies the epilogue.
        const int num_kb = (int)((d.K + bke - 1) / bke);
        const int64_t tiles = tiles_m * tiles_n;
        const int sms = dev->prop.multiProcessorCount;
        int splits = 1, kb_per_split = num_kb;
        const bool worth_it = (int64_t)d.K * d.N * es_in >= (4ll << 20);    // below 4 MiB of weights a second launch costs more than it saves
        const bool can_split = !pair && !dual && d.n_peers == 0;
        int want = 1;
        if (tune.splits > 0) {      // a tuned count (1 = never split), kept to at most four units per SM
            if (can_split && tiles <= sms) want = (int)std::min<int64_t>(std::min<int64_t>(tune.splits, num_kb), std::max<int64_t>(1, 4 * sms / tiles));
        } else if (split_k_enabled() && worth_it && can_split && tiles * 4 <= 3ll * sms && num_kb >= 8) {
            want = (int)std::min<int64_t>(sms / tiles, num_kb / 4);      // at most one unit per SM, at least 4 k-blocks each
        }
        if (want > 1) {
            kb_per_split = (num_kb + want - 1) / want;
            splits = (num_kb + kb_per_split - 1) / kb_per_split;
        }
        if (splits > 1) {
            float* ws = nullptr;
            mk_status sw = stream_scratch(dev, st, (size_t)splits * d.M * d.N * sizeof(float), (void**)&ws);
            if (sw != MK_OK) return sw;
            TcParams ps = p;
            ps.C = ws;
            ps.ldc = d.N;
            ps.D = nullptr;
            ps.scaled = 0;
            ps.splits = splits;
            ps.kb_per_split = kb_per_split;
            ps.staged = staged_ok(ps, 4);
            mk_status s3;
            if (f8 && !d.trans_b) s3 = launch_tc<false, MK_F32, true>(dev, st, ta, tb, ps);
            else if (f8) s3 = launch_tc<true, MK_F32, true>(dev, st, ta, tb, ps);
            else if (d.trans_b) s3 = launch_tc<true, MK_F32>(dev, st, ta, tb, ps);
            else s3 = launch_tc<false, MK_F32>(dev, st, ta, tb, ps);
            if (s3 == MK_OK) {
                MergeParams mp{ws, p.C, p.D, d.M, d.N, d.N, p.ldc, p.ldd, splits, p.alpha, p.beta};
                const int64_t work = d.M * ((d.N + 3) / 4);
                const int grid = (int)std::min<int64_t>((work + 255) / 256, (int64_t)sms * 8);
                cudaError_t le;
                if (d.dtype_out == MK_F32) le = launch_dependent(gemm_split_merge_kernel<MK_F32>, dim3(grid), dim3(256), st, mp);
                else if (d.dtype_out == MK_BF16) le = launch_dependent(gemm_split_merge_kernel<MK_BF16>, dim3(grid), dim3(256), st, mp);
                else le = launch_dependent(gemm_split_merge_kernel<MK_F16>, dim3(grid), dim3(256), st, mp);
                if (le != cudaSuccess || cudaGetLastError() != cudaSuccess) s3 = fail(MK_ERR_CUDA, "mk_gemm: the split-K merge kernel failed to launch");
                note_launch(dev, st, "gemm_split_merge");
            }
            if (s3 != MK_OK) return s3;
            continue;
        }

        // N-sharded delivery: 16-bit tiles leave through tile stores, one per destination
        if (pair && !dual && !f8 && d.n_peers > 0 && d.dtype_out != MK_F32 && p.staged && peer_tma_enabled()) {
            alignas(64) CStoreMaps maps;
            mk_status sm = MK_OK;
            for (int q = 0; q <= d.n_peers && sm == MK_OK; ++q)
                sm = encode_2d(&maps.m[q], d.dtype_out, q == 0 ? p.C : p.peer_C[q - 1], (uint64_t)d.N, (uint64_t)d.M, (uint64_t)d.ldc * 2, 64, 32);
            if (sm != MK_OK) return sm;
            mk_status sd;
            if (d.trans_b) sd = d.dtype_out == MK_BF16 ? launch_tc_pair_deliver<true, MK_BF16>(dev, st, ta, tb, p, maps) : launch_tc_pair_deliver<true, MK_F16>(dev, st, ta, tb, p, maps);
            else sd = d.dtype_out == MK_BF16 ? launch_tc_pair_deliver<false, MK_BF16>(dev, st, ta, tb, p, maps) : launch_tc_pair_deliver<false, MK_F16>(dev, st, ta, tb, p, maps);
            if (sd != MK_OK) return sd;
            continue;
        }

        mk_status s2;
#define MK_TC(TB, OUT) s2 = pair ? launch_tc_pair<TB, OUT>(dev, st, ta, tb, tb2, p) : launch_tc<TB, OUT>(dev, st, ta, tb, p)
#define MK_TC8(OUT) s2 = pair ? launch_tc_pair<true, OUT, true>(dev, st, ta, tb, tb2, p) : launch_tc<true, OUT, true>(dev, st, ta, tb, p)
#define MK_TC8N(OUT) s2 = pair ? launch_tc_pair<false, OUT, true>(dev, st, ta, tb, tb2, p) : launch_tc<false, OUT, true>(dev, st, ta, tb, p)
        if (f8 && !d.trans_b) {
            if (d.dtype_out == MK_F32) MK_TC8N(MK_F32); else if (d.dtype_out == MK_BF16) MK_TC8N(MK_BF16); else MK_TC8N(MK_F16);
        } else if (f8) {
            if (d.dtype_out == MK_F32) MK_TC8(MK_F32); else if (d.dtype_out == MK_BF16) MK_TC8(MK_BF16); else MK_TC8(MK_F16);
        } else if (d.trans_b) {
            if (d.dtype_out == MK_F32) MK_TC(true, MK_F32); else if (d.dtype_out == MK_BF16) MK_TC(true, MK_BF16); else MK_TC(true, MK_F16);
        } else {
            if (d.dtype_out == MK_F32) MK_TC(false, MK_F32); else if (d.dtype_out == MK_BF16) MK_TC(false, MK_BF16); else MK_TC(false, MK_F16);
        }
#undef MK_TC8N
#undef MK_TC8
#undef MK_TC
        if (s2 != MK_OK) return s2;
    }
    *handled = true;
    return MK_OK;
}

// =================================================================================================
// mk_gemm_static -- the tensor-core GEMM for callers that must not allocate device memory.
//
// Who needs it: code that runs inside somebody else's memory budget.  A plugin loaded into an
// inference server, or an operator called from a framework whose caching allocator has already
// reserved (nearly) all of HBM, cannot count on cudaMalloc succeeding; and even when it succeeds,
// cudaMalloc / cudaFree synchronise the whole device, which a latency-critical caller must not
// trigger from its hot path.  mk_gemm itself allocates nothing, but it needs an mk_device, and
// mk_device_open reserves the kernel error word with cudaMalloc.  This entry point needs no
// mk_device: the only global memory the kernel uses besides the caller's A, B, C (and D) -- the
// error words that record a pipeline wait that gave up -- lives in the array below, which is part
// of the library image.  Every GPU that loads the library holds these 4 KiB until the process exits.
//
// The array's name is a device symbol.  In host code it is only a handle for the runtime, not an
// address a kernel could use, so the address is looked up once per device with
// cudaGetSymbolAddress (with that device current) and that pointer is what the kernel receives.
// =================================================================================================
namespace {
constexpr int kStaticMaxBatch = MK_STATIC_GEMM_MAX_BATCH;             // one error word per batch item
static __device__ __align__(256) KernelError g_static_error_words[kStaticMaxBatch];   // 256 x 16 B = 4 KiB

constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
KernelError* g_static_ptr[kMaxDevices] = {};     // device address of g_static_error_words, per device
int g_static_sms[kMaxDevices] = {};
int g_static_cc_major[kMaxDevices] = {};

// First call on a device: resolve the symbol's device address and cache the device attributes.
mk_status static_setup(int ordinal) {
    std::lock_guard<std::mutex> lk(g_static_mu);
    if (g_static_ptr[ordinal]) return MK_OK;
    void* p = nullptr;
    MK_CUDA(cudaGetSymbolAddress(&p, g_static_error_words));
    if (!p) return fail(MK_ERR_CUDA, "mk_gemm_static: cudaGetSymbolAddress returned a null address");
    MK_CUDA(cudaDeviceGetAttribute(&g_static_sms[ordinal], cudaDevAttrMultiProcessorCount, ordinal));
    MK_CUDA(cudaDeviceGetAttribute(&g_static_cc_major[ordinal], cudaDevAttrComputeCapabilityMajor, ordinal));
    g_static_ptr[ordinal] = static_cast<KernelError*>(p);
    return MK_OK;
}

template <bool TRANS_B, int OUT>
mk_status launch_tc_static(int sms, bool pair, cudaStream_t st, const CUtensorMap& ta, const CUtensorMap& tb, const TcParams& p) {
    if (pair) {
        auto kern = gemm_tc_pair_kernel<TRANS_B, OUT, false, false>;
        MK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PairCfg<false>::SMEM_BYTES));
        const int tiles = p.tiles_m2 * p.tiles_n;
        const int clusters = tiles < sms / 2 ? tiles : sms / 2;
        static const CStoreMaps no_maps{};
        kern<<<2 * clusters, NUM_THREADS, PairCfg<false>::SMEM_BYTES, st>>>(ta, tb, tb, p, no_maps);
    } else {
        auto kern = gemm_tc_kernel<TRANS_B, OUT>;
        MK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        const int tiles = p.tiles_m * p.tiles_n;
        kern<<<tiles < sms ? tiles : sms, NUM_THREADS, SMEM_BYTES, st>>>(ta, tb, p);
    }
    MK_CUDA(cudaGetLastError());
    return MK_OK;
}

// Restores the calling thread's current device on every exit path.
struct DeviceGuard {
    int prev = -1;
    mk_status enter(int ordinal) {
        MK_CUDA(cudaGetDevice(&prev));
        if (prev != ordinal) MK_CUDA(cudaSetDevice(ordinal));
        else prev = -1;
        return MK_OK;
    }
    ~DeviceGuard() {
        if (prev >= 0) {
            cudaSetDevice(prev);
            cudaGetLastError();
        }
    }
};

// Waits for the stream and reports the first non-zero word among the first `batch`.
mk_status read_static_words(KernelError* words, int batch, cudaStream_t stream, uint32_t* kernel_error, const char* who) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    MK_CUDA(cudaStreamIsCapturing(stream, &cs));
    if (cs != cudaStreamCaptureStatusNone)
        return fail(MK_ERR_INVALID, "%s: the stream is capturing; the error words can only be read from a stream that runs", who);
    MK_CUDA(cudaStreamSynchronize(stream));
    KernelError host[kStaticMaxBatch];
    MK_CUDA(cudaMemcpy(host, words, sizeof(KernelError) * batch, cudaMemcpyDeviceToHost));
    *kernel_error = 0;
    for (int b = 0; b < batch; ++b)
        if (host[b].code) {
            *kernel_error = host[b].code;
            return fail(MK_ERR_KERNEL, "%s: batch item %d reported error word 0x%x (block %u, detail %u)", who, b, host[b].code,
                        host[b].block, host[b].detail);
        }
    return MK_OK;
}
}  // namespace
}  // namespace mk

extern "C" mk_status mk_gemm_static(int32_t device_ordinal, void* cuda_stream, const mk_gemm_desc* desc, uint32_t* kernel_error) {
    using namespace mk;
    MK_REQUIRE(desc, "mk_gemm_static: null descriptor");
    MK_REQUIRE(device_ordinal >= 0 && device_ordinal < kMaxDevices, "mk_gemm_static: device ordinal %d out of range", device_ordinal);
    mk_gemm_desc d = *desc;
    // the rules of mk_gemm first (dtypes, leading dimensions, epilogue / flag combinations, non-null peers) ...
    bool nothing_to_do = false;
    mk_status st = validate_gemm_desc(d, "mk_gemm_static", &nothing_to_do);
    if (st != MK_OK) return st;
    // ... then what this entry point adds: the static scratch bounds the batch, and only the tensor-core kernel runs
    if (d.batch > kStaticMaxBatch)
        return fail(MK_ERR_INVALID, "mk_gemm_static: batch %d exceeds the static scratch (one error word per batch item, at most %d)", d.batch,
                    kStaticMaxBatch);
    MK_REQUIRE(d.dtype_in == MK_BF16 || d.dtype_in == MK_F16, "mk_gemm_static: only bf16 / f16 inputs run on the tensor-core kernel");
    MK_REQUIRE(d.M > 0 && d.N > 0 && d.K > 0, "mk_gemm_static: M, N, K must be positive");
    MK_REQUIRE(d.epilogue != MK_EPI_SWIGLU, "mk_gemm_static: the gated pair of products is not available here; use mk_gemm");
    if ((reinterpret_cast<uintptr_t>(d.A) & 15) || (reinterpret_cast<uintptr_t>(d.B) & 15) || (d.lda % 8) || (d.ldb % 8) || (d.stride_a % 8) ||
        (d.stride_b % 8))
        return fail(MK_ERR_UNSUPPORTED, "mk_gemm_static: A and B need 16-byte aligned bases and row pitches (TMA); use mk_gemm for other layouts");
    MK_REQUIRE(d.M <= 0x7fffff00ll && d.N <= 0x7fffff00ll && d.K <= 0x7fffff00ll, "mk_gemm_static: dimension too large");
    const int64_t tiles_m = (d.M + BM - 1) / BM, tiles_n = (d.N + BN - 1) / BN;
    MK_REQUIRE(tiles_m * tiles_n <= 0x7fffffffll, "mk_gemm_static: too many tiles");
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);

    DeviceGuard guard;
    st = guard.enter(device_ordinal);
    if (st != MK_OK) return st;
    if (kernel_error) {     // the synchronous form cannot run inside a capture
        cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
        MK_CUDA(cudaStreamIsCapturing(stream, &cs));
        if (cs != cudaStreamCaptureStatusNone)
            return fail(MK_ERR_INVALID, "mk_gemm_static: kernel_error asks for a stream synchronisation, which a capturing stream cannot do; pass NULL");
    }
    st = static_setup(device_ordinal);
    if (st != MK_OK) return st;
    if (g_static_cc_major[device_ordinal] != 10) return fail(MK_ERR_UNSUPPORTED, "mk_gemm_static: needs an sm_100 device");
    KernelError* words = g_static_ptr[device_ordinal];
    const int sms = g_static_sms[device_ordinal];
    const bool pair = use_pair(d, sms);

    // The kernel only writes an error word when a wait gives up (compare-and-swap against 0), and the
    // array keeps whatever the previous call left: clear the words this call uses, in stream order.
    MK_CUDA(cudaMemsetAsync(words, 0, sizeof(KernelError) * d.batch, stream));

    const size_t es_out = dtype_size(d.dtype_out);
    for (int b = 0; b < d.batch; ++b) {
        const char* A = (const char*)d.A + (size_t)b * d.stride_a * 2;
        const char* B = (const char*)d.B + (size_t)b * d.stride_b * 2;
        alignas(64) CUtensorMap ta, tb;
        st = encode_2d(&ta, d.dtype_in, A, (uint64_t)d.K, (uint64_t)d.M, (uint64_t)d.lda * 2, BK, BM);
        if (st != MK_OK) return st;
        st = d.trans_b ? encode_2d(&tb, d.dtype_in, B, (uint64_t)d.K, (uint64_t)d.N, (uint64_t)d.ldb * 2, BK, pair ? BN / 2 : BN)
                       : encode_2d(&tb, d.dtype_in, B, (uint64_t)d.N, (uint64_t)d.K, (uint64_t)d.ldb * 2, 64, BK);
        if (st != MK_OK) return st;
        TcParams p{};
        p.M = d.M; p.N = d.N; p.K = d.K;
        p.C = (char*)d.C + (size_t)b * d.stride_c * es_out;
        p.D = d.epilogue == MK_EPI_ADD ? (const char*)d.D + (size_t)b * d.stride_c * es_out : d.epilogue == MK_EPI_ADD_ROW ? (const char*)d.D : nullptr;
        p.ldc = d.ldc;
        p.ldd = d.epilogue == MK_EPI_ADD_ROW ? 0 : d.ldc;
        p.scaled = (d.flags & MK_GEMM_SCALED) ? 1 : 0;
        p.alpha = p.scaled ? d.alpha : 1.0f;
        p.beta = p.scaled ? d.beta : 1.0f;
        const uint32_t fmt = d.dtype_in == MK_BF16 ? 1u : 0u;
        p.idesc = idesc_f16(fmt, 0u, d.trans_b ? 0u : 1u, BM, BN);
        p.idesc2 = idesc_f16(fmt, 0u, d.trans_b ? 0u : 1u, 2 * BM, BN);
        p.tiles_m = (int)tiles_m;
        p.tiles_m2 = (int)((d.M + 2 * BM - 1) / (2 * BM));
        p.tiles_n = (int)tiles_n;
        p.group_m = group_m_setting();
        p.n_peers = d.n_peers;
        for (int q = 0; q < d.n_peers; ++q) p.peer_C[q] = (char*)d.peer_C[q] + (size_t)b * d.stride_c * es_out;
        p.staged = staged_ok(p, es_out);
        p.kerr = words + b;
#define MK_TCS(TB, OUT) st = launch_tc_static<TB, OUT>(sms, pair, stream, ta, tb, p)
        if (d.trans_b) {
            if (d.dtype_out == MK_F32) MK_TCS(true, MK_F32); else if (d.dtype_out == MK_BF16) MK_TCS(true, MK_BF16); else MK_TCS(true, MK_F16);
        } else {
            if (d.dtype_out == MK_F32) MK_TCS(false, MK_F32); else if (d.dtype_out == MK_BF16) MK_TCS(false, MK_BF16); else MK_TCS(false, MK_F16);
        }
#undef MK_TCS
        if (st != MK_OK) return st;
    }
    if (kernel_error) return read_static_words(words, d.batch, stream, kernel_error, "mk_gemm_static");
    return MK_OK;
}

extern "C" mk_status mk_gemm_static_status(int32_t device_ordinal, void* cuda_stream, int32_t batch, uint32_t* kernel_error) {
    using namespace mk;
    MK_REQUIRE(kernel_error, "mk_gemm_static_status: null output");
    MK_REQUIRE(device_ordinal >= 0 && device_ordinal < kMaxDevices, "mk_gemm_static_status: device ordinal %d out of range", device_ordinal);
    if (batch <= 0) batch = 1;
    MK_REQUIRE(batch <= kStaticMaxBatch, "mk_gemm_static_status: batch %d exceeds the static scratch (at most %d)", batch, kStaticMaxBatch);
    DeviceGuard guard;
    mk_status st = guard.enter(device_ordinal);
    if (st != MK_OK) return st;
    st = static_setup(device_ordinal);
    if (st != MK_OK) return st;
    return read_static_words(g_static_ptr[device_ordinal], batch, static_cast<cudaStream_t>(cuda_stream), kernel_error, "mk_gemm_static_status");
}
