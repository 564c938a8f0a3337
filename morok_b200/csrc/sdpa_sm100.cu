// Fused attention forward on Blackwell tensor cores (sm_100a): head sizes up to 128 (built for 64 and 128 columns;
// other multiples of 8 run zero-padded on the next larger one) and 256.
//
// One kernel replaces the >= 5 kernels (and the materialised [Sq,Sk] score matrix) that morok
// schedules for `scaled_dot_product_attention` (tensor/src/transformer.rs:78-137):
// O = softmax(causal(Q K^T * scale)) V with an online softmax whose running maximum and sum stay
// in f32 registers.
//
// A CTA owns 256 query rows of one (batch, head) as two 128-row tiles that ping-pong (one tile for 256-wide heads).
// Twelve warps = three warpgroups; the control warpgroup gives registers to the two softmax warpgroups (setmaxnreg):
//
//   warps 0-3 / 4-7  softmax of tile 0 / tile 1: one thread per query row.  The row's 128 scores of a key block
//                    are read from tensor memory once and stay in registers: row maximum, exp2 (three pairs in
//                    four on the special-function unit, the fourth as a polynomial on the FMA pipes), P (16 bit)
//                    written back over S -- for 128-wide heads published in two halves of 64 keys; m and l in
//                    registers; O is rescaled only when the maximum moved by > 2^8; finally O is normalised and
//                    stored -- 128-bit stores of each thread's row, or into a staging tile that leaves by tile
//                    stores (peer GPUs receive copies, padded head sizes, long key ranges)
//   warp 8           TMA producer: claims work items, Q per item, then K / V blocks of 128 keys
//                    through a ring that runs on across items
//   warp 9           MMA issuer: S_t = Q_t K^T and O_t += P_t V, tile 0 and tile 1 interleaved so the
//                    tensor pipe works on one tile while the other is in softmax.  All 32 lanes run
//                    the loops and waits (descriptors then live in uniform registers); one elected
//                    lane is predicated on the tcgen05 instructions
//   warp 10          tensor-memory allocation (512 columns: S0 S1 at 0 / 128, O0 O1 at 256 / 384); then, for
//                    staged output, one tile store per destination (local O and every peer's O over
//                    NVLink) of each staged tile
//   warp 11          idle (register rebalancing works per warpgroup of four warps)
//
// K is a K-major B operand, V an MN-major one (read as stored, no transpose), P is the A operand
// taken from tensor memory.  Key blocks entirely above the causal diagonal are never loaded.
// A mask (additive or bool, any shape that broadcasts against the scores) and a softcap run in the same
// kernel: its general form rewrites the scores of a block where they sit, in the softmax warps' registers.
// All barrier waits are bounded; a wait that gives up records a code in the device error word.
#include <cstdlib>
#include <type_traits>

#include "ptx_sm100.cuh"

namespace mk {
namespace {

using namespace ptx;

constexpr int BQ = 128;                 // query rows per tile (two tiles per CTA)
constexpr int BKV = 128;                // keys per block
// Per head size (D == Dv: 64, 128 or 256).  A tile of 128 rows is HD / 64 boxes of 64 columns (16 KiB each,
// 128-byte swizzled); with 64-wide heads the K / V ring is four stages deep in the same 128 KiB.  256-wide heads
// run one query tile per CTA: O alone takes 256 of the 512 tensor-memory columns, and Q, one K block and one V block
// (64 KiB each) fill shared memory, so the K / V "rings" are a single stage -- which is enough for one tile, because
// the next K is only needed after this block's softmax and P V, and the next V after the next S and softmax.
template <int HD>
struct Cfg {
    static constexpr int TILE_BYTES = BQ * HD * 2;
    static constexpr int HALF_BYTES = BQ * 64 * 2;
    static constexpr int TILES = HD == 256 ? 1 : 2;                       // query tiles per CTA (see below)
    static constexpr int KV_STAGES = HD == 64 ? 4 : (HD == 256 ? 1 : 2);
    static constexpr int SMEM_Q = TILES * TILE_BYTES;
    static constexpr int SMEM_K = KV_STAGES * TILE_BYTES;
    static constexpr int SMEM_V = KV_STAGES * TILE_BYTES;
    static constexpr int NUM_BARS = 1 + 4 * KV_STAGES + 6 + 1 + 2 + 4 + 1 + 2;
    static constexpr int SMEM_BYTES = SMEM_Q + SMEM_K + SMEM_V + 1024 + 512;      // + alignment slack + barriers and slots
    // (runs whose output leaves by tile stores add one 128-row staging tile beside the operands: the launcher asks for it)
};
// Tensor maps of the output as every destination sees it: [0] the local O, [1 ..] the peers' O
// ([B, H, S, D] with the caller's strides; box of 64 columns x 128 rows, 128-byte swizzle).
struct OStoreMaps {
    CUtensorMap m[1 + MK_MAX_PEERS];
};
constexpr int NUM_THREADS = 384;        // 12 warps = 3 warpgroups (register rebalancing works per warpgroup); warp 11 idles
// 384 threads start with 168 registers each.  The control warpgroup keeps 56, which frees 128 * 112 = 14336 registers;
// the two softmax warpgroups take 224 each: 2 * 128 * 56 = 14336.
constexpr int REGS_LAUNCH = 168, REGS_CONTROL = 56, REGS_SOFTMAX = 224;
static_assert(2 * 128 * (REGS_SOFTMAX - REGS_LAUNCH) <= 128 * (REGS_LAUNCH - REGS_CONTROL), "register budget of the rebalancing");
template <int N>
__device__ __forceinline__ void setmaxnreg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }
constexpr int TMEM_COLS = 512;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_THRESHOLD = 8.0f;  // log2 domain: P stays below 2^8

struct FaParams {
    int B, Hq, Hkv, Sq, Sk;
    int causal;
    int causal_offset;  // >= 0: row i sees columns <= i + causal_offset
    float scale_log2;   // scale * log2(e)
    // general form (mask and / or softcap): the scores are rewritten in tensor memory as
    // log2(e) * softcap(scale * s + causal rule + mask) before the softmax proper
    float scale;            // natural scale
    float softcap;          // <= 0: none
    const void* mask;       // null: none
    int mask_bool;          // one byte per element, zero adds -inf
    int mask_vec;           // rows may be read 16 bytes at a time
    int64_t mask_strides[3];    // batch, head, query row (elements)
    void* O;
    float* lse;
    int64_t o_strides[3];
    uint32_t idesc_qk, idesc_pv;
    int q_pairs;        // work items per (batch, head): ceil(Sq / (tiles * 128))
    int tiles;          // query tiles of 128 rows per work item: 2, or 1 for 256-wide heads
    unsigned int* work_counter;   // device-wide claim counter, zeroed before the launch
    int tma_o;          // stage O in a tile of shared memory from which warp 10 issues one tile store per destination
                        // (always when peers receive copies, and for head sizes the kernel pads)
    int n_peers;
    void* peer_O[MK_MAX_PEERS];
    KernelError* kerr;
};

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint64_t pack_f32x2(float a, float b) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ float lo_f32(uint64_t v) { return __uint_as_float((uint32_t)v); }
__device__ __forceinline__ float hi_f32(uint64_t v) { return __uint_as_float((uint32_t)(v >> 32)); }
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// Scores past the last visible column of this row become -inf.
__device__ __forceinline__ void mask_chunk(uint32_t (&s)[32], int col, int col_limit) {
#pragma unroll
    for (int i = 0; i < 32; ++i)
        if (col + i > col_limit) s[i] = 0xff800000u;
}

// Maximum of 32 scores with 3-input max instructions.
__device__ __forceinline__ float max_chunk(const uint32_t (&s)[32]) {
    float m = fmaxf(__uint_as_float(s[0]), __uint_as_float(s[1]));
#pragma unroll
    for (int i = 2; i < 32; i += 2) m = max3(m, __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
    return m;
}

// 32 scores -> 16 packed 16-bit pairs of exp2(s * scale - m); the two-lane f32 sum accumulates the
// unrounded values.  Scale-and-shift and the sum run as packed f32x2 instructions.
template <bool BF16>
__device__ __forceinline__ void exp_chunk(const uint32_t (&s)[32], float scale_log2, float neg_m, uint64_t& sum2, uint32_t* pk) {
    const uint64_t sc2 = pack_f32x2(scale_log2, scale_log2), nm2 = pack_f32x2(neg_m, neg_m);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        uint64_t v = (uint64_t)s[2 * i] | ((uint64_t)s[2 * i + 1] << 32);
        asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(v) : "l"(v), "l"(sc2), "l"(nm2));
        const float a = fast_exp2(lo_f32(v)), b = fast_exp2(hi_f32(v));
        const uint64_t e = pack_f32x2(a, b);
        asm("add.rn.f32x2 %0, %1, %2;" : "=l"(sum2) : "l"(sum2), "l"(e));
        if constexpr (BF16) {
            __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
            pk[i] = *reinterpret_cast<uint32_t*>(&h);
        } else {
            __half2 h = __floats2half2_rn(a, b);
            pk[i] = *reinterpret_cast<uint32_t*>(&h);
        }
    }
}

// The same with every POLY_EVERY-th pair evaluated on the FMA pipes instead of the special-function unit.
// That unit delivers 4 results per clock per SM sub-partition, so the two softmax warps that share one
// need 2048 clocks per key block for their exponentials alone -- as long as the tensor core needs for
// the block's MMAs.  Moving a quarter of the pairs to a degree-3 polynomial (x = n + f, n = round(x),
// f in [-0.5, 0.5]; 2^f by minimax polynomial, relative error 7.5e-5, far below the 16-bit rounding of P;
// 2^n by adding n to the exponent field) balances the two pipes: 1738 instead of 2083 clocks for two
// warps in isolation.
template <bool BF16, int POLY_EVERY>
__device__ __forceinline__ void exp_chunk_mixed(const uint32_t (&s)[32], float scale_log2, float neg_m, uint64_t& sum2, uint32_t* pk) {
    const uint64_t sc2 = pack_f32x2(scale_log2, scale_log2), nm2 = pack_f32x2(neg_m, neg_m);
    const uint64_t magic2 = pack_f32x2(12582912.0f, 12582912.0f);
    const uint64_t c0 = pack_f32x2(9.999280572e-01f, 9.999280572e-01f), c1 = pack_f32x2(6.932609677e-01f, 6.932609677e-01f);
    const uint64_t c2 = pack_f32x2(2.426111251e-01f, 2.426111251e-01f), c3 = pack_f32x2(5.517162010e-02f, 5.517162010e-02f);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        uint64_t v = (uint64_t)s[2 * i] | ((uint64_t)s[2 * i + 1] << 32);
        asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(v) : "l"(v), "l"(sc2), "l"(nm2));
        float a, b;
        if (i % POLY_EVERY == POLY_EVERY - 1) {
            v = pack_f32x2(fmaxf(lo_f32(v), -125.0f), fmaxf(hi_f32(v), -125.0f));   // keeps 2^n a normal number; -inf -> ~0
            uint64_t xf, n, f, q;
            asm("add.rn.f32x2 %0, %1, %2;" : "=l"(xf) : "l"(v), "l"(magic2));      // integer part lands in the low mantissa bits
            asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(n) : "l"(xf), "l"(magic2));
            asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(f) : "l"(v), "l"(n));
            asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(q) : "l"(c3), "l"(f), "l"(c2));
            asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(q) : "l"(q), "l"(f), "l"(c1));
            asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(q) : "l"(q), "l"(f), "l"(c0));
            a = __uint_as_float((uint32_t)q + ((uint32_t)xf << 23));
            b = __uint_as_float((uint32_t)(q >> 32) + ((uint32_t)(xf >> 32) << 23));
        } else {
            a = fast_exp2(lo_f32(v));
            b = fast_exp2(hi_f32(v));
        }
        const uint64_t e = pack_f32x2(a, b);
        asm("add.rn.f32x2 %0, %1, %2;" : "=l"(sum2) : "l"(sum2), "l"(e));
        if constexpr (BF16) {
            __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
            pk[i] = *reinterpret_cast<uint32_t*>(&h);
        } else {
            __half2 h = __floats2half2_rn(a, b);
            pk[i] = *reinterpret_cast<uint32_t*>(&h);
        }
    }
}

// 2^x on the FMA pipes (the polynomial of exp_chunk_mixed, one value), x clamped to [-125, 125].
__device__ __forceinline__ float poly_exp2(float x) {
    x = fminf(fmaxf(x, -125.0f), 125.0f);
    const float xf = x + 12582912.0f;        // integer part lands in the low mantissa bits
    const float n = xf - 12582912.0f;
    const float f = x - n;
    float q = fmaf(5.517162010e-02f, f, 2.426111251e-01f);
    q = fmaf(q, f, 6.932609677e-01f);
    q = fmaf(q, f, 9.999280572e-01f);
    return __uint_as_float(__float_as_uint(q) + (__float_as_uint(xf) << 23));
}
__device__ __forceinline__ float fast_rcp(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// 32 consecutive mask values of one row as additive terms (bool: 0 where set, -inf where clear); columns >= Sk read as 0.
template <bool BOOLM>
__device__ __forceinline__ void load_mask_chunk(const void* row_ptr, int col, int Sk, bool vec, float (&add)[32]) {
    if (vec && col + 32 <= Sk) {
        if constexpr (BOOLM) {
            const uint4* p4 = reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned char*>(row_ptr) + col);
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const uint4 v = __ldg(p4 + i);
                const uint32_t ws[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int j = 0; j < 16; ++j) add[16 * i + j] = ((ws[j >> 2] >> (8 * (j & 3))) & 0xffu) ? 0.0f : -INFINITY;
            }
        } else {
            const float4* p4 = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(row_ptr) + col);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float4 v = __ldg(p4 + i);
                add[4 * i] = v.x; add[4 * i + 1] = v.y; add[4 * i + 2] = v.z; add[4 * i + 3] = v.w;
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            float a = 0.0f;
            if (col + i < Sk) {
                if constexpr (BOOLM) a = __ldg(reinterpret_cast<const unsigned char*>(row_ptr) + col + i) ? 0.0f : -INFINITY;
                else a = __ldg(reinterpret_cast<const float*>(row_ptr) + col + i);
            }
            add[i] = a;
        }
    }
}

// Does the mask change anything in columns col0 .. col0 + 127 for the rows of this warp?  (additive: any value other
// than +0; bool: any element clear.)  When every row reads the same values (a key-padding mask: row stride 0) the 32
// lanes share the scan, four values each; otherwise every thread scans its own row.  Warp-uniform result.
template <bool BOOLM>
__device__ __forceinline__ bool mask_block_active(const char* row_ptr, bool rows_shared, int col0, int Sk, bool vec, int lane) {
    bool any = false;
    if (rows_shared) {
        const int c = col0 + 4 * lane;
        if constexpr (BOOLM) {
            const unsigned char* m = reinterpret_cast<const unsigned char*>(row_ptr) + c;
            if (vec && c + 4 <= Sk) any = __vcmpeq4(__ldg(reinterpret_cast<const unsigned int*>(m)), 0u) != 0u;
            else
                for (int i = 0; i < 4; ++i) any |= (c + i < Sk) && __ldg(m + i) == 0;
        } else {
            const float* m = reinterpret_cast<const float*>(row_ptr) + c;
            if (vec && c + 4 <= Sk) {
                const uint4 v = __ldg(reinterpret_cast<const uint4*>(m));
                any = (v.x | v.y | v.z | v.w) != 0u;
            } else {
                for (int i = 0; i < 4; ++i) any |= (c + i < Sk) && __float_as_uint(__ldg(m + i)) != 0u;
            }
        }
    } else {
#pragma unroll 1
        for (int c = 0; c < BKV / 32; ++c) {
            float add[32];
            load_mask_chunk<BOOLM>(row_ptr, col0 + c * 32, Sk, vec, add);
            uint32_t bits = 0;
#pragma unroll
            for (int i = 0; i < 32; ++i) bits |= __float_as_uint(add[i]);
            any |= bits != 0u;
        }
    }
    return __any_sync(0xffffffffu, any);
}

// General form of a key block: rewrites 32 scores of this thread's row, held in registers, as
// log2(e) * softcap(scale * s, causal rule, mask).  Order as in the reference (tensor/src/transformer.rs:98-132):
// scale, causal -inf, mask added, softcap last (which turns the -inf of masked positions into -softcap); columns
// past Sk do not exist and stay -inf.  `add` holds the chunk's 32 mask values when there is a mask.
struct RewriteConsts {
    bool edge, has_mask;
    int causal_limit;
    float cap, k2;
};
__device__ __forceinline__ RewriteConsts rewrite_consts(const FaParams& p, const char* mask_row, int col0, int qrow, int tile_row0) {
    RewriteConsts c;
    const bool causal_here = p.causal && col0 + BKV - 1 > tile_row0 + p.causal_offset;
    c.edge = causal_here || col0 + BKV > p.Sk;
    c.has_mask = mask_row != nullptr;
    c.causal_limit = p.causal ? qrow + p.causal_offset : 0x7fffffff;
    c.cap = p.softcap;
    c.k2 = p.softcap > 0.0f ? 2.0f * LOG2E / p.softcap : 0.0f;
    return c;
}
__device__ __forceinline__ void load_mask_values(const FaParams& p, const char* mask_row, int cbase, float (&add)[32]) {
    if (!mask_row) return;
    if (p.mask_bool) load_mask_chunk<true>(mask_row, cbase, p.Sk, p.mask_vec != 0, add);
    else load_mask_chunk<false>(mask_row, cbase, p.Sk, p.mask_vec != 0, add);
}
template <bool CAP>
__device__ __forceinline__ void rewrite_chunk(const FaParams& p, const RewriteConsts& c, uint32_t (&s)[32], const float (&add)[32], int cbase) {
    if constexpr (CAP) {
        // log2(e) * cap * tanh(x / cap) with tanh(z) = 1 - 2 / (1 + 2^(z * 2 log2 e)): the power of two alternately on the
        // special-function unit and on the FMA pipes, like the exponentials of P; one rcp.approx per score; -inf (a masked
        // position) gives -cap as in the reference.  Plain f32 instructions: the packed f32x2 form of this chain measured
        // 40 % slower (the clamp, the exponent arithmetic and the reciprocal have no packed form; the pairs are taken apart
        // and put together again around them).
        const float cap_l2 = c.cap * LOG2E;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const int col = cbase + i;
            float x = __uint_as_float(s[i]) * p.scale;
            if (c.edge && col > c.causal_limit) x = -INFINITY;
            if (c.has_mask) x += add[i];
            const float t2 = x * c.k2;
            const float e = (i & 1) ? poly_exp2(t2) : fast_exp2(t2);      // ex2.approx: -inf -> 0, overflow -> inf -> rcp 0
            x = fmaf(fast_rcp(1.0f + e), -2.0f * cap_l2, cap_l2);
            if (c.edge && col >= p.Sk) x = -INFINITY;
            s[i] = __float_as_uint(x);
        }
    } else {
        // no cap: log2(e) * (scale * s + mask) on packed pairs; -inf (a causal or a masked position)
        // survives the addition either way round
        const uint64_t sc2 = pack_f32x2(p.scale_log2, p.scale_log2), l2e2 = pack_f32x2(LOG2E, LOG2E);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            uint64_t v = (uint64_t)s[2 * i] | ((uint64_t)s[2 * i + 1] << 32);
            if (c.has_mask) {
                uint64_t m2 = pack_f32x2(add[2 * i], add[2 * i + 1]);
                asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(m2) : "l"(m2), "l"(l2e2));
                asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(v) : "l"(v), "l"(sc2), "l"(m2));
            } else {
                asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(v) : "l"(v), "l"(sc2));
            }
            s[2 * i] = (uint32_t)v;
            s[2 * i + 1] = (uint32_t)(v >> 32);
        }
        if (c.edge) mask_chunk(s, cbase, min(c.causal_limit, p.Sk - 1));
    }
}

// Number of key blocks a query tile starting at row q0 needs.
__device__ __forceinline__ int blocks_for_tile(const FaParams& p, int q0) {
    if (q0 >= p.Sq) return 0;
    const int all = (p.Sk + BKV - 1) / BKV;
    // with a softcap the causally masked scores become -softcap instead of -inf and take part: no block is skipped
    if (!p.causal || p.softcap > 0.0f) return all;
    const int last_col = min(q0 + BQ, p.Sq) - 1 + p.causal_offset;   // the tile's last row sees columns <= last_col
    return min(all, last_col / BKV + 1);
}

// One unit of work: 256 query rows (two tiles) of one (batch, head).
struct WorkItem {
    int batch, head, kv_head, q0;
    int nblk[2], nmax;
};

__device__ __forceinline__ WorkItem decode_item(const FaParams& p, int idx) {
    WorkItem w;
    // heaviest first within a head: under a causal mask the last query rows need the most key blocks
    const int pair = p.q_pairs - 1 - idx % p.q_pairs;
    const int bh = idx / p.q_pairs;
    w.head = bh % p.Hq;
    w.batch = bh / p.Hq;
    w.kv_head = w.head / (p.Hq / p.Hkv);
    w.q0 = pair * p.tiles * BQ;
    w.nblk[0] = blocks_for_tile(p, w.q0);
    w.nblk[1] = p.tiles == 2 ? blocks_for_tile(p, w.q0 + BQ) : 0;
    w.nmax = max(w.nblk[0], w.nblk[1]);
    return w;
}

// FORM 0: plain (scale and the causal rule only); 1: with a mask (only the blocks it changes are rewritten); 2: with a
// softcap (every block is rewritten), with or without a mask.
template <bool BF16, int HD, int FORM>
__global__ void __launch_bounds__(NUM_THREADS, 1)
sdpa_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
               const __grid_constant__ FaParams p, const __grid_constant__ OStoreMaps omaps) {
    constexpr int TILE_BYTES = Cfg<HD>::TILE_BYTES, HALF_BYTES = Cfg<HD>::HALF_BYTES, KV_STAGES = Cfg<HD>::KV_STAGES;
    constexpr int SMEM_Q = Cfg<HD>::SMEM_Q, SMEM_K = Cfg<HD>::SMEM_K, SMEM_V = Cfg<HD>::SMEM_V, NUM_BARS = Cfg<HD>::NUM_BARS;
    constexpr int NH = HD / 64;      // 64-column boxes per tile
    constexpr bool GENERAL = FORM != 0;
    // P is published in two halves of 64 keys, so that the first four P V steps run while the second half is exponentiated.
    // 64-wide heads are bound by the softmax warps, not by the chain softmax -> P V -> next S: there the second barrier only costs.
    constexpr bool P_HALVES = HD >= 128;
    constexpr int PE = HD == 64 ? 3 : 4;     // every PE-th pair of exponentials runs on the FMA pipes (measured best per head size)
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t sQ = smem_u32(smem), sK = sQ + SMEM_Q, sV = sK + SMEM_K;
    uint8_t* stageO = smem + SMEM_Q + SMEM_K + SMEM_V;      // present only when p.tma_o (the launch then asks for TILE_BYTES more)
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SMEM_Q + SMEM_K + SMEM_V + (p.tma_o ? TILE_BYTES : 0));
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NUM_BARS);
    static_assert(NUM_BARS * 8 + 32 <= 512, "barrier area");
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const uint32_t bar_q = smem_u32(bars);                   // Q tiles of the current work item landed
    const uint32_t bar_kfull = bar_q + 8, bar_kempty = bar_kfull + 8 * KV_STAGES;
    const uint32_t bar_vfull = bar_kempty + 8 * KV_STAGES, bar_vempty = bar_vfull + 8 * KV_STAGES;
    const uint32_t bar_sfull = bar_vempty + 8 * KV_STAGES;   // [2] S_t written by the tensor core
    const uint32_t bar_pfull = bar_sfull + 16;               // [2] P_t written (and O_t rescaled) by the softmax warps
    const uint32_t bar_pvdone = bar_pfull + 16;              // [2] O_t += P_t V retired
    const uint32_t bar_qempty = bar_pvdone + 16;             // Q tiles may be overwritten (the item's last S MMA was issued)
    const uint32_t bar_ofree = bar_qempty + 8;               // [2] O_t drained by the epilogue of the previous item
    const uint32_t bar_ifull = bar_ofree + 16;               // [2] work-item slot published by the producer
    const uint32_t bar_iempty = bar_ifull + 16;              // [2] work-item slot read by every consumer
    const uint32_t bar_ostage_full = bar_iempty + 16;        // output staging tile written by the four warps of a query tile
    const uint32_t bar_phalf = bar_ostage_full + 8;          // [2] first 64 keys of P_t written (only when P is published in halves)
    // "The staging tile is free again" is a counter, not a barrier: the number of uses the tile stores of warp 10 have
    // read out.  The warps of a query tile wait until it has reached their use number.  A barrier would not do: its
    // waits see the parity of a phase only, and a waiter here can be two or more uses behind -- a tile that sat out an
    // item or two (a last, half-filled pair of tiles), or one that comes to wait while the copy engine is still busy with
    // the use before the other tile's -- and would take an old phase for its own.
    const uint32_t stage_freed = smem_u32(tmem_slot + 4);
    volatile int* item_slot = reinterpret_cast<volatile int*>(tmem_slot + 2);   // [2] claimed item indices

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_items = p.q_pairs * p.B * p.Hq;

    if (threadIdx.x == 0) {
        mbar_init(bar_q, 1);
        mbar_init(bar_qempty, 1);     // Q tiles are free once the item's last S MMA retired (one commit)
        mbar_init(bar_ostage_full, 128);
        for (int i = 0; i < KV_STAGES; ++i) {
            mbar_init(bar_kfull + 8 * i, 1);
            mbar_init(bar_kempty + 8 * i, 1);
            mbar_init(bar_vfull + 8 * i, 1);
            mbar_init(bar_vempty + 8 * i, 1);
        }
        for (int t = 0; t < 2; ++t) {
            mbar_init(bar_sfull + 8 * t, 1);
            mbar_init(bar_pfull + 8 * t, 128);
            mbar_init(bar_phalf + 8 * t, 128);
            mbar_init(bar_pvdone + 8 * t, 1);
            mbar_init(bar_ofree + 8 * t, 4);   // one lane per softmax warp of the tile
            mbar_init(bar_ifull + 8 * t, 1);
            mbar_init(bar_iempty + 8 * t, 1 + 8 + (p.tma_o ? 1 : 0));    // MMA warp, eight softmax warps, and the store warp when it takes part
        }
        *abort_flag = 0;
        tmem_slot[4] = 0;
        fence_barrier_init();
        prefetch_tensormap(&tmQ);
        prefetch_tensormap(&tmK);
        prefetch_tensormap(&tmV);
        if (p.tma_o)
            for (int d = 0; d <= p.n_peers; ++d) prefetch_tensormap(&omaps.m[d]);
    }
    if (warp == 10) {
        tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // tensor-memory columns: S_t / P_t at t*128, O_t at 256 + t*128

    // The CTA is persistent: it claims work items -- (batch, head, pair of query tiles) -- from a
    // device-wide counter until none are left.  Items are numbered head-major with the heaviest pair
    // of a head first, so the CTAs running at any moment share few heads (K/V stay in L2), the
    // cheapest items come last (short tail), and the epilogue of one item overlaps the loads and
    // first MMAs of the next.  The producer publishes each claimed index through a two-slot ring.
    // Registers are rebalanced between the warpgroups first: warps 8-11 (producer, MMA issuer, allocation / stores, one
    // idle warp) keep REGS_CONTROL each, and the two softmax warpgroups take REGS_SOFTMAX -- every warp of a warpgroup
    // executes the same instruction, before anything that could make another warp wait.
    if (warp >= 8) {
      setmaxnreg_dec<REGS_CONTROL>();
      if (warp == 8) {
        // ---------------------------------------------------------------- TMA producer + item claims
        // Warp-uniform like the MMA issuer: all lanes run the loops and waits, lane 0 claims and copies.
        {
            const bool leader = lane == 0;
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int n = 0; ok; ++n) {
                const int slot = n & 1;
                const uint32_t ipar = (n >> 1) & 1;
                ok = __all_sync(0xffffffffu, mbar_wait(bar_iempty + 8 * slot, ipar ^ 1, abort_flag, p.kerr, KERR_SDPA_PRODUCER_WAIT, 500000 + n));
                if (!ok) break;
                int claimed = 0;
                if (leader) claimed = (n == 0) ? (int)blockIdx.x : (int)(atomicAdd(p.work_counter, 1u) + gridDim.x);
                const int idx = __reduce_max_sync(0xffffffffu, claimed);     // item indices are >= 0
                if (leader) {
                    item_slot[slot] = idx;
                    mbar_arrive(bar_ifull + 8 * slot);      // release: consumers acquire through their wait
                }
                if (idx >= total_items) break;
                const WorkItem w = decode_item(p, idx);
                ok = __all_sync(0xffffffffu, mbar_wait(bar_qempty, (n & 1) ^ 1, abort_flag, p.kerr, KERR_SDPA_PRODUCER_WAIT, 600000 + n));
                if (!ok) break;
                if (leader) {
                    mbar_arrive_expect_tx(bar_q, Cfg<HD>::TILES * TILE_BYTES);
#pragma unroll
                    for (int t = 0; t < Cfg<HD>::TILES; ++t)
#pragma unroll
                        for (int h = 0; h < NH; ++h)
                            tma_load_4d(sQ + t * TILE_BYTES + h * HALF_BYTES, &tmQ, bar_q, h * 64, w.q0 + t * BQ, w.head, w.batch);
                }
                for (int j = 0; j < w.nmax; ++j) {
                    if (!__all_sync(0xffffffffu, mbar_wait(bar_kempty + 8 * stage, phase ^ 1, abort_flag, p.kerr, KERR_SDPA_PRODUCER_WAIT, j))) { ok = false; break; }
                    if (leader) {
                        mbar_arrive_expect_tx(bar_kfull + 8 * stage, TILE_BYTES);
#pragma unroll
                        for (int h = 0; h < NH; ++h)
                            tma_load_4d(sK + stage * TILE_BYTES + h * HALF_BYTES, &tmK, bar_kfull + 8 * stage, h * 64, j * BKV, w.kv_head, w.batch);
                    }
                    if (!__all_sync(0xffffffffu, mbar_wait(bar_vempty + 8 * stage, phase ^ 1, abort_flag, p.kerr, KERR_SDPA_PRODUCER_WAIT, 100000 + j))) { ok = false; break; }
                    if (leader) {
                        mbar_arrive_expect_tx(bar_vfull + 8 * stage, TILE_BYTES);
#pragma unroll
                        for (int h = 0; h < NH; ++h)
                            tma_load_4d(sV + stage * TILE_BYTES + h * HALF_BYTES, &tmV, bar_vfull + 8 * stage, h * 64, j * BKV, w.kv_head, w.batch);
                    }
                    if (++stage == KV_STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
      } else if (warp == 9) {
        // ---------------------------------------------------------------- MMA issuer
        // All 32 lanes run the loops and the waits so that descriptors and addresses stay warp-uniform;
        // one elected lane issues the tensor-core instructions.
        {
            const uint32_t leader = elect_one_u32();
            const uint32_t tm = __reduce_max_sync(0xffffffffu, tmem_base);
            const uint64_t desc_q = smem_desc_sw128(sQ, 16, 1024), desc_k = smem_desc_sw128(sK, 16, 1024);
            const uint64_t desc_v = smem_desc_sw128(sV, HALF_BYTES, 1024);
            auto issue_s = [&](int t, int kstage) {
                const uint64_t qd = desc_q + (uint32_t)((t * TILE_BYTES) >> 4), kd = desc_k + (uint32_t)((kstage * TILE_BYTES) >> 4);
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks) {
                    const uint32_t off = ((ks >> 2) * HALF_BYTES + (ks & 3) * 32) >> 4;
                    mma_f16_ss_lead(tm + t * 128, qd + off, kd + off, p.idesc_qk, ks != 0 ? 1u : 0u, leader);
                }
                mma_commit_lead(bar_sfull + 8 * t, leader);
            };
            auto issue_pv_steps = [&](int t, int vstage, bool accumulate, int ks0, int ks1) {
                const uint64_t vd = desc_v + (uint32_t)((vstage * TILE_BYTES) >> 4);
#pragma unroll
                for (int ks = ks0; ks < ks1; ++ks) {
                    mma_f16_ts_lead(tm + 256 + t * 128, tm + t * 128 + ks * 8, vd + (uint32_t)((ks * (16 * 128)) >> 4), p.idesc_pv,
                                    (accumulate || ks != 0) ? 1u : 0u, leader);
                }
            };
            int stage = 0;            // K/V ring position, carried across work items
            uint32_t phase = 0;
            uint32_t cum[2] = {0, 0}; // key blocks issued so far per tile (barrier phases are cumulative)
            uint32_t used[2] = {0, 0};   // items so far in which the tile had any work (phases of bar_ofree)
            bool ok = true;
            for (int n = 0; ok; ++n) {
                const int slot = n & 1;
                ok = __all_sync(0xffffffffu, mbar_wait(bar_ifull + 8 * slot, (n >> 1) & 1, abort_flag, p.kerr, KERR_SDPA_MMA_WAIT, 500000 + n));
                if (!ok) break;
                const int idx = __reduce_max_sync(0xffffffffu, (int)item_slot[slot]);
                if (leader) mbar_arrive(bar_iempty + 8 * slot);
                if (idx >= total_items) break;
                const WorkItem w = decode_item(p, idx);
                ok = __all_sync(0xffffffffu, mbar_wait(bar_q, n & 1, abort_flag, p.kerr, KERR_SDPA_MMA_WAIT, 900000) &&
                                                 mbar_wait(bar_kfull + 8 * stage, phase, abort_flag, p.kerr, KERR_SDPA_MMA_WAIT, 0));
                if (!ok) break;
                tc_fence_after();
                for (int t = 0; t < 2; ++t)
                    if (w.nblk[t] > 0) issue_s(t, stage);
                mma_commit_lead(bar_kempty + 8 * stage, leader);
                if (w.nmax == 1) mma_commit_lead(bar_qempty, leader);     // no further S of this item reads Q
                for (int j = 0; j < w.nmax && ok; ++j) {
                    const int nstage = (stage + 1 == KV_STAGES) ? 0 : stage + 1;
                    const uint32_t nphase = (stage + 1 == KV_STAGES) ? phase ^ 1 : phase;
                    ok = __all_sync(0xffffffffu, mbar_wait(bar_vfull + 8 * stage, phase, abort_flag, p.kerr, KERR_SDPA_MMA_WAIT, 200000 + j));
                    bool k_next_ready = false;
                    for (int t = 0; t < 2 && ok; ++t) {
                        if (j >= w.nblk[t]) continue;
                        if (j == 0) {   // the first P V of an item overwrites O_t: the previous item's epilogue must have drained it
                            ok = __all_sync(0xffffffffu, mbar_wait(bar_ofree + 8 * t, (used[t] & 1) ^ 1, abort_flag, p.kerr, KERR_SDPA_MMA_WAIT, 700000 + n));
                            if (!ok) break;
                        }
                        if constexpr (P_HALVES) {
                            ok = __all_sync(0xffffffffu, mbar_wait(bar_phalf + 8 * t, (cum[t] + j) & 1, abort_flag, p.kerr, KERR_SDPA_MMA_WAIT, 350000 + j));
                            if (!ok) break;
                            tc_fence_after();
                            issue_pv_steps(t, stage, j > 0, 0, BKV / 32);
                        }
                        ok = __all_sync(0xffffffffu, mbar_wait(bar_pfull + 8 * t, (cum[t] + j) & 1, abort_flag, p.kerr, KERR_SDPA_MMA_WAIT, 300000 + j));
                        if (!ok) break;
                        tc_fence_after();
                        issue_pv_steps(t, stage, j > 0, P_HALVES ? BKV / 32 : 0, BKV / 16);
                        mma_commit_lead(bar_pvdone + 8 * t, leader);
                        if (j + 1 < w.nblk[t]) {
                            if (!k_next_ready) {
                                ok = __all_sync(0xffffffffu, mbar_wait(bar_kfull + 8 * nstage, nphase, abort_flag, p.kerr, KERR_SDPA_MMA_WAIT, 400000 + j));
                                if (!ok) break;
                                tc_fence_after();
                                k_next_ready = true;
                            }
                            issue_s(t, nstage);
                        }
                    }
                    if (!ok) break;
                    mma_commit_lead(bar_vempty + 8 * stage, leader);
                    if (k_next_ready) mma_commit_lead(bar_kempty + 8 * nstage, leader);
                    if (j + 2 == w.nmax) mma_commit_lead(bar_qempty, leader);   // the S MMAs of the item's last block have just been issued
                    stage = nstage;
                    phase = nphase;
                }
                for (int t = 0; t < 2; ++t) {
                    cum[t] += w.nblk[t];
                    used[t] += w.nblk[t] > 0 ? 1u : 0u;
                }
            }
        }
      } else if (warp == 10 && p.tma_o) {
        // ---------------------------------------------------------------- tile stores of finished output tiles
        // Follows the work items like every other consumer; for each query tile that had work it waits until the four
        // softmax warps have staged the tile, issues one tile store per 64-column box and destination (the local O and
        // every peer's O over NVLink), and frees the staging tile once the copy engine has read it.
        uint32_t u = 0;
        bool ok = true;
        for (int n = 0; ok; ++n) {
            const int slot = n & 1;
            ok = __all_sync(0xffffffffu, mbar_wait(bar_ifull + 8 * slot, (n >> 1) & 1, abort_flag, p.kerr, KERR_SDPA_STORE_WAIT, 500000 + n));
            if (!ok) break;
            const int idx = __reduce_max_sync(0xffffffffu, (int)item_slot[slot]);
            if (lane == 0) mbar_arrive(bar_iempty + 8 * slot);
            if (idx >= total_items) break;
            const WorkItem w = decode_item(p, idx);
            for (int t = 0; t < 2 && ok; ++t) {
                if (w.nblk[t] == 0) continue;
                ok = __all_sync(0xffffffffu, mbar_wait(bar_ostage_full, u & 1, abort_flag, p.kerr, KERR_SDPA_STORE_WAIT, n));
                if (!ok) break;
                if (lane == 0) {
                    const uint32_t src = smem_u32(stageO);
#pragma unroll
                    for (int h = 0; h < NH; ++h)
                        for (int d = 0; d <= p.n_peers; ++d) tma_store_4d(&omaps.m[d], src + h * HALF_BYTES, h * 64, w.q0 + t * BQ, w.head, w.batch);
                    bulk_commit_group();
                    bulk_wait_group_read<0>();
                    st_release_shared_u32(stage_freed, u + 1);
                }
                __syncwarp();
                ++u;
            }
        }
        if (lane == 0) bulk_wait_group<0>();     // every tile store has completed before the CTA may leave
        __syncwarp();
    
      }
    } else {
        setmaxnreg_inc<REGS_SOFTMAX>();
        // ---------------------------------------------------------------- softmax / correction / epilogue
        const int t = warp >> 2;                 // query tile
        const int quarter = warp & 3;            // tensor-memory lane quarter of this warp
        const int row_in_tile = quarter * 32 + lane;
        const uint32_t lane_base = uint32_t(quarter * 32) << 16;
        const uint32_t tS = tmem_base + lane_base + t * 128;
        const uint32_t tO = tmem_base + lane_base + 256 + t * 128;
        uint32_t cum = 0;                        // key blocks of this tile processed in earlier items
        uint32_t stage_uses = 0;                 // uses of the output staging tile in earlier items (tile-store delivery)
        bool ok = true;
      for (int n = 0; ok; ++n) {
        const int slot = n & 1;
        ok = mbar_wait(bar_ifull + 8 * slot, (n >> 1) & 1, abort_flag, p.kerr, KERR_SDPA_SOFTMAX_WAIT, 500000 + n);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const int idx = item_slot[slot];
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_iempty + 8 * slot);
        if (idx >= total_items) break;
        const WorkItem w = decode_item(p, idx);
        const int nblk = w.nblk[t], q0 = w.q0, head = w.head, batch = w.batch;
        const int qrow = q0 + t * BQ + row_in_tile;
        // This query row's mask values (rows past Sq read the last row: their output is never stored).  Computed where it is
        // needed, so that nothing of the mask stays live across the plain blocks.
        auto mask_row_of = [&]() -> const char* {
            if (!GENERAL || !p.mask) return nullptr;
            return (const char*)p.mask + ((int64_t)batch * p.mask_strides[0] + (int64_t)head * p.mask_strides[1] +
                                          (int64_t)min(qrow, p.Sq - 1) * p.mask_strides[2]) * (p.mask_bool ? 1 : 4);
        };
        const char* mask_row = nullptr;
        // A mask whose rows are all the same (a key-padding mask): the 32 lanes share the scan "does it change anything
        // in this block", four values each, fetched one block ahead.  A block that is not whole counts as changed.
        bool mask_shared = false;
        auto scan_fetch = [&](const char* row, int jb) {
            const int c = jb * BKV + 4 * lane;
            if (c + 4 > p.Sk) return p.mask_bool ? make_uint4(0u, 0u, 0u, 0u) : make_uint4(1u, 0u, 0u, 0u);
            if (p.mask_bool) return make_uint4(__ldg(reinterpret_cast<const unsigned int*>(row + c)), 0u, 0u, 0u);
            return __ldg(reinterpret_cast<const uint4*>(row + 4 * c));
        };
        uint4 scan_next = make_uint4(0u, 0u, 0u, 0u);
        float m_used = -INFINITY;   // maximum the stored P and O are expressed against (log2 domain)
        float l = 0.0f;
        // One key block of this tile.  `general` (a compile-time tag) selects the form with the per-block question and the
        // rewrite; the plain form is the whole loop of a run without mask or softcap, and the leading blocks a key-padding
        // mask leaves alone run through it too.  Returns false when a wait gave up.
        auto block = [&](auto general, int j) -> bool {
            constexpr bool G = decltype(general)::value;
            ok = mbar_wait(bar_sfull + 8 * t, (cum + j) & 1, abort_flag, p.kerr, KERR_SDPA_SOFTMAX_WAIT, j);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) return false;
            tc_fence_after();
            const int col0 = j * BKV;
            // Only the diagonal block and a ragged last block need element-wise masking.
            // General form: does this block need its scores rewritten (a softcap, or a mask that is not all "attend"
            // here)?  Blocks a mask leaves alone -- all of them but the boundary for a key-padding mask -- take the plain path.
            bool rewrite = false;
            if constexpr (G) {
                rewrite = FORM == 2;        // a softcap rewrites every block
                if (!rewrite && mask_shared) {
                    // the lanes' four values each of this block were requested one block ago; request the next block's now
                    const uint4 cur = scan_next;
                    if (j + 1 < nblk) scan_next = scan_fetch(mask_row, j + 1);
                    const bool any = p.mask_bool ? __vcmpeq4(cur.x, 0u) != 0u : (cur.x | cur.y | cur.z | cur.w) != 0u;
                    rewrite = __any_sync(0xffffffffu, any);
                } else if (!rewrite && mask_row) {
                    rewrite = p.mask_bool ? mask_block_active<true>(mask_row, p.mask_strides[2] == 0, col0, p.Sk, p.mask_vec != 0, lane)
                                          : mask_block_active<false>(mask_row, p.mask_strides[2] == 0, col0, p.Sk, p.mask_vec != 0, lane);
                }
            }
            const bool need_mask = !rewrite && ((p.causal && col0 + BKV - 1 > q0 + t * BQ + p.causal_offset) || (col0 + BKV > p.Sk));
            const int col_limit = p.causal ? min(p.Sk - 1, qrow + p.causal_offset) : p.Sk - 1;   // last visible column of this row
            const float sc = rewrite ? 1.0f : p.scale_log2;     // a rewritten block holds log2-domain scores

            // One pass over the row: with the registers the rebalancing gives the softmax warps, all 128 scores stay in
            // registers from the row maximum through the exponentials -- no second read of S from tensor memory.
            uint32_t s0[32], s1[32], s2[32], s3[32];
            {
                tmem_ld_32x32b_x32(tS, s0);
                tmem_ld_32x32b_x32(tS + 32, s1);
                tmem_ld_32x32b_x32(tS + 64, s2);
                tmem_ld_32x32b_x32(tS + 96, s3);
                if (G && (FORM == 2 || rewrite)) {
                    // every block under a softcap; for a key-padding mask its boundary blocks only.  The row is rewritten
                    // where it sits (registers), one chunk of mask values at a time; the first is requested before the wait.
                    const RewriteConsts rc = rewrite_consts(p, mask_row, col0, qrow, q0 + t * BQ);
                    float add[32];
                    load_mask_values(p, mask_row, col0, add);
                    tmem_wait_ld();
                    if constexpr (FORM == 2) {
                        // Every block is rewritten: one copy of the transform in the instruction stream, run four times.  The
                        // chunk to rewrite is always s0 and the four chunks rotate through it (four rotations put every chunk
                        // back where it was).  Unrolled four times the block loop outgrows the instruction cache: measured,
                        // the warps then wait for instructions more often than for anything else.
#pragma unroll 1
                        for (int c = 0; c < 4; ++c) {
                            if (c > 0) load_mask_values(p, mask_row, col0 + 32 * c, add);
                            rewrite_chunk<true>(p, rc, s0, add, col0 + 32 * c);
#pragma unroll
                            for (int i = 0; i < 32; ++i) {
                                const uint32_t first = s0[i];
                                s0[i] = s1[i];
                                s1[i] = s2[i];
                                s2[i] = s3[i];
                                s3[i] = first;
                            }
                        }
                    } else {
                        // Mask form: a rewritten block is the exception (the boundary of a key-padding mask), straight-line
                        // code off the hot path costs the plain blocks nothing.
                        rewrite_chunk<false>(p, rc, s0, add, col0);
                        load_mask_values(p, mask_row, col0 + 32, add);
                        rewrite_chunk<false>(p, rc, s1, add, col0 + 32);
                        load_mask_values(p, mask_row, col0 + 64, add);
                        rewrite_chunk<false>(p, rc, s2, add, col0 + 64);
                        load_mask_values(p, mask_row, col0 + 96, add);
                        rewrite_chunk<false>(p, rc, s3, add, col0 + 96);
                    }
                } else {
                    tmem_wait_ld();
                    if (need_mask) {   // masked scores become -inf: they drop out of the max and exponentiate to 0
                        mask_chunk(s0, col0, col_limit);
                        mask_chunk(s1, col0 + 32, col_limit);
                        mask_chunk(s2, col0 + 64, col_limit);
                        mask_chunk(s3, col0 + 96, col_limit);
                    }
                }
            }
            const float mx = fmaxf(fmaxf(max_chunk(s0), max_chunk(s1)), fmaxf(max_chunk(s2), max_chunk(s3)));
            const float m_new = fmaxf(m_used, mx * sc);
            float alpha = 1.0f;
            bool need = false;
            if (m_new > m_used + RESCALE_THRESHOLD) {
                alpha = fast_exp2(m_used - m_new);   // exp2(-inf) = 0 on the first block
                m_used = m_new;
                need = true;
            }
            if (j > 0 && __any_sync(0xffffffffu, need)) {
                // O_t is only touched between "P V of block j-1 retired" and "P of block j published".
                ok = mbar_wait(bar_pvdone + 8 * t, (cum + j - 1) & 1, abort_flag, p.kerr, KERR_SDPA_SOFTMAX_WAIT, 100000 + j);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) return false;
                tc_fence_after();
#pragma unroll 1
                for (int c = 0; c < HD / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld_32x32b_x32(tO + c * 32, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                    tmem_st_32x32b_x32(tO + c * 32, r);
                }
            }
            l *= alpha;

            // P = exp2(S * scale_log2 - m) on packed f32 pairs, rounded to 16 bit, written over S (every score has
            // been read by now, so P can land anywhere in the S columns).
            const float neg_m = (m_used == -INFINITY) ? 0.0f : -m_used;   // a fully masked row keeps P = 0
            uint64_t sum2 = 0;                                            // two partial row sums (f32x2)
            uint32_t pk[32];
            exp_chunk_mixed<BF16, PE>(s0, sc, neg_m, sum2, pk);
            exp_chunk_mixed<BF16, PE>(s1, sc, neg_m, sum2, pk + 16);
            tmem_st_32x32b_x32(tS, pk);
            exp_chunk_mixed<BF16, PE>(s2, sc, neg_m, sum2, pk);
            if constexpr (P_HALVES) {
                tmem_wait_st();                  // the first store has long landed: publish the first 64 keys of P
                tc_fence_before();
                mbar_arrive(bar_phalf + 8 * t);
            }
            exp_chunk_mixed<BF16, PE>(s3, sc, neg_m, sum2, pk + 16);
            tmem_st_32x32b_x32(tS + 32, pk);
            l += lo_f32(sum2) + hi_f32(sum2);
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(bar_pfull + 8 * t);
            return true;
        };
        // Under a softcap the blocks above the causal diagonal are not skipped: every score there is -inf before the cap
        // and -cap after it (the reference applies tanh last), whatever Q K^T and the mask say.  Such a block needs no
        // read of S and one exponential per row: P is the same value in all 128 columns.
        auto capped_block = [&](int j) -> bool {
            ok = mbar_wait(bar_sfull + 8 * t, (cum + j) & 1, abort_flag, p.kerr, KERR_SDPA_SOFTMAX_WAIT, j);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) return false;
            tc_fence_after();
            const float capped = -p.softcap * LOG2E;
            const float m_new = fmaxf(m_used, capped);
            float alpha = 1.0f;
            bool need = false;
            if (m_new > m_used + RESCALE_THRESHOLD) {
                alpha = fast_exp2(m_used - m_new);
                m_used = m_new;
                need = true;
            }
            if (j > 0 && __any_sync(0xffffffffu, need)) {
                ok = mbar_wait(bar_pvdone + 8 * t, (cum + j - 1) & 1, abort_flag, p.kerr, KERR_SDPA_SOFTMAX_WAIT, 100000 + j);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) return false;
                tc_fence_after();
#pragma unroll 1
                for (int c = 0; c < HD / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld_32x32b_x32(tO + c * 32, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                    tmem_st_32x32b_x32(tO + c * 32, r);
                }
            }
            const float e = fast_exp2(capped - m_used);
            l = l * alpha + float(BKV) * e;
            uint32_t pe;
            if constexpr (BF16) {
                __nv_bfloat162 h = __floats2bfloat162_rn(e, e);
                pe = *reinterpret_cast<uint32_t*>(&h);
            } else {
                __half2 h = __floats2half2_rn(e, e);
                pe = *reinterpret_cast<uint32_t*>(&h);
            }
            uint32_t pk[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) pk[i] = pe;
            tmem_st_32x32b_x32(tS, pk);
            tmem_st_32x32b_x32(tS + 32, pk);
            tmem_wait_st();
            tc_fence_before();
            if constexpr (P_HALVES) mbar_arrive(bar_phalf + 8 * t);
            mbar_arrive(bar_pfull + 8 * t);
            return true;
        };
        // Leading blocks that a key-padding mask leaves alone (all of them but the last one or two, usually) take the plain
        // form: the lanes scan eight blocks at a time, four mask values each, until the first block that changes anything.
        int j_plain = FORM == 0 ? nblk : 0;
        if (FORM == 1 && p.mask_strides[2] == 0 && p.mask_vec != 0) {
            const char* row = mask_row_of();
            j_plain = nblk;
            for (int jb = 0; jb < nblk && j_plain == nblk; jb += 8) {
                uint4 v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    v[u] = jb + u < nblk ? scan_fetch(row, jb + u) : (p.mask_bool ? make_uint4(0x01010101u, 0u, 0u, 0u) : make_uint4(0u, 0u, 0u, 0u));
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const bool any = p.mask_bool ? __vcmpeq4(v[u].x, 0u) != 0u : (v[u].x | v[u].y | v[u].z | v[u].w) != 0u;
                    if (__any_sync(0xffffffffu, any)) j_plain = min(j_plain, jb + u);
                }
            }
        }
        for (int j = 0; j < j_plain && ok; ++j) ok = block(std::false_type{}, j);
        if constexpr (GENERAL) {
            if (j_plain < nblk) {
                mask_row = mask_row_of();
                mask_shared = FORM == 1 && mask_row != nullptr && p.mask_strides[2] == 0 && p.mask_vec != 0;
                if (mask_shared) scan_next = scan_fetch(mask_row, j_plain);
            }
            // first key block that lies entirely above the causal diagonal of this tile and is whole (softcap form only)
            int j_capped = nblk;
            if (FORM == 2 && p.causal) j_capped = min(nblk, max(0, (q0 + t * BQ + BQ - 1 + p.causal_offset) / BKV + 1));
            for (int j = j_plain; j < nblk && ok; ++j)
                ok = (j >= j_capped && (j + 1) * BKV <= p.Sk) ? capped_block(j) : block(std::true_type{}, j);
        }

        // epilogue: O / l -> global
        if (ok && nblk > 0) {
            ok = mbar_wait(bar_pvdone + 8 * t, (cum + nblk - 1) & 1, abort_flag, p.kerr, KERR_SDPA_SOFTMAX_WAIT, 200000);
            ok = __all_sync(0xffffffffu, ok);
        }
        if (ok && nblk > 0) {
            tc_fence_after();
            const float inv = l > 0.0f ? 1.0f / l : __int_as_float(0x7fc00000);
            const bool in_range = qrow < p.Sq;
            if (p.tma_o) {
                // Head-sharded delivery: the normalised tile goes to the staging tile in the layout of a 128-byte-swizzled
                // tile store (two boxes of 64 columns for 128-wide heads); warp 10 then issues one store per destination
                // while these warps move on to their next item.  The staging tile serves both query tiles in turn:
                // use u = uses of earlier items + (tile 1 after a tile 0 that had work).
                const uint32_t u = stage_uses + ((t == 1 && w.nblk[0] > 0) ? 1u : 0u);
                ok = counter_wait_ge(stage_freed, u, abort_flag, p.kerr, KERR_SDPA_SOFTMAX_WAIT, 900000 + n);
                ok = __all_sync(0xffffffffu, ok);
                if (ok) {
    #pragma unroll 1
                    for (int c = 0; c < HD / 32; ++c) {
                        uint32_t r[32];
                        tmem_ld_32x32b_x32(tO + c * 32, r);
                        tmem_wait_ld();
                        uint32_t pk[16];
    #pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const float a = __uint_as_float(r[2 * i]) * inv, b = __uint_as_float(r[2 * i + 1]) * inv;
                            if constexpr (BF16) {
                                __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
                                pk[i] = *reinterpret_cast<uint32_t*>(&h);
                            } else {
                                __half2 h = __floats2half2_rn(a, b);
                                pk[i] = *reinterpret_cast<uint32_t*>(&h);
                            }
                        }
                        uint8_t* box = stageO + (c >> 1) * HALF_BYTES + row_in_tile * 128;     // 64-column box c / 2, this thread's row
    #pragma unroll
                        for (int i = 0; i < 4; ++i)
                            *reinterpret_cast<uint4*>(box + ((((c & 1) * 4 + i) ^ (row_in_tile & 7)) << 4)) = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
                    }
                    tc_fence_before();
                    fence_proxy_async_smem();           // the staged rows become visible to the copy engine
                    mbar_arrive(bar_ostage_full);
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_ofree + 8 * t);   // O_t is in shared memory now: the next item may overwrite it
                }
            } else {   // every thread stores its own row directly
                const int64_t off = batch * p.o_strides[0] + head * p.o_strides[1] + (int64_t)qrow * p.o_strides[2];
    #pragma unroll 1
                for (int c = 0; c < HD / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld_32x32b_x32(tO + c * 32, r);
                    tmem_wait_ld();
                    uint32_t pk[16];
    #pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float a = __uint_as_float(r[2 * i]) * inv, b = __uint_as_float(r[2 * i + 1]) * inv;
                        if constexpr (BF16) {
                            __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
                            pk[i] = *reinterpret_cast<uint32_t*>(&h);
                        } else {
                            __half2 h = __floats2half2_rn(a, b);
                            pk[i] = *reinterpret_cast<uint32_t*>(&h);
                        }
                    }
                    if (in_range) {
                        uint16_t* dst = reinterpret_cast<uint16_t*>(p.O) + off + c * 32;
    #pragma unroll
                        for (int i = 0; i < 4; ++i)
                            reinterpret_cast<uint4*>(dst)[i] = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_ofree + 8 * t);
            }
            if (p.lse && in_range)
                p.lse[((int64_t)batch * p.Hq + head) * p.Sq + qrow] = (l > 0.0f) ? (m_used + log2f(l)) * 0.6931471805599453f : -INFINITY;
        }
        stage_uses += (w.nblk[0] > 0 ? 1u : 0u) + (w.nblk[1] > 0 ? 1u : 0u);
        cum += nblk;
      }
    }

    if (*abort_flag) __nanosleep(2000000);
    tc_fence_before();
    __syncthreads();
    if (warp == 10) tmem_dealloc(tmem_base, TMEM_COLS);
}

typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// [B, H, S, D] tensor with element strides (batch, head, row); box = 64 columns x 128 rows.
mk_status encode_bhsd(CUtensorMap* map, int dtype, const void* base, int B, int H, int S, int D, const int64_t* strides) {
    static PFN_encodeTiled encode = (PFN_encodeTiled)driver_entry("cuTensorMapEncodeTiled");
    if (!encode) return fail(MK_ERR_CUDA, "cuTensorMapEncodeTiled is unavailable (driver too old?)");
    cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)S, (cuuint64_t)H, (cuuint64_t)B};
    cuuint64_t str[3] = {(cuuint64_t)strides[2] * 2, (cuuint64_t)strides[1] * 2, (cuuint64_t)strides[0] * 2};
    cuuint32_t box[4] = {64, 128, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = encode(map, dtype == MK_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                        const_cast<void*>(base), dims, str, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(MK_ERR_CUDA, "cuTensorMapEncodeTiled (attention operand) failed with %d", (int)r);
    return MK_OK;
}

bool strides_ok(const int64_t* s, int D) { return s[0] % 8 == 0 && s[1] % 8 == 0 && s[2] % 8 == 0 && s[2] >= D; }

}  // namespace

// Runs the tensor-core kernel when the problem qualifies; otherwise leaves *handled = false and
// the caller uses the general kernel.
mk_status sdpa_sm100(mk_device* dev, cudaStream_t st, const mk_sdpa_desc& d, float scale, bool* handled) {
    *handled = false;
    if (dev->prop.major != 10) return MK_OK;
    if (d.dtype != MK_BF16 && d.dtype != MK_F16) return MK_OK;
    // Head sizes: the kernel is built for 64 and 128 columns; any head size that is a multiple of 8 (16-byte rows) up to 128
    // runs on the next larger one -- the tile loads zero-fill the columns past D (zero products in Q K^T, zero
    // columns of O) and the stores of O drop them.
    if (d.D != d.Dv || d.D % 8 != 0 || d.D < 8 || (d.D > 128 && d.D != 256)) return MK_OK;
    const int HDk = d.D <= 64 ? 64 : (d.D <= 128 ? 128 : 256);
    // 256-wide heads: no room for an output staging tile, so no peers and no padded head sizes there
    if (HDk == 256 && d.n_peers > 0) return MK_OK;
    if (d.Sk <= 0 || d.Sq <= 0) return MK_OK;
    if (d.causal && d.causal_offset < 0) return MK_OK;   // rows without any visible key (NaN rows) are the general kernel's business
    if (!strides_ok(d.q_strides, d.D) || !strides_ok(d.k_strides, d.D) || !strides_ok(d.v_strides, d.D)) return MK_OK;
    if (d.o_strides[0] % 8 || d.o_strides[1] % 8 || d.o_strides[2] % 8) return MK_OK;
    if ((reinterpret_cast<uintptr_t>(d.Q) | reinterpret_cast<uintptr_t>(d.K) | reinterpret_cast<uintptr_t>(d.V) |
         reinterpret_cast<uintptr_t>(d.O)) & 15)
        return MK_OK;
    for (int i = 0; i < d.n_peers; ++i)
        if (reinterpret_cast<uintptr_t>(d.peer_O[i]) & 15) return MK_OK;
    const int tiles = HDk == 256 ? 1 : 2;
    const int64_t q_pairs = (d.Sq + tiles * BQ - 1) / (tiles * BQ);
    const int64_t items = q_pairs * d.B * d.Hq;
    if (items > 0x7fffffffll) return MK_OK;
    const int64_t grid = items < dev->prop.multiProcessorCount ? items : dev->prop.multiProcessorCount;

    alignas(64) CUtensorMap tq, tk, tv;
    mk_status s1 = encode_bhsd(&tq, d.dtype, d.Q, d.B, d.Hq, d.Sq, d.D, d.q_strides);
    if (s1 != MK_OK) return s1;
    s1 = encode_bhsd(&tk, d.dtype, d.K, d.B, d.Hkv, d.Sk, d.D, d.k_strides);
    if (s1 != MK_OK) return s1;
    s1 = encode_bhsd(&tv, d.dtype, d.V, d.B, d.Hkv, d.Sk, d.D, d.v_strides);
    if (s1 != MK_OK) return s1;

    FaParams p{};
    p.B = d.B; p.Hq = d.Hq; p.Hkv = d.Hkv; p.Sq = d.Sq; p.Sk = d.Sk;
    p.causal = d.causal ? 1 : 0;
    p.causal_offset = d.causal ? d.causal_offset : 0;
    p.scale_log2 = scale * LOG2E;
    p.scale = scale;
    p.softcap = d.softcap > 0.0f ? d.softcap : 0.0f;
    p.mask = d.mask;
    p.mask_bool = d.mask_kind == MK_MASK_BOOL ? 1 : 0;
    if (d.mask_kind == MK_MASK_SQ_SK) {
        p.mask_strides[0] = p.mask_strides[1] = 0;
        p.mask_strides[2] = d.Sk;
    } else {
        for (int i = 0; i < 3; ++i) p.mask_strides[i] = d.mask_strides[i];
    }
    {   // rows may be read 16 bytes at a time when every row starts on a 16-byte boundary
        const int64_t per16 = p.mask_bool ? 16 : 4;
        p.mask_vec = d.mask && (reinterpret_cast<uintptr_t>(d.mask) & 15) == 0 && p.mask_strides[0] % per16 == 0 &&
                     p.mask_strides[1] % per16 == 0 && p.mask_strides[2] % per16 == 0;
    }
    const int form = p.softcap > 0.0f ? 2 : (d.mask != nullptr ? 1 : 0);
    const bool general = form != 0;
    p.O = d.O;
    p.lse = d.lse;
    for (int i = 0; i < 3; ++i) p.o_strides[i] = d.o_strides[i];
    const uint32_t fmt = d.dtype == MK_BF16 ? 1u : 0u;
    p.idesc_qk = idesc_f16(fmt, 0u, 0u, BQ, BKV);
    p.idesc_pv = idesc_f16(fmt, 0u, 1u, BQ, (uint32_t)HDk);
    p.q_pairs = (int)q_pairs;
    p.tiles = tiles;
    // Peers receive their copies as tile stores issued from a staging tile; without peers every thread stores its
    // own row (MOROK_B200_ATTN_TMA_O forces the staged form for measurements).
    // ... and for head sizes the kernel pads to 64 / 128 columns: the tile store drops the padding columns
    // ... and for 128-wide heads with long key ranges, where a work item lasts long enough for the one staging tile not
    // to be contended: the staged tile leaves through the copy engine in 128-byte rows, while row-per-thread stores
    // cost the softmax warps ~3000 cycles per tile (measured: +1.5 % causal and +2 % non-causal at S = 4096, +1 % at
    // 8192; -2 % at S = 2048 and -11 % at 1024, -2 % for 64-wide heads -- hence the rule).  MOROK_B200_ATTN_TMA_O=1 / 0
    // forces the staged / the direct form where both are possible.
    p.tma_o = d.n_peers > 0 || d.D != HDk || (HDk == 128 && d.Sk >= 4096);
    if (const char* e = getenv("MOROK_B200_ATTN_TMA_O")) {
        if (atoi(e) != 0 && HDk != 256) p.tma_o = 1;
        else if (d.n_peers == 0 && d.D == HDk) p.tma_o = 0;
    }
    alignas(64) OStoreMaps omaps{};
    if (p.tma_o) {
        const bool optional = d.n_peers == 0 && d.D == HDk;     // the staged form is a choice here, not a need
        for (int i = 0; i <= d.n_peers; ++i) {
            s1 = encode_bhsd(&omaps.m[i], d.dtype, i == 0 ? d.O : d.peer_O[i - 1], d.B, d.Hq, d.Sq, d.Dv, d.o_strides);
            if (s1 != MK_OK && optional) {       // an output layout the tile store cannot describe: direct stores take any
                p.tma_o = 0;
                break;
            }
            if (s1 != MK_OK) return s1;
        }
    }
    p.n_peers = d.n_peers;
    for (int i = 0; i < d.n_peers; ++i) p.peer_O[i] = d.peer_O[i];
    p.kerr = stream_kerr(dev, st);
    // The claim counter of this stream, zeroed in stream order before the launch.  Launches on one stream
    // run one after the other; other streams -- and recorded plans, which keep their capture stream for
    // life -- have counters of their own, so concurrent kernels never consume each other's claims.
    p.work_counter = stream_work_counter(dev, st);
    MK_CUDA(cudaMemsetAsync(p.work_counter, 0, sizeof(unsigned int), st));

    auto launch = [&](auto kernel, int smem_bytes) -> cudaError_t {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
        if (e != cudaSuccess) return e;
        // the register increase of the softmax warpgroups is only satisfiable if the kernel starts with REGS_LAUNCH
        // registers per thread: checked here, never assumed
        cudaFuncAttributes fa{};
        e = cudaFuncGetAttributes(&fa, kernel);
        if (e != cudaSuccess) return e;
        if (fa.numRegs < REGS_LAUNCH) return cudaErrorLaunchOutOfResources;
        kernel<<<(unsigned)grid, NUM_THREADS, smem_bytes, st>>>(tq, tk, tv, p, omaps);
        return cudaSuccess;
    };
    const bool bf = d.dtype == MK_BF16;
    const int smem128 = Cfg<128>::SMEM_BYTES + (p.tma_o ? Cfg<128>::TILE_BYTES : 0), smem64 = Cfg<64>::SMEM_BYTES + (p.tma_o ? Cfg<64>::TILE_BYTES : 0);
#define MK_FA(BF, HD_, FORM_, SMEM) MK_CUDA(launch(sdpa_tc_kernel<BF, HD_, FORM_>, SMEM))
#define MK_FA_FORMS(BF, HD_, SMEM)                          \
    do {                                                    \
        if (form == 2) MK_FA(BF, HD_, 2, SMEM);             \
        else if (form == 1) MK_FA(BF, HD_, 1, SMEM);        \
        else MK_FA(BF, HD_, 0, SMEM);                       \
    } while (0)
    if (HDk == 256) {
        if (bf) MK_FA_FORMS(true, 256, Cfg<256>::SMEM_BYTES); else MK_FA_FORMS(false, 256, Cfg<256>::SMEM_BYTES);
    } else if (HDk == 128) {
        if (bf) MK_FA_FORMS(true, 128, smem128); else MK_FA_FORMS(false, 128, smem128);
    } else {
        if (bf) MK_FA_FORMS(true, 64, smem64); else MK_FA_FORMS(false, 64, smem64);
    }
#undef MK_FA_FORMS
#undef MK_FA
    MK_CUDA(cudaGetLastError());
    note_launch(dev, st, HDk == 256 ? (general ? "sdpa_tc_d256_general" : "sdpa_tc_d256")
                         : HDk == 128 ? (general ? "sdpa_tc_d128_general" : "sdpa_tc_d128") : (general ? "sdpa_tc_d64_general" : "sdpa_tc_d64"));
    *handled = true;
    return MK_OK;
}

}  // namespace mk
