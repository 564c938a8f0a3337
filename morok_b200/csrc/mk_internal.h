// Internal declarations shared by the host runtime and the kernel launchers of libmorok_b200.
#pragma once

#include <cuda_runtime.h>

#include <array>
#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <list>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/morok_b200.h"

namespace mk {

// ---- thread-local error message --------------------------------------------------------------
void set_error(const char* fmt, ...) __attribute__((format(printf, 1, 2)));
mk_status fail(mk_status code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));
mk_status cuda_fail(cudaError_t e, const char* what);

#define MK_CUDA(expr)                                           \
    do {                                                        \
        cudaError_t _e = (expr);                                \
        if (_e != cudaSuccess) return ::mk::cuda_fail(_e, #expr); \
    } while (0)

#define MK_REQUIRE(cond, ...)                                   \
    do {                                                        \
        if (!(cond)) return ::mk::fail(MK_ERR_INVALID, __VA_ARGS__); \
    } while (0)

inline bool dtype_is_fp8(int32_t dt) { return dt == MK_F8E4M3 || dt == MK_F8E5M2; }
inline size_t dtype_size(int32_t dt) { return dt == MK_F32 ? 4 : (dtype_is_fp8(dt) || dt == MK_BOOL) ? 1 : 2; }
// The types every operation computes in; the 8-bit floats are storage types that only mk_gemm (as
// inputs) and mk_cast accept.
inline bool dtype_valid(int32_t dt) { return dt == MK_F32 || dt == MK_BF16 || dt == MK_F16; }

// ---- device-side error word --------------------------------------------------------------------
// Kernels that wait on barriers record (code, block, detail) here instead of trapping.
struct KernelError {
    unsigned int code;     // 0 = none
    unsigned int block;
    unsigned int detail;
    unsigned int pad;
};

enum : unsigned int {
    KERR_NONE = 0,
    KERR_GEMM_PRODUCER_WAIT = 0x101,
    KERR_GEMM_MMA_WAIT = 0x102,
    KERR_GEMM_EPILOGUE_WAIT = 0x103,
    KERR_SDPA_PRODUCER_WAIT = 0x201,
    KERR_SDPA_MMA_WAIT = 0x202,
    KERR_SDPA_SOFTMAX_WAIT = 0x203,
    KERR_SDPA_STORE_WAIT = 0x204,
    KERR_SKINNY_PRODUCER_WAIT = 0x301,
    KERR_SKINNY_CONSUMER_WAIT = 0x302,
    KERR_SKINNY_REDUCE_WAIT = 0x303,
    KERR_SELFTEST_WAIT = 0x901,
};

}  // namespace mk

// ---- opaque handle definitions -------------------------------------------------------------------
namespace mk {
// An event recorded on one stream when a block went back to the allocator cache; shared by every block
// parked since the stream last received work.
struct StreamFence {
    cudaStream_t stream = nullptr;
    cudaEvent_t event = nullptr;
    ~StreamFence() {
        if (event) cudaEventDestroy(event);
    }
};
// What the library keeps per CUDA stream it has enqueued work on.  `slot` indexes the device arrays of
// kernel error words and claim counters, so that launches on different streams (and recorded plans, which
// own their capture stream for life) never share either.
struct StreamState {
    int slot = 0;                          // 0 is also the shared fallback when every slot is taken
    void* scratch = nullptr;               // two-launch kernels (K-split GEMM, key-split attention): grown on demand
    size_t scratch_bytes = 0;
    bool dirty = false;                    // work was enqueued since the last fence
    bool plan = false;                     // capture stream of a recorded plan
    std::shared_ptr<StreamFence> fence;    // completes when everything enqueued before the last release has run
};
}  // namespace mk

struct mk_device {
    int ordinal = 0;
    bool mock = false;  // host-memory stand-in for allocator / copy tests; cannot run kernels
    cudaDeviceProp prop{};
    std::mutex mu;  // guards the allocator state, the stream table and the tuning records below
    // LRU free lists keyed by allocation size; each list newest-first, at most kMaxPerKey entries.  A parked
    // block carries the fences of the streams that may still be using it (stream-ordered reuse).
    struct Parked {
        void* ptr;
        std::vector<std::shared_ptr<mk::StreamFence>> fences;
    };
    std::map<size_t, std::list<Parked>> free_lists;
    mk_alloc_stats_t stats{};
    int inject_oom = 0;
    // per-stream slots (device memory): kernel error words and the claim counters of persistent kernels
    static constexpr int kStreamSlots = 256;
    mk::KernelError* kerr_words = nullptr;      // [kStreamSlots]
    unsigned int* work_counters = nullptr;      // [kStreamSlots], one zeroed (in stream order) per launch
    std::map<cudaStream_t, mk::StreamState> streams;
    std::vector<int> free_slots;                // slots 1 .. kStreamSlots-1 not in use
    std::vector<void*> retired_scratch;   // outgrown blocks: work already enqueued (or recorded in a plan) may still use them
    // schedule choices found by mk_gemm_autotune (or loaded from a file), keyed by the problem; guarded by mu
    std::map<std::array<int64_t, 9>, mk_gemm_tuning> gemm_tunes;
    // kernels launched through this device (all entry points)
    std::atomic<uint64_t> launches{0};
    static constexpr size_t kMaxPerKey = 32;
};

struct mk_stream {
    mk_device* dev;
    cudaStream_t s;
};

struct mk_event {
    mk_device* dev;
    cudaEvent_t e;
    bool recorded;
};

// Allocation shared by a buffer and its views.
struct BufData {
    mk_device* dev = nullptr;
    size_t bytes = 0;
    uint32_t flags = 0;
    std::mutex mu;
    void* ptr = nullptr;     // null until first use (lazy)
    bool ipc_mapped = false; // opened from a peer's handle: unmap instead of caching
    ~BufData();
};

struct mk_buf {
    std::shared_ptr<BufData> data;
    size_t offset = 0;
    size_t bytes = 0;
};

namespace mk {

inline cudaStream_t raw(mk_stream* s) { return s ? s->s : (cudaStream_t)0; }

mk_status device_alloc(mk_device* dev, size_t bytes, uint32_t flags, void** out);
void device_release(mk_device* dev, void* ptr, size_t bytes);
mk_status buf_ptr(mk_buf* b, void** out);

// Descriptor rules shared by mk_gemm and mk_gemm_static (dispatch.cpp).
mk_status validate_gemm_desc(mk_gemm_desc& d, const char* who, bool* nothing_to_do);

// kernel launchers implemented in the .cu files
mk_status gemm_simt(mk_device* dev, cudaStream_t st, const mk_gemm_desc& d);
mk_status gemm_sm100(mk_device* dev, cudaStream_t st, const mk_gemm_desc& d, bool* handled);
mk_status gemm_skinny(mk_device* dev, cudaStream_t st, const mk_gemm_desc& d, bool* handled, bool dry_run = false);
mk_status sdpa_simt(mk_device* dev, cudaStream_t st, const mk_sdpa_desc& d, float scale);
mk_status sdpa_sm100(mk_device* dev, cudaStream_t st, const mk_sdpa_desc& d, float scale, bool* handled);
mk_status sdpa_decode(mk_device* dev, cudaStream_t st, const mk_sdpa_desc& d, float scale, bool* handled);
// The tuning record of this problem: the one mk_gemm_autotune is trying on this thread, else the stored one.
bool gemm_tuning_for(mk_device* dev, const mk_gemm_desc& d, mk_gemm_tuning* out);
// Counts one kernel launch and, while the calling thread records a profile of this stream, stamps an event
// behind it; `name` must be a string literal.
void note_launch(mk_device* dev, cudaStream_t st, const char* name);
// At least `bytes` of device memory that belongs to work enqueued on `st` (valid until the next call for the same stream).
mk_status stream_scratch(mk_device* dev, cudaStream_t st, size_t bytes, void** out);
// The error word and the claim counter of the stream's slot (device pointers).
KernelError* stream_kerr(mk_device* dev, cudaStream_t st);
unsigned int* stream_work_counter(mk_device* dev, cudaStream_t st);
// Marks the stream as carrying work the allocator must order block reuse after (launches do this through
// note_launch; copies and memsets call it directly).
void touch_stream(mk_device* dev, cudaStream_t st);
// Marks the stream as the capture stream of a recorded plan (its error word is reported by every status query).
void mark_plan_stream(mk_device* dev, cudaStream_t st);
// Drops everything kept for a stream that is about to be destroyed: scratch block (cudaFree waits for work
// that still uses it), slot, fence.
void release_stream_state(mk_device* dev, cudaStream_t st);
// While alive, allocations made by the calling thread are ordered on `st`: a cached block that another
// stream may still be using makes `st` wait for that stream's fence instead of blocking the host, and
// zero-initialisation runs on `st`.
struct AllocStreamScope {
    explicit AllocStreamScope(cudaStream_t st);
    ~AllocStreamScope();
    bool prev_set;
    cudaStream_t prev;
};

mk_status ew_silu(mk_device* dev, cudaStream_t s, int32_t dtype, const void* x, void* y, int64_t n);
mk_status ew_sigmoid(mk_device* dev, cudaStream_t s, int32_t dtype, const void* x, void* y, int64_t n);
mk_status ew_glu(mk_device* dev, cudaStream_t s, int32_t dtype, const void* gate, const void* value, void* y, int64_t n);
mk_status ew_mul(mk_device* dev, cudaStream_t s, int32_t dtype, const void* a, const void* b, void* y, int64_t n);
mk_status ew_binary_bcast(mk_device* dev, cudaStream_t s, int32_t dtype, int is_mul, const void* a, const void* b, void* y, int64_t n,
                          int64_t nb);
mk_status strided_copy(mk_device* dev, cudaStream_t s, int elem_size, const void* src, void* dst, int ndim, const int64_t* shape,
                       const int64_t* strides);

// cuTensorMapEncodeTiled fetched through the runtime (the library does not link libcuda).
void* driver_entry(const char* name);
// A 2-D tiled tensor map (CUtensorMap behind `map`) of 16- or 8-bit elements with the 128-byte swizzle.
mk_status tma_encode_2d(void* map, int dtype, const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                        uint32_t box_inner, uint32_t box_outer);

#ifdef __CUDACC__
// Kernels that work in two launches (partials, then a merge) chain the second launch programmatically: the
// merge grid may become resident while the first grid still runs (which calls grid_launch_dependents()
// early) and blocks in grid_dependency_wait() until that grid has completed and its writes are visible.
// This takes the launch latency of the merge off the critical path; both instructions do nothing in a
// kernel launched the ordinary way.  MOROK_B200_PDL=0 launches the merge the ordinary way.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

bool dependent_launch_enabled();
template <typename P>
cudaError_t launch_dependent(void (*kern)(const P), dim3 grid, dim3 block, cudaStream_t st, const P& params) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dependent_launch_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, params);
}
#endif

}  // namespace mk
