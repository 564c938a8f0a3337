/*
 * morok_b200.h -- C ABI of libmorok_b200: a B200 (sm_100a) device for morok's dense hot path.
 *
 * This is the boundary a morok `Device` for `DeviceSpec::Cuda` binds to: allocator, buffers,
 * copies, streams/events, module load + launch, and the hand-written kernels that replace the
 * code morok would otherwise generate for matmul and scaled-dot-product attention.
 *
 * Conventions
 *   - Every function returns an mk_status (0 = MK_OK, negative = error).  No exceptions cross the
 *     boundary and nothing aborts; mk_last_error() returns a thread-local message for the last
 *     failing call on the calling thread (the reference reports errors as snafu enums,
 *     device/src/error.rs:5-51).
 *   - Plain pointers and sizes only.  The caller owns all host memory; the library owns device
 *     memory from mk_alloc until mk_free.
 *   - Handles may be used from any thread; one stream is one ordered queue; the allocator is
 *     internally locked (the reference shares kernels and allocators across threads:
 *     runtime/src/kernel_cache.rs:26-49, device/src/allocator.rs:72-112).
 *   - There is no CPU fallback: without a CUDA device every compute entry point fails with
 *     MK_ERR_CUDA.
 *   - Paths in comments ("device/src/...") are relative to the reference project's root.
 */
#ifndef MOROK_B200_H
#define MOROK_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define MK_API
#else
#define MK_API __attribute__((visibility("default")))
#endif

typedef int32_t mk_status;

enum {
    MK_OK = 0,
    MK_ERR_INVALID = -1,        /* bad argument (null handle, negative size, unsupported combination) */
    MK_ERR_CUDA = -2,           /* a CUDA call failed; message carries cudaGetErrorString            */
    MK_ERR_OOM = -3,            /* allocation failed even after the cache was flushed                */
    MK_ERR_SIZE_MISMATCH = -4,  /* copy size != buffer size (device/src/error.rs SizeMismatch)       */
    MK_ERR_NOT_ALLOCATED = -5,  /* operation needs an allocated buffer                               */
    MK_ERR_TIMEOUT = -6,        /* bounded wait ran out                                              */
    MK_ERR_UNSUPPORTED = -7,    /* dtype / layout the kernels do not cover                           */
    MK_ERR_KERNEL = -8          /* a kernel reported a device-side error word (e.g. a pipeline wait
                                   gave up); the CUDA context stays usable                           */
};

/* Element types of the dense path (dtype/src/lib.rs:145 ScalarDType::{Float32,BFloat16,Float16}).
 * MK_F8E4M3 / MK_F8E5M2 (dtype/src/lib.rs:142-143, 234-256: finite range +-448 / +-57344) are storage
 * types: inputs of mk_gemm (f32 accumulation, f32 / bf16 / f16 output) and either side of mk_cast. */
typedef enum { MK_F32 = 0, MK_BF16 = 1, MK_F16 = 2, MK_F8E4M3 = 3, MK_F8E5M2 = 4,
               MK_BOOL = 5 /* one byte per element; tensors of this type are attention masks only (DType::Bool) */ } mk_dtype;

typedef struct mk_device mk_device;
typedef struct mk_stream mk_stream;
typedef struct mk_buf mk_buf;
typedef struct mk_event mk_event;
typedef struct mk_module mk_module;
typedef struct mk_function mk_function;

MK_API const char* mk_last_error(void);
MK_API int32_t mk_abi_version(void);
/* sizeof of a descriptor struct as this library was compiled (0 = mk_gemm_desc, 1 = mk_sdpa_desc),
 * for bindings that mirror the structs by hand; -1 for an unknown index. */
MK_API int32_t mk_abi_struct_size(int32_t which);

/* ---------------------------------------------------------------------------------------------
 * Device  (replaces the commented-out CUDA factory of runtime/src/device_registry.rs:66-67 and
 * `CudaAllocator::new(device_id)` of device/src/allocator.rs:256-275)
 * ------------------------------------------------------------------------------------------- */
typedef struct {
    int32_t ordinal;
    int32_t sm_count;
    int32_t cc_major, cc_minor;
    int32_t max_smem_per_block;   /* opt-in dynamic shared memory limit, bytes */
    int32_t l2_bytes;
    int64_t total_mem;
    char name[128];
} mk_device_info;

MK_API mk_status mk_device_count(int32_t* count);
MK_API mk_status mk_device_open(int32_t ordinal, mk_device** out);
/* Test fake (the reference's tests use fakes such as MockKernel, runtime/src/benchmark.rs:150-168):
 * a device whose "HBM" is host memory, so that the allocator policy, views, size checks and
 * copies can be exercised on a machine without a GPU.  It cannot create streams or run any
 * kernel: every compute entry point fails on it with MK_ERR_CUDA. */
MK_API mk_status mk_device_open_mock(mk_device** out);
MK_API mk_status mk_device_close(mk_device* dev);
MK_API mk_status mk_device_get_info(mk_device* dev, mk_device_info* info);
/* Allocator::synchronize (device/src/allocator.rs:186): waits for all work on the device. */
MK_API mk_status mk_device_sync(mk_device* dev);

/* ---------------------------------------------------------------------------------------------
 * Streams and events  (HardwareQueue wait/signal/submit: device/src/queue.rs:83-133;
 * CudaTimelineSignal record / bounded wait: device/src/sync.rs:185-310)
 * A NULL mk_stream* anywhere below means the device's default stream.
 * ------------------------------------------------------------------------------------------- */
MK_API mk_status mk_stream_create(mk_device* dev, mk_stream** out);
MK_API mk_status mk_stream_destroy(mk_stream* s);
MK_API mk_status mk_stream_sync(mk_stream* s);
MK_API mk_status mk_stream_wait_event(mk_stream* s, mk_event* ev);
/* Raw cudaStream_t of a stream (for callers that interoperate with other CUDA libraries). */
MK_API mk_status mk_stream_raw(mk_stream* s, void** cuda_stream);

MK_API mk_status mk_event_create(mk_device* dev, mk_event** out);
MK_API mk_status mk_event_destroy(mk_event* ev);
MK_API mk_status mk_event_record(mk_event* ev, mk_stream* s);
/* TimelineSignal::wait(value, timeout_ms) (device/src/sync.rs:248-306): polls, never blocks
 * without bound.  Returns MK_ERR_TIMEOUT when the event has not completed in time. */
MK_API mk_status mk_event_wait(mk_event* ev, int32_t timeout_ms);
MK_API mk_status mk_event_elapsed_ms(mk_event* start, mk_event* stop, float* ms);

/* ---------------------------------------------------------------------------------------------
 * HBM allocator with lazy allocation and LRU reuse
 *   Allocator::alloc/free (device/src/allocator.rs:164-190), CudaAllocator::alloc
 *   (device/src/allocator.rs:276-296), LruAllocator: free lists keyed by size, at most 32 cached
 *   buffers per key, flush-and-retry on out-of-memory (device/src/allocator.rs:322-442),
 *   lazy OnceLock allocation on first use (device/src/buffer.rs:58-73),
 *   views sharing the allocation (device/src/buffer.rs:136-150).
 * ------------------------------------------------------------------------------------------- */
enum { MK_ALLOC_ZERO_INIT = 1u };   /* BufferOptions::zero_init */

typedef struct {
    uint64_t device_allocs;     /* cudaMalloc calls that succeeded           */
    uint64_t device_frees;      /* cudaFree calls                            */
    uint64_t cache_hits;        /* allocations served from the free lists    */
    uint64_t cache_returns;     /* frees parked in the free lists            */
    uint64_t oom_flushes;       /* times the cache was flushed to retry      */
    uint64_t bytes_in_use;      /* handed out and not yet freed              */
    uint64_t bytes_cached;      /* parked in the free lists                  */
    uint64_t peak_bytes_in_use;
} mk_alloc_stats_t;

/* Reuse is stream-ordered.  The reference issues every CUDA call on one stream and leaves ordering to its
 * scheduler (device/src/allocator.rs:72-112); here kernels run on several non-blocking streams, so a block
 * that goes back to the cache remembers, for every stream of this device that had work enqueued through the
 * library, an event behind that work, and the caller that takes the block out of the cache waits for those
 * events first (usually they completed long ago).  mk_free therefore never needs a preceding sync -- as long
 * as the work that uses the buffer was enqueued through this library (mk_launch included) before the free.
 * MK_ALLOC_ZERO_INIT zeros are in place when the allocating call returns.
 *
 * Creates a lazy buffer: no device memory is reserved until the first mk_buf_ptr /
 * mk_buf_ensure / copy.  size may be 0. */
MK_API mk_status mk_alloc(mk_device* dev, size_t bytes, uint32_t flags, mk_buf** out);
/* Forces allocation (BufferData::ensure_allocated). */
MK_API mk_status mk_buf_ensure(mk_buf* buf);
/* Buffer::as_raw_ptr (device/src/buffer.rs:567-572, `unimplemented!` for CUDA in the
 * reference): device pointer + view offset.  Allocates on first use. */
MK_API mk_status mk_buf_ptr(mk_buf* buf, void** dptr);
MK_API mk_status mk_buf_size(mk_buf* buf, size_t* bytes);
MK_API mk_status mk_buf_is_allocated(mk_buf* buf, int32_t* allocated);
/* Buffer::view(offset, size): shares the parent's allocation; the parent stays alive until the
 * last view is freed. */
MK_API mk_status mk_buf_view(mk_buf* buf, size_t offset, size_t bytes, mk_buf** out);
/* Drop: returns the allocation to the LRU free lists (or releases a view's reference). */
MK_API mk_status mk_free(mk_buf* buf);
MK_API mk_status mk_alloc_stats(mk_device* dev, mk_alloc_stats_t* stats);
/* Releases every cached allocation back to the driver (LruAllocator::free_cache). */
MK_API mk_status mk_alloc_trim(mk_device* dev);
/* Test hook for host-side failure injection: the next `count` device allocations of this
 * device fail as if the driver were out of memory (exercises flush-and-retry without
 * exhausting a shared GPU). */
MK_API mk_status mk_alloc_inject_oom(mk_device* dev, int32_t count);

/* ---------------------------------------------------------------------------------------------
 * Copies  (Buffer::copyin / copyout / copy_from: device/src/buffer.rs:332-534).
 * `bytes` must equal the buffer's size (views: the view's size) or MK_ERR_SIZE_MISMATCH.
 * copyin returns once the source may be reused (pageable memory is staged by the driver, pinned
 * memory from mk_host_alloc is read asynchronously on the stream -- keep it unchanged until the
 * stream reaches the copy); copyout returns after the bytes have arrived.
 * ------------------------------------------------------------------------------------------- */
MK_API mk_status mk_copy_h2d(mk_buf* dst, const void* src, size_t bytes, mk_stream* s);
MK_API mk_status mk_copy_d2h(void* dst, mk_buf* src, size_t bytes, mk_stream* s);
MK_API mk_status mk_copy_d2d(mk_buf* dst, mk_buf* src, size_t bytes, mk_stream* s);
/* Device to device across GPUs of one node (NVLink); dst/src may belong to different devices. */
MK_API mk_status mk_copy_p2p(mk_buf* dst, mk_buf* src, size_t bytes, mk_stream* s);
/* Pinned host memory for callers that overlap their own transfers. */
MK_API mk_status mk_host_alloc(size_t bytes, void** out);
MK_API mk_status mk_host_free(void* p);
/* Raw async copies between caller-managed pointers (pinned host or device). kind: 0 = H2D,
 * 1 = D2H, 2 = D2D. */
MK_API mk_status mk_memcpy_async(mk_device* dev, void* dst, const void* src, size_t bytes, int32_t kind,
                                 mk_stream* s);
/* CudaAllocator::memset_zeros (device/src/allocator.rs:256-309) for any byte value: fills `bytes` bytes at
 * the device pointer `dst` on stream s. */
MK_API mk_status mk_memset_async(mk_device* dev, void* dst, int32_t byte_value, size_t bytes, mk_stream* s);
/* Free and total device memory as the driver reports them (cudaMemGetInfo). */
MK_API mk_status mk_mem_info(mk_device* dev, size_t* free_bytes, size_t* total_bytes);

/* ---------------------------------------------------------------------------------------------
 * Module load and launch  (JitKernel compile+load+fn pointer: runtime/src/jit_loader.rs:31-38;
 * KernelCif::dispatch, buffers first then i64 values: runtime/src/dispatch.rs:45-83;
 * Program::execute(buffers, vals, global_size, local_size): device/src/device.rs:34-60).
 * Images are cubin/fatbin/PTX built ahead of time for sm_100a.
 * ------------------------------------------------------------------------------------------- */
MK_API mk_status mk_module_load(mk_device* dev, const void* image, size_t bytes, mk_module** out);
MK_API mk_status mk_module_unload(mk_module* m);
MK_API mk_status mk_get_function(mk_module* m, const char* name, mk_function** out);
/* args: one pointer per kernel parameter, buffers (PARAM slot order) first, then values. */
MK_API mk_status mk_launch(mk_function* f, const uint32_t grid[3], const uint32_t block[3], uint32_t smem_bytes,
                           mk_stream* s, void** args);

/* ---------------------------------------------------------------------------------------------
 * GEMM -- replaces the kernel morok generates for `Tensor::matmul` / `dot` / `linear`
 * (tensor/src/matmul.rs:54-56,82-110,161-187) and the tensor-core rewrite of that kernel
 * (schedule/src/optimizer/tc.rs:358-674, dtype routing 126-168):
 *   C[m,n] = alpha * sum_k A[m,k] * B[k,n]  + beta * D[m,n] (MK_EPI_ADD) or beta * D[n] (MK_EPI_ADD_ROW)
 * with alpha = beta = 1 unless MK_GEMM_SCALED is set -- `Tensor::gemm` (tensor/src/matmul.rs:112-133:
 * alpha * A @ B + beta * C) and the bias of `linear` (161-187) in the store of one kernel;
 * accumulated in f32 (tensor/src/reduce.rs:101-117) and cast to dtype_out on store.
 *   bf16/f16 inputs: tcgen05 tensor cores (exact products, f32 accumulators in TMEM).
 *   f32 inputs:      exact fp32 FMA, one accumulator per output, k increasing (TF32 is never
 *                    used; the reference keeps allow_tf32 = false, renderer.rs:153,173,680).
 * Any M, N, K >= 0 is accepted (tails are predicated; K = 0 yields zeros or D).
 * ------------------------------------------------------------------------------------------- */
enum { MK_EPI_NONE = 0, MK_EPI_ADD = 1, MK_EPI_ADD_ROW = 2, MK_EPI_SWIGLU = 3 };
enum {
    MK_GEMM_SCALED = 1,        /* mk_gemm_desc.flags: alpha and beta are meaningful */
    MK_GEMM_GATE_SIGMOID = 2   /* MK_EPI_SWIGLU: the gate is sigmoid(g) instead of silu(g) = g * sigmoid(g) */
};
enum { MK_MAX_PEERS = 8 };

typedef struct {
    int32_t dtype_in;     /* mk_dtype of A and B */
    int32_t dtype_out;    /* mk_dtype of C (and D) */
    int64_t M, N, K;
    const void* A;        /* device pointer, row-major [M,K]; element stride between rows = lda */
    int64_t lda;
    const void* B;        /* trans_b = 0: row-major [K,N] (morok matmul); trans_b = 1: row-major [N,K]
                             (`linear` weights, tensor/src/matmul.rs:161-177) */
    int64_t ldb;
    void* C;              /* row-major [M,N], row stride ldc */
    int64_t ldc;
    int32_t trans_b;
    int32_t batch;        /* >= 1; leading batch dims flattened by the caller */
    int64_t stride_a;     /* elements between consecutive batch items; 0 broadcasts */
    int64_t stride_b;
    int64_t stride_c;
    int32_t epilogue;     /* MK_EPI_* */
    const void* D;        /* MK_EPI_ADD: same shape/strides/dtype as C (residual add fused into
                             the store, as pm_wmma_accumulate keeps `+ c` inside the kernel:
                             schedule/src/devectorize.rs:1017-1038) */
    /* Sharded delivery (N split across GPUs): when n_peers > 0 every finished tile is also
     * stored at the same [m, n] position of each peer_C[i] (peer-mapped device pointers, row
     * stride ldc).  C and peer_C then address the full gathered matrix and the shard's columns
     * start at column 0 of the pointers passed (pre-offset by the caller). */
    int32_t n_peers;
    void* peer_C[MK_MAX_PEERS];
    /* C = alpha * (A B) + beta * D when flags has MK_GEMM_SCALED (otherwise both count as 1).  With
     * MK_EPI_ADD_ROW, D holds N elements of dtype_out and is added to every row (a bias). */
    float alpha, beta;
    uint32_t flags;
    /* MK_EPI_SWIGLU: C[m,n] = silu(sum_k A[m,k] B[k,n]) * (sum_k A[m,k] B2[k,n]) -- the gated feed-forward
     * `x.matmul(w_gate).silu() * x.matmul(w_up)`, which the reference keeps in one kernel with two reduces
     * (tensor/src/test/unit/fusion.rs:58-67, 106-114).  B2 has the shape, layout and leading dimension of B; both
     * products stay in f32 until the gate is applied.  16-bit inputs and outputs on the tensor cores only
     * (MK_ERR_UNSUPPORTED otherwise: run the two products and mk_swiglu instead); no scaling, no peers.
     * Biases: D (NULL or N elements of dtype_out, 16-byte aligned) is added to the first product before the
     * gate function, D2 likewise to the second -- with MK_GEMM_GATE_SIGMOID this is the reference's gate
     * block `(x @ w1 + b1).sigmoid() * (x @ w2 + b2)`, one kernel there as well
     * (tensor/src/test/unit/fusion.rs:58-67). */
    const void* B2;
    const void* D2;
} mk_gemm_desc;

MK_API mk_status mk_gemm(mk_device* dev, mk_stream* s, const mk_gemm_desc* desc);

/* GEMM tuning.  The reference searches the schedule of each new kernel by timing candidates on the
 * device and keeps the winner in a cache on disk, keyed by the kernel's structure
 * (schedule/src/optimizer/beam.rs:223-291 the search, 390-397 and 445-524 the cache).  The tensor-core
 * GEMM here has three schedule choices per problem -- one CTA per 128 x 256 tile or a CTA pair per
 * 256 x 256 tile, the number of row tiles per raster group, and the number of K ranges for problems with
 * few rows -- which a built-in rule sets.  mk_gemm_autotune times the candidates for one problem on the
 * device and records the fastest; later mk_gemm calls (and Tensor matmuls) with the same
 * M, N, K, dtypes, trans_b, epilogue, scaling flag and batch use it.  Records live in the mk_device and
 * can be written to and read from a text file.
 *   pair      -1: rule, 0: one CTA per tile, 1: CTA pairs (ignored where M <= 128)
 *   group_m    0: rule, else row tiles per raster group
 *   splits     0: rule, 1: never split K, n > 1: n ranges (ignored where the problem cannot be split:
 *              CTA pairs, the gated pair of products, peers)
 * A different number of K ranges changes the summation order: results then differ from the untuned call
 * in the last bits, within the same error bound.  The candidates overwrite C `iters + 1` times each, so the
 * problem must be idempotent: an epilogue whose D overlaps C is refused (MK_ERR_INVALID). */
typedef struct mk_gemm_tuning {
    int32_t pair, group_m, splits;
    int32_t candidates;         /* out: how many candidates mk_gemm_autotune timed */
    float best_ms, default_ms;  /* out: per launch, the winner and the built-in rule */
} mk_gemm_tuning;
MK_API mk_status mk_gemm_autotune(mk_device* dev, mk_stream* s, const mk_gemm_desc* desc, int32_t iters,
                                  mk_gemm_tuning* result /* may be NULL */);
MK_API mk_status mk_gemm_tuning_set(mk_device* dev, const mk_gemm_desc* desc, const mk_gemm_tuning* t /* NULL: forget */);
MK_API mk_status mk_gemm_tuning_get(mk_device* dev, const mk_gemm_desc* desc, mk_gemm_tuning* t, int32_t* found);
MK_API mk_status mk_tuning_save(mk_device* dev, const char* path);
MK_API mk_status mk_tuning_load(mk_device* dev, const char* path, int32_t* entries /* may be NULL */);
MK_API mk_status mk_tuning_clear(mk_device* dev);

/* mk_gemm_static -- the tensor-core GEMM for callers that must not allocate device memory.
 * (No counterpart in the reference: morok's allocator is the only thing there that allocates, and
 * its kernels never need memory of their own.)
 *
 * For whom: code that lives inside another owner's memory budget -- a plugin in an inference server,
 * an operator under a framework's caching allocator that has already reserved HBM -- where a
 * cudaMalloc can fail, and latency-critical callers that cannot afford the device-wide
 * synchronisation cudaMalloc / cudaFree imply.  mk_gemm needs an mk_device, and opening one reserves
 * the kernel error word with cudaMalloc; this call needs no mk_device and calls no cudaMalloc,
 * cudaFree or any allocating routine.  The kernel's only memory besides the caller's A, B, C (D) --
 * one 16-byte error word per batch item -- is a fixed 4 KiB array inside the library image, held by
 * every GPU that loads the library until the process exits.
 *
 *   device_ordinal  CUDA device the pointers in `desc` belong to
 *   cuda_stream     a cudaStream_t (NULL = default stream); the launch is asynchronous
 *   desc            as for mk_gemm, restricted to what the tensor-core kernel takes: bf16 / f16
 *                   inputs, M, N, K > 0, A and B 16-byte aligned with row pitches that are multiples
 *                   of 8 elements (anything else: MK_ERR_UNSUPPORTED -- use mk_gemm), and
 *                   batch <= MK_STATIC_GEMM_MAX_BATCH (more: MK_ERR_INVALID, nothing is launched)
 *   kernel_error    NULL, or where to store the kernel error word: when given, the call waits for the
 *                   stream and returns MK_ERR_KERNEL if a pipeline wait gave up (not allowed while the
 *                   stream is capturing: MK_ERR_INVALID).  With NULL the call only enqueues; a wait that
 *                   gave up then stays unreported until mk_gemm_static_status (or the next call with a
 *                   pointer) reads the words.
 *
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress) and the
 * device's attributes, and the first launch of each kernel variant makes the driver load that kernel's
 * image; make that first call before any stream capture begins.  The calling thread's current device is
 * left as it was.  Problems with more than 128 rows and enough 256 x 256 tiles run on the CTA-pair kernel,
 * like mk_gemm.
 * All calls on a device share the array.  Each call clears, in stream order, the words it uses, so
 * calls queued on one stream are fine; calls that overlap on the GPU (different streams, different
 * host threads) race on the error words -- results in C stay correct, error reporting does not. */
#define MK_STATIC_GEMM_MAX_BATCH 256
MK_API mk_status mk_gemm_static(int32_t device_ordinal, void* cuda_stream, const mk_gemm_desc* desc, uint32_t* kernel_error);
/* Waits for `cuda_stream` and reads the first `batch` error words of the static array (what the last
 * mk_gemm_static call with that batch wrote): *kernel_error receives the first non-zero word and the call
 * returns MK_ERR_KERNEL, or 0 and MK_OK.  Allocates nothing.  (No counterpart in the reference.) */
MK_API mk_status mk_gemm_static_status(int32_t device_ordinal, void* cuda_stream, int32_t batch, uint32_t* kernel_error);

/* ---------------------------------------------------------------------------------------------
 * Attention forward -- replaces the >= 5 kernels morok schedules for
 * `Tensor::scaled_dot_product_attention` (tensor/src/transformer.rs:78-137):
 *   O = softmax(mask(Q K^T * scale)) V
 * scale: lines 90-100; causal = keep col <= row, top-left aligned (lines 103-109,
 * tensor/src/shape_ops.rs:780-807); additive mask: lines 112-124; softcap: lines 127-132;
 * softmax: tensor/src/activation.rs:90-101.  One fused kernel with online softmax; the
 * [Sq,Sk] score matrix is never written to memory.  Softmax statistics are f32.
 * GQA: h_kv < h_q maps query head h to kv head h / (h_q / h_kv) -- the repeat-interleave the
 * reference builds with unsqueeze/expand/reshape (onnx/src/registry/transformer.rs:80-103)
 * without materialising the expanded K/V.
 * Layout: Q [B,Hq,Sq,D], K [B,Hkv,Sk,D], V [B,Hkv,Sk,Dv], O [B,Hq,Sq,Dv]; the last dimension
 * is contiguous and each tensor gives its batch / head / row strides in elements, so
 * [B,S,H,D]-stored activations are read in place.
 * ------------------------------------------------------------------------------------------- */
typedef struct {
    int32_t dtype;        /* mk_dtype of Q, K, V and O */
    int32_t B, Hq, Hkv;
    int32_t Sq, Sk, D, Dv;
    float scale;          /* <= 0 selects 1/sqrt(D) */
    int32_t causal;
    float softcap;        /* <= 0 disables */
    const void *Q, *K, *V;
    void* O;
    int64_t q_strides[3]; /* batch, head, row (elements) */
    int64_t k_strides[3];
    int64_t v_strides[3];
    int64_t o_strides[3];
    const void* mask;     /* optional mask added to the scaled scores; shape and element type: mask_kind below */
    float* lse;           /* optional [B,Hq,Sq] f32: max + log(sum) of the scaled, masked scores */
    /* Sharded delivery (heads split across GPUs): finished O tiles are also stored at the same
     * element offset of each peer_O[i]. */
    int32_t n_peers;
    void* peer_O[MK_MAX_PEERS];
    /* With causal != 0, query row i sees keys j <= i + causal_offset.  0 is the Tensor method's tril(0)
     * (tensor/src/transformer.rs:103-110); a key/value cache of past_seq_len entries in front of the
     * current keys uses past_seq_len (onnx/src/registry/transformer.rs:155-162), so a single new
     * query row (Sq = 1, causal_offset = Sk - 1) sees the whole cache. */
    int32_t causal_offset;
    /* The reference adds any mask that broadcasts against the [B, H, Sq, Sk] scores, and turns a bool mask into
     * 0 where it is true and -inf where it is false first (tensor/src/transformer.rs:112-124).
     *   MK_MASK_SQ_SK (0)  additive f32 [Sq, Sk], shared by every batch element and head (mask_strides ignored)
     *   MK_MASK_F32   (1)  additive f32, element (b, h, i, j) at mask[b * s0 + h * s1 + i * s2 + j]
     *   MK_MASK_BOOL  (2)  one byte per element at the same index, non-zero = attend, zero = add -inf
     * with s0, s1, s2 = mask_strides in elements; 0 broadcasts that dimension (a key-padding mask [B, 1, 1, Sk] has
     * strides {Sk, 0, 0}).  Keys are contiguous.  Masks and softcap run on the tensor-core kernel as well. */
    int32_t mask_kind;
    int64_t mask_strides[3];
} mk_sdpa_desc;
enum { MK_MASK_SQ_SK = 0, MK_MASK_F32 = 1, MK_MASK_BOOL = 2 };

MK_API mk_status mk_sdpa_fwd(mk_device* dev, mk_stream* s, const mk_sdpa_desc* desc);

/* ---------------------------------------------------------------------------------------------
 * Element-wise / row-wise kernels of the decoder layer (HBM-bound, 128-bit vectorised)
 * ------------------------------------------------------------------------------------------- */
/* y = x * rsqrt(mean(x^2) + eps) [* gain], statistics in f32 (tensor/src/nn/norm.rs:92-110;
 * gain multiply: onnx/src/registry/transformer.rs:13-20). x [rows, cols] contiguous. */
MK_API mk_status mk_rms_norm(mk_device* dev, mk_stream* s, int32_t dtype_in, int32_t dtype_out, const void* x,
                             const void* gain /* dtype_in, [cols], or NULL */, void* y, int64_t rows, int64_t cols,
                             float eps);
/* apply_rotary_emb (tensor/src/transformer.rs:32-69). x, y [rows, D]; cos/sin f32 [rows_cs, D/2];
 * row r uses table row (r / row_div) % rows_cs. In place allowed (x == y). */
MK_API mk_status mk_rope(mk_device* dev, mk_stream* s, int32_t dtype, const void* x, const float* cosv,
                         const float* sinv, void* y, int64_t rows, int32_t D, int64_t rows_cs, int64_t row_div,
                         int32_t interleaved);
/* y = silu(gate) * up with silu(x) = x / (1 + exp2(-x / ln 2)) (tensor/src/activation.rs:42-52,309-318). */
MK_API mk_status mk_swiglu(mk_device* dev, mk_stream* s, int32_t dtype, const void* gate, const void* up, void* y,
                           int64_t n);
MK_API mk_status mk_add(mk_device* dev, mk_stream* s, int32_t dtype, const void* a, const void* b, void* y,
                        int64_t n);
/* Tensor::cast between f32 / bf16 / f16 (round to nearest even). */
MK_API mk_status mk_cast(mk_device* dev, mk_stream* s, int32_t dtype_in, int32_t dtype_out, const void* x, void* y,
                         int64_t n);

/* ---------------------------------------------------------------------------------------------
 * Multi-GPU plumbing for sharded outputs (one process per GPU).  The reference has no
 * communication backend (its multi-device IR ops are never executed: ir/src/op.rs:67-70);
 * these calls let ranks map each other's output buffers so that GEMM / attention epilogues can
 * deliver tiles to peers over NVLink, and provide a copy-engine all-gather over the same
 * mappings.
 * ------------------------------------------------------------------------------------------- */
typedef struct { unsigned char bytes[64]; } mk_ipc_handle;

/* Handle for a buffer allocated by mk_alloc (allocates it if still lazy).  The handle's bytes
 * are sent to the peer process by the caller (any transport). */
MK_API mk_status mk_ipc_export(mk_buf* buf, mk_ipc_handle* handle, size_t* offset);
/* Maps a peer's buffer into this process; the result behaves like a buffer of `bytes` bytes
 * whose mk_free unmaps it. */
MK_API mk_status mk_ipc_open(mk_device* dev, const mk_ipc_handle* handle, size_t offset, size_t bytes,
                             mk_buf** out);
/* All-gather by peer stores: copies this rank's `bytes`-byte shard (src) to byte offset
 * `dst_offset` of every dst[i] (n_dst mapped buffers, the local one included) on stream s. */
MK_API mk_status mk_all_gather_push(mk_device* dev, mk_stream* s, const void* src, size_t bytes,
                                    void* const* dst, int32_t n_dst, size_t dst_offset);
/* Strided variant for column shards of a row-major matrix: rows x row_bytes block, source row
 * pitch src_pitch, written at dst[i] + dst_offset with row pitch dst_pitch. */
MK_API mk_status mk_all_gather_push_2d(mk_device* dev, mk_stream* s, const void* src, size_t src_pitch,
                                       size_t row_bytes, size_t rows, void* const* dst, int32_t n_dst,
                                       size_t dst_offset, size_t dst_pitch);

/* ---------------------------------------------------------------------------------------------
 * Kernel error words.  Kernels never trap or spin without bound: a pipeline wait that runs out
 * records a code in the error word of the stream the kernel was launched on (every stream has its own
 * word; a recorded plan has one too, whichever stream replays it) and the kernel returns.
 * mk_kernel_status synchronises stream `s`, then reads and clears the word of `s` and the words of
 * recorded plans; non-zero yields MK_ERR_KERNEL.  Words of other streams stay for their own queries.  Codes name the kernel and the waiting
 * role: 0x101-0x103 tensor-core GEMM (producer, MMA issuer, epilogue), 0x201-0x203 tensor-core
 * attention (producer, MMA issuer, softmax), 0x301-0x303 few-row GEMM (producer, consumer, reduction),
 * 0x901 the self-test below.
 * ------------------------------------------------------------------------------------------- */
MK_API mk_status mk_kernel_status(mk_device* dev, mk_stream* s, uint32_t* code);
/* Self-test of that mechanism, safe to run anywhere: launches one warp that waits, for limit_ms
 * milliseconds (1..1000), on a barrier nothing ever signals.  The wait runs out, the kernel records
 * code 0x901 and returns normally.  Returns MK_OK when the kernel behaved that way; the caller then
 * reads the recorded error with mk_kernel_status (MK_ERR_KERNEL, code 0x901, which also clears it).
 * No reference counterpart on the device side; the host-side analogue is the deadline polling of
 * device/src/sync.rs:248-306. */
#define MK_KERR_SELFTEST_WAIT 0x901u
MK_API mk_status mk_selftest_bounded_wait(mk_device* dev, mk_stream* s, uint32_t limit_ms);
/* Number of kernels this library has launched on the device since it was opened. */
MK_API mk_status mk_launch_count(mk_device* dev, uint64_t* launches);

/* Per-kernel timing: what ExecutionPlan::execute_profiled reports (runtime/src/execution_plan.rs:200-221),
 * measured on the device.  Between begin and end every kernel the CALLING THREAD launches on stream `s`
 * through this library (mk_gemm, mk_sdpa_fwd, the glue kernels, mk_launch, mk_tensor_realize) is stamped
 * with an event; mk_profile_end waits for the last one and returns the kernels in launch order with the
 * time from the previous stamp to theirs.  `*count` receives the number of kernels seen; at most
 * `capacity` entries are written.  Kernels recorded into a plan are not stamped, and a replayed plan is
 * one opaque graph launch. */
typedef struct mk_kernel_profile {
    char name[56];      /* which kernel, e.g. "gemm_tc_pair", "sdpa_tc_d128", "rms_norm" */
    float elapsed_ms;
    int32_t reserved;
} mk_kernel_profile;
MK_API mk_status mk_profile_begin(mk_device* dev, mk_stream* s /* NULL: the default stream */);
MK_API mk_status mk_profile_end(mk_device* dev, mk_kernel_profile* out, int32_t capacity, int32_t* count);

/* ---------------------------------------------------------------------------------------------
 * Lazy Tensor mirror.  morok's user-facing API builds a graph and computes on `realize()`
 * (tensor/src/realize.rs:83-127); the functions below mirror that for the dense path so a
 * binding can keep `Tensor::matmul(..)`, `scaled_dot_product_attention`, `realize()` and
 * `as_vec` semantics while every kernel comes from this library:
 *   from_raw_bytes / from_slice      tensor/src/data.rs:23-139
 *   matmul                           tensor/src/matmul.rs:82-110   (1-D operands as there)
 *   scaled_dot_product_attention     tensor/src/transformer.rs:78-137
 *   rms_norm, apply_rotary_emb       tensor/src/nn/norm.rs:92-110, tensor/src/transformer.rs:32-69
 *   silu, add, mul, cast             tensor/src/activation.rs:309-318
 *   reshape / permute (metadata)     views; copies are made only where a kernel needs them
 *   realize                          schedules the graph into an execution plan (kernel calls
 *                                    in topological order, buffers from the LRU allocator) and
 *                                    runs it (runtime/src/execution_plan.rs:168-181)
 *   as_vec (copyout)                 tensor/src/data.rs:165-262, device/src/buffer.rs:391-397
 * ------------------------------------------------------------------------------------------- */
typedef struct mk_tensor mk_tensor;
enum { MK_MAX_DIMS = 6 };

MK_API mk_status mk_tensor_from_bytes(mk_device* dev, const void* data, int32_t dtype, const int64_t* shape,
                                      int32_t ndim, mk_tensor** out);
MK_API mk_status mk_tensor_free(mk_tensor* t);
MK_API mk_status mk_tensor_shape(mk_tensor* t, int64_t* shape /* MK_MAX_DIMS */, int32_t* ndim, int32_t* dtype);
MK_API mk_status mk_tensor_matmul(mk_tensor* a, mk_tensor* b, mk_tensor** out);
/* mask: NULL, or a tensor of 2 to 4 dimensions that broadcasts against [B, H, Sq, Sk] (each dimension equal to the
 * score's or 1; missing leading dimensions count as 1), floating point (added) or MK_BOOL (true attends). */
MK_API mk_status mk_tensor_sdpa(mk_tensor* q, mk_tensor* k, mk_tensor* v, mk_tensor* mask /* or NULL */,
                                float scale /* <= 0: default */, int32_t causal, float softcap, mk_tensor** out);
MK_API mk_status mk_tensor_rms_norm(mk_tensor* x, float eps, mk_tensor** out);
MK_API mk_status mk_tensor_rope(mk_tensor* x, mk_tensor* cosv, mk_tensor* sinv, int32_t interleaved,
                                mk_tensor** out);
MK_API mk_status mk_tensor_silu(mk_tensor* x, mk_tensor** out);
/* tensor/src/activation.rs:42 (1 / (1 + 2^(-x / ln 2))); mul(sigmoid(x), x) and mul(sigmoid(g), u) realise as one kernel */
MK_API mk_status mk_tensor_sigmoid(mk_tensor* x, mk_tensor** out);
MK_API mk_status mk_tensor_add(mk_tensor* a, mk_tensor* b, mk_tensor** out);
MK_API mk_status mk_tensor_mul(mk_tensor* a, mk_tensor* b, mk_tensor** out);
MK_API mk_status mk_tensor_cast(mk_tensor* x, int32_t dtype, mk_tensor** out);
MK_API mk_status mk_tensor_reshape(mk_tensor* x, const int64_t* shape, int32_t ndim, mk_tensor** out);
MK_API mk_status mk_tensor_permute(mk_tensor* x, const int32_t* axes, int32_t ndim, mk_tensor** out);
/* Computes the tensor (and everything it depends on) on the device. */
MK_API mk_status mk_tensor_realize(mk_tensor* t);
/* Number of kernel launches the last realize() of this tensor issued (the reference asserts
 * kernel counts in tensor/src/test/unit/fusion.rs). */
MK_API mk_status mk_tensor_last_launches(mk_tensor* t, int32_t* launches);
/* Copies a realized tensor to host memory (`bytes` must equal numel * element size). */
MK_API mk_status mk_tensor_copyout(mk_tensor* t, void* dst, size_t bytes);
/* Overwrites the data of a realized, contiguous tensor (normally a leaf made by mk_tensor_from_bytes)
 * with `bytes` host bytes; a plan that reads the tensor sees the new data on its next replay. */
MK_API mk_status mk_tensor_write(mk_tensor* t, const void* data, size_t bytes);

/* Plans: prepare once, execute many times (runtime/src/execution_plan.rs:88-106 builds an
 * ExecutionPlan, 168-181 executes it).  mk_tensor_compile records the kernels that realising `t`
 * would launch into a CUDA graph instead of running them; `t` then counts as realized, but holds
 * results only after the plan has run.  mk_plan_launch replays the plan on stream `s` (NULL = default
 * stream) with one launch call; launches on one stream run in order, and a plan must not run
 * concurrently with itself.  The plan keeps every intermediate buffer allocated until mk_plan_free. */
typedef struct mk_plan mk_plan;
MK_API mk_status mk_tensor_compile(mk_tensor* t, mk_plan** out);
MK_API mk_status mk_plan_launch(mk_plan* plan, mk_stream* s);
MK_API mk_status mk_plan_kernel_count(mk_plan* plan, int32_t* kernels);
MK_API mk_status mk_plan_free(mk_plan* plan);

#ifdef __cplusplus
}
#endif
#endif /* MOROK_B200_H */
