// Host runtime of libmorok_b200: errors, devices, streams, events, the lazy + LRU HBM allocator,
// copies, IPC peer mappings, and module load / launch.  Mirrors the `Device` bundle of the
// reference (allocator + runtime, device/src/device.rs:255-298) for a CUDA device.
#include <cuda.h>

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <thread>

#include "mk_internal.h"

namespace mk {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

mk_status fail(mk_status code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

mk_status cuda_fail(cudaError_t e, const char* what) {
    // Clear the sticky-free "last error" so that the next runtime call does not report it again.
    cudaGetLastError();
    snprintf(g_err, sizeof(g_err), "CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
    return e == cudaErrorMemoryAllocation ? MK_ERR_OOM : MK_ERR_CUDA;
}

void* driver_entry(const char* name) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return fn;
}

static size_t size_key(size_t bytes) { return (bytes + 511) & ~size_t(511); }

// Raw memory back end.  A mock device (mk_device_open_mock) keeps the allocator and copy logic
// testable on machines without a GPU by backing "device" memory with host memory; it cannot
// run kernels.
static cudaError_t raw_malloc(mk_device* dev, void** p, size_t bytes) {
    if (dev->mock) {
        *p = aligned_alloc(512, bytes);
        return *p ? cudaSuccess : cudaErrorMemoryAllocation;
    }
    return cudaMalloc(p, bytes);
}
static void raw_free(mk_device* dev, void* p) {
    if (dev->mock) free(p); else cudaFree(p);
}
static cudaError_t raw_memset0(mk_device* dev, void* p, size_t bytes) {
    if (dev->mock) { memset(p, 0, bytes); return cudaSuccess; }
    return cudaMemset(p, 0, bytes);
}
static cudaError_t raw_copy(mk_device* dev, void* dst, const void* src, size_t bytes, cudaMemcpyKind kind, cudaStream_t st) {
    if (dev->mock) { memmove(dst, src, bytes); return cudaSuccess; }
    return cudaMemcpyAsync(dst, src, bytes, kind, st);
}
static cudaError_t raw_stream_sync(mk_device* dev, cudaStream_t st) {
    if (dev->mock) return cudaSuccess;
    return cudaStreamSynchronize(st);
}

// ---- stream-ordered reuse ------------------------------------------------------------------------------
// The reference's LRU allocator hands a cached block to the next caller at once and leaves ordering to its
// scheduler ("scheduler guarantees exclusive access", device/src/allocator.rs:72-112); its CUDA calls all
// run on one stream.  Here kernels run on several non-blocking streams, so a parked block remembers, per
// stream that had work in flight when it was released, an event behind that work; whoever takes the block
// from the cache waits for the events of the other streams first (on the consumer's stream when the
// calling thread declared one with AllocStreamScope, else on the host -- usually the events have long
// completed and the query costs a microsecond).
static thread_local bool t_alloc_set = false;
static thread_local cudaStream_t t_alloc_stream = nullptr;

AllocStreamScope::AllocStreamScope(cudaStream_t st) : prev_set(t_alloc_set), prev(t_alloc_stream) {
    t_alloc_set = true;
    t_alloc_stream = st;
}
AllocStreamScope::~AllocStreamScope() {
    t_alloc_set = prev_set;
    t_alloc_stream = prev;
}

static bool stream_is_capturing(cudaStream_t st) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cs) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return cs != cudaStreamCaptureStatusNone;
}

// Fences of every stream that may still be working on memory released now (caller holds dev->mu).
static void collect_fences_locked(mk_device* dev, std::vector<std::shared_ptr<StreamFence>>* out) {
    if (dev->mock) return;
    for (auto& kv : dev->streams) {
        StreamState& ss = kv.second;
        if (ss.dirty) {
            if (stream_is_capturing(kv.first)) continue;     // recorded work runs later; a plan retains what it uses
            auto f = std::make_shared<StreamFence>();
            f->stream = kv.first;
            if (cudaEventCreateWithFlags(&f->event, cudaEventDisableTiming) != cudaSuccess || cudaEventRecord(f->event, kv.first) != cudaSuccess) {
                cudaGetLastError();
                cudaStreamSynchronize(kv.first);             // no event to be had: make the release itself safe
                cudaGetLastError();
                f.reset();
            }
            ss.fence = f;
            ss.dirty = false;
        }
        if (ss.fence) out->push_back(ss.fence);
    }
}

// Orders the calling thread's next use of a block after the work its fences stand for.
static void wait_fences(const std::vector<std::shared_ptr<StreamFence>>& fences) {
    for (const auto& f : fences) {
        if (!f || !f->event) continue;
        if (t_alloc_set && f->stream == t_alloc_stream) continue;        // same queue: already ordered
        cudaError_t q = cudaEventQuery(f->event);
        if (q == cudaSuccess) continue;
        cudaGetLastError();
        if (t_alloc_set && !stream_is_capturing(t_alloc_stream)) cudaStreamWaitEvent(t_alloc_stream, f->event, 0);
        else cudaEventSynchronize(f->event);
        cudaGetLastError();
    }
}

// cudaMalloc with the reference's LRU policy in front of it (device/src/allocator.rs:383-442):
// reuse a cached block of the same size class, else allocate; on out-of-memory flush the whole
// cache and retry once.
mk_status device_alloc(mk_device* dev, size_t bytes, uint32_t flags, void** out) {
    const size_t key = size_key(bytes);
    void* p = nullptr;
    std::vector<std::shared_ptr<StreamFence>> fences;
    {
        std::lock_guard<std::mutex> lk(dev->mu);
        auto it = dev->free_lists.find(key);
        if (it != dev->free_lists.end() && !it->second.empty()) {
            p = it->second.front().ptr;
            fences = std::move(it->second.front().fences);
            it->second.pop_front();
            dev->stats.cache_hits++;
            dev->stats.bytes_cached -= key;
        }
    }
    if (p && !fences.empty()) {
        cudaSetDevice(dev->ordinal);
        wait_fences(fences);
        fences.clear();
    }
    if (!p) {
        if (!dev->mock) MK_CUDA(cudaSetDevice(dev->ordinal));
        bool injected = false;
        {
            std::lock_guard<std::mutex> lk(dev->mu);
            if (dev->inject_oom > 0) {
                dev->inject_oom--;
                injected = true;
            }
        }
        cudaError_t e = injected ? cudaErrorMemoryAllocation : raw_malloc(dev, &p, key);
        if (e == cudaErrorMemoryAllocation) {
            cudaGetLastError();
            std::vector<void*> victims;
            {
                std::lock_guard<std::mutex> lk(dev->mu);
                for (auto& kv : dev->free_lists)
                    for (auto& v : kv.second) victims.push_back(v.ptr);
                dev->free_lists.clear();
                dev->stats.bytes_cached = 0;
                dev->stats.oom_flushes++;
                dev->stats.device_frees += victims.size();
            }
            for (void* v : victims) raw_free(dev, v);       // cudaFree waits for work that still uses the block
            bool injected_again = false;
            {
                std::lock_guard<std::mutex> lk(dev->mu);
                if (dev->inject_oom > 0) {
                    dev->inject_oom--;
                    injected_again = true;
                }
            }
            e = injected_again ? cudaErrorMemoryAllocation : raw_malloc(dev, &p, key);
        }
        if (e != cudaSuccess) {
            cudaGetLastError();
            return fail(e == cudaErrorMemoryAllocation ? MK_ERR_OOM : MK_ERR_CUDA,
                        "device allocation of %zu bytes failed: %s", key, cudaGetErrorString(e));
        }
        std::lock_guard<std::mutex> lk(dev->mu);
        dev->stats.device_allocs++;
    }
    if (flags & MK_ALLOC_ZERO_INIT) {
        // Zeroed on the consumer's stream when the thread declared one, else finished before this returns, so that
        // the zeros are in place whichever stream touches the buffer first.
        cudaError_t e;
        if (dev->mock) {
            e = raw_memset0(dev, p, key);
        } else if (t_alloc_set) {
            e = cudaMemsetAsync(p, 0, key, t_alloc_stream);
            touch_stream(dev, t_alloc_stream);
        } else {
            e = cudaMemsetAsync(p, 0, key, (cudaStream_t)0);
            if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)0);
        }
        if (e != cudaSuccess) {
            device_release(dev, p, bytes);
            return cuda_fail(e, "cudaMemset(zero_init)");
        }
    }
    {
        std::lock_guard<std::mutex> lk(dev->mu);
        dev->stats.bytes_in_use += key;
        if (dev->stats.bytes_in_use > dev->stats.peak_bytes_in_use) dev->stats.peak_bytes_in_use = dev->stats.bytes_in_use;
    }
    *out = p;
    return MK_OK;
}

void device_release(mk_device* dev, void* ptr, size_t bytes) {
    if (!ptr) return;
    const size_t key = size_key(bytes);
    bool park = false;
    if (!dev->mock) cudaSetDevice(dev->ordinal);
    {
        std::lock_guard<std::mutex> lk(dev->mu);
        if (dev->stats.bytes_in_use >= key) dev->stats.bytes_in_use -= key;
        auto& lst = dev->free_lists[key];
        if (lst.size() < mk_device::kMaxPerKey) {
            mk_device::Parked blk{ptr, {}};
            collect_fences_locked(dev, &blk.fences);
            lst.push_front(std::move(blk));
            dev->stats.cache_returns++;
            dev->stats.bytes_cached += key;
            park = true;
        } else {
            dev->stats.device_frees++;
        }
    }
    if (!park) raw_free(dev, ptr);
}

mk_status buf_ptr(mk_buf* b, void** out) {
    BufData* d = b->data.get();
    std::lock_guard<std::mutex> lk(d->mu);
    if (!d->ptr && d->bytes > 0) {
        mk_status st = device_alloc(d->dev, d->bytes, d->flags, &d->ptr);
        if (st != MK_OK) return st;
    }
    *out = d->ptr ? (void*)((char*)d->ptr + b->offset) : nullptr;
    return MK_OK;
}

}  // namespace mk

BufData::~BufData() {
    if (!ptr) return;
    if (ipc_mapped) {
        cudaSetDevice(dev->ordinal);
        cudaIpcCloseMemHandle(ptr);
        cudaGetLastError();
    } else {
        mk::device_release(dev, ptr, bytes);
    }
}

using namespace mk;

extern "C" {

const char* mk_last_error(void) { return g_err; }
int32_t mk_abi_version(void) { return 4; }
int32_t mk_abi_struct_size(int32_t which) {
    return which == 0 ? (int32_t)sizeof(mk_gemm_desc) : which == 1 ? (int32_t)sizeof(mk_sdpa_desc) : -1;
}

// ---- device ------------------------------------------------------------------------------------
mk_status mk_device_count(int32_t* count) {
    MK_REQUIRE(count, "mk_device_count: null output");
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) {
        *count = 0;
        return cuda_fail(e, "cudaGetDeviceCount");
    }
    *count = n;
    return MK_OK;
}

mk_status mk_device_open(int32_t ordinal, mk_device** out) {
    MK_REQUIRE(out, "mk_device_open: null output");
    *out = nullptr;
    int n = 0;
    MK_CUDA(cudaGetDeviceCount(&n));
    MK_REQUIRE(ordinal >= 0 && ordinal < n, "mk_device_open: ordinal %d out of range (%d devices)", ordinal, n);
    MK_CUDA(cudaSetDevice(ordinal));
    MK_CUDA(cudaFree(0));  // create the primary context
    std::unique_ptr<mk_device> dev(new mk_device());
    dev->ordinal = ordinal;
    MK_CUDA(cudaGetDeviceProperties(&dev->prop, ordinal));
    MK_CUDA(cudaMalloc((void**)&dev->kerr_words, sizeof(KernelError) * mk_device::kStreamSlots));
    MK_CUDA(cudaMemset(dev->kerr_words, 0, sizeof(KernelError) * mk_device::kStreamSlots));
    MK_CUDA(cudaMalloc((void**)&dev->work_counters, sizeof(unsigned int) * mk_device::kStreamSlots));
    MK_CUDA(cudaMemset(dev->work_counters, 0, sizeof(unsigned int) * mk_device::kStreamSlots));
    for (int i = mk_device::kStreamSlots - 1; i >= 1; --i) dev->free_slots.push_back(i);
    *out = dev.release();
    return MK_OK;
}

mk_status mk_device_open_mock(mk_device** out) {
    MK_REQUIRE(out, "mk_device_open_mock: null output");
    auto* dev = new mk_device();
    dev->mock = true;
    dev->ordinal = -1;
    snprintf(dev->prop.name, sizeof(dev->prop.name), "mock (host memory, no kernels)");
    *out = dev;
    return MK_OK;
}

mk_status mk_device_close(mk_device* dev) {
    MK_REQUIRE(dev, "mk_device_close: null device");
    if (!dev->mock) {
        cudaSetDevice(dev->ordinal);
        cudaDeviceSynchronize();
    }
    mk_alloc_trim(dev);
    if (dev->kerr_words) cudaFree(dev->kerr_words);
    if (dev->work_counters) cudaFree(dev->work_counters);
    for (auto& kv : dev->streams)
        if (kv.second.scratch) cudaFree(kv.second.scratch);
    dev->streams.clear();
    for (void* p : dev->retired_scratch) cudaFree(p);
    cudaGetLastError();
    delete dev;
    return MK_OK;
}

mk_status mk_device_get_info(mk_device* dev, mk_device_info* info) {
    MK_REQUIRE(dev && info, "mk_device_get_info: null argument");
    memset(info, 0, sizeof(*info));
    info->ordinal = dev->ordinal;
    info->sm_count = dev->prop.multiProcessorCount;
    info->cc_major = dev->prop.major;
    info->cc_minor = dev->prop.minor;
    info->max_smem_per_block = (int32_t)dev->prop.sharedMemPerBlockOptin;
    info->l2_bytes = dev->prop.l2CacheSize;
    info->total_mem = (int64_t)dev->prop.totalGlobalMem;
    snprintf(info->name, sizeof(info->name), "%s", dev->prop.name);
    return MK_OK;
}

mk_status mk_device_sync(mk_device* dev) {
    MK_REQUIRE(dev, "mk_device_sync: null device");
    if (dev->mock) return MK_OK;
    MK_CUDA(cudaSetDevice(dev->ordinal));
    MK_CUDA(cudaDeviceSynchronize());
    return MK_OK;
}

// ---- streams / events ----------------------------------------------------------------------------
mk_status mk_stream_create(mk_device* dev, mk_stream** out) {
    MK_REQUIRE(dev && out, "mk_stream_create: null argument");
    if (dev->mock) return fail(MK_ERR_CUDA, "mk_stream_create: mock device has no streams");
    MK_CUDA(cudaSetDevice(dev->ordinal));
    cudaStream_t s;
    MK_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    *out = new mk_stream{dev, s};
    return MK_OK;
}

mk_status mk_stream_destroy(mk_stream* s) {
    MK_REQUIRE(s, "mk_stream_destroy: null stream");
    if (s->dev && !s->dev->mock) mk::release_stream_state(s->dev, s->s);
    cudaError_t e = cudaStreamDestroy(s->s);
    delete s;
    if (e != cudaSuccess) return cuda_fail(e, "cudaStreamDestroy");
    return MK_OK;
}

mk_status mk_stream_sync(mk_stream* s) {
    MK_CUDA(cudaStreamSynchronize(raw(s)));
    return MK_OK;
}

mk_status mk_stream_wait_event(mk_stream* s, mk_event* ev) {
    MK_REQUIRE(ev, "mk_stream_wait_event: null event");
    MK_CUDA(cudaStreamWaitEvent(raw(s), ev->e, 0));
    return MK_OK;
}

mk_status mk_stream_raw(mk_stream* s, void** cuda_stream) {
    MK_REQUIRE(cuda_stream, "mk_stream_raw: null output");
    *cuda_stream = (void*)raw(s);
    return MK_OK;
}

mk_status mk_event_create(mk_device* dev, mk_event** out) {
    MK_REQUIRE(dev && out, "mk_event_create: null argument");
    if (dev->mock) return fail(MK_ERR_CUDA, "mk_event_create: mock device has no events");
    MK_CUDA(cudaSetDevice(dev->ordinal));
    cudaEvent_t e;
    MK_CUDA(cudaEventCreate(&e));
    *out = new mk_event{dev, e, false};
    return MK_OK;
}

mk_status mk_event_destroy(mk_event* ev) {
    MK_REQUIRE(ev, "mk_event_destroy: null event");
    cudaEventDestroy(ev->e);
    cudaGetLastError();
    delete ev;
    return MK_OK;
}

mk_status mk_event_record(mk_event* ev, mk_stream* s) {
    MK_REQUIRE(ev, "mk_event_record: null event");
    MK_CUDA(cudaEventRecord(ev->e, raw(s)));
    ev->recorded = true;
    return MK_OK;
}

mk_status mk_event_wait(mk_event* ev, int32_t timeout_ms) {
    MK_REQUIRE(ev, "mk_event_wait: null event");
    MK_REQUIRE(ev->recorded, "mk_event_wait: event was never recorded");
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms < 0 ? 0 : timeout_ms);
    for (;;) {
        cudaError_t e = cudaEventQuery(ev->e);
        if (e == cudaSuccess) return MK_OK;
        if (e != cudaErrorNotReady) return cuda_fail(e, "cudaEventQuery");
        cudaGetLastError();
        if (std::chrono::steady_clock::now() >= deadline)
            return fail(MK_ERR_TIMEOUT, "mk_event_wait: not complete after %d ms", timeout_ms);
        std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
}

mk_status mk_event_elapsed_ms(mk_event* start, mk_event* stop, float* ms) {
    MK_REQUIRE(start && stop && ms, "mk_event_elapsed_ms: null argument");
    MK_CUDA(cudaEventElapsedTime(ms, start->e, stop->e));
    return MK_OK;
}

// ---- allocator -------------------------------------------------------------------------------------
mk_status mk_alloc(mk_device* dev, size_t bytes, uint32_t flags, mk_buf** out) {
    MK_REQUIRE(dev && out, "mk_alloc: null argument");
    MK_REQUIRE((flags & ~MK_ALLOC_ZERO_INIT) == 0, "mk_alloc: unknown flags 0x%x", flags);
    auto* b = new mk_buf();
    b->data = std::make_shared<BufData>();
    b->data->dev = dev;
    b->data->bytes = bytes;
    b->data->flags = flags;
    b->offset = 0;
    b->bytes = bytes;
    *out = b;
    return MK_OK;
}

mk_status mk_buf_ensure(mk_buf* buf) {
    MK_REQUIRE(buf, "mk_buf_ensure: null buffer");
    void* p;
    return buf_ptr(buf, &p);
}

mk_status mk_buf_ptr(mk_buf* buf, void** dptr) {
    MK_REQUIRE(buf && dptr, "mk_buf_ptr: null argument");
    return buf_ptr(buf, dptr);
}

mk_status mk_buf_size(mk_buf* buf, size_t* bytes) {
    MK_REQUIRE(buf && bytes, "mk_buf_size: null argument");
    *bytes = buf->bytes;
    return MK_OK;
}

mk_status mk_buf_is_allocated(mk_buf* buf, int32_t* allocated) {
    MK_REQUIRE(buf && allocated, "mk_buf_is_allocated: null argument");
    std::lock_guard<std::mutex> lk(buf->data->mu);
    *allocated = buf->data->ptr != nullptr;
    return MK_OK;
}

mk_status mk_buf_view(mk_buf* buf, size_t offset, size_t bytes, mk_buf** out) {
    MK_REQUIRE(buf && out, "mk_buf_view: null argument");
    MK_REQUIRE(offset <= buf->bytes && bytes <= buf->bytes - offset, "mk_buf_view: [%zu, +%zu) exceeds buffer of %zu bytes",
               offset, bytes, buf->bytes);
    auto* v = new mk_buf();
    v->data = buf->data;
    v->offset = buf->offset + offset;
    v->bytes = bytes;
    *out = v;
    return MK_OK;
}

mk_status mk_free(mk_buf* buf) {
    MK_REQUIRE(buf, "mk_free: null buffer");
    delete buf;  // the shared allocation returns to the cache when its last handle goes
    return MK_OK;
}

mk_status mk_alloc_stats(mk_device* dev, mk_alloc_stats_t* stats) {
    MK_REQUIRE(dev && stats, "mk_alloc_stats: null argument");
    std::lock_guard<std::mutex> lk(dev->mu);
    *stats = dev->stats;
    return MK_OK;
}

mk_status mk_alloc_trim(mk_device* dev) {
    MK_REQUIRE(dev, "mk_alloc_trim: null device");
    std::vector<void*> victims;
    {
        std::lock_guard<std::mutex> lk(dev->mu);
        for (auto& kv : dev->free_lists)
            for (auto& v : kv.second) victims.push_back(v.ptr);
        dev->free_lists.clear();
        dev->stats.bytes_cached = 0;
        dev->stats.device_frees += victims.size();
    }
    if (!dev->mock) cudaSetDevice(dev->ordinal);
    for (void* v : victims) raw_free(dev, v);
    if (!dev->mock) cudaGetLastError();
    return MK_OK;
}

mk_status mk_alloc_inject_oom(mk_device* dev, int32_t count) {
    MK_REQUIRE(dev && count >= 0, "mk_alloc_inject_oom: bad argument");
    std::lock_guard<std::mutex> lk(dev->mu);
    dev->inject_oom = count;
    return MK_OK;
}

// ---- copies ------------------------------------------------------------------------------------------
mk_status mk_copy_h2d(mk_buf* dst, const void* src, size_t bytes, mk_stream* s) {
    MK_REQUIRE(dst && (src || bytes == 0), "mk_copy_h2d: null argument");
    if (bytes != dst->bytes)
        return fail(MK_ERR_SIZE_MISMATCH, "mk_copy_h2d: %zu bytes into a buffer of %zu", bytes, dst->bytes);
    if (bytes == 0) return MK_OK;
    void* d;
    mk_status st = buf_ptr(dst, &d);
    if (st != MK_OK) return st;
    MK_CUDA(raw_copy(dst->data->dev, d, src, bytes, cudaMemcpyHostToDevice, raw(s)));
    touch_stream(dst->data->dev, raw(s));
    return MK_OK;
}

mk_status mk_copy_d2h(void* dst, mk_buf* src, size_t bytes, mk_stream* s) {
    MK_REQUIRE(src && (dst || bytes == 0), "mk_copy_d2h: null argument");
    if (bytes != src->bytes)
        return fail(MK_ERR_SIZE_MISMATCH, "mk_copy_d2h: %zu bytes from a buffer of %zu", bytes, src->bytes);
    if (bytes == 0) return MK_OK;
    {
        std::lock_guard<std::mutex> lk(src->data->mu);
        // A zero-initialised buffer has defined contents before its first use; anything else has not.
        if (!src->data->ptr && !(src->data->flags & MK_ALLOC_ZERO_INIT))
            return fail(MK_ERR_NOT_ALLOCATED, "mk_copy_d2h: source buffer was never written");
    }
    void* p;
    mk_status st = buf_ptr(src, &p);
    if (st != MK_OK) return st;
    MK_CUDA(raw_copy(src->data->dev, dst, p, bytes, cudaMemcpyDeviceToHost, raw(s)));
    MK_CUDA(raw_stream_sync(src->data->dev, raw(s)));
    return MK_OK;
}

static mk_status copy_dd(mk_buf* dst, mk_buf* src, size_t bytes, mk_stream* s, const char* who) {
    MK_REQUIRE(dst && src, "%s: null argument", who);
    if (bytes != dst->bytes || bytes != src->bytes)
        return fail(MK_ERR_SIZE_MISMATCH, "%s: %zu bytes, dst %zu, src %zu", who, bytes, dst->bytes, src->bytes);
    if (bytes == 0) return MK_OK;
    void *d, *p;
    mk_status st = buf_ptr(dst, &d);
    if (st != MK_OK) return st;
    st = buf_ptr(src, &p);
    if (st != MK_OK) return st;
    MK_CUDA(raw_copy(dst->data->dev, d, p, bytes, cudaMemcpyDefault, raw(s)));
    touch_stream(dst->data->dev, raw(s));
    return MK_OK;
}

mk_status mk_copy_d2d(mk_buf* dst, mk_buf* src, size_t bytes, mk_stream* s) { return copy_dd(dst, src, bytes, s, "mk_copy_d2d"); }

mk_status mk_copy_p2p(mk_buf* dst, mk_buf* src, size_t bytes, mk_stream* s) {
    MK_REQUIRE(dst && src, "mk_copy_p2p: null argument");
    const int a = dst->data->dev->ordinal, b = src->data->dev->ordinal;
    if (a != b && !dst->data->dev->mock && !src->data->dev->mock) {
        int can = 0;
        MK_CUDA(cudaDeviceCanAccessPeer(&can, a, b));
        if (can) {
            cudaSetDevice(a);
            cudaError_t e = cudaDeviceEnablePeerAccess(b, 0);
            if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) return cuda_fail(e, "cudaDeviceEnablePeerAccess");
            cudaGetLastError();
        }
    }
    return copy_dd(dst, src, bytes, s, "mk_copy_p2p");
}

mk_status mk_host_alloc(size_t bytes, void** out) {
    MK_REQUIRE(out, "mk_host_alloc: null output");
    MK_CUDA(cudaHostAlloc(out, bytes ? bytes : 1, cudaHostAllocDefault));
    return MK_OK;
}

mk_status mk_host_free(void* p) {
    if (!p) return MK_OK;
    MK_CUDA(cudaFreeHost(p));
    return MK_OK;
}

mk_status mk_memcpy_async(mk_device* dev, void* dst, const void* src, size_t bytes, int32_t kind, mk_stream* s) {
    MK_REQUIRE(dev, "mk_memcpy_async: null device");
    MK_REQUIRE(kind >= 0 && kind <= 2, "mk_memcpy_async: kind %d", kind);
    if (bytes == 0) return MK_OK;
    MK_REQUIRE(dst && src, "mk_memcpy_async: null pointer");
    static const cudaMemcpyKind kinds[3] = {cudaMemcpyHostToDevice, cudaMemcpyDeviceToHost, cudaMemcpyDeviceToDevice};
    MK_CUDA(cudaMemcpyAsync(dst, src, bytes, kinds[kind], raw(s)));
    touch_stream(dev, raw(s));
    return MK_OK;
}

// CudaAllocator::memset_zeros (device/src/allocator.rs:256-309) generalised to any byte value.
mk_status mk_memset_async(mk_device* dev, void* dst, int32_t byte_value, size_t bytes, mk_stream* s) {
    MK_REQUIRE(dev, "mk_memset_async: null device");
    MK_REQUIRE(byte_value >= 0 && byte_value <= 255, "mk_memset_async: byte value %d", byte_value);
    if (bytes == 0) return MK_OK;
    MK_REQUIRE(dst, "mk_memset_async: null pointer");
    if (dev->mock) {
        memset(dst, byte_value, bytes);
        return MK_OK;
    }
    MK_CUDA(cudaSetDevice(dev->ordinal));
    MK_CUDA(cudaMemsetAsync(dst, byte_value, bytes, raw(s)));
    touch_stream(dev, raw(s));
    return MK_OK;
}

mk_status mk_mem_info(mk_device* dev, size_t* free_bytes, size_t* total_bytes) {
    MK_REQUIRE(dev && free_bytes && total_bytes, "mk_mem_info: null argument");
    if (dev->mock) return fail(MK_ERR_CUDA, "mk_mem_info: mock device has no device memory");
    MK_CUDA(cudaSetDevice(dev->ordinal));
    MK_CUDA(cudaMemGetInfo(free_bytes, total_bytes));
    return MK_OK;
}

// ---- IPC peer mappings and push all-gather ----------------------------------------------------------------
mk_status mk_ipc_export(mk_buf* buf, mk_ipc_handle* handle, size_t* offset) {
    MK_REQUIRE(buf && handle && offset, "mk_ipc_export: null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == sizeof(mk_ipc_handle), "handle size");
    MK_REQUIRE(!buf->data->ipc_mapped, "mk_ipc_export: buffer is itself a peer mapping");
    if (buf->data->dev->mock) return fail(MK_ERR_CUDA, "mk_ipc_export: mock device");
    void* p;
    mk_status st = buf_ptr(buf, &p);
    if (st != MK_OK) return st;
    MK_REQUIRE(buf->data->ptr, "mk_ipc_export: empty buffer");
    cudaIpcMemHandle_t h;
    MK_CUDA(cudaIpcGetMemHandle(&h, buf->data->ptr));
    memcpy(handle->bytes, &h, sizeof(h));
    *offset = buf->offset;
    return MK_OK;
}

mk_status mk_ipc_open(mk_device* dev, const mk_ipc_handle* handle, size_t offset, size_t bytes, mk_buf** out) {
    MK_REQUIRE(dev && handle && out, "mk_ipc_open: null argument");
    if (dev->mock) return fail(MK_ERR_CUDA, "mk_ipc_open: mock device");
    MK_CUDA(cudaSetDevice(dev->ordinal));
    cudaIpcMemHandle_t h;
    memcpy(&h, handle->bytes, sizeof(h));
    void* p = nullptr;
    MK_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    auto* b = new mk_buf();
    b->data = std::make_shared<BufData>();
    b->data->dev = dev;
    b->data->bytes = offset + bytes;
    b->data->ptr = p;
    b->data->ipc_mapped = true;
    b->offset = offset;
    b->bytes = bytes;
    *out = b;
    return MK_OK;
}

mk_status mk_all_gather_push(mk_device* dev, mk_stream* s, const void* src, size_t bytes, void* const* dst, int32_t n_dst,
                             size_t dst_offset) {
    MK_REQUIRE(dev && dst && n_dst >= 0, "mk_all_gather_push: bad argument");
    if (bytes == 0) return MK_OK;
    MK_REQUIRE(src, "mk_all_gather_push: null source");
    for (int i = 0; i < n_dst; ++i) {
        MK_REQUIRE(dst[i], "mk_all_gather_push: dst[%d] is null", i);
        char* d = (char*)dst[i] + dst_offset;
        if ((const void*)d == src) continue;
        MK_CUDA(cudaMemcpyAsync(d, src, bytes, cudaMemcpyDefault, raw(s)));
    }
    touch_stream(dev, raw(s));
    return MK_OK;
}

mk_status mk_all_gather_push_2d(mk_device* dev, mk_stream* s, const void* src, size_t src_pitch, size_t row_bytes, size_t rows,
                                void* const* dst, int32_t n_dst, size_t dst_offset, size_t dst_pitch) {
    MK_REQUIRE(dev && dst && n_dst >= 0, "mk_all_gather_push_2d: bad argument");
    if (row_bytes == 0 || rows == 0) return MK_OK;
    MK_REQUIRE(src && src_pitch >= row_bytes && dst_pitch >= row_bytes, "mk_all_gather_push_2d: bad pitch");
    for (int i = 0; i < n_dst; ++i) {
        MK_REQUIRE(dst[i], "mk_all_gather_push_2d: dst[%d] is null", i);
        char* d = (char*)dst[i] + dst_offset;
        if ((const void*)d == src) continue;
        MK_CUDA(cudaMemcpy2DAsync(d, dst_pitch, src, src_pitch, row_bytes, rows, cudaMemcpyDefault, raw(s)));
    }
    touch_stream(dev, raw(s));
    return MK_OK;
}

// ---- kernel error word ---------------------------------------------------------------------------------------
mk_status mk_kernel_status(mk_device* dev, mk_stream* s, uint32_t* code) {
    MK_REQUIRE(dev, "mk_kernel_status: null device");
    if (dev->mock) return fail(MK_ERR_CUDA, "mk_kernel_status: mock device runs no kernels");
    MK_CUDA(cudaSetDevice(dev->ordinal));
    MK_CUDA(cudaStreamSynchronize(raw(s)));
    // Every stream has its own word.  This query reports the word of `s` and the words of recorded plans
    // (their kernels write to the slot of the plan's capture stream whichever stream replays them); words of
    // other streams are left for the queries of those streams.
    std::vector<int> slots;
    {
        std::lock_guard<std::mutex> lk(dev->mu);
        auto it = dev->streams.find(raw(s));
        slots.push_back(it != dev->streams.end() ? it->second.slot : 0);
        for (auto& kv : dev->streams)
            if (kv.second.plan && kv.second.slot != slots[0]) slots.push_back(kv.second.slot);
    }
    static thread_local std::vector<KernelError> host;
    host.resize(mk_device::kStreamSlots);
    MK_CUDA(cudaMemcpy(host.data(), dev->kerr_words, sizeof(KernelError) * mk_device::kStreamSlots, cudaMemcpyDeviceToHost));
    if (code) *code = 0;
    for (int slot : slots) {
        const KernelError h = host[slot];
        if (h.code == 0) continue;
        if (code) *code = h.code;
        cudaMemset(dev->kerr_words + slot, 0, sizeof(KernelError));
        return fail(MK_ERR_KERNEL, "kernel error word 0x%x (block %u, detail %u): a bounded pipeline wait gave up", h.code,
                    h.block, h.detail);
    }
    return MK_OK;
}

// ---- module load / launch (driver API through runtime entry points) -----------------------------------------------
struct mk_module_impl {
    mk_device* dev;
    CUmodule mod;
};
struct mk_function_impl {
    mk_module_impl* m;
    CUfunction fn;
};

typedef CUresult (*PFN_cuModuleLoadData)(CUmodule*, const void*);
typedef CUresult (*PFN_cuModuleUnload)(CUmodule);
typedef CUresult (*PFN_cuModuleGetFunction)(CUfunction*, CUmodule, const char*);
typedef CUresult (*PFN_cuLaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream,
                                       void**, void**);
typedef CUresult (*PFN_cuFuncSetAttribute)(CUfunction, CUfunction_attribute, int);

static mk_status cu_fail(CUresult r, const char* what) { return fail(MK_ERR_CUDA, "driver error %d in %s", (int)r, what); }

mk_status mk_module_load(mk_device* dev, const void* image, size_t bytes, mk_module** out) {
    MK_REQUIRE(dev && image && bytes > 0 && out, "mk_module_load: bad argument");
    if (dev->mock) return fail(MK_ERR_CUDA, "mk_module_load: mock device cannot load modules");
    MK_CUDA(cudaSetDevice(dev->ordinal));
    MK_CUDA(cudaFree(0));
    auto load = (PFN_cuModuleLoadData)driver_entry("cuModuleLoadData");
    if (!load) return fail(MK_ERR_CUDA, "mk_module_load: cuModuleLoadData unavailable");
    // PTX images must be NUL-terminated; copy so that the caller's size is honoured.
    std::string copy((const char*)image, bytes);
    CUmodule mod;
    CUresult r = load(&mod, copy.c_str());
    if (r != CUDA_SUCCESS) return cu_fail(r, "cuModuleLoadData");
    *out = (mk_module*)new mk_module_impl{dev, mod};
    return MK_OK;
}

mk_status mk_module_unload(mk_module* m_) {
    MK_REQUIRE(m_, "mk_module_unload: null module");
    auto* m = (mk_module_impl*)m_;
    auto unload = (PFN_cuModuleUnload)driver_entry("cuModuleUnload");
    CUresult r = unload ? unload(m->mod) : CUDA_ERROR_NOT_FOUND;
    delete m;
    if (r != CUDA_SUCCESS) return cu_fail(r, "cuModuleUnload");
    return MK_OK;
}

mk_status mk_get_function(mk_module* m_, const char* name, mk_function** out) {
    MK_REQUIRE(m_ && name && out, "mk_get_function: null argument");
    auto* m = (mk_module_impl*)m_;
    auto get = (PFN_cuModuleGetFunction)driver_entry("cuModuleGetFunction");
    if (!get) return fail(MK_ERR_CUDA, "mk_get_function: cuModuleGetFunction unavailable");
    CUfunction fn;
    CUresult r = get(&fn, m->mod, name);
    if (r != CUDA_SUCCESS) return cu_fail(r, "cuModuleGetFunction");
    *out = (mk_function*)new mk_function_impl{m, fn};  // freed with the process; functions are cached by callers
    return MK_OK;
}

mk_status mk_launch(mk_function* f_, const uint32_t grid[3], const uint32_t block[3], uint32_t smem_bytes, mk_stream* s,
                    void** args) {
    MK_REQUIRE(f_ && grid && block, "mk_launch: null argument");
    auto* f = (mk_function_impl*)f_;
    MK_REQUIRE(grid[0] && grid[1] && grid[2] && block[0] && block[1] && block[2], "mk_launch: zero-sized launch");
    auto launch = (PFN_cuLaunchKernel)driver_entry("cuLaunchKernel");
    if (!launch) return fail(MK_ERR_CUDA, "mk_launch: cuLaunchKernel unavailable");
    if (smem_bytes > 48 * 1024) {
        auto setattr = (PFN_cuFuncSetAttribute)driver_entry("cuFuncSetAttribute");
        if (setattr) setattr(f->fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, (int)smem_bytes);
    }
    CUresult r = launch(f->fn, grid[0], grid[1], grid[2], block[0], block[1], block[2], smem_bytes, (CUstream)raw(s), args, nullptr);
    if (r != CUDA_SUCCESS) return cu_fail(r, "cuLaunchKernel");
    note_launch(f->m->dev, raw(s), "module_function");
    return MK_OK;
}

}  // extern "C"

// ---- per-stream state: slot (error word, claim counter), scratch, fence ------------------------------------------
namespace mk {
// Caller holds dev->mu.
static StreamState& stream_state_locked(mk_device* dev, cudaStream_t st) {
    auto it = dev->streams.find(st);
    if (it != dev->streams.end()) return it->second;
    StreamState ss;
    if (st != nullptr && !dev->free_slots.empty()) {     // the legacy stream keeps slot 0; so does everyone once the slots run out
        ss.slot = dev->free_slots.back();
        dev->free_slots.pop_back();
    }
    return dev->streams.emplace(st, std::move(ss)).first->second;
}

mk_status stream_scratch(mk_device* dev, cudaStream_t st, size_t bytes, void** out) {
    std::lock_guard<std::mutex> lk(dev->mu);
    StreamState& ss = stream_state_locked(dev, st);
    if (ss.scratch_bytes < bytes) {
        // Growing: work already enqueued on this stream, or recorded in a plan, may still use the old block,
        // so it is kept until the device is closed (no synchronisation here: this also runs during capture).
        if (ss.scratch) dev->retired_scratch.push_back(ss.scratch);
        ss.scratch = nullptr;
        ss.scratch_bytes = 0;
        const size_t want = (bytes + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);   // whole MiB
        void* p = nullptr;
        MK_CUDA(cudaMalloc(&p, want));
        ss.scratch = p;
        ss.scratch_bytes = want;
    }
    *out = ss.scratch;
    return MK_OK;
}

KernelError* stream_kerr(mk_device* dev, cudaStream_t st) {
    std::lock_guard<std::mutex> lk(dev->mu);
    return dev->kerr_words + stream_state_locked(dev, st).slot;
}

unsigned int* stream_work_counter(mk_device* dev, cudaStream_t st) {
    std::lock_guard<std::mutex> lk(dev->mu);
    return dev->work_counters + stream_state_locked(dev, st).slot;
}

void touch_stream(mk_device* dev, cudaStream_t st) {
    if (dev->mock) return;
    std::lock_guard<std::mutex> lk(dev->mu);
    stream_state_locked(dev, st).dirty = true;
}

void mark_plan_stream(mk_device* dev, cudaStream_t st) {
    std::lock_guard<std::mutex> lk(dev->mu);
    stream_state_locked(dev, st).plan = true;
}

void release_stream_state(mk_device* dev, cudaStream_t st) {
    std::lock_guard<std::mutex> lk(dev->mu);
    auto it = dev->streams.find(st);
    if (it == dev->streams.end()) return;
    if (it->second.scratch) cudaFree(it->second.scratch);
    if (it->second.slot != 0) dev->free_slots.push_back(it->second.slot);
    // Parked blocks may still hold this stream's fence: the event stays valid after the stream is destroyed
    // (work that was enqueued still completes), so waiting on it later is fine.
    dev->streams.erase(it);
}
}  // namespace mk


// ---- per-kernel timing -------------------------------------------------------------------------------------------
// The reference times each kernel of a plan on the host around a blocking call
// (runtime/src/execution_plan.rs:200-221).  Launches here are asynchronous, so a profile is a chain of
// events on one stream: one before the first kernel and one after each kernel this thread launches on that
// stream; a kernel's time is the span between its event and the one before it.
namespace mk {
namespace {
struct LaunchProfile {
    mk_device* dev = nullptr;
    cudaStream_t stream = nullptr;
    std::vector<cudaEvent_t> events;     // events[0] = start marker, events[i] = after kernel i-1
    std::vector<const char*> names;      // string literals of the launch sites
    bool failed = false;
};
thread_local LaunchProfile* t_profile = nullptr;

void drop_profile() {
    if (!t_profile) return;
    for (cudaEvent_t e : t_profile->events) cudaEventDestroy(e);
    delete t_profile;
    t_profile = nullptr;
}
}  // namespace

void note_launch(mk_device* dev, cudaStream_t st, const char* name) {
    dev->launches++;
    touch_stream(dev, st);
    LaunchProfile* p = t_profile;
    if (!p || p->dev != dev || p->stream != st) return;
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone) return;   // a recording plan is not timed
    cudaEvent_t e = nullptr;
    if (cudaEventCreate(&e) != cudaSuccess || cudaEventRecord(e, st) != cudaSuccess) {
        if (e) cudaEventDestroy(e);
        p->failed = true;
        return;
    }
    p->events.push_back(e);
    p->names.push_back(name);
}
}  // namespace mk

extern "C" {

mk_status mk_profile_begin(mk_device* dev, mk_stream* s) {
    MK_REQUIRE(dev, "mk_profile_begin: null device");
    MK_REQUIRE(!s || s->dev == dev, "mk_profile_begin: the stream belongs to another device");
    if (dev->mock) return fail(MK_ERR_CUDA, "mk_profile_begin: no CUDA device (mock devices run no kernels)");
    if (t_profile) return fail(MK_ERR_INVALID, "mk_profile_begin: this thread already records a profile");
    MK_CUDA(cudaSetDevice(dev->ordinal));
    cudaEvent_t e = nullptr;
    MK_CUDA(cudaEventCreate(&e));
    cudaError_t err = cudaEventRecord(e, raw(s));
    if (err != cudaSuccess) {
        cudaEventDestroy(e);
        return cuda_fail(err, "cudaEventRecord");
    }
    t_profile = new LaunchProfile();
    t_profile->dev = dev;
    t_profile->stream = raw(s);
    t_profile->events.push_back(e);
    return MK_OK;
}

mk_status mk_profile_end(mk_device* dev, mk_kernel_profile* out, int32_t capacity, int32_t* count) {
    MK_REQUIRE(dev && count && capacity >= 0 && (out || capacity == 0), "mk_profile_end: bad argument");
    if (!t_profile || t_profile->dev != dev) return fail(MK_ERR_INVALID, "mk_profile_end: this thread records no profile on this device");
    LaunchProfile& p = *t_profile;
    mk_status st = MK_OK;
    if (p.failed) st = fail(MK_ERR_CUDA, "mk_profile_end: an event could not be recorded; the profile is incomplete");
    cudaError_t err = st == MK_OK ? cudaEventSynchronize(p.events.back()) : cudaSuccess;
    if (err != cudaSuccess) st = cuda_fail(err, "cudaEventSynchronize");
    const int32_t n = (int32_t)p.names.size();
    for (int32_t i = 0; st == MK_OK && i < n && i < capacity; ++i) {
        std::memset(&out[i], 0, sizeof(out[i]));
        std::strncpy(out[i].name, p.names[i], sizeof(out[i].name) - 1);
        err = cudaEventElapsedTime(&out[i].elapsed_ms, p.events[i], p.events[i + 1]);
        if (err != cudaSuccess) st = cuda_fail(err, "cudaEventElapsedTime");
    }
    *count = n;
    drop_profile();
    return st;
}

}  // extern "C"
