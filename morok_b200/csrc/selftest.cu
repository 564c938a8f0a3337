// Self-test of the bounded pipeline wait.
//
// Every barrier wait of the tensor-core kernels goes through ptx::mbar_wait, which gives up after a
// time limit, records a code in the device's error word and lets the kernel return, so a pipeline
// that lost a signal costs one failed call instead of a hung GPU.  This file exercises exactly that
// path without any fault: one warp waits, with a limit of milliseconds, on a barrier that no thread
// and no copy ever signals.  The wait runs out, the kernel records KERR_SELFTEST_WAIT and exits
// normally; the host then sees MK_ERR_KERNEL from mk_kernel_status and the context stays usable.
// The reference has no device-side waits of its own (its kernels are generated straight-line code);
// the host-side counterpart is the deadline polling of device/src/sync.rs:248-306.
#include "mk_internal.h"
#include "ptx_sm100.cuh"

namespace mk {
namespace {

__global__ void __launch_bounds__(32) bounded_wait_selftest_kernel(KernelError* kerr, uint64_t limit_ns, uint32_t* outcome) {
    __shared__ uint64_t bar;
    __shared__ uint32_t abort_flag;
    if (threadIdx.x == 0) {
        ptx::mbar_init(ptx::smem_u32(&bar), 1);   // one arrival expected; nothing ever arrives
        abort_flag = 0;
        ptx::fence_barrier_init();
    }
    __syncwarp();
    bool done = true;
    if (threadIdx.x == 0)
        done = ptx::mbar_wait(ptx::smem_u32(&bar), 0, &abort_flag, kerr, KERR_SELFTEST_WAIT, 0, limit_ns);
    done = __shfl_sync(0xffffffffu, done ? 1 : 0, 0) != 0;
    // Lanes that did not wait observe the CTA-wide abort flag, as the other roles of a real kernel do.
    if (threadIdx.x == 1) *outcome = (done ? 1u : 0u) | (abort_flag ? 2u : 0u);
}

}  // namespace
}  // namespace mk

using namespace mk;

extern "C" mk_status mk_selftest_bounded_wait(mk_device* dev, mk_stream* s, uint32_t limit_ms) {
    MK_REQUIRE(dev, "mk_selftest_bounded_wait: null device");
    if (dev->mock) return fail(MK_ERR_CUDA, "mk_selftest_bounded_wait: mock device runs no kernels");
    MK_REQUIRE(limit_ms >= 1 && limit_ms <= 1000, "mk_selftest_bounded_wait: limit_ms must be in 1..1000, got %u", limit_ms);
    MK_CUDA(cudaSetDevice(dev->ordinal));
    // four bytes from the allocator cache receive what the non-waiting lanes saw
    mk_buf* out = nullptr;
    mk_status st = mk_alloc(dev, sizeof(uint32_t), 0, &out);
    if (st != MK_OK) return st;
    void* out_ptr = nullptr;
    st = mk_buf_ptr(out, &out_ptr);
    if (st != MK_OK) { mk_free(out); return st; }
    bounded_wait_selftest_kernel<<<1, 32, 0, raw(s)>>>(stream_kerr(dev, raw(s)), (uint64_t)limit_ms * 1000000ull, (uint32_t*)out_ptr);
    cudaError_t e = cudaGetLastError();
    note_launch(dev, raw(s), "bounded_wait_selftest");
    uint32_t outcome = 0;
    if (e == cudaSuccess) e = cudaMemcpyAsync(&outcome, out_ptr, sizeof(outcome), cudaMemcpyDeviceToHost, raw(s));
    if (e == cudaSuccess) e = cudaStreamSynchronize(raw(s));
    mk_free(out);
    if (e != cudaSuccess) return fail(MK_ERR_CUDA, "mk_selftest_bounded_wait: %s", cudaGetErrorString(e));
    // Expected: the wait returned false (bit 0 clear) and the abort flag was raised (bit 1 set).
    if (outcome != 2u) return fail(MK_ERR_CUDA, "mk_selftest_bounded_wait: the wait did not run out as designed (outcome %u)", outcome);
    return MK_OK;
}
