//! B200 device for morok, bound to `libmorok_b200.so` (C ABI in `include/morok_b200.h`).
//!
//! UNCOMPILED: the environment this library was built in has no Rust toolchain.  The file is the glue a
//! maintainer adds to the `device` / `runtime` crates: (1) the `extern "C"` declarations, one per symbol of the
//! header, with `#[repr(C)]` mirrors of its structs; (2) the `Allocator`, `Renderer`, `Program` implementations
//! and the factory registered for `DeviceSpec::Cuda`.  The same calls, in the same order, are exercised from
//! Python ctypes (`morok_b200/_ffi.py`) and from the C++ Tensor mirror (`morok_b200/csrc/tensor.cpp`) by the
//! test-suite; a test keeps the symbol list below in step with the header.
//!
//! Reference interfaces this replaces (paths relative to the morok repository):
//!   runtime/src/device_registry.rs:66-67   the commented-out CUDA factory
//!   device/src/buffer.rs:567-572           `Buffer::as_raw_ptr`, `unimplemented!()` for CUDA
//!   device/src/allocator.rs:164-190,256-309,322-442   `Allocator`, `CudaAllocator`, `LruAllocator`
//!   device/src/device.rs:34-60,186-222,255-298         `Program`, `Renderer`, `Device`
#![allow(non_camel_case_types, dead_code)]

use std::ffi::{c_char, c_void, CStr};
use std::ptr;
use std::sync::Arc;

// ---------------------------------------------------------------------------------------------------------
// 1. FFI surface
// ---------------------------------------------------------------------------------------------------------
pub const MK_MAX_PEERS: usize = 8;
pub const MK_MAX_DIMS: usize = 6;

#[repr(C)] pub struct MkDeviceInfo { pub ordinal: i32, pub sm_count: i32, pub cc_major: i32, pub cc_minor: i32,
    pub max_smem_per_block: i32, pub l2_bytes: i32, pub total_mem: i64, pub name: [c_char; 128] }
#[repr(C)] pub struct MkAllocStats { pub device_allocs: u64, pub device_frees: u64, pub cache_hits: u64, pub cache_returns: u64,
    pub oom_flushes: u64, pub bytes_in_use: u64, pub bytes_cached: u64, pub peak_bytes_in_use: u64 }
#[repr(C)] #[derive(Clone)] pub struct MkGemmDesc { pub dtype_in: i32, pub dtype_out: i32, pub m: i64, pub n: i64, pub k: i64,
    pub a: *const u8, pub lda: i64, pub b: *const u8, pub ldb: i64, pub c: *mut u8, pub ldc: i64,
    pub trans_b: i32, pub batch: i32, pub stride_a: i64, pub stride_b: i64, pub stride_c: i64,
    pub epilogue: i32, pub d: *const u8, pub n_peers: i32, pub peer_c: [*mut u8; MK_MAX_PEERS],
    pub alpha: f32, pub beta: f32, pub flags: u32,           // flags & 1 (MK_GEMM_SCALED): alpha, beta are used
    pub b2: *const u8,                                        // MK_EPI_SWIGLU: act(A B + d) * (A B2 + d2)
    pub d2: *const u8 }                                       //   flags & 2 (MK_GEMM_GATE_SIGMOID): act = sigmoid, else silu
#[repr(C)] #[derive(Clone)] pub struct MkSdpaDesc { pub dtype: i32, pub b: i32, pub hq: i32, pub hkv: i32, pub sq: i32, pub sk: i32,
    pub d: i32, pub dv: i32, pub scale: f32, pub causal: i32, pub softcap: f32,
    pub q: *const u8, pub k: *const u8, pub v: *const u8, pub o: *mut u8,
    pub q_strides: [i64; 3], pub k_strides: [i64; 3], pub v_strides: [i64; 3], pub o_strides: [i64; 3],
    pub mask: *const c_void, pub lse: *mut f32, pub n_peers: i32, pub peer_o: [*mut u8; MK_MAX_PEERS],
    pub causal_offset: i32,                                   // past_seq_len of a key/value cache
    pub mask_kind: i32,                                       // 0: f32 [Sq,Sk]; 1: f32 with strides; 2: bool with strides
    pub mask_strides: [i64; 3] }                              // batch, head, query row (0 broadcasts)
#[repr(C)] pub struct MkGemmTuning { pub pair: i32, pub group_m: i32, pub splits: i32, pub candidates: i32,
    pub best_ms: f32, pub default_ms: f32 }
#[repr(C)] pub struct MkKernelProfile { pub name: [c_char; 56], pub elapsed_ms: f32, pub reserved: i32 }
#[repr(C)] pub struct MkIpcHandle { pub bytes: [u8; 64] }

pub enum MkDevice {} pub enum MkStream {} pub enum MkBuf {} pub enum MkEvent {} pub enum MkModule {} pub enum MkFunction {}
pub enum MkTensor {} pub enum MkPlan {}

#[link(name = "morok_b200")]
extern "C" {
    pub fn mk_last_error() -> *const c_char;
    pub fn mk_abi_version() -> i32;
    pub fn mk_abi_struct_size(which: i32) -> i32;
    // device
    pub fn mk_device_count(count: *mut i32) -> i32;
    pub fn mk_device_open(ordinal: i32, out: *mut *mut MkDevice) -> i32;
    pub fn mk_device_open_mock(out: *mut *mut MkDevice) -> i32;
    pub fn mk_device_close(dev: *mut MkDevice) -> i32;
    pub fn mk_device_get_info(dev: *mut MkDevice, info: *mut MkDeviceInfo) -> i32;
    pub fn mk_device_sync(dev: *mut MkDevice) -> i32;
    // streams and events
    pub fn mk_stream_create(dev: *mut MkDevice, out: *mut *mut MkStream) -> i32;
    pub fn mk_stream_destroy(s: *mut MkStream) -> i32;
    pub fn mk_stream_sync(s: *mut MkStream) -> i32;
    pub fn mk_stream_wait_event(s: *mut MkStream, ev: *mut MkEvent) -> i32;
    pub fn mk_stream_raw(s: *mut MkStream, cuda_stream: *mut *mut c_void) -> i32;
    pub fn mk_event_create(dev: *mut MkDevice, out: *mut *mut MkEvent) -> i32;
    pub fn mk_event_destroy(ev: *mut MkEvent) -> i32;
    pub fn mk_event_record(ev: *mut MkEvent, s: *mut MkStream) -> i32;
    pub fn mk_event_wait(ev: *mut MkEvent, timeout_ms: i32) -> i32;
    pub fn mk_event_elapsed_ms(start: *mut MkEvent, stop: *mut MkEvent, ms: *mut f32) -> i32;
    // allocator
    pub fn mk_alloc(dev: *mut MkDevice, bytes: usize, flags: u32, out: *mut *mut MkBuf) -> i32;
    pub fn mk_buf_ensure(buf: *mut MkBuf) -> i32;
    pub fn mk_buf_ptr(buf: *mut MkBuf, dptr: *mut *mut u8) -> i32;
    pub fn mk_buf_size(buf: *mut MkBuf, bytes: *mut usize) -> i32;
    pub fn mk_buf_is_allocated(buf: *mut MkBuf, allocated: *mut i32) -> i32;
    pub fn mk_buf_view(buf: *mut MkBuf, off: usize, len: usize, out: *mut *mut MkBuf) -> i32;
    pub fn mk_free(buf: *mut MkBuf) -> i32;
    pub fn mk_alloc_stats(dev: *mut MkDevice, stats: *mut MkAllocStats) -> i32;
    pub fn mk_alloc_trim(dev: *mut MkDevice) -> i32;
    pub fn mk_alloc_inject_oom(dev: *mut MkDevice, count: i32) -> i32;
    pub fn mk_mem_info(dev: *mut MkDevice, free_bytes: *mut usize, total_bytes: *mut usize) -> i32;
    // copies
    pub fn mk_copy_h2d(dst: *mut MkBuf, src: *const u8, bytes: usize, s: *mut MkStream) -> i32;
    pub fn mk_copy_d2h(dst: *mut u8, src: *mut MkBuf, bytes: usize, s: *mut MkStream) -> i32;
    pub fn mk_copy_d2d(dst: *mut MkBuf, src: *mut MkBuf, bytes: usize, s: *mut MkStream) -> i32;
    pub fn mk_copy_p2p(dst: *mut MkBuf, src: *mut MkBuf, bytes: usize, s: *mut MkStream) -> i32;
    pub fn mk_host_alloc(bytes: usize, out: *mut *mut c_void) -> i32;
    pub fn mk_host_free(p: *mut c_void) -> i32;
    pub fn mk_memcpy_async(dev: *mut MkDevice, dst: *mut c_void, src: *const c_void, bytes: usize, kind: i32, s: *mut MkStream) -> i32;
    pub fn mk_memset_async(dev: *mut MkDevice, dst: *mut c_void, byte_value: i32, bytes: usize, s: *mut MkStream) -> i32;
    // module load and launch
    pub fn mk_module_load(dev: *mut MkDevice, image: *const c_void, bytes: usize, out: *mut *mut MkModule) -> i32;
    pub fn mk_module_unload(m: *mut MkModule) -> i32;
    pub fn mk_get_function(m: *mut MkModule, name: *const c_char, out: *mut *mut MkFunction) -> i32;
    pub fn mk_launch(f: *mut MkFunction, grid: *const u32, block: *const u32, smem_bytes: u32, s: *mut MkStream, args: *mut *mut c_void) -> i32;
    // kernels
    pub fn mk_gemm(dev: *mut MkDevice, s: *mut MkStream, d: *const MkGemmDesc) -> i32;
    pub fn mk_gemm_static(device_ordinal: i32, cuda_stream: *mut c_void, d: *const MkGemmDesc, kernel_error: *mut u32) -> i32;
    pub fn mk_gemm_static_status(device_ordinal: i32, cuda_stream: *mut c_void, batch: i32, kernel_error: *mut u32) -> i32;
    pub fn mk_gemm_autotune(dev: *mut MkDevice, s: *mut MkStream, d: *const MkGemmDesc, iters: i32, out: *mut MkGemmTuning) -> i32;
    pub fn mk_gemm_tuning_set(dev: *mut MkDevice, d: *const MkGemmDesc, t: *const MkGemmTuning) -> i32;
    pub fn mk_gemm_tuning_get(dev: *mut MkDevice, d: *const MkGemmDesc, t: *mut MkGemmTuning, found: *mut i32) -> i32;
    pub fn mk_tuning_save(dev: *mut MkDevice, path: *const c_char) -> i32;          // the beam cache's file
    pub fn mk_tuning_load(dev: *mut MkDevice, path: *const c_char, entries: *mut i32) -> i32;
    pub fn mk_tuning_clear(dev: *mut MkDevice) -> i32;
    pub fn mk_sdpa_fwd(dev: *mut MkDevice, s: *mut MkStream, d: *const MkSdpaDesc) -> i32;
    pub fn mk_rms_norm(dev: *mut MkDevice, s: *mut MkStream, dt_in: i32, dt_out: i32, x: *const u8, gain: *const u8,
                       y: *mut u8, rows: i64, cols: i64, eps: f32) -> i32;
    pub fn mk_rope(dev: *mut MkDevice, s: *mut MkStream, dtype: i32, x: *const u8, cosv: *const f32, sinv: *const f32, y: *mut u8,
                   rows: i64, d: i32, rows_cs: i64, row_div: i64, interleaved: i32) -> i32;
    pub fn mk_swiglu(dev: *mut MkDevice, s: *mut MkStream, dtype: i32, gate: *const u8, up: *const u8, y: *mut u8, n: i64) -> i32;
    pub fn mk_add(dev: *mut MkDevice, s: *mut MkStream, dtype: i32, a: *const u8, b: *const u8, y: *mut u8, n: i64) -> i32;
    pub fn mk_cast(dev: *mut MkDevice, s: *mut MkStream, dt_in: i32, dt_out: i32, x: *const u8, y: *mut u8, n: i64) -> i32;
    // multi-GPU plumbing
    pub fn mk_ipc_export(buf: *mut MkBuf, handle: *mut MkIpcHandle, offset: *mut usize) -> i32;
    pub fn mk_ipc_open(dev: *mut MkDevice, handle: *const MkIpcHandle, offset: usize, bytes: usize, out: *mut *mut MkBuf) -> i32;
    pub fn mk_all_gather_push(dev: *mut MkDevice, s: *mut MkStream, src: *const c_void, bytes: usize, dst: *const *mut c_void, n_dst: i32,
                              dst_offset: usize) -> i32;
    pub fn mk_all_gather_push_2d(dev: *mut MkDevice, s: *mut MkStream, src: *const c_void, src_pitch: usize, row_bytes: usize, rows: usize,
                                 dst: *const *mut c_void, n_dst: i32, dst_offset: usize, dst_pitch: usize) -> i32;
    // kernel error words, launch counter, per-kernel profiles
    pub fn mk_kernel_status(dev: *mut MkDevice, s: *mut MkStream, code: *mut u32) -> i32;
    pub fn mk_selftest_bounded_wait(dev: *mut MkDevice, s: *mut MkStream, limit_ms: u32) -> i32;
    pub fn mk_launch_count(dev: *mut MkDevice, launches: *mut u64) -> i32;
    pub fn mk_profile_begin(dev: *mut MkDevice, s: *mut MkStream) -> i32;           // ExecutionPlan::execute_profiled
    pub fn mk_profile_end(dev: *mut MkDevice, out: *mut MkKernelProfile, capacity: i32, count: *mut i32) -> i32;
    // lazy Tensor mirror and plans
    pub fn mk_tensor_from_bytes(dev: *mut MkDevice, data: *const c_void, dtype: i32, shape: *const i64, ndim: i32, out: *mut *mut MkTensor) -> i32;
    pub fn mk_tensor_free(t: *mut MkTensor) -> i32;
    pub fn mk_tensor_shape(t: *mut MkTensor, shape: *mut i64, ndim: *mut i32, dtype: *mut i32) -> i32;
    pub fn mk_tensor_matmul(a: *mut MkTensor, b: *mut MkTensor, out: *mut *mut MkTensor) -> i32;
    pub fn mk_tensor_sdpa(q: *mut MkTensor, k: *mut MkTensor, v: *mut MkTensor, mask: *mut MkTensor, scale: f32, causal: i32, softcap: f32,
                          out: *mut *mut MkTensor) -> i32;
    pub fn mk_tensor_rms_norm(x: *mut MkTensor, eps: f32, out: *mut *mut MkTensor) -> i32;
    pub fn mk_tensor_rope(x: *mut MkTensor, cosv: *mut MkTensor, sinv: *mut MkTensor, interleaved: i32, out: *mut *mut MkTensor) -> i32;
    pub fn mk_tensor_silu(x: *mut MkTensor, out: *mut *mut MkTensor) -> i32;
    pub fn mk_tensor_sigmoid(x: *mut MkTensor, out: *mut *mut MkTensor) -> i32;
    pub fn mk_tensor_add(a: *mut MkTensor, b: *mut MkTensor, out: *mut *mut MkTensor) -> i32;
    pub fn mk_tensor_mul(a: *mut MkTensor, b: *mut MkTensor, out: *mut *mut MkTensor) -> i32;
    pub fn mk_tensor_cast(x: *mut MkTensor, dtype: i32, out: *mut *mut MkTensor) -> i32;
    pub fn mk_tensor_reshape(x: *mut MkTensor, shape: *const i64, ndim: i32, out: *mut *mut MkTensor) -> i32;
    pub fn mk_tensor_permute(x: *mut MkTensor, axes: *const i32, ndim: i32, out: *mut *mut MkTensor) -> i32;
    pub fn mk_tensor_realize(t: *mut MkTensor) -> i32;
    pub fn mk_tensor_last_launches(t: *mut MkTensor, launches: *mut i32) -> i32;
    pub fn mk_tensor_copyout(t: *mut MkTensor, dst: *mut c_void, bytes: usize) -> i32;
    pub fn mk_tensor_write(t: *mut MkTensor, data: *const c_void, bytes: usize) -> i32;
    pub fn mk_tensor_compile(t: *mut MkTensor, out: *mut *mut MkPlan) -> i32;
    pub fn mk_plan_launch(plan: *mut MkPlan, s: *mut MkStream) -> i32;
    pub fn mk_plan_kernel_count(plan: *mut MkPlan, kernels: *mut i32) -> i32;
    pub fn mk_plan_free(plan: *mut MkPlan) -> i32;
}

/// Status code -> morok's error enum (device/src/error.rs:5-51).  No panic crosses the boundary.
fn check(st: i32) -> morok_device::Result<()> {
    if st == 0 { return Ok(()) }
    let message = unsafe { CStr::from_ptr(mk_last_error()) }.to_string_lossy().into_owned();
    Err(match st {
        -4 => morok_device::Error::SizeMismatch { message },
        -5 => morok_device::Error::NotAllocated,
        _ => morok_device::Error::Runtime { message },       // -8 (MK_ERR_KERNEL): a bounded pipeline wait gave up
    })
}

// ---------------------------------------------------------------------------------------------------------
// 2. The `Device` bundle (runtime/src/devices/b200.rs)
// ---------------------------------------------------------------------------------------------------------
use morok_device::{Allocator, BufferOptions, Compiler, Device, Program, ProgramSpec, RawBuffer, Renderer};
use morok_dtype::DeviceSpec;
use morok_ir::UOp;

struct B200Allocator { dev: *mut MkDevice, spec: DeviceSpec }
unsafe impl Send for B200Allocator {}
unsafe impl Sync for B200Allocator {}                                 // handles are usable from any thread; the allocator locks internally

impl Allocator for B200Allocator {                                    // device/src/allocator.rs:164-190
    fn alloc(&self, size: usize, opts: &BufferOptions) -> morok_device::Result<RawBuffer> {
        let mut b = ptr::null_mut();
        check(unsafe { mk_alloc(self.dev, size, opts.zero_init as u32, &mut b) })?;    // lazy + LRU + stream-ordered reuse inside
        Ok(RawBuffer::B200(b))
    }
    fn free(&self, buf: RawBuffer, _: &BufferOptions) { if let RawBuffer::B200(b) = buf { unsafe { mk_free(b); } } }
    fn synchronize(&self) -> morok_device::Result<()> { check(unsafe { mk_device_sync(self.dev) }) }
    fn name(&self) -> &'static str { "B200" }
    fn device_spec(&self) -> DeviceSpec { self.spec.clone() }
}
// Buffer::as_raw_ptr (device/src/buffer.rs:567-572):   RawBuffer::B200(b) => { mk_buf_ptr(b, &mut p); p.add(offset) }
// Buffer::copyin / copyout / copy_from (332-534):       mk_copy_h2d / mk_copy_d2h / mk_copy_d2d (size-checked there as here)

/// What a compiled "kernel" is on this device: a call descriptor instead of source code.
#[derive(Clone)]
enum KernelCall { Gemm(MkGemmDesc), Sdpa(MkSdpaDesc) }

/// "Rendering" a kernel AST = recognising it and emitting the call descriptor (device/src/device.rs:186-222).
struct B200Renderer;
impl Renderer for B200Renderer {
    fn render(&self, ast: &Arc<UOp>, _name: Option<&str>) -> morok_device::Result<ProgramSpec> {
        if let Some(mm) = morok_schedule::optimizer::tc::detect_matmul(ast) {            // schedule/src/optimizer/tc.rs:36-94
            return Ok(ProgramSpec::call("mk_gemm", encode_gemm(&mm)));                    // dtypes, M/N/K, strides, fused `+ c`
        }
        Err(morok_device::Error::Runtime { message: "B200 device runs matmul and attention kernels only".into() })
    }
}

struct B200Program { dev: *mut MkDevice, call: KernelCall }
unsafe impl Send for B200Program {}
unsafe impl Sync for B200Program {}
impl Program for B200Program {                                        // device/src/device.rs:34-60
    unsafe fn execute(&self, buffers: &[*mut u8], _vals: &[i64], _g: Option<[usize; 3]>, _l: Option<[usize; 3]>) -> morok_device::Result<()> {
        match &self.call {   // buffers arrive in PARAM-slot order: output first, then inputs (tensor/src/realize.rs:877-915)
            KernelCall::Gemm(d) => { let mut d = d.clone(); d.c = buffers[0]; d.a = buffers[1]; d.b = buffers[2];
                                     check(mk_gemm(self.dev, ptr::null_mut(), &d)) }
            KernelCall::Sdpa(d) => { let mut d = d.clone(); d.o = buffers[0]; d.q = buffers[1]; d.k = buffers[2]; d.v = buffers[3];
                                     check(mk_sdpa_fwd(self.dev, ptr::null_mut(), &d)) }
        }
    }
    fn name(&self) -> &str { match self.call { KernelCall::Gemm(_) => "mk_gemm", KernelCall::Sdpa(_) => "mk_sdpa_fwd" } }
}

/// runtime/src/device_registry.rs:81-83 -- replaces the commented-out line 66-67.
pub fn register() {
    morok_runtime::DEVICE_FACTORIES.register_factory("CUDA", Arc::new(|spec, _reg| {
        let DeviceSpec::Cuda { device_id } = spec else { unreachable!() };
        debug_assert_eq!(unsafe { mk_abi_struct_size(0) } as usize, std::mem::size_of::<MkGemmDesc>());
        debug_assert_eq!(unsafe { mk_abi_struct_size(1) } as usize, std::mem::size_of::<MkSdpaDesc>());
        let mut dev = ptr::null_mut();
        check(unsafe { mk_device_open(*device_id as i32, &mut dev) })?;
        Ok(Device { device: spec.clone(), allocator: Arc::new(B200Allocator { dev, spec: spec.clone() }),
                    renderer: Arc::new(B200Renderer), compiler: Arc::new(PassThroughCompiler),
                    runtime: Arc::new(move |c| Ok(Box::new(B200Program { dev, call: decode(c)? }))) })
    }));
}
// Attention has no single kernel AST in the reference (it schedules >= 5 kernels), so its matcher sits one level up,
// where the graph is still whole: in `prepare_with` (tensor/src/realize.rs:299-357) match
// matmul -> mul(scale) -> where(tril) -> [mask] -> [softcap] -> softmax -> matmul and emit one KernelCall::Sdpa.
