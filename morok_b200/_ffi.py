"""ctypes binding of libmorok_b200.so -- one Python prototype per symbol of include/morok_b200.h.

This is the same kind of stub a morok maintainer would write in Rust (`extern "C"` block) to
bind the library; Python is used here because it drives the tests and the benchmark.
The library is loaded from the package directory.  There is no fallback: if the shared object
is missing or does not load, importing the compute API raises.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("MOROK_B200_LIB") or os.path.join(HERE, "libmorok_b200.so")   # override: A/B builds

MK_OK, MK_ERR_INVALID, MK_ERR_CUDA, MK_ERR_OOM = 0, -1, -2, -3
MK_ERR_SIZE_MISMATCH, MK_ERR_NOT_ALLOCATED, MK_ERR_TIMEOUT, MK_ERR_UNSUPPORTED, MK_ERR_KERNEL = -4, -5, -6, -7, -8
MK_F32, MK_BF16, MK_F16, MK_F8E4M3, MK_F8E5M2, MK_BOOL = 0, 1, 2, 3, 4, 5
MK_MASK_SQ_SK, MK_MASK_F32, MK_MASK_BOOL = 0, 1, 2
MK_ALLOC_ZERO_INIT = 1
MK_EPI_NONE, MK_EPI_ADD, MK_EPI_ADD_ROW, MK_EPI_SWIGLU = 0, 1, 2, 3
MK_GEMM_SCALED, MK_GEMM_GATE_SIGMOID = 1, 2
MK_MAX_PEERS = 8
MK_MAX_DIMS = 6
MK_STATIC_GEMM_MAX_BATCH = 256

vp, i32, i64, u32, u64, f32, sz = C.c_void_p, C.c_int32, C.c_int64, C.c_uint32, C.c_uint64, C.c_float, C.c_size_t
P = C.POINTER


class DeviceInfo(C.Structure):
    _fields_ = [("ordinal", i32), ("sm_count", i32), ("cc_major", i32), ("cc_minor", i32),
                ("max_smem_per_block", i32), ("l2_bytes", i32), ("total_mem", i64), ("name", C.c_char * 128)]


class AllocStats(C.Structure):
    _fields_ = [(n, u64) for n in ("device_allocs", "device_frees", "cache_hits", "cache_returns", "oom_flushes",
                                   "bytes_in_use", "bytes_cached", "peak_bytes_in_use")]


class GemmDesc(C.Structure):
    _fields_ = [("dtype_in", i32), ("dtype_out", i32), ("M", i64), ("N", i64), ("K", i64),
                ("A", vp), ("lda", i64), ("B", vp), ("ldb", i64), ("C", vp), ("ldc", i64),
                ("trans_b", i32), ("batch", i32), ("stride_a", i64), ("stride_b", i64), ("stride_c", i64),
                ("epilogue", i32), ("D", vp), ("n_peers", i32), ("peer_C", vp * MK_MAX_PEERS),
                ("alpha", f32), ("beta", f32), ("flags", u32), ("B2", vp), ("D2", vp)]


class SdpaDesc(C.Structure):
    _fields_ = [("dtype", i32), ("B", i32), ("Hq", i32), ("Hkv", i32), ("Sq", i32), ("Sk", i32), ("D", i32),
                ("Dv", i32), ("scale", f32), ("causal", i32), ("softcap", f32),
                ("Q", vp), ("K", vp), ("V", vp), ("O", vp),
                ("q_strides", i64 * 3), ("k_strides", i64 * 3), ("v_strides", i64 * 3), ("o_strides", i64 * 3),
                ("mask", vp), ("lse", vp), ("n_peers", i32), ("peer_O", vp * MK_MAX_PEERS), ("causal_offset", i32),
                ("mask_kind", i32), ("mask_strides", i64 * 3)]


class GemmTuning(C.Structure):
    _fields_ = [("pair", i32), ("group_m", i32), ("splits", i32), ("candidates", i32), ("best_ms", f32), ("default_ms", f32)]


class KernelProfile(C.Structure):
    _fields_ = [("name", C.c_char * 56), ("elapsed_ms", f32), ("reserved", i32)]


class IpcHandle(C.Structure):
    _fields_ = [("bytes", C.c_ubyte * 64)]


# name -> (restype, argtypes); every exported symbol of include/morok_b200.h
PROTOTYPES = {
    "mk_last_error": (C.c_char_p, []),
    "mk_abi_version": (i32, []),
    "mk_abi_struct_size": (i32, [i32]),
    "mk_device_count": (i32, [P(i32)]),
    "mk_device_open": (i32, [i32, P(vp)]),
    "mk_device_open_mock": (i32, [P(vp)]),
    "mk_device_close": (i32, [vp]),
    "mk_device_get_info": (i32, [vp, P(DeviceInfo)]),
    "mk_device_sync": (i32, [vp]),
    "mk_stream_create": (i32, [vp, P(vp)]),
    "mk_stream_destroy": (i32, [vp]),
    "mk_stream_sync": (i32, [vp]),
    "mk_stream_wait_event": (i32, [vp, vp]),
    "mk_stream_raw": (i32, [vp, P(vp)]),
    "mk_event_create": (i32, [vp, P(vp)]),
    "mk_event_destroy": (i32, [vp]),
    "mk_event_record": (i32, [vp, vp]),
    "mk_event_wait": (i32, [vp, i32]),
    "mk_event_elapsed_ms": (i32, [vp, vp, P(f32)]),
    "mk_alloc": (i32, [vp, sz, u32, P(vp)]),
    "mk_buf_ensure": (i32, [vp]),
    "mk_buf_ptr": (i32, [vp, P(vp)]),
    "mk_buf_size": (i32, [vp, P(sz)]),
    "mk_buf_is_allocated": (i32, [vp, P(i32)]),
    "mk_buf_view": (i32, [vp, sz, sz, P(vp)]),
    "mk_free": (i32, [vp]),
    "mk_alloc_stats": (i32, [vp, P(AllocStats)]),
    "mk_alloc_trim": (i32, [vp]),
    "mk_alloc_inject_oom": (i32, [vp, i32]),
    "mk_copy_h2d": (i32, [vp, vp, sz, vp]),
    "mk_copy_d2h": (i32, [vp, vp, sz, vp]),
    "mk_copy_d2d": (i32, [vp, vp, sz, vp]),
    "mk_copy_p2p": (i32, [vp, vp, sz, vp]),
    "mk_host_alloc": (i32, [sz, P(vp)]),
    "mk_host_free": (i32, [vp]),
    "mk_memcpy_async": (i32, [vp, vp, vp, sz, i32, vp]),
    "mk_memset_async": (i32, [vp, vp, i32, sz, vp]),
    "mk_mem_info": (i32, [vp, P(sz), P(sz)]),
    "mk_module_load": (i32, [vp, vp, sz, P(vp)]),
    "mk_module_unload": (i32, [vp]),
    "mk_get_function": (i32, [vp, C.c_char_p, P(vp)]),
    "mk_launch": (i32, [vp, P(u32), P(u32), u32, vp, P(vp)]),
    "mk_gemm": (i32, [vp, vp, P(GemmDesc)]),
    "mk_gemm_static": (i32, [i32, vp, P(GemmDesc), P(u32)]),
    "mk_gemm_static_status": (i32, [i32, vp, i32, P(u32)]),
    "mk_gemm_autotune": (i32, [vp, vp, P(GemmDesc), i32, P(GemmTuning)]),
    "mk_gemm_tuning_set": (i32, [vp, P(GemmDesc), P(GemmTuning)]),
    "mk_gemm_tuning_get": (i32, [vp, P(GemmDesc), P(GemmTuning), P(i32)]),
    "mk_tuning_save": (i32, [vp, C.c_char_p]),
    "mk_tuning_load": (i32, [vp, C.c_char_p, P(i32)]),
    "mk_tuning_clear": (i32, [vp]),
    "mk_sdpa_fwd": (i32, [vp, vp, P(SdpaDesc)]),
    "mk_rms_norm": (i32, [vp, vp, i32, i32, vp, vp, vp, i64, i64, f32]),
    "mk_rope": (i32, [vp, vp, i32, vp, vp, vp, vp, i64, i32, i64, i64, i32]),
    "mk_swiglu": (i32, [vp, vp, i32, vp, vp, vp, i64]),
    "mk_add": (i32, [vp, vp, i32, vp, vp, vp, i64]),
    "mk_cast": (i32, [vp, vp, i32, i32, vp, vp, i64]),
    "mk_ipc_export": (i32, [vp, P(IpcHandle), P(sz)]),
    "mk_ipc_open": (i32, [vp, P(IpcHandle), sz, sz, P(vp)]),
    "mk_all_gather_push": (i32, [vp, vp, vp, sz, P(vp), i32, sz]),
    "mk_all_gather_push_2d": (i32, [vp, vp, vp, sz, sz, sz, P(vp), i32, sz, sz]),
    "mk_kernel_status": (i32, [vp, vp, P(u32)]),
    "mk_selftest_bounded_wait": (i32, [vp, vp, u32]),
    "mk_launch_count": (i32, [vp, P(u64)]),
    "mk_profile_begin": (i32, [vp, vp]),
    "mk_profile_end": (i32, [vp, P(KernelProfile), i32, P(i32)]),
    "mk_tensor_from_bytes": (i32, [vp, vp, i32, P(i64), i32, P(vp)]),
    "mk_tensor_free": (i32, [vp]),
    "mk_tensor_shape": (i32, [vp, P(i64), P(i32), P(i32)]),
    "mk_tensor_matmul": (i32, [vp, vp, P(vp)]),
    "mk_tensor_sdpa": (i32, [vp, vp, vp, vp, f32, i32, f32, P(vp)]),
    "mk_tensor_rms_norm": (i32, [vp, f32, P(vp)]),
    "mk_tensor_rope": (i32, [vp, vp, vp, i32, P(vp)]),
    "mk_tensor_silu": (i32, [vp, P(vp)]),
    "mk_tensor_sigmoid": (i32, [vp, P(vp)]),
    "mk_tensor_add": (i32, [vp, vp, P(vp)]),
    "mk_tensor_mul": (i32, [vp, vp, P(vp)]),
    "mk_tensor_cast": (i32, [vp, i32, P(vp)]),
    "mk_tensor_reshape": (i32, [vp, P(i64), i32, P(vp)]),
    "mk_tensor_permute": (i32, [vp, P(i32), i32, P(vp)]),
    "mk_tensor_realize": (i32, [vp]),
    "mk_tensor_last_launches": (i32, [vp, P(i32)]),
    "mk_tensor_copyout": (i32, [vp, vp, sz]),
    "mk_tensor_write": (i32, [vp, vp, sz]),
    "mk_tensor_compile": (i32, [vp, P(vp)]),
    "mk_plan_launch": (i32, [vp, vp]),
    "mk_plan_kernel_count": (i32, [vp, P(i32)]),
    "mk_plan_free": (i32, [vp]),
}

_lib = None


class MorokError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"[mk_status {status}] {message}")
        self.status = status


def load() -> C.CDLL:
    """Loads the shared library and binds every prototype.  Raises when it is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m morok_b200._build` (needs nvcc). "
                "There is no CPU fallback for the compute path.")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def check(status: int):
    if status != MK_OK:
        raise MorokError(status, load().mk_last_error().decode(errors="replace"))
