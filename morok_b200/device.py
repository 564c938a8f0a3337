"""Thin object layer over the C ABI: Device, Buffer, Stream, Event and the compute calls.

Mirrors the pieces of morok's `device` and `runtime` crates that the dense path touches
(`Buffer` with lazy allocation / views / copyin / copyout: device/src/buffer.rs:39-603;
allocator statistics and LRU reuse: device/src/allocator.rs:322-442; streams and events:
device/src/queue.rs, device/src/sync.rs).  All work happens in libmorok_b200.so; nothing here
computes on the host.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import numpy as np

from . import _ffi
from ._ffi import MK_BF16, MK_BOOL, MK_F16, MK_F32, MK_F8E4M3, MK_F8E5M2, check

_NP_OF = {MK_F32: np.float32, MK_BF16: np.uint16, MK_F16: np.float16, MK_F8E4M3: np.uint8, MK_F8E5M2: np.uint8, MK_BOOL: np.bool_}
_SIZE_OF = {MK_F32: 4, MK_BF16: 2, MK_F16: 2, MK_F8E4M3: 1, MK_F8E5M2: 1, MK_BOOL: 1}


def dtype_size(dt: int) -> int:
    return _SIZE_OF[dt]


class Stream:
    def __init__(self, dev: "Device"):
        self.dev = dev
        h = C.c_void_p()
        check(dev.lib.mk_stream_create(dev.h, C.byref(h)))
        self.h = h

    def sync(self):
        check(self.dev.lib.mk_stream_sync(self.h))

    def raw(self) -> int:
        p = C.c_void_p()
        check(self.dev.lib.mk_stream_raw(self.h, C.byref(p)))
        return p.value or 0

    def close(self):
        if self.h:
            check(self.dev.lib.mk_stream_destroy(self.h))
            self.h = None


class Event:
    def __init__(self, dev: "Device"):
        self.dev = dev
        h = C.c_void_p()
        check(dev.lib.mk_event_create(dev.h, C.byref(h)))
        self.h = h

    def record(self, stream: Optional[Stream] = None):
        check(self.dev.lib.mk_event_record(self.h, stream.h if stream else None))

    def wait(self, timeout_ms: int = 10000):
        check(self.dev.lib.mk_event_wait(self.h, timeout_ms))

    def elapsed_ms(self, stop: "Event") -> float:
        ms = C.c_float()
        check(self.dev.lib.mk_event_elapsed_ms(self.h, stop.h, C.byref(ms)))
        return ms.value

    def close(self):
        if self.h:
            self.dev.lib.mk_event_destroy(self.h)
            self.h = None


class Buffer:
    """Lazy device buffer (no memory until first use) or a view into one."""

    def __init__(self, dev: "Device", handle, nbytes: int):
        self.dev, self.h, self.nbytes = dev, handle, nbytes

    @property
    def ptr(self) -> int:
        p = C.c_void_p()
        check(self.dev.lib.mk_buf_ptr(self.h, C.byref(p)))
        return p.value or 0

    @property
    def is_allocated(self) -> bool:
        a = C.c_int32()
        check(self.dev.lib.mk_buf_is_allocated(self.h, C.byref(a)))
        return bool(a.value)

    def view(self, offset: int, nbytes: int) -> "Buffer":
        h = C.c_void_p()
        check(self.dev.lib.mk_buf_view(self.h, offset, nbytes, C.byref(h)))
        return Buffer(self.dev, h, nbytes)

    def copyin(self, arr: np.ndarray, stream: Optional[Stream] = None):
        arr = np.ascontiguousarray(arr)
        check(self.dev.lib.mk_copy_h2d(self.h, arr.ctypes.data_as(C.c_void_p), arr.nbytes, stream.h if stream else None))

    def copyout(self, dtype, shape, stream: Optional[Stream] = None) -> np.ndarray:
        out = np.empty(shape, dtype=dtype)
        check(self.dev.lib.mk_copy_d2h(out.ctypes.data_as(C.c_void_p), self.h, out.nbytes, stream.h if stream else None))
        return out

    def copy_from(self, src: "Buffer", stream: Optional[Stream] = None):
        check(self.dev.lib.mk_copy_d2d(self.h, src.h, src.nbytes, stream.h if stream else None))

    def free(self):
        if self.h:
            check(self.dev.lib.mk_free(self.h))
            self.h = None


class Device:
    """An opened B200 (or, with mock=True, the host-memory test fake that runs no kernels)."""

    def __init__(self, ordinal: int = 0, mock: bool = False):
        self.lib = _ffi.load()
        h = C.c_void_p()
        if mock:
            check(self.lib.mk_device_open_mock(C.byref(h)))
        else:
            check(self.lib.mk_device_open(ordinal, C.byref(h)))
        self.h = h
        self.mock = mock

    # -- housekeeping ---------------------------------------------------------------------------
    def close(self):
        if self.h:
            check(self.lib.mk_device_close(self.h))
            self.h = None

    def info(self) -> _ffi.DeviceInfo:
        inf = _ffi.DeviceInfo()
        check(self.lib.mk_device_get_info(self.h, C.byref(inf)))
        return inf

    def sync(self):
        check(self.lib.mk_device_sync(self.h))

    def stats(self) -> dict:
        s = _ffi.AllocStats()
        check(self.lib.mk_alloc_stats(self.h, C.byref(s)))
        return {n: getattr(s, n) for n, _ in s._fields_}

    def trim(self):
        check(self.lib.mk_alloc_trim(self.h))

    def inject_oom(self, count: int):
        check(self.lib.mk_alloc_inject_oom(self.h, count))

    def kernel_status(self, stream: Optional[Stream] = None) -> int:
        code = C.c_uint32()
        check(self.lib.mk_kernel_status(self.h, stream.h if stream else None, C.byref(code)))
        return code.value

    def selftest_bounded_wait(self, limit_ms: int = 50, stream: Optional[Stream] = None):
        """Runs the kernel whose barrier wait is designed to run out after `limit_ms`; the recorded
        error is then read (and cleared) with `kernel_status`, which raises MorokError(MK_ERR_KERNEL)."""
        check(self.lib.mk_selftest_bounded_wait(self.h, stream.h if stream else None, limit_ms))

    def launch_count(self) -> int:
        n = C.c_uint64()
        check(self.lib.mk_launch_count(self.h, C.byref(n)))
        return n.value

    def profile_begin(self, stream=None):
        """Starts stamping the kernels this thread launches on `stream` (runtime/src/execution_plan.rs:200-221)."""
        check(self.lib.mk_profile_begin(self.h, stream.h if stream else None))

    def profile_end(self, capacity: int = 256):
        """Ends the profile: [(kernel name, milliseconds)] in launch order."""
        out = (_ffi.KernelProfile * capacity)()
        n = C.c_int32()
        check(self.lib.mk_profile_end(self.h, out, capacity, C.byref(n)))
        return [(out[i].name.decode(), float(out[i].elapsed_ms)) for i in range(min(n.value, capacity))]

    # -- memory -----------------------------------------------------------------------------------
    def alloc(self, nbytes: int, zero: bool = False) -> Buffer:
        h = C.c_void_p()
        check(self.lib.mk_alloc(self.h, nbytes, _ffi.MK_ALLOC_ZERO_INIT if zero else 0, C.byref(h)))
        return Buffer(self, h, nbytes)

    def from_numpy(self, arr: np.ndarray, stream: Optional[Stream] = None) -> Buffer:
        arr = np.ascontiguousarray(arr)
        b = self.alloc(arr.nbytes)
        b.copyin(arr, stream)
        return b

    # -- compute ------------------------------------------------------------------------------------
    @staticmethod
    def gemm_desc(a: Buffer, b: Buffer, c: Buffer, M: int, N: int, K: int, dtype_in: int, dtype_out: Optional[int] = None,
                  trans_b: bool = False, lda: Optional[int] = None, ldb: Optional[int] = None, ldc: Optional[int] = None,
                  add: Optional[Buffer] = None, batch: int = 1, stride_a: int = 0, stride_b: int = 0, stride_c: int = 0,
                  peers: Sequence[int] = (), c_ptr: Optional[int] = None,
                  bias: Optional[Buffer] = None, alpha: Optional[float] = None, beta: Optional[float] = None,
                  swiglu_with: Optional[Buffer] = None, gate: str = "silu", gate_bias: Optional[Buffer] = None,
                  up_bias: Optional[Buffer] = None) -> "_ffi.GemmDesc":
        """The mk_gemm_desc of C = alpha * A B + beta * add (full matrix) or + beta * bias (one row of N elements);
        with swiglu_with = B2: C = gate(A B + gate_bias) * (A B2 + up_bias), gate "silu" or "sigmoid"."""
        d = _ffi.GemmDesc()
        d.dtype_in, d.dtype_out = dtype_in, dtype_in if dtype_out is None else dtype_out
        d.M, d.N, d.K = M, N, K
        d.A, d.lda = a.ptr, K if lda is None else lda
        d.B, d.ldb = b.ptr, (K if trans_b else N) if ldb is None else ldb
        d.C, d.ldc = (c.ptr if c_ptr is None else c_ptr), N if ldc is None else ldc
        d.trans_b, d.batch = int(trans_b), batch
        d.stride_a, d.stride_b, d.stride_c = stride_a, stride_b, stride_c
        d.epilogue, d.D = (_ffi.MK_EPI_ADD, add.ptr) if add is not None else \
            (_ffi.MK_EPI_ADD_ROW, bias.ptr) if bias is not None else (_ffi.MK_EPI_NONE, None)
        if swiglu_with is not None:       # C = silu(A B) * (A B2)
            d.epilogue, d.B2 = _ffi.MK_EPI_SWIGLU, swiglu_with.ptr
            d.D = gate_bias.ptr if gate_bias is not None else None
            d.D2 = up_bias.ptr if up_bias is not None else None
            if gate == "sigmoid":
                d.flags |= _ffi.MK_GEMM_GATE_SIGMOID
            elif gate != "silu":
                raise ValueError(f"gate must be 'silu' or 'sigmoid', not {gate!r}")
        if alpha is not None or beta is not None:
            d.flags |= _ffi.MK_GEMM_SCALED
            d.alpha, d.beta = (1.0 if alpha is None else alpha), (1.0 if beta is None else beta)
        d.n_peers = len(peers)
        for i, p in enumerate(peers):
            d.peer_C[i] = p
        return d

    def gemm(self, *args, stream: Optional[Stream] = None, **kw):
        """mk_gemm; the arguments are gemm_desc's."""
        d = self.gemm_desc(*args, **kw)
        check(self.lib.mk_gemm(self.h, stream.h if stream else None, C.byref(d)))

    # -- GEMM schedule tuning (schedule/src/optimizer/beam.rs:223-291, 390-397, 445-524) ------------
    def gemm_autotune(self, *args, iters: int = 10, stream: Optional[Stream] = None, **kw) -> dict:
        """Times the schedule candidates of this problem and keeps the fastest for later calls."""
        d = self.gemm_desc(*args, **kw)
        t = _ffi.GemmTuning()
        check(self.lib.mk_gemm_autotune(self.h, stream.h if stream else None, C.byref(d), iters, C.byref(t)))
        return {n: getattr(t, n) for n, _ in _ffi.GemmTuning._fields_}

    def gemm_tuning_get(self, *args, **kw) -> Optional[dict]:
        d = self.gemm_desc(*args, **kw)
        t, found = _ffi.GemmTuning(), C.c_int32()
        check(self.lib.mk_gemm_tuning_get(self.h, C.byref(d), C.byref(t), C.byref(found)))
        return {n: getattr(t, n) for n, _ in _ffi.GemmTuning._fields_} if found.value else None

    def gemm_tuning_set(self, tuning: Optional[dict], *args, **kw):
        d = self.gemm_desc(*args, **kw)
        if tuning is None:
            check(self.lib.mk_gemm_tuning_set(self.h, C.byref(d), None))
            return
        t = _ffi.GemmTuning(tuning.get("pair", -1), tuning.get("group_m", 0), tuning.get("splits", 0), 0,
                            tuning.get("best_ms", 0.0), tuning.get("default_ms", 0.0))
        check(self.lib.mk_gemm_tuning_set(self.h, C.byref(d), C.byref(t)))

    def tuning_save(self, path: str):
        check(self.lib.mk_tuning_save(self.h, path.encode()))

    def tuning_load(self, path: str) -> int:
        n = C.c_int32()
        check(self.lib.mk_tuning_load(self.h, path.encode(), C.byref(n)))
        return n.value

    def tuning_clear(self):
        check(self.lib.mk_tuning_clear(self.h))

    def sdpa(self, q: Buffer, k: Buffer, v: Buffer, o: Buffer, B: int, Hq: int, Hkv: int, Sq: int, Sk: int, D: int,
             Dv: Optional[int] = None, dtype: int = MK_BF16, scale: float = 0.0, causal: bool = False,
             softcap: float = 0.0, mask: Optional[Buffer] = None, lse: Optional[Buffer] = None,
             q_strides=None, k_strides=None, v_strides=None, o_strides=None, peers: Sequence[int] = (),
             stream: Optional[Stream] = None, o_ptr: Optional[int] = None, causal_offset: int = 0,
             mask_strides: Optional[Sequence[int]] = None, mask_bool: bool = False):
        """mk_sdpa_fwd.  mask: additive f32 [Sq, Sk] by default; with mask_strides = (batch, head, row) element strides
        (0 broadcasts) any shape that broadcasts against [B, Hq, Sq, Sk]; mask_bool: one byte per element, non-zero attends."""
        Dv = D if Dv is None else Dv
        d = _ffi.SdpaDesc()
        d.dtype, d.B, d.Hq, d.Hkv, d.Sq, d.Sk, d.D, d.Dv = dtype, B, Hq, Hkv, Sq, Sk, D, Dv
        d.scale, d.causal, d.softcap, d.causal_offset = scale, int(causal), softcap, causal_offset
        d.Q, d.K, d.V, d.O = q.ptr, k.ptr, v.ptr, (o.ptr if o_ptr is None else o_ptr)

        def contiguous(H, S, dim):
            return (H * S * dim, S * dim, dim)
        for name, val, dflt in (("q_strides", q_strides, contiguous(Hq, Sq, D)), ("k_strides", k_strides, contiguous(Hkv, Sk, D)),
                                ("v_strides", v_strides, contiguous(Hkv, Sk, Dv)), ("o_strides", o_strides, contiguous(Hq, Sq, Dv))):
            arr = getattr(d, name)
            for i, x in enumerate(val if val is not None else dflt):
                arr[i] = x
        d.mask = mask.ptr if mask is not None else None
        if mask is not None and (mask_strides is not None or mask_bool):
            d.mask_kind = _ffi.MK_MASK_BOOL if mask_bool else _ffi.MK_MASK_F32
            for i, x in enumerate(mask_strides if mask_strides is not None else (0, 0, Sk)):
                d.mask_strides[i] = x
        d.lse = lse.ptr if lse is not None else None
        d.n_peers = len(peers)
        for i, p in enumerate(peers):
            d.peer_O[i] = p
        check(self.lib.mk_sdpa_fwd(self.h, stream.h if stream else None, C.byref(d)))

    def rms_norm(self, x: Buffer, y: Buffer, rows: int, cols: int, eps: float, dtype_in: int, dtype_out: Optional[int] = None,
                 gain: Optional[Buffer] = None, stream: Optional[Stream] = None):
        check(self.lib.mk_rms_norm(self.h, stream.h if stream else None, dtype_in, dtype_in if dtype_out is None else dtype_out,
                                   x.ptr, gain.ptr if gain is not None else None, y.ptr, rows, cols, eps))

    def rope(self, x: Buffer, cos: Buffer, sin: Buffer, y: Buffer, rows: int, D: int, rows_cs: int, row_div: int,
             dtype: int, interleaved: bool = False, stream: Optional[Stream] = None):
        check(self.lib.mk_rope(self.h, stream.h if stream else None, dtype, x.ptr, cos.ptr, sin.ptr, y.ptr, rows, D,
                               rows_cs, row_div, int(interleaved)))

    def swiglu(self, gate: Buffer, up: Buffer, y: Buffer, n: int, dtype: int, stream: Optional[Stream] = None):
        check(self.lib.mk_swiglu(self.h, stream.h if stream else None, dtype, gate.ptr, up.ptr, y.ptr, n))

    def add(self, a: Buffer, b: Buffer, y: Buffer, n: int, dtype: int, stream: Optional[Stream] = None):
        check(self.lib.mk_add(self.h, stream.h if stream else None, dtype, a.ptr, b.ptr, y.ptr, n))

    def cast(self, x: Buffer, y: Buffer, n: int, dtype_in: int, dtype_out: int, stream: Optional[Stream] = None):
        check(self.lib.mk_cast(self.h, stream.h if stream else None, dtype_in, dtype_out, x.ptr, y.ptr, n))


def device_count() -> int:
    n = C.c_int32()
    st = _ffi.load().mk_device_count(C.byref(n))
    return n.value if st == _ffi.MK_OK else 0
