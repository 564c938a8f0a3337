"""`Tensor`: the reference's lazy user API for the dense path, over libmorok_b200's graph mirror.

Method names, argument meaning and error behaviour follow morok's `Tensor`
(tensor/src/matmul.rs, tensor/src/transformer.rs, tensor/src/nn/norm.rs, tensor/src/activation.rs,
tensor/src/data.rs, tensor/src/realize.rs): operations only record a graph; `realize()` runs it
on the GPU; `as_vec` / `as_ndarray` read a realized tensor back and fail on an unrealized one.
bf16 has no host type in the reference either -- bf16 data goes in and out as raw 16-bit
patterns (`from_raw_bytes`, numpy uint16).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import numpy as np

from . import _ffi
from ._ffi import MK_BF16, MK_BOOL, MK_F16, MK_F32, check
from .device import Device

_NP = {MK_F32: np.float32, MK_BF16: np.uint16, MK_F16: np.float16, MK_BOOL: np.bool_}


def _i64(vals: Sequence[int]):
    return (C.c_int64 * max(len(vals), 1))(*vals)


class Tensor:
    def __init__(self, dev: Device, handle):
        self._dev, self._h = dev, handle

    def __del__(self):
        try:
            if self._h and self._dev.h:
                self._dev.lib.mk_tensor_free(self._h)
        except Exception:
            pass
        self._h = None

    # ---- construction (tensor/src/data.rs:23-139) -----------------------------------------------
    @staticmethod
    def from_raw_bytes(dev: Device, data: bytes, shape: Sequence[int], dtype: int) -> "Tensor":
        h = C.c_void_p()
        buf = (C.c_char * max(len(data), 1)).from_buffer_copy(data if len(data) else b"\0")
        check(dev.lib.mk_tensor_from_bytes(dev.h, buf, dtype, _i64(list(shape)), len(shape), C.byref(h)))
        return Tensor(dev, h)

    @staticmethod
    def from_ndarray(dev: Device, arr: np.ndarray, dtype: Optional[int] = None) -> "Tensor":
        """f32 / f16 arrays map to their dtype; uint16 arrays are bf16 bit patterns."""
        arr = np.ascontiguousarray(arr)
        if dtype is None:
            dtype = {np.dtype(np.float32): MK_F32, np.dtype(np.float16): MK_F16, np.dtype(np.uint16): MK_BF16,
                     np.dtype(np.bool_): MK_BOOL}.get(arr.dtype)      # bool arrays are attention masks (DType::Bool)
            if dtype is None:
                raise TypeError(f"unsupported array dtype {arr.dtype}")
        h = C.c_void_p()
        check(dev.lib.mk_tensor_from_bytes(dev.h, arr.ctypes.data_as(C.c_void_p), dtype, _i64(list(arr.shape)), arr.ndim,
                                           C.byref(h)))
        return Tensor(dev, h)

    @staticmethod
    def from_slice(dev: Device, values: Sequence[float]) -> "Tensor":
        return Tensor.from_ndarray(dev, np.asarray(values, dtype=np.float32))

    # ---- metadata ----------------------------------------------------------------------------------
    def _meta(self):
        shape = (C.c_int64 * _ffi.MK_MAX_DIMS)()
        nd, dt = C.c_int32(), C.c_int32()
        check(self._dev.lib.mk_tensor_shape(self._h, shape, C.byref(nd), C.byref(dt)))
        return tuple(shape[i] for i in range(nd.value)), dt.value

    def shape(self):
        return self._meta()[0]

    def ndim(self) -> int:
        return len(self.shape())

    def dtype(self) -> int:
        return self._meta()[1]

    def _unary(self, fn, *args) -> "Tensor":
        h = C.c_void_p()
        check(fn(self._h, *args, C.byref(h)))
        return Tensor(self._dev, h)

    # ---- dense ops ------------------------------------------------------------------------------------
    def matmul(self, other: "Tensor") -> "Tensor":
        """tensor/src/matmul.rs:54-56,82-110."""
        return self._unary(self._dev.lib.mk_tensor_matmul, other._h)

    dot = matmul

    def linear(self, weight: "Tensor", bias: Optional["Tensor"] = None) -> "Tensor":
        """x @ weight^T (+ bias); weight is stored [out, in]; a 1-D weight multiplies element-wise
        (tensor/src/matmul.rs:161-187)."""
        y = self.try_mul(weight) if weight.ndim() == 1 else self.matmul(weight.try_transpose(-1, -2))
        return y.try_add(bias) if bias is not None else y

    def gemm(self, b: "Tensor", alpha: float = 1.0, beta: float = 1.0, trans_a: bool = False, trans_b: bool = False,
             c: Optional["Tensor"] = None) -> "Tensor":
        """alpha * A @ B + beta * C, composed like the reference does (tensor/src/matmul.rs:112-133): transposes
        are views, the scale factors are one-element tensors multiplied in, and the add of an unscaled C
        lands in the GEMM's store."""
        a = self.try_transpose(0, 1) if trans_a else self
        bb = b.try_transpose(0, 1) if trans_b else b
        y = a.matmul(bb)
        _, dt = y._meta()
        scalar = {_ffi.MK_F32: np.float32, _ffi.MK_F16: np.float16}.get(dt)

        def const(v):
            if scalar is not None:
                return Tensor.from_ndarray(self._dev, np.array([v], scalar))
            bits = (np.array([v], np.float32).view(np.uint32) + 0x7FFF + ((np.array([v], np.float32).view(np.uint32) >> 16) & 1)) >> 16
            return Tensor.from_ndarray(self._dev, bits.astype(np.uint16))

        if alpha != 1.0:
            y = y.try_mul(const(alpha))
        if c is not None:
            y = y.try_add(c.try_mul(const(beta)) if beta != 1.0 else c)
        return y

    def scaled_dot_product_attention(self, key: "Tensor", value: "Tensor", attn_mask: Optional["Tensor"] = None,
                                     scale: Optional[float] = None, is_causal: bool = False,
                                     softcap: Optional[float] = None) -> "Tensor":
        """tensor/src/transformer.rs:78-137.  Q [B,H,Sq,D], K [B,Hkv,Sk,D], V [B,Hkv,Sk,Dv]; Hkv may
        divide H (the caller-side GQA expansion of the reference is folded into the kernel).  attn_mask: 2 to 4
        dimensions broadcastable against [B,H,Sq,Sk]; a bool tensor attends where true, any other is added."""
        return self._unary(self._dev.lib.mk_tensor_sdpa, key._h, value._h, attn_mask._h if attn_mask is not None else None,
                           float(scale) if scale else 0.0, int(is_causal), float(softcap) if softcap else 0.0)

    def rms_norm(self, axis: int = -1, eps: float = 1e-5) -> "Tensor":
        """tensor/src/nn/norm.rs:92-110 over the last axis; the result is f32 for 16-bit inputs."""
        if axis not in (-1, self.ndim() - 1):
            raise _ffi.MorokError(_ffi.MK_ERR_UNSUPPORTED, "rms_norm: only the last axis is supported")
        return self._unary(self._dev.lib.mk_tensor_rms_norm, float(eps))

    def apply_rotary_emb(self, cos: "Tensor", sin: "Tensor", interleaved: bool = False) -> "Tensor":
        """tensor/src/transformer.rs:32-69."""
        return self._unary(self._dev.lib.mk_tensor_rope, cos._h, sin._h, int(interleaved))

    def silu(self) -> "Tensor":
        return self._unary(self._dev.lib.mk_tensor_silu)

    swish = silu

    def sigmoid(self) -> "Tensor":
        """tensor/src/activation.rs:42."""
        return self._unary(self._dev.lib.mk_tensor_sigmoid)

    def try_add(self, other: "Tensor") -> "Tensor":
        return self._unary(self._dev.lib.mk_tensor_add, other._h)

    def try_mul(self, other: "Tensor") -> "Tensor":
        return self._unary(self._dev.lib.mk_tensor_mul, other._h)

    __add__ = try_add
    __mul__ = try_mul
    __matmul__ = matmul

    def cast(self, dtype: int) -> "Tensor":
        return self._unary(self._dev.lib.mk_tensor_cast, dtype)

    # ---- movement ops (views) -------------------------------------------------------------------------
    def try_reshape(self, shape: Sequence[int]) -> "Tensor":
        shape = list(shape)
        if -1 in shape:
            known = int(np.prod([s for s in shape if s != -1])) or 1
            shape[shape.index(-1)] = int(np.prod(self.shape())) // known
        return self._unary(self._dev.lib.mk_tensor_reshape, _i64(shape), len(shape))

    def try_permute(self, axes: Sequence[int]) -> "Tensor":
        nd = self.ndim()
        axes = [a % nd for a in axes]
        return self._unary(self._dev.lib.mk_tensor_permute, (C.c_int32 * max(nd, 1))(*axes), len(axes))

    def try_transpose(self, a: int, b: int) -> "Tensor":
        nd = self.ndim()
        axes = list(range(nd))
        axes[a % nd], axes[b % nd] = axes[b % nd], axes[a % nd]
        return self.try_permute(axes)

    # ---- execution and extraction (tensor/src/realize.rs:83, tensor/src/data.rs:165-262) ----------------
    def realize(self) -> "Tensor":
        check(self._dev.lib.mk_tensor_realize(self._h))
        return self

    def realize_profiled(self):
        """realize() with per-kernel device times: [(kernel name, milliseconds)] in launch order, the
        counterpart of ExecutionPlan::execute_profiled (runtime/src/execution_plan.rs:200-221)."""
        self._dev.profile_begin()
        try:
            check(self._dev.lib.mk_tensor_realize(self._h))
        finally:
            prof = self._dev.profile_end()
        return prof

    def last_launches(self) -> int:
        n = C.c_int32()
        check(self._dev.lib.mk_tensor_last_launches(self._h, C.byref(n)))
        return n.value

    def as_ndarray(self) -> np.ndarray:
        """Realized tensors only.  bf16 comes back as uint16 bit patterns."""
        shape, dt = self._meta()
        out = np.empty(shape, dtype=_NP[dt])
        check(self._dev.lib.mk_tensor_copyout(self._h, out.ctypes.data_as(C.c_void_p), out.nbytes))
        return out

    def as_vec(self) -> np.ndarray:
        return self.as_ndarray().reshape(-1)

    def write(self, arr: np.ndarray) -> "Tensor":
        """Overwrites the data of a realized tensor in place (the input side of a plan replay)."""
        arr = np.ascontiguousarray(arr)
        check(self._dev.lib.mk_tensor_write(self._h, arr.ctypes.data_as(C.c_void_p), arr.nbytes))
        return self

    # ---- prepare once, execute many (runtime/src/execution_plan.rs:88-106, 168-181) ----------------------
    def compile(self) -> "Plan":
        """Records the kernels that realize() would launch into a plan instead of running them."""
        h = C.c_void_p()
        check(self._dev.lib.mk_tensor_compile(self._h, C.byref(h)))
        return Plan(self._dev, h, self)


class Plan:
    """A recorded realisation: `launch()` replays all of its kernels with one call."""

    def __init__(self, dev: Device, handle, result: Tensor):
        self._dev, self._h, self.result = dev, handle, result

    def launch(self, stream=None) -> "Plan":
        check(self._dev.lib.mk_plan_launch(self._h, stream.h if stream else None))
        return self

    def kernel_count(self) -> int:
        n = C.c_int32()
        check(self._dev.lib.mk_plan_kernel_count(self._h, C.byref(n)))
        return n.value

    def free(self):
        if self._h:
            self._dev.lib.mk_plan_free(self._h)
            self._h = None

    def __del__(self):
        try:
            if self._dev.h:
                self.free()
        except Exception:
            pass
