"""The C-ABI library loads without a GPU and exports every symbol include/morok_b200.h declares;
host-side logic (allocator policy, views, size checks, error reporting) runs on the mock device."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import morok_b200 as mk
from morok_b200 import _ffi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "morok_b200.h")).read()
    return sorted(set(re.findall(r"MK_API\s+[\w\s\*]+?\b(mk_\w+)\s*\(", text)))


def test_header_symbols_exported_and_bound():
    lib = _ffi.load()
    names = declared_symbols()
    assert len(names) >= 60
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
        assert n in _ffi.PROTOTYPES, f"{n} has no ctypes prototype"
    assert set(_ffi.PROTOTYPES) <= set(names), set(_ffi.PROTOTYPES) - set(names)
    assert lib.mk_abi_version() == 4


def test_rust_shim_declares_every_header_symbol():
    """ffi/morok_b200_device.rs (uncompiled: no Rust toolchain here) stays in step with the header."""
    text = open(os.path.join(ROOT, "ffi", "morok_b200_device.rs")).read()
    declared = set(re.findall(r"pub fn (mk_\w+)\(", text))
    assert declared == set(declared_symbols()), (set(declared_symbols()) - declared, declared - set(declared_symbols()))
    # the struct mirrors carry the fields the header added last
    for field in ("mask_kind", "mask_strides", "causal_offset", "b2", "d2"):
        assert f"pub {field}:" in text


def test_struct_layouts_match_header():
    lib = _ffi.load()
    # the natural-alignment sizes of the declared field lists ...
    assert C.sizeof(_ffi.GemmDesc) == 8 + 24 + 6 * 8 + 8 + 24 + 8 + 8 + 8 + 8 * 8 + 16 + 8 + 8
    assert C.sizeof(_ffi.IpcHandle) == 64
    # ... and the hand-written ctypes mirrors against what the C compiler made of the header
    assert lib.mk_abi_struct_size(0) == C.sizeof(_ffi.GemmDesc)
    assert lib.mk_abi_struct_size(1) == C.sizeof(_ffi.SdpaDesc)
    assert lib.mk_abi_struct_size(7) == -1
    assert C.sizeof(_ffi.AllocStats) == 64


def test_no_gpu_fails_loudly():
    if mk.device_count() > 0:
        pytest.skip("a GPU is present")
    with pytest.raises(mk.MorokError) as e:
        mk.Device(0)
    assert e.value.status == _ffi.MK_ERR_CUDA


def test_mock_device_lazy_alloc_and_lru_reuse():
    dev = mk.Device(mock=True)
    b = dev.alloc(4096)
    assert not b.is_allocated                      # lazy: nothing reserved yet
    assert dev.stats()["device_allocs"] == 0
    p1 = b.ptr
    assert b.is_allocated and dev.stats()["device_allocs"] == 1
    b.free()
    s = dev.stats()
    assert s["cache_returns"] == 1 and s["bytes_cached"] == 4096 and s["bytes_in_use"] == 0
    b2 = dev.alloc(4096)
    assert b2.ptr == p1                            # LRU reuse by pointer identity
    assert dev.stats()["cache_hits"] == 1
    b3 = dev.alloc(8192)                           # other size class: fresh allocation
    assert b3.ptr != p1 and dev.stats()["device_allocs"] == 2
    b2.free(); b3.free()
    dev.trim()
    assert dev.stats()["bytes_cached"] == 0
    dev.close()


def test_mock_device_cache_cap_32_per_size():
    dev = mk.Device(mock=True)
    bufs = [dev.alloc(1024) for _ in range(40)]
    for b in bufs:
        b.ptr
    for b in bufs:
        b.free()
    s = dev.stats()
    assert s["cache_returns"] == 32 and s["device_frees"] == 8
    dev.close()


def test_mock_device_oom_flush_and_retry():
    dev = mk.Device(mock=True)
    a = dev.alloc(2048); a.ptr; a.free()           # one block parked in the cache
    dev.inject_oom(1)
    b = dev.alloc(1 << 20)
    assert b.ptr != 0                              # first try "fails", cache is flushed, retry succeeds
    s = dev.stats()
    assert s["oom_flushes"] == 1 and s["bytes_cached"] == 0
    dev.inject_oom(2)                              # both tries fail -> MK_ERR_OOM, no crash
    c = dev.alloc(1 << 20)
    with pytest.raises(mk.MorokError) as e:
        c.ptr
    assert e.value.status == _ffi.MK_ERR_OOM
    assert c.ptr != 0                              # and the allocator recovers afterwards
    dev.close()


def test_mock_device_views_copies_and_size_checks():
    dev = mk.Device(mock=True)
    x = np.arange(64, dtype=np.float32)
    b = dev.from_numpy(x)
    assert np.array_equal(b.copyout(np.float32, (64,)), x)
    v = b.view(64, 128)                            # elements 16..47
    assert v.ptr == b.ptr + 64
    assert np.array_equal(v.copyout(np.float32, (32,)), x[16:48])
    with pytest.raises(mk.MorokError) as e:
        b.copyin(np.zeros(3, np.float32))
    assert e.value.status == _ffi.MK_ERR_SIZE_MISMATCH
    with pytest.raises(mk.MorokError) as e:
        b.view(200, 100)
    assert e.value.status == _ffi.MK_ERR_INVALID
    fresh = dev.alloc(16)
    with pytest.raises(mk.MorokError) as e:
        fresh.copyout(np.float32, (4,))
    assert e.value.status == _ffi.MK_ERR_NOT_ALLOCATED
    z = dev.alloc(256, zero=True)
    assert np.all(z.copyout(np.uint8, (256,)) == 0)
    # a view keeps the allocation alive after the parent handle is freed
    b.free()
    assert np.array_equal(v.copyout(np.float32, (32,)), x[16:48])
    v.free()
    assert dev.stats()["bytes_in_use"] == 512      # only z remains (sizes round up to 512-byte classes)
    dev.close()


def test_mock_device_runs_no_kernels():
    dev = mk.Device(mock=True)
    a = dev.alloc(64); b = dev.alloc(64); c = dev.alloc(64)
    for fn in (lambda: dev.gemm(a, b, c, 4, 4, 4, mk.MK_F32),
               lambda: dev.sdpa(a, b, c, c, 1, 1, 1, 2, 2, 2, dtype=mk.MK_F32),
               lambda: dev.add(a, b, c, 16, mk.MK_F32),
               lambda: dev.rms_norm(a, c, 4, 4, 1e-5, mk.MK_F32)):
        with pytest.raises(mk.MorokError) as e:
            fn()
        assert e.value.status == _ffi.MK_ERR_CUDA
    dev.close()


def test_argument_validation_reports_messages():
    dev = mk.Device(mock=True)
    a = dev.alloc(64)
    with pytest.raises(mk.MorokError) as e:
        dev.gemm(a, a, a, -1, 4, 4, mk.MK_F32)
    assert e.value.status == _ffi.MK_ERR_INVALID and "negative" in str(e.value)
    with pytest.raises(mk.MorokError) as e:
        dev.gemm(a, a, a, 4, 4, 4, 7)
    assert e.value.status == _ffi.MK_ERR_INVALID
    with pytest.raises(mk.MorokError) as e:
        dev.sdpa(a, a, a, a, 1, 3, 2, 2, 2, 2, dtype=mk.MK_F32)   # Hq not a multiple of Hkv
    assert "multiple" in str(e.value)
    with pytest.raises(mk.MorokError) as e:                        # a mask that broadcasts is described by strides >= 0
        dev.sdpa(a, a, a, a, 1, 2, 2, 2, 2, 8, dtype=mk.MK_BF16, mask=a, mask_strides=(-4, 0, 2))
    assert e.value.status == _ffi.MK_ERR_INVALID and "mask stride" in str(e.value)
    with pytest.raises(mk.MorokError) as e:                        # every announced peer needs a buffer
        dev.sdpa(a, a, a, a, 1, 2, 2, 2, 2, 8, dtype=mk.MK_BF16, peers=[0])
    assert e.value.status == _ffi.MK_ERR_INVALID and "peer_O" in str(e.value)
    dev.close()


def test_profile_needs_a_cuda_device_and_a_begin():
    dev = mk.Device(mock=True)
    with pytest.raises(mk.MorokError) as e:
        dev.profile_begin()
    assert e.value.status == _ffi.MK_ERR_CUDA
    with pytest.raises(mk.MorokError) as e:
        dev.profile_end()
    assert e.value.status == _ffi.MK_ERR_INVALID and "no profile" in str(e.value)
    dev.close()


def test_allocator_is_safe_under_racing_threads():
    """Handles are usable from any thread and the allocator locks internally: the reference's buffers
    race the same way (device/src/buffer.rs:58-73, a double allocation is freed again)."""
    import threading
    dev = mk.Device(mock=True)
    errors = []

    def worker(seed):
        try:
            rng = np.random.default_rng(seed)
            held = []
            for _ in range(300):
                if held and rng.random() < 0.5:
                    held.pop(int(rng.integers(len(held)))).free()
                else:
                    b = dev.alloc(int(rng.choice([512, 1024, 4096, 65536])))
                    assert b.ptr != 0
                    held.append(b)
            for b in held:
                b.free()
        except Exception as ex:     # noqa: BLE001
            errors.append(ex)

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(8)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    s = dev.stats()
    assert s["bytes_in_use"] == 0
    assert s["device_allocs"] + s["cache_hits"] >= 8          # every first touch either allocated or reused
    # one shared buffer first touched by many threads resolves to a single allocation
    shared = dev.alloc(2048)
    before = dev.stats()["device_allocs"] + dev.stats()["cache_hits"]
    ptrs = []
    ts = [threading.Thread(target=lambda: ptrs.append(shared.ptr)) for _ in range(8)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    assert len(set(ptrs)) == 1
    assert dev.stats()["device_allocs"] + dev.stats()["cache_hits"] == before + 1
    shared.free()
    dev.trim()
    s = dev.stats()
    assert s["bytes_cached"] == 0 and s["device_allocs"] == s["device_frees"]
    dev.close()


def test_gemm_tuning_records_round_trip_through_a_file(tmp_path):
    """The tuning cache: records keyed by the problem, kept in the device, saved to and loaded from a
    file (the reference's beam-search cache: schedule/src/optimizer/beam.rs:390-397, 445-524)."""
    dev = mk.Device(mock=True)
    a = dev.alloc(64)
    prob = (a, a, a, 16, 4096, 4096, mk.MK_BF16)
    assert dev.gemm_tuning_get(*prob) is None
    dev.gemm_tuning_set({"pair": 0, "group_m": 8, "splits": 6, "best_ms": 0.02, "default_ms": 0.03}, *prob)
    dev.gemm_tuning_set({"pair": 1, "group_m": 16}, a, a, a, 8192, 14336, 4096, mk.MK_BF16, mk.MK_F32, trans_b=True)
    got = dev.gemm_tuning_get(*prob)
    assert (got["pair"], got["group_m"], got["splits"]) == (0, 8, 6)
    assert dev.gemm_tuning_get(a, a, a, 16, 4096, 4096, mk.MK_F16) is None            # another dtype: another problem
    assert dev.gemm_tuning_get(a, a, a, 16, 4096, 4096, mk.MK_BF16, trans_b=True) is None
    path = str(tmp_path / "tuning.txt")
    dev.tuning_save(path)
    dev.tuning_clear()
    assert dev.gemm_tuning_get(*prob) is None
    assert dev.tuning_load(path) == 2
    got = dev.gemm_tuning_get(*prob)
    assert (got["pair"], got["group_m"], got["splits"]) == (0, 8, 6) and abs(got["best_ms"] - 0.02) < 1e-6
    got = dev.gemm_tuning_get(a, a, a, 8192, 14336, 4096, mk.MK_BF16, mk.MK_F32, trans_b=True)
    assert (got["pair"], got["group_m"], got["splits"]) == (1, 16, 0)
    dev.gemm_tuning_set(None, *prob)                                                   # forget one record
    assert dev.gemm_tuning_get(*prob) is None
    # values out of range, malformed and foreign files are refused with a message, nothing is half-loaded
    with pytest.raises(mk.MorokError) as e:
        dev.gemm_tuning_set({"pair": 2}, *prob)
    assert e.value.status == _ffi.MK_ERR_INVALID
    lines = open(path).read().splitlines()
    bad = str(tmp_path / "bad.txt")
    open(bad, "w").write("\n".join([lines[0], lines[1], "16 4096 4096 1 1 0 0 0 1 0 8"]) + "\n")
    dev.tuning_clear()
    with pytest.raises(mk.MorokError) as e:
        dev.tuning_load(bad)
    assert "line 3" in str(e.value) and dev.gemm_tuning_get(*prob) is None
    open(bad, "w").write(lines[0].replace("sm_count 0", "sm_count 7") + "\n" + lines[1] + "\n")
    with pytest.raises(mk.MorokError) as e:
        dev.tuning_load(bad)
    assert "SMs" in str(e.value)
    open(bad, "w").write("something else\n")
    with pytest.raises(mk.MorokError):
        dev.tuning_load(bad)
    with pytest.raises(mk.MorokError):
        dev.tuning_load(str(tmp_path / "missing.txt"))
    with pytest.raises(mk.MorokError) as e:                                            # no kernels on the mock device
        dev.gemm_autotune(*prob)
    assert e.value.status == _ffi.MK_ERR_CUDA
    dev.close()
