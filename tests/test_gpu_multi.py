"""Sharded GEMM and attention across 2 GPUs with the all-gather fused into the kernels' epilogues
(peer stores over NVLink): every rank must end up with the full, oracle-matching output.
Ranks run as child processes (one per GPU) that rendezvous over gloo; needs >= 2 GPUs."""
import ctypes as C
import os
import socket
import sys

import numpy as np
import pytest

import morok_b200 as mk

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _open_peers(dev, dist, rank, world, bufs):
    """Exports each buffer, gathers all ranks' handles, maps every peer's copy.  Returns
    {name: [ptr of rank 0's buffer, ptr of rank 1's, ...]} (own entry = local pointer) and the mappings."""
    from morok_b200 import _ffi
    mine = {}
    for name, b in bufs.items():
        h, off = _ffi.IpcHandle(), C.c_size_t()
        _ffi.check(dev.lib.mk_ipc_export(b.h, C.byref(h), C.byref(off)))
        mine[name] = (bytes(h.bytes), off.value, b.nbytes)
    gathered = [None] * world
    dist.all_gather_object(gathered, mine)
    ptrs, keep = {n: [] for n in bufs}, []
    for r in range(world):
        for name, b in bufs.items():
            if r == rank:
                ptrs[name].append(b.ptr)
                continue
            hb, off, nbytes = gathered[r][name]
            h = _ffi.IpcHandle()
            C.memmove(h.bytes, hb, 64)
            out = C.c_void_p()
            _ffi.check(dev.lib.mk_ipc_open(dev.h, C.byref(h), off, nbytes, C.byref(out)))
            pb = mk.Buffer(dev, out, nbytes)
            keep.append(pb)
            ptrs[name].append(pb.ptr)
    return ptrs, keep


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from morok_b200 import sharding
    from oracle import oracle as orc
    dist.init_process_group("gloo", rank=rank, world_size=world)
    dev = mk.Device(rank)
    rng = np.random.default_rng(0)                       # identical inputs on every rank

    # ---- GEMM split along N: a small problem (single-CTA kernel, peers written by the epilogue warps) ----
    M, K, N = 384, 256, 1280
    a, b = orc.normal_bf16(rng, (M, K), 1.0), orc.normal_bf16(rng, (K, N), 0.05)
    A, B = dev.from_numpy(a), dev.from_numpy(b)
    Cfull = dev.from_numpy(np.full((M, N), 0xFFFF, np.uint16))          # poison: every element must be overwritten
    # ---- ... and one with enough 256 x 256 tiles per rank for the CTA-pair kernel, whose epilogue delivers tiles by
    # tile stores; rows and columns are ragged against the tile and against the 32 x 64 store boxes ----
    M2, K2, N2 = 2040, 320, 5128
    a2, b2 = orc.normal_bf16(rng, (M2, K2), 1.0), orc.normal_bf16(rng, (K2, N2), 0.05)
    A2, B2 = dev.from_numpy(a2), dev.from_numpy(b2)
    C2full = dev.from_numpy(np.full((M2, N2), 0xFFFF, np.uint16))
    # ---- attention split by head (GQA 8:4, two kv heads per rank) ----
    Bt, Hq, Hkv, S, D = 1, 8, 4, 320, 128
    q, k, v = orc.normal_bf16(rng, (Bt, Hq, S, D)), orc.normal_bf16(rng, (Bt, Hkv, S, D)), orc.normal_bf16(rng, (Bt, Hkv, S, D))
    Q, Kb, V = dev.from_numpy(q), dev.from_numpy(k), dev.from_numpy(v)
    Ofull = dev.from_numpy(np.full((Bt, Hq, S, D), 0xFFFF, np.uint16))
    dev.sync()
    ptrs, keep = _open_peers(dev, dist, rank, world, {"c": Cfull, "o": Ofull, "c2": C2full})
    dist.barrier()                                       # poison is in place everywhere before anyone stores

    col0, ncols = sharding.gemm_column_shard(N, rank, world)
    peers_c = [p + col0 * 2 for r, p in enumerate(ptrs["c"]) if r != rank]
    dev.gemm(A, B.view(col0 * 2, K * N * 2 - col0 * 2), Cfull, M, ncols, K, mk.MK_BF16, ldb=N, ldc=N,
             c_ptr=Cfull.ptr + col0 * 2, peers=peers_c)
    c20, n2cols = sharding.gemm_column_shard(N2, rank, world)
    peers_c2 = [p + c20 * 2 for r, p in enumerate(ptrs["c2"]) if r != rank]
    dev.profile_begin()
    dev.gemm(A2, B2.view(c20 * 2, K2 * N2 * 2 - c20 * 2), C2full, M2, n2cols, K2, mk.MK_BF16, ldb=N2, ldc=N2,
             c_ptr=C2full.ptr + c20 * 2, peers=peers_c2)
    launched = [name for name, _ in dev.profile_end()]
    if os.environ.get("MOROK_B200_PEER_TMA", "1") != "0":
        assert launched == ["gemm_tc_pair_deliver"], launched
    q0, nq, kv0, nkv = sharding.head_shard(Hq, Hkv, rank, world)
    qv = Q.view(q0 * S * D * 2, (Hq - q0) * S * D * 2)
    kv, vv = (t.view(kv0 * S * D * 2, (Hkv - kv0) * S * D * 2) for t in (Kb, V))
    peers_o = [p + q0 * S * D * 2 for r, p in enumerate(ptrs["o"]) if r != rank]
    dev.sdpa(qv, kv, vv, Ofull, Bt, nq, nkv, S, S, D, dtype=mk.MK_BF16, causal=True,
             q_strides=(Hq * S * D, S * D, D), k_strides=(Hkv * S * D, S * D, D), v_strides=(Hkv * S * D, S * D, D),
             o_strides=(Hq * S * D, S * D, D), o_ptr=Ofull.ptr + q0 * S * D * 2, peers=peers_o)
    assert dev.kernel_status() == 0                      # synchronises this rank's stream
    dist.barrier()                                       # ... and every other rank has finished storing to us

    bf = orc.bf16_to_f32
    c = Cfull.copyout(np.uint16, (M, N))
    ref = orc.matmul_f32(bf(a), bf(b))
    assert np.all(np.abs(bf(c) - ref) <= 1e-2 + 2e-2 * np.abs(ref)), "gathered C differs from the oracle"
    c2 = C2full.copyout(np.uint16, (M2, N2))
    assert not np.any(c2 == 0xFFFF), "an element of the gathered C (CTA-pair kernel) was never written"
    ref2 = orc.matmul_f32(bf(a2), bf(b2))
    assert np.all(np.abs(bf(c2) - ref2) <= 1e-2 + 2e-2 * np.abs(ref2)), "gathered C (tile-store delivery) differs from the oracle"
    o = Ofull.copyout(np.uint16, (Bt, Hq, S, D))
    ref_o = orc.sdpa_f32(bf(q), bf(k), bf(v), causal=True)
    assert np.all(np.abs(bf(o) - ref_o) <= 1e-2 + 2e-2 * np.abs(ref_o)), "gathered O differs from the oracle"
    dist.barrier()
    for pb in keep:
        pb.free()
    dist.barrier()
    dev.close()
    dist.destroy_process_group()
    open(os.path.join(out_dir, f"ok{rank}"), "w").close()


def test_two_gpu_sharded_gemm_and_attention_deliver_full_outputs(tmp_path):
    if mk.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_worker, args=(r, 2, port, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    for r, p in enumerate(procs):
        if p.is_alive():
            p.kill()
        assert p.exitcode == 0, f"rank {r} exited with {p.exitcode}"
        assert (tmp_path / f"ok{r}").exists()
