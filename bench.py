#!/usr/bin/env python3
"""Benchmark of the dense hot path: bf16 GEMM + causal flash-attention forward, in TFLOP/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --probe NAME [args]        small single-kernel workloads for profiler captures (bench_probes.py)

A step is one pass of the hot path over one batch of synthetic input:
  N = 1  "headline": bf16 GEMM M=8192 K=4096 N=14336 (f32 accumulate, bf16 out, row-major A and B)
         followed by causal attention B=4 H=32 S=4096 D=128 (bf16, f32 statistics).
  N > 1  "sharded":  bf16 GEMM M=16384 K=8192 N=28672 split along N over the ranks and causal
         attention B=8 H=64 S=8192 D=128 split by head; every rank's epilogue stores its finished
         tiles into all ranks' output buffers over NVLink (the all-gather of the sharded outputs is
         fused into the kernels), total work fixed => strong scaling.
`value` is algorithmic TFLOP/s of the whole job (2MNK for the GEMM, 2*B*H*S^2*D for causal
attention = half of the dense 4*B*H*S^2*D), inputs resident in HBM, device-timed with CUDA events,
max over ranks.  `sustained` repeats the same step for at least two seconds (power-capped clocks).
`e2e` is the same metric through the C ABI with host buffers: pinned-host -> HBM copies of every
input and the HBM -> host read of every output inside the timed region.  At N > 1 the line also
carries `delivery_check` (every rank compares what the peers delivered into its buffers with the CPU
oracle), `nvlink` (bytes received per rank and step, the link bound) and `parts.nccl_allgather`
(the same kernels without delivery followed by NCCL all-gathers of the shards).
`--impl reference` times the CPU restatement of morok's own path (the reference itself needs
rustc + clang, which this image lacks) on the host cores, on a bounded sample of the same work.
Rank 0 prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import datetime
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "bf16 GEMM & causal flash-attn TFLOP/s"
UNIT = "TFLOP/s"

# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture each) at the headline
# shapes: gemm_tc_pair_kernel 387.5 MB + 218.1 MB against 419.4 MB algorithmic; sdpa_tc_kernel 402.7 MB +
# 115.8 MB against 536.9 MB algorithmic (Q, K, V and O once).
GEMM_C2_DRAM_TRAFFIC_BYTES = 605_636_096
ATTN_C3_DRAM_TRAFFIC_BYTES = 518_552_064

HEADLINE = dict(gemm=(8192, 4096, 14336), attn=(4, 32, 4096, 128))
SHARDED = dict(gemm=(16384, 8192, 28672), attn=(8, 64, 8192, 128))

# peer-copy bandwidth measured on this pool (GB/s per direction per GPU) and the nominal NVLink 5 figure
NVLINK_MEASURED_GBS, NVLINK_NOMINAL_GBS = 770.0, 900.0


def gemm_flops(M, K, N):
    return 2.0 * M * N * K


def attn_flops(B, H, S, D):
    return 2.0 * B * H * S * S * D        # causal: half of 4*B*H*S^2*D


def workload_config(sharded: bool, world: int) -> dict:
    """The `config` object both arms print (the reference arm times a bounded sample of this workload)."""
    cfg = SHARDED if sharded else HEADLINE
    M, K, N = cfg["gemm"]
    B, H, S, D = cfg["attn"]
    per_gpu_mb = ((M * K + K * N // world + M * N // world + 4 * B * (H // world) * S * D) * 2) / 1e6
    return {
        "workload": ("sharded: bf16 GEMM M16384 K8192 N28672 split along N + causal attention B8 H64 S8192 D128 split by head, "
                     "outputs gathered on every rank" if sharded else
                     "headline: bf16 GEMM M8192 K4096 N14336 (f32 acc, bf16 out) + causal attention B4 H32 S4096 D128"),
        "parallelism": f"shard{world}" if world > 1 else "single",
        "l2": "no flush: each step streams %.0f MB of operands and results per GPU, L2 is 126 MB" % per_gpu_mb,
    }


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"burst": float(p["bf16_tflops"]), "sustained": float(p["bf16_tflops_sustained"]), "hbm_gbs": float(p["hbm_gbs"]),
                "source": "measured"}
    return {"burst": 1590.0, "sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons every 50 ms.  It is started before the warm-up (the
    tool needs a few hundred milliseconds before its first line) and the samples are cut to the marked
    regions by their timestamps.  Read-only queries; no setting of the GPU is touched."""
    FIELDS = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.path = gpu_index, None, None
        self.rows = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "50"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    @staticmethod
    def now():
        return datetime.datetime.now()

    def stop(self):
        if not self.proc:
            self.rows = []
            return
        time.sleep(0.06)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        rows = []
        try:
            with open(self.path) as f:
                for line in f:
                    parts = [x.strip() for x in line.split(",")]
                    if len(parts) < 10:
                        continue
                    try:
                        ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f")
                        rows.append((ts, float(parts[2]), float(parts[3]), float(parts[4]), parts[6:10]))
                    except ValueError:
                        continue
            os.unlink(self.path)
        except Exception:
            pass
        self.rows = rows

    def region(self, t_begin, t_end) -> dict:
        """Median SM clock and the throttle reasons seen between the two marks."""
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        rows = self.rows or []
        if not rows:
            return out
        slack = datetime.timedelta(milliseconds=25)
        inside = [r for r in rows if t_begin - slack <= r[0] <= t_end + slack]
        if not inside:
            # a region shorter than the sampling period: take the sample closest to its middle
            mid = t_begin + (t_end - t_begin) / 2
            inside = [min(rows, key=lambda r: abs((r[0] - mid).total_seconds()))]
            out["note"] = "region shorter than the 50 ms sampling period: nearest sample"
        reasons = set()
        for r in inside:
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[4]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        out["sm_mhz"] = statistics.median(r[1] for r in inside)
        out["sm_max_mhz"] = inside[-1][2]
        out["power_w"] = round(statistics.median(r[3] for r in inside), 1)
        out["samples"] = len(inside)
        out["reasons"] = sorted(reasons)
        return out


# ---------------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------------
def run_ours(args, rank, world, local_rank, dist):
    import morok_b200 as mk
    from morok_b200 import sharding, synth
    if mk.device_count() == 0:
        raise SystemExit("bench.py: no CUDA device -- the library has no CPU fallback")
    dev = mk.Device(local_rank)
    stream = mk.Stream(dev)
    sharded = world > 1 or args.workload == "sharded"
    cfg = SHARDED if sharded else HEADLINE
    M, K, N = cfg["gemm"]
    B, H, S, D = cfg["attn"]
    col0, Nl = sharding.gemm_column_shard(N, rank, world)      # this rank's columns of B and C
    h0, Hl, _, _ = sharding.head_shard(H, H, rank, world)      # ... and its heads
    check = world > 1 and not args.no_delivery_check

    # Inputs.  Every tensor is drawn chunk by chunk, each chunk from its own generator (seed, chunk index): A in
    # blocks of 64 rows, B in panels of 128 columns, Q / K / V per (batch, head).  A rank draws what it reads -- all
    # of A, its column block of B, its heads -- and the delivery check later re-draws the pieces it samples.
    SEED_A, SEED_B, SEED_Q = 1, 2, 3
    assert col0 % synth.COL_PANEL == 0 and Nl % synth.COL_PANEL == 0, "column shards are whole panels of the generator"
    A = dev.alloc(M * K * 2)
    for r in range(0, M, 2048):
        rows = min(2048, M - r)
        A.view(r * K * 2, rows * K * 2).copyin(synth.matrix_rows_bf16(SEED_A, K, r, rows, 1.0))
    Bw = dev.alloc(K * N * 2)                                   # full-size B; this rank fills and reads its column block in place
    shard = dev.from_numpy(synth.matrix_panels_bf16(SEED_B, K, col0, Nl, 0.02))
    dst = (C.c_void_p * 1)(Bw.ptr)
    mk._ffi.check(dev.lib.mk_all_gather_push_2d(dev.h, None, shard.ptr, Nl * 2, Nl * 2, K, dst, 1, col0 * 2, N * 2))
    dev.sync()
    shard.free()
    Q, Kt, V = (dev.alloc(B * H * S * D * 2) for _ in range(3))
    for i, t in enumerate((Q, Kt, V)):
        for b in range(B):
            heads = np.stack([synth.head_slice_bf16(SEED_Q + i, H, b, h, S, D) for h in range(h0, h0 + Hl)])
            t.view((b * H + h0) * S * D * 2, Hl * S * D * 2).copyin(heads)
    dev.sync()
    Cfull = dev.alloc(M * N * 2)
    Ofull = dev.alloc(B * H * S * D * 2)

    # peers: every rank maps every other rank's C and O
    peer_c, peer_o, peer_bufs = [], [], []
    if world > 1:
        handles = []
        for buf in (Cfull, Ofull):
            h, off = mk._ffi.IpcHandle(), C.c_size_t()
            mk._ffi.check(dev.lib.mk_ipc_export(buf.h, C.byref(h), C.byref(off)))
            handles.append((bytes(h.bytes), off.value))
        gathered = [None] * world
        dist.all_gather_object(gathered, handles)
        for r in [(rank + 1 + i) % world for i in range(world - 1)]:    # rotated: ranks never all target one GPU first
            for which, (hb, off) in enumerate(gathered[r]):
                h = mk._ffi.IpcHandle()
                C.memmove(h.bytes, hb, 64)
                out = C.c_void_p()
                nbytes = (M * N * 2) if which == 0 else (B * H * S * D * 2)
                mk._ffi.check(dev.lib.mk_ipc_open(dev.h, C.byref(h), off, nbytes, C.byref(out)))
                pb = mk.Buffer(dev, out, nbytes)
                peer_bufs.append(pb)
                (peer_c if which == 0 else peer_o).append(pb.ptr)

    b_view = Bw.view(col0 * 2, K * N * 2 - col0 * 2)
    c_off = col0 * 2
    hs = (H * S * D, S * D, D)
    q_view, k_view, v_view = (t.view(h0 * S * D * 2, (B * H * S * D - h0 * S * D) * 2) for t in (Q, Kt, V))
    o_off = h0 * S * D * 2

    def gemm(deliver=True, c_ptr=None, ldc=None):
        dev.gemm(A, b_view, Cfull, M, Nl, K, mk.MK_BF16, ldb=N, ldc=N if ldc is None else ldc,
                 c_ptr=(Cfull.ptr + c_off) if c_ptr is None else c_ptr,
                 peers=[p + c_off for p in peer_c] if deliver else [], stream=stream)

    def attn(deliver=True, o_ptr=None, o_strides=None):
        dev.sdpa(q_view, k_view, v_view, Ofull, B, Hl, Hl, S, S, D, dtype=mk.MK_BF16, causal=True,
                 q_strides=hs, k_strides=hs, v_strides=hs, o_strides=hs if o_strides is None else o_strides,
                 o_ptr=(Ofull.ptr + o_off) if o_ptr is None else o_ptr,
                 peers=[p + o_off for p in peer_o] if deliver else [], stream=stream)

    def step(ev=None, deliver=True, do_gemm=True, do_attn=True):
        if do_gemm:
            gemm(deliver)
        if ev:
            ev[1].record(stream)
        if do_attn:
            attn(deliver)

    def barrier():
        stream.sync()
        if world > 1:
            dist.barrier()

    def max_over_ranks(vals):
        if world == 1:
            return list(vals)
        import torch
        t = torch.tensor(list(vals), dtype=torch.float64, device=f"cuda:{local_rank}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(x) for x in t.tolist()]

    def timed(n, fn=None, **kw):
        """Device milliseconds per step of n back-to-back steps (max over ranks)."""
        a, b = mk.Event(dev), mk.Event(dev)
        barrier()
        a.record(stream)
        for _ in range(n):
            fn() if fn else step(**kw)
        b.record(stream)
        barrier()
        return max_over_ranks([a.elapsed_ms(b) / n])[0]

    def check_status(where):
        if dev.kernel_status(stream) != 0:
            raise SystemExit(f"bench.py: a kernel reported a device-side error {where}")

    warmup = max(args.warmup, 3)
    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(warmup):
        step()
    barrier()
    check_status("during warm-up")

    # ---- timed region: exactly K steps, device time from CUDA events on the launching stream ----
    evs = [[mk.Event(dev) for _ in range(3)] for _ in range(args.steps)]
    launches0 = dev.launch_count()
    barrier()
    t_begin = sampler.now()
    t_wall0 = time.perf_counter()
    for i in range(args.steps):
        evs[i][0].record(stream)
        step(evs[i])
        evs[i][2].record(stream)
    barrier()
    t_wall = time.perf_counter() - t_wall0
    t_end = sampler.now()
    launches = dev.launch_count() - launches0
    total_ms = evs[0][0].elapsed_ms(evs[-1][2])
    gemm_ms = statistics.mean(e[0].elapsed_ms(e[1]) for e in evs)
    attn_ms = statistics.mean(e[1].elapsed_ms(e[2]) for e in evs)
    check_status("in the timed region")
    total_ms, gemm_ms, attn_ms = max_over_ranks([total_ms, gemm_ms, attn_ms])

    # ---- sustained: the same step back to back for >= 2 s; every 16th step carries per-kernel events ----
    sus = None
    if args.sustain_seconds > 0:
        n_target = max(args.steps, int(args.sustain_seconds * 1e3 / (total_ms / args.steps)) + 1)
        marks = []
        s0, s1 = mk.Event(dev), mk.Event(dev)
        barrier()
        ts_begin = sampler.now()
        s0.record(stream)
        for i in range(n_target):
            if i % 16 == 0:
                e = [mk.Event(dev) for _ in range(3)]
                e[0].record(stream)
                step(e)
                e[2].record(stream)
                marks.append(e)
            else:
                step()
        s1.record(stream)
        barrier()
        ts_end = sampler.now()
        check_status("in the sustained loop")
        half = marks[len(marks) // 2:]                 # second half: the power state has settled
        sus_ms, sus_g, sus_a = max_over_ranks([s0.elapsed_ms(s1) / n_target, statistics.mean(e[0].elapsed_ms(e[1]) for e in half),
                                               statistics.mean(e[1].elapsed_ms(e[2]) for e in half)])
        sus = (n_target, sus_ms, sus_g, sus_a, ts_begin, ts_end)

    fl_gemm, fl_attn = gemm_flops(M, K, N), attn_flops(B, H, S, D)     # whole job, all ranks
    ms_per_step = total_ms / args.steps
    value = (fl_gemm + fl_attn) / (ms_per_step * 1e-3) / 1e12
    peaks = measured_peaks()
    peak_kind = "burst" if total_ms * 1e-3 < 1.0 else "sustained"
    of = "of measured" if peaks["source"] == "measured" else "of fallback"

    def tf(flops, ms):
        return flops / world / (ms * 1e-3) / 1e12

    gemm_tf, attn_tf = tf(fl_gemm, gemm_ms), tf(fl_attn, attn_ms)

    def roofline(kernel, achieved, traffic):
        frac = achieved / peaks[peak_kind]
        r = {"kernel": kernel, "bound": "tensor", "achieved": round(achieved, 1), "peak": peaks[peak_kind], "unit": "TFLOP/s",
             "frac": round(frac, 4), "peak_source": f"{of}: {peak_kind} bf16 GEMM figure of MEASURED_PEAKS.json" if peaks["source"] == "measured" else of,
             "frac_of_burst": round(achieved / peaks["burst"], 4), "frac_of_sustained": round(achieved / peaks["sustained"], 4),
             "traffic": traffic}
        if frac > 1.0:
            # the denominator is a cuBLAS GEMM timed by the driver in another process at its own clocks; a kernel in a
            # short burst at full clocks can read slightly above it -- the sustained block below is the like-for-like figure
            r["note"] = "above the measured denominator (a library GEMM at that run's clocks): read as 'at the denominator', see sustained"
        return r

    result = {
        "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": warmup, "ms_per_step": round(ms_per_step, 5), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(sharded, world),
        "timing": "CUDA events on the launching stream, max over ranks",
        "parts": {
            "gemm": {"ms": round(gemm_ms, 5), "tflops_per_gpu": round(gemm_tf, 1),
                     "frac_of_%s_peak_%s" % (peaks["source"], peak_kind): round(gemm_tf / peaks[peak_kind], 4)},
            "attn": {"ms": round(attn_ms, 5), "tflops_per_gpu": round(attn_tf, 1),
                     "frac_of_%s_peak_%s" % (peaks["source"], peak_kind): round(attn_tf / peaks[peak_kind], 4)},
        },
        "roofline": roofline("gemm_tc_pair_kernel", gemm_tf, GEMM_C2_DRAM_TRAFFIC_BYTES if not sharded else None),
        "roofline_attention": roofline("sdpa_tc_kernel", attn_tf, ATTN_C3_DRAM_TRAFFIC_BYTES if not sharded else None),
        "gpu_launches": int(launches),
        "wall_s": round(t_wall, 4),
    }

    # ---- side measurements (not the headline): each kernel alone, and the sharded step without delivery ----
    n_side = max(5, min(args.steps, 30))
    time.sleep(0.5)                      # let the power state relax so "alone" is not measured under the step's cap
    g_alone = timed(n_side, do_attn=False, deliver=False)
    time.sleep(0.5)
    a_alone = timed(n_side, do_gemm=False, deliver=False)
    result["parts"]["gemm"]["alone"] = {"ms": round(g_alone, 5), "tflops_per_gpu": round(tf(fl_gemm, g_alone), 1),
                                        "frac_of_%s_peak_burst" % peaks["source"]: round(tf(fl_gemm, g_alone) / peaks["burst"], 4)}
    result["parts"]["attn"]["alone"] = {"ms": round(a_alone, 5), "tflops_per_gpu": round(tf(fl_attn, a_alone), 1),
                                        "frac_of_%s_peak_burst" % peaks["source"]: round(tf(fl_attn, a_alone) / peaks["burst"], 4)}
    if world == 1 and not sharded:
        result["parts"]["gemm_f8e4m3_alone"] = f8_side(mk, dev, stream, Cfull, M, K, N, n_side, fl_gemm, barrier)
        if not args.no_t1_sharded:
            # free the headline tensors first: the sharded shapes take ~6 GB
            result["t1_sharded"] = t1_sharded(mk, synth, dev, stream, n_side)
    if world > 1:
        c_ms = timed(n_side, deliver=False)
        result["compute_only"] = {"value": round((fl_gemm + fl_attn) / (c_ms * 1e-3) / 1e12, 2), "unit": UNIT, "ms_per_step": round(c_ms, 5),
                                  "note": "same sharded step with peer delivery off: every rank keeps only its own shard"}
        rx = (world - 1) / world * (M * N * 2 + B * H * S * D * 2)      # bytes every rank receives per step
        result["nvlink"] = {"rx_bytes_per_rank_per_step": int(rx), "achieved_ingress_gbs": round(rx / (ms_per_step * 1e-3) / 1e9, 1),
                            "link_bound_ms": round(rx / (NVLINK_MEASURED_GBS * 1e9) * 1e3, 4),
                            "link_bound_ms_nominal": round(rx / (NVLINK_NOMINAL_GBS * 1e9) * 1e3, 4),
                            "peer_copy_gbs_measured": NVLINK_MEASURED_GBS, "nominal_gbs": NVLINK_NOMINAL_GBS,
                            "step_bound_ms": round(max(c_ms, rx / (NVLINK_MEASURED_GBS * 1e9) * 1e3), 4),
                            "note": "step_bound = max(compute-only step, bytes received / measured peer-copy bandwidth)"}
        if not args.no_nccl_leg:
            result["parts"]["nccl_allgather"] = nccl_leg(mk, dev, stream, dist, local_rank, world, gemm, attn, timed, n_side,
                                                         dict(M=M, Nl=Nl, B=B, Hl=Hl, S=S, D=D), fl_gemm + fl_attn)
        if check:
            result["delivery_check"] = delivery_check(mk, dev, stream, dist, local_rank, rank, world, step, barrier, Cfull, Ofull,
                                                      dict(M=M, K=K, N=N, B=B, H=H, S=S, D=D), (SEED_A, SEED_B, SEED_Q))

    sampler.stop()
    result["clocks"] = sampler.region(t_begin, t_end)
    if sus:
        n_target, sus_ms, sus_g, sus_a, ts_begin, ts_end = sus
        sv = (fl_gemm + fl_attn) / (sus_ms * 1e-3) / 1e12
        result["sustained"] = {
            "value": round(sv, 2), "unit": UNIT, "steps": n_target, "seconds": round(sus_ms * n_target * 1e-3, 3), "ms_per_step": round(sus_ms, 5),
            "gemm": {"ms": round(sus_g, 5), "tflops_per_gpu": round(tf(fl_gemm, sus_g), 1),
                     "frac_of_%s_peak_burst" % peaks["source"]: round(tf(fl_gemm, sus_g) / peaks["burst"], 4),
                     "frac_of_%s_peak_sustained" % peaks["source"]: round(tf(fl_gemm, sus_g) / peaks["sustained"], 4)},
            "attn": {"ms": round(sus_a, 5), "tflops_per_gpu": round(tf(fl_attn, sus_a), 1),
                     "frac_of_%s_peak_burst" % peaks["source"]: round(tf(fl_attn, sus_a) / peaks["burst"], 4),
                     "frac_of_%s_peak_sustained" % peaks["source"]: round(tf(fl_attn, sus_a) / peaks["sustained"], 4)},
            "clocks": sampler.region(ts_begin, ts_end),
            "note": "same step back to back; per-kernel times from events around every 16th step, second half of the loop"}

    # ---- end to end through the C ABI with host buffers (rank-local shard, copies inside the timed region) ----
    result["e2e"] = run_e2e(mk, dev, stream, dict(M=M, K=K, N=N, Nl=Nl, B=B, H=H, Hl=Hl, S=S, D=D, col0=col0, h0=h0),
                            world, dist, local_rank, args.steps, fl_gemm + fl_attn)
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        result["cpu_baseline"] = cpu_baseline(sharded, args.cpu_seconds)
    for pb in peer_bufs:
        pb.free()
    return result


def f8_side(mk, dev, stream, Cfull, M, K, N, n_side, fl_gemm, barrier):
    """The same GEMM shape with 8-bit float inputs (e4m3, weights stored [N, K]) on tcgen05 kind::f8f6f4: a
    capability beyond the bf16 headline, reported beside it and not part of `value`."""
    rng = np.random.default_rng(9)
    a8 = dev.from_numpy(rng.integers(0, 0x78, (M, K), dtype=np.uint8) | (rng.integers(0, 2, (M, K), dtype=np.uint8) << 7))
    w8 = dev.from_numpy(rng.integers(0, 0x40, (N, K), dtype=np.uint8) | (rng.integers(0, 2, (N, K), dtype=np.uint8) << 7))

    def f8_step():
        dev.gemm(a8, w8, Cfull, M, N, K, mk.MK_F8E4M3, mk.MK_BF16, trans_b=True, stream=stream)

    for _ in range(3):
        f8_step()
    time.sleep(0.5)
    e_a, e_b = mk.Event(dev), mk.Event(dev)
    barrier()
    e_a.record(stream)
    for _ in range(n_side):
        f8_step()
    e_b.record(stream)
    barrier()
    f8_ms = e_a.elapsed_ms(e_b) / n_side
    if dev.kernel_status(stream) != 0:
        raise SystemExit("bench.py: the 8-bit float GEMM reported a device-side error")
    a8.free()
    w8.free()
    return {"ms": round(f8_ms, 5), "tflops_per_gpu": round(fl_gemm / (f8_ms * 1e-3) / 1e12, 1),
            "note": "same M, K, N; e4m3 inputs, f32 accumulation, bf16 output; not part of value"}


def t1_sharded(mk, synth, dev, stream, n_side):
    """One-GPU time of the sharded workload (config 5 fits one GPU: ~6 GB), so that the N-GPU values of the
    scaling run have a like-for-like denominator.  Timing only: inputs are one random chunk repeated."""
    M, K, N = SHARDED["gemm"]
    B, H, S, D = SHARDED["attn"]

    def tensor(n, sigma, seed):
        buf = dev.alloc(n * 2)
        synth.fill_normal_bf16(dev, buf, n, sigma, seed, tile=True)
        return buf

    A, Bw = tensor(M * K, 1.0, 11), tensor(K * N, 0.02, 12)
    Q, Kt, V = (tensor(B * H * S * D, 1.0, 13 + i) for i in range(3))
    Cb, Ob = dev.alloc(M * N * 2), dev.alloc(B * H * S * D * 2)

    def step(ev=None):
        dev.gemm(A, Bw, Cb, M, N, K, mk.MK_BF16, stream=stream)
        if ev:
            ev.record(stream)
        dev.sdpa(Q, Kt, V, Ob, B, H, H, S, S, D, dtype=mk.MK_BF16, causal=True, stream=stream)

    for _ in range(2):
        step()
    stream.sync()
    n = max(3, min(n_side, 10))
    e0, e1, mids = mk.Event(dev), mk.Event(dev), [mk.Event(dev) for _ in range(n)]
    starts = [mk.Event(dev) for _ in range(n)]
    e0.record(stream)
    for i in range(n):
        starts[i].record(stream)
        step(mids[i])
    e1.record(stream)
    stream.sync()
    if dev.kernel_status(stream) != 0:
        raise SystemExit("bench.py: a kernel reported a device-side error in the one-GPU run of the sharded workload")
    ms = e0.elapsed_ms(e1) / n
    g_ms = statistics.mean(starts[i].elapsed_ms(mids[i]) for i in range(n))
    fl = gemm_flops(M, K, N) + attn_flops(B, H, S, D)
    for b in (A, Bw, Q, Kt, V, Cb, Ob):
        b.free()
    dev.trim()
    return {"value": round(fl / (ms * 1e-3) / 1e12, 2), "unit": UNIT, "ms_per_step": round(ms, 4), "gemm_ms": round(g_ms, 4), "attn_ms": round(ms - g_ms, 4),
            "steps": n, "note": "the N > 1 workload (GEMM 16384x8192x28672 + attention B8 H64 S8192 D128) on one GPU: "
                                "strong-scaling efficiency at N GPUs = value_N / (N * this value)"}


def nccl_leg(mk, dev, stream, dist, local_rank, world, gemm, attn, timed, n_side, s, total_flops):
    """The collective the headline names, as a baseline beside the fused delivery: the same kernels store only
    their own shard (contiguous [M, N/g] and [B, H/g, S, D] blocks), and NCCL all-gathers of C and O follow;
    the gather of C is asynchronous so that it overlaps the attention kernel.  The gathered layouts are
    [g][M][N/g] and [g][B][H/g][S][D] (no de-interleave pass is charged to NCCL)."""
    import torch
    M, Nl, B, Hl, S, D = s["M"], s["Nl"], s["B"], s["Hl"], s["S"], s["D"]
    tdev = torch.device(f"cuda:{local_rank}")
    c_shard = torch.empty((M, Nl), dtype=torch.bfloat16, device=tdev)
    o_shard = torch.empty((B, Hl, S, D), dtype=torch.bfloat16, device=tdev)
    c_all = torch.empty((world, M, Nl), dtype=torch.bfloat16, device=tdev)
    o_all = torch.empty((world, B, Hl, S, D), dtype=torch.bfloat16, device=tdev)
    ext = torch.cuda.ExternalStream(stream.raw(), device=tdev)
    o_str = (Hl * S * D, S * D, D)

    def nccl_step():
        with torch.cuda.stream(ext):
            gemm(False, c_ptr=c_shard.data_ptr(), ldc=Nl)
            w1 = dist.all_gather_into_tensor(c_all, c_shard, async_op=True)
            attn(False, o_ptr=o_shard.data_ptr(), o_strides=o_str)
            w2 = dist.all_gather_into_tensor(o_all, o_shard, async_op=True)
            w1.wait()
            w2.wait()

    for _ in range(2):
        nccl_step()
    ms = timed(n_side, fn=nccl_step)
    del c_shard, o_shard, c_all, o_all
    torch.cuda.empty_cache()
    return {"value": round(total_flops / (ms * 1e-3) / 1e12, 2), "unit": UNIT, "ms_per_step": round(ms, 5),
            "note": "kernels without delivery + ncclAllGather of the C and O shards (gather of C overlaps attention); gathered as [g][shard]"}


def delivery_check(mk, dev, stream, dist, local_rank, rank, world, step, barrier, Cfull, Ofull, s, seeds):
    """Correctness of what the peers delivered.  C and O are filled with a poison pattern on every rank, one
    delivered step runs, and every rank compares -- for EVERY rank's column block of C and head slice of O as
    they now stand in ITS OWN buffers -- sampled rows / column panels / heads with the CPU oracle (the checker;
    outside any timed region), on inputs re-drawn from the generators' chunk seeds.  Pass / fail is reduced over
    the ranks."""
    import torch
    from morok_b200 import sharding, synth
    from oracle import oracle as orc
    orc.lib().orc_set_threads(max(1, (os.cpu_count() or 1) // world))       # torchrun exports OMP_NUM_THREADS=1
    M, K, N, B, H, S, D = (s[k] for k in ("M", "K", "N", "B", "H", "S", "D"))
    seed_a, seed_b, seed_q = seeds
    for buf, nbytes in ((Cfull, M * N * 2), (Ofull, B * H * S * D * 2)):
        mk._ffi.check(dev.lib.mk_memset_async(dev.h, buf.ptr, 0xFF, nbytes, stream.h))
    barrier()                           # poison is in place everywhere before anyone stores
    step()
    barrier()                           # every rank's stores have landed everywhere
    bf = orc.bf16_to_f32
    rng = np.random.default_rng(1234)   # the same sample on every rank
    rows = np.unique(np.concatenate([[0, 255, 256, 8191, 8192, M - 257, M - 256, M - 1], rng.integers(0, M, 12)]))
    failures, n_rows, n_heads, worst = [], 0, 0, 0.0
    a_rows = bf(np.concatenate([synth.matrix_rows_bf16(seed_a, K, int(r), 1, 1.0) for r in rows]))
    c_rows = np.stack([Cfull.view(int(r) * N * 2, N * 2).copyout(np.uint16, (N,)) for r in rows])
    P = synth.COL_PANEL
    for r in range(world):
        c0, nc = sharding.gemm_column_shard(N, r, world)
        # the first, the last and one random panel of 128 columns of this rank's block: tile seams and the block's edges
        panels = sorted({c0 // P, (c0 + nc) // P - 1, c0 // P + int(rng.integers(0, nc // P))})
        for pidx in panels:
            ref = orc.matmul_f32(a_rows, bf(synth.matrix_panels_bf16(seed_b, K, pidx * P, P, 0.02)))
            got_bits = c_rows[:, pidx * P:(pidx + 1) * P]
            got = bf(got_bits)
            bad = (np.abs(got - ref) > 1e-2 + 2e-2 * np.abs(ref)) | (got_bits == 0xFFFF)
            worst = max(worst, float(np.max(np.abs(got - ref) / (1e-2 + 2e-2 * np.abs(ref)))))
            if bad.any():
                failures.append(f"rank {rank}: C columns {pidx * P}..{pidx * P + P - 1} (rank {r}'s block): {int(bad.sum())} of {bad.size} sampled elements off")
        # poison anywhere in the sampled rows of this block means a tile was never delivered
        if np.any(c_rows[:, c0:c0 + nc] == 0xFFFF):
            failures.append(f"rank {rank}: poison left in rank {r}'s column block of C")
        n_rows += len(rows)
    row_blocks = [(0, 64), (S // 2 - 32, 64), (S - 64, 64)]     # per head: first rows, a tile seam in the middle, the last rows
    for r in range(world):
        q0, nq, _, _ = sharding.head_shard(H, H, r, world)
        for (b, h) in ((int(rng.integers(0, B)), q0), (int(rng.integers(0, B)), q0 + nq - 1)):
            qh, kh, vh = (bf(synth.head_slice_bf16(seed_q + i, H, b, h, S, D)) for i in range(3))
            for (r0, nr) in row_blocks:
                off = ((b * H + h) * S + r0) * D * 2
                got_bits = Ofull.view(off, nr * D * 2).copyout(np.uint16, (nr, D))
                ref = orc.sdpa_f32(qh[None, None, r0:r0 + nr], kh[None, None, :r0 + nr], vh[None, None, :r0 + nr], causal=True, causal_offset=r0)[0, 0]
                got = bf(got_bits)
                bad = (np.abs(got - ref) > 1e-2 + 2e-2 * np.abs(ref)) | (got_bits == 0xFFFF)
                worst = max(worst, float(np.max(np.abs(got - ref) / (1e-2 + 2e-2 * np.abs(ref)))))
                if bad.any():
                    failures.append(f"rank {rank}: O head ({b},{h}) of rank {r}, rows {r0}..{r0 + nr - 1}: {int(bad.sum())} of {bad.size} elements off")
            n_heads += 1
    ok = torch.tensor([0 if failures else 1], dtype=torch.int32, device=f"cuda:{local_rank}")
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    all_fail = [None] * world
    dist.all_gather_object(all_fail, failures[:4])
    return {"ok": bool(ok.item() == 1), "rows": n_rows, "heads": n_heads, "ranks": world,
            "worst_error_over_bar": round(worst, 3),
            "what": "after a poison fill and one delivered step, every rank checked, in its own buffers, sampled rows of every rank's column "
                    "block of C (first, last and a random 128-column panel against the oracle; no poison anywhere in those rows) and two heads "
                    "(three 64-row blocks each) of every rank's slice of O, at 2e-2 rel + 1e-2 abs",
            "failures": [f for fs in all_fail for f in (fs or [])][:8]}


def run_e2e(mk, dev, stream, s, world, dist, local_rank, steps, total_flops):
    """Host buffers in, host buffers out: every step copies this rank's inputs from pinned host
    memory to HBM, runs the two kernels through the C ABI, and reads both outputs back."""
    M, K, Nl, B, Hl, S, D = s["M"], s["K"], s["Nl"], s["B"], s["Hl"], s["S"], s["D"]
    sizes_in = [M * K * 2, K * Nl * 2] + [B * Hl * S * D * 2] * 3
    sizes_out = [M * Nl * 2, B * Hl * S * D * 2]
    lib = dev.lib

    def pinned(nbytes):
        p = C.c_void_p()
        mk._ffi.check(lib.mk_host_alloc(nbytes, C.byref(p)))
        return p

    host_in = [pinned(n) for n in sizes_in]
    host_out = [pinned(n) for n in sizes_out]
    rng = np.random.default_rng(7)
    for p, n in zip(host_in, sizes_in):       # bf16 values in [1, 2) patterns scaled small: finite, non-trivial
        arr = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint16)), shape=(n // 2,))
        arr[:] = (rng.integers(0, 1 << 7, size=n // 2, dtype=np.uint16) | np.uint16(0x3C00)) ^ \
                 (rng.integers(0, 2, size=n // 2, dtype=np.uint16) << np.uint16(15))
    # Three ordered queues -- uploads, kernels, downloads -- over two sets of device buffers, so that
    # step i+1's host->device copies and step i-1's device->host copies run under step i's kernels
    # (PCIe is full duplex).  Every step still moves all of its inputs and outputs.
    NBUF = 2
    dev_in = [[dev.alloc(n) for n in sizes_in] for _ in range(NBUF)]
    dev_out = [[dev.alloc(n) for n in sizes_out] for _ in range(NBUF)]
    for group in dev_in + dev_out:
        for b in group:
            b.ptr
    hs = (Hl * S * D, S * D, D)
    s_in, s_out = mk.Stream(dev), mk.Stream(dev)
    ev_in = [mk.Event(dev) for _ in range(NBUF)]      # inputs of the set are on the device
    ev_comp = [mk.Event(dev) for _ in range(NBUF)]    # kernels of the set are done (inputs reusable, outputs ready)
    ev_out = [mk.Event(dev) for _ in range(NBUF)]     # outputs of the set are on the host (outputs reusable)

    def step(i):
        k = i % NBUF
        if i >= NBUF:
            mk._ffi.check(lib.mk_stream_wait_event(s_in.h, ev_comp[k].h))
        for hb, db, n in zip(host_in, dev_in[k], sizes_in):
            mk._ffi.check(lib.mk_memcpy_async(dev.h, db.ptr, hb, n, 0, s_in.h))
        ev_in[k].record(s_in)
        mk._ffi.check(lib.mk_stream_wait_event(stream.h, ev_in[k].h))
        if i >= NBUF:
            mk._ffi.check(lib.mk_stream_wait_event(stream.h, ev_out[k].h))
        dev.gemm(dev_in[k][0], dev_in[k][1], dev_out[k][0], M, Nl, K, mk.MK_BF16, stream=stream)
        dev.sdpa(dev_in[k][2], dev_in[k][3], dev_in[k][4], dev_out[k][1], B, Hl, Hl, S, S, D, dtype=mk.MK_BF16, causal=True,
                 q_strides=hs, k_strides=hs, v_strides=hs, o_strides=hs, stream=stream)
        ev_comp[k].record(stream)
        mk._ffi.check(lib.mk_stream_wait_event(s_out.h, ev_comp[k].h))
        for hb, db, n in zip(host_out, dev_out[k], sizes_out):
            mk._ffi.check(lib.mk_memcpy_async(dev.h, hb, db.ptr, n, 1, s_out.h))
        ev_out[k].record(s_out)

    def barrier():
        s_in.sync(); stream.sync(); s_out.sync()
        if world > 1:
            dist.barrier()

    for i in range(NBUF):
        step(i)
    barrier()
    e0, e1 = mk.Event(dev), mk.Event(dev)
    barrier()
    e0.record(s_in)
    for i in range(NBUF, NBUF + steps):    # i >= NBUF: every reuse of a buffer set waits for its previous user
        step(i)
    mk._ffi.check(lib.mk_stream_wait_event(s_out.h, ev_out[(NBUF + steps - 2) % NBUF].h))
    e1.record(s_out)                      # after the last download (downloads are ordered on s_out)
    barrier()
    ms = e0.elapsed_ms(e1) / steps
    if world > 1:
        import torch
        t = torch.tensor([ms], dtype=torch.float64, device=f"cuda:{local_rank}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    if dev.kernel_status(stream) != 0:
        raise SystemExit("bench.py: a kernel reported a device-side error in the end-to-end leg")
    for p in host_in + host_out:
        lib.mk_host_free(p)
    for group in dev_in + dev_out:
        for b in group:
            b.free()
    return {"value": round(total_flops / (ms * 1e-3) / 1e12, 3), "unit": UNIT, "ms_per_step": round(ms, 4), "steps": steps,
            "h2d_bytes_per_step": int(sum(sizes_in)), "d2h_bytes_per_step": int(sum(sizes_out)),
            "path": "per rank and step: mk_memcpy_async(pinned host -> HBM) of every input, mk_gemm + mk_sdpa_fwd, mk_memcpy_async(HBM -> pinned host) of every output; "
                    "uploads, kernels and downloads on three streams over two buffer sets"}


# ---------------------------------------------------------------------------------------------------
# CPU baseline / reference arm: the oracle port of morok's CPU path on a bounded sample of the workload
# ---------------------------------------------------------------------------------------------------
class CpuSample:
    """Bounded sample of one workload for the CPU restatement of the reference's path.

    GEMM: `rows` rows of A against the full B, rows a multiple of the thread count the reference's THREAD
    rule gives the FULL problem (schedule/src/optimizer/heuristics.rs:485-535: the largest of
    [32,16,12,8,6,5,4,3,2] that fits the cores and divides M), one contiguous chunk of rows per thread.
    Attention: `qrows` query rows of one (batch, head) against all S keys -- the reference evaluates every
    score row in full before masking, so every row costs the same -- with every thread busy.
    The two rates are combined in the proportion of the full workload, value = (F_gemm + F_attn) /
    (F_gemm / rate_gemm + F_attn / rate_attn), so the figure does not depend on how large the sample was."""

    def __init__(self, sharded: bool):
        from oracle import oracle as orc
        self.orc = orc
        try:
            self.lib = orc.lib(native=True)      # -march=native build made on the machine that runs the timing
        except Exception:
            self.lib = orc.lib()
        cfg = SHARDED if sharded else HEADLINE
        self.M, self.K, self.N = cfg["gemm"]
        self.B, self.H, self.S, self.D = cfg["attn"]
        cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
        self.cores = int(self.lib.orc_set_threads(cores))            # a launcher may have exported OMP_NUM_THREADS=1
        self.gemm_threads = int(self.lib.orc_thread_count(self.M * self.N * self.K, self.M, self.cores))
        rng = np.random.default_rng(0)
        self.max_rows = 64 * self.gemm_threads
        self.a = orc.bf16_to_f32(orc.normal_bf16(rng, (self.max_rows, self.K), 1.0))
        self.b = orc.bf16_to_f32(orc.normal_bf16(rng, (self.K, self.N), 0.02))
        self.q, self.k, self.v = (orc.bf16_to_f32(orc.normal_bf16(rng, (1, 1, self.S, self.D))) for _ in range(3))
        self.rows, self.qrows = self.gemm_threads, self.cores

    def gemm_seconds(self, rows):
        a = self.a[:rows]
        c = np.empty((rows, self.N), dtype=np.float32)
        t0 = time.perf_counter()
        used = self.lib.orc_matmul_f32(a.ctypes.data_as(C.c_void_p), self.b.ctypes.data_as(C.c_void_p), c.ctypes.data_as(C.c_void_p),
                                       rows, self.N, self.K, self.K, self.N, self.N, self.gemm_threads)
        dt = time.perf_counter() - t0
        assert used == self.gemm_threads, f"the GEMM sample ran on {used} threads, not {self.gemm_threads}"
        return dt

    def attn_seconds(self, qrows):
        # rows r0 .. r0 + qrows - 1 of the head; keys beyond a row's position are masked after the full score row
        q = np.ascontiguousarray(self.q[:, :, :qrows])
        o = np.empty((1, 1, qrows, self.D), dtype=np.float32)
        t0 = time.perf_counter()
        r = self.lib.orc_sdpa_f32_offset(q.ctypes.data_as(C.c_void_p), self.k.ctypes.data_as(C.c_void_p), self.v.ctypes.data_as(C.c_void_p),
                                         o.ctypes.data_as(C.c_void_p), None, 1, 1, 1, qrows, self.S, self.D, self.D,
                                         C.c_float(1.0 / np.sqrt(self.D)), 1, self.S - qrows, None, C.c_float(0.0))
        assert r == 0
        return time.perf_counter() - t0

    def size(self, budget_s):
        """Sizes the sample for about budget_s seconds per evaluation (half per op)."""
        self.gemm_seconds(self.gemm_threads)                 # thread pool up, pages touched
        self.attn_seconds(self.cores)
        t_g = max(self.gemm_seconds(self.gemm_threads), 1e-4)
        t_a = max(self.attn_seconds(self.cores), 1e-4)
        self.rows = self.gemm_threads * int(min(64, max(1, (budget_s / 2) / t_g)))
        self.qrows = int(min(self.S, self.cores * max(1, int((budget_s / 2) / t_a))))

    def run(self):
        """One evaluation of the sample: (seconds, workload-proportion TFLOP/s)."""
        t_g, t_a = self.gemm_seconds(self.rows), self.attn_seconds(self.qrows)
        rate_g = gemm_flops(self.rows, self.K, self.N) / t_g
        rate_a = attn_flops(1, 1, self.S, self.D) * (self.qrows / self.S) / t_a       # same flop convention as the GPU arm
        Fg, Fa = gemm_flops(self.M, self.K, self.N), attn_flops(self.B, self.H, self.S, self.D)
        return t_g + t_a, (Fg + Fa) / (Fg / rate_g + Fa / rate_a) / 1e12, rate_g / 1e12, rate_a / 1e12

    def describe(self):
        return (f"{self.rows} of {self.M} rows of the GEMM on {self.gemm_threads} threads (the reference's thread rule for M={self.M}) + "
                f"{self.qrows} of {self.S} query rows of one of {self.B * self.H} (batch, head) pairs of the attention on {self.cores} threads; "
                "the two rates are combined in the proportion of the full workload "
                "(oracle/morok_oracle.c, the C restatement of morok's clang CPU path)")


def cpu_baseline(sharded, budget_s=12.0):
    cs = CpuSample(sharded)
    cs.size(budget_s / 3)
    runs = [cs.run() for _ in range(3)]
    value = statistics.median(r[1] for r in runs)
    return {"value": round(value, 6), "unit": UNIT, "cores": cs.cores, "kind": "port",
            "gemm_tflops": round(statistics.median(r[2] for r in runs), 6), "attn_tflops": round(statistics.median(r[3] for r in runs), 6),
            "threads": {"gemm": cs.gemm_threads, "attention": cs.cores},
            "sample": cs.describe() + f"; median of 3 evaluations of {sum(r[0] for r in runs) / 3:.1f} s"}


def run_reference(args, rank, world):
    """Reference arm: the reference's own CPU implementation cannot be built in this image (no
    rustc / cargo / clang), so its restatement in oracle/ is timed, with all host threads, on the
    configuration our arm runs at this N (headline at N = 1, sharded shapes at N > 1)."""
    if rank != 0:
        return None
    sharded = world > 1 or args.gpus > 1 or args.workload == "sharded"
    cs = CpuSample(sharded)
    cs.size(max(0.5, args.cpu_seconds / max(args.steps + args.warmup, 1)))   # whole arm within a few minutes at any step count
    for _ in range(args.warmup):
        cs.run()
    runs = [cs.run() for _ in range(args.steps)]
    value = statistics.median(r[1] for r in runs)
    t = sum(r[0] for r in runs)
    return {
        "impl": "reference", "metric": METRIC, "value": round(value, 6), "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(t / args.steps * 1e3, 3), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32 on bf16-rounded inputs", "data": "synthetic",
        "config": workload_config(sharded, max(world, args.gpus)),
        "timing": "host clock around each evaluation of the sample; value = median over the steps",
        "note": "morok's Rust + clang toolchain is absent from this image; oracle/morok_oracle.c restates its CPU path. each step = " + cs.describe(),
        "cpu_baseline": {"value": round(value, 6), "unit": UNIT, "cores": cs.cores, "kind": "port",
                         "threads": {"gemm": cs.gemm_threads, "attention": cs.cores}, "sample": "each step = " + cs.describe()},
        "e2e": {"value": round(value, 6), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def main():
    if "--probe" in sys.argv:
        import bench_probes
        i = sys.argv.index("--probe")
        bench_probes.main(sys.argv[i + 1:])
        return
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=["auto", "headline", "sharded"], default="auto")
    ap.add_argument("--cpu-seconds", type=float, default=None, help="CPU time budget of the cpu_baseline sample / reference arm")
    ap.add_argument("--sustain-seconds", type=float, default=2.0, help="length of the sustained loop (0: skip)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-delivery-check", action="store_true")
    ap.add_argument("--no-nccl-leg", action="store_true")
    ap.add_argument("--no-t1-sharded", action="store_true")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        args.steps = 3 if args.steps is None else args.steps
        args.warmup = 1 if args.warmup is None else args.warmup
        args.cpu_seconds = 60.0 if args.cpu_seconds is None else args.cpu_seconds
        out = run_reference(args, rank, world)
        if out is not None:
            print(json.dumps(out), flush=True)
        return

    args.steps = 300 if args.steps is None else args.steps
    args.warmup = 5 if args.warmup is None else args.warmup
    args.cpu_seconds = 12.0 if args.cpu_seconds is None else args.cpu_seconds
    dist = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        import torch
        import torch.distributed as dist_mod
        torch.cuda.set_device(local_rank)
        dist_mod.init_process_group("nccl", device_id=torch.device(f"cuda:{local_rank}"))
        dist = dist_mod
    if world != args.gpus and rank == 0:
        print(f"bench.py: --gpus {args.gpus} but WORLD_SIZE={world}; launch with torchrun for N > 1", file=sys.stderr)
    out = run_ours(args, rank, world, local_rank, dist)
    if rank == 0:
        print(json.dumps(out), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
