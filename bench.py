#!/usr/bin/env python
"""Benchmark of the horizontally fused kernel pairs on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--only PAIR --mode fused|b2b|a|b] [--no-extras]

Prints ONE JSON line.  The headline workload is configuration 1 of the
benchmark list (bilinear x2 upsample of [16,128,56,56] + batch-norm statistics
of [32,256,28,28], fp32): one step = one launch of the fused pair over one
batch.  `value` is the algorithmic HBM traffic of the pair (each input read
once, each output written once: 154,142,720 B) times the steps, divided by
the device time of the timed region, summed over GPUs.  `pairs` carries, for
every benchmark configuration, the fused time, the time of the same two
kernels launched back to back on one stream, their ratio, and GB/s or GH/s
with the roofline fraction.

Timing: the K steps of one pass are replayed from a CUDA graph; the timed region is R
such passes (R chosen so that the region lasts about a second, at least 50), every pass
bracketed by CUDA events on the launching stream (for small K several passes share one
graph, with event-record nodes between them), barrier + synchronize on both sides of
the region; every rank takes the median of its passes and the maximum over ranks is
reported (mean, min and max beside it).  The steps rotate over several independent buffer sets whose combined
footprint is several times the L2, so no step finds its inputs in cache.  After the timed
region the results left in the buffers are compared with the oracle (`parity_ok`).

With N > 1 (one process per GPU under torch.distributed.run) every rank runs the full
per-GPU configuration on its own batch shard (weak scaling); the per-channel batch-norm
moments are summed over ranks INSIDE the fused kernel over NVLink peer memory
(`--collective nccl`: with an NCCL all-reduce and a finalize kernel instead).  The line
then also carries configuration 2 split over the ranks (`dl_sharded`, strong scaling) and
the nonce-sharded searches (`crypto_sharded`).

`--impl reference` times the CPU restatement of the same pair (PyTorch CPU
operators on all host cores) instead: the reference ships no CPU or GPU code
for these kernels, so the oracle port is the only CPU implementation there is.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG1_BYTES = 154_142_720
CFG0_BYTES = 218_365_952
CFG2_BYTES = 324_011_008
ETHASH_BYTES_PER_HASH = 8192
# both arms (this library, and --impl reference) report under the same names
METRIC = "fused upsample_bilinear2d + batch_norm_collect_statistics pair, HBM throughput"
WORKLOAD = "config 1: bilinear x2 upsample [16,128,56,56] + batch-norm statistics [32,256,28,28], fp32, per GPU"
# 32-bit operations per nonce, counted from the specifications.
# SPEC_OPS: every add, xor, rotate and boolean separate (no three-input adds, no merged logic):
#   BLAKE-256   14 rounds x 8 G x (6 add + 6 xor + 4 rotate)
#   SHA-256d    2 compressions x (64 rounds x 25 + 48 schedule words x 13)
#   BLAKE2b     12 rounds x 8 G x (6 add + 4 xor + 4 rotate) on 64-bit words = 2 x 32-bit each
# LOGIC_OPS: what is left for the logic/shift pipe when adds issue elsewhere and three-input
# logic is merged (a SHA-256 Sigma = 3 funnel shifts + 1 three-input xor, Ch and Maj = 1 each;
# the message-word xors of BLAKE are precomputed): the pipe that saturates first.
#   BLAKE-256   14 x 8 x (4 xor + 4 rotate)
#   SHA-256d    2 x (64 x 10 + 48 x 8)
#   BLAKE2b     12 x 8 x (4 xor x 2 halves + rotations 32/24/16/63 = 0 + 2 + 2 + 2)
SPEC_OPS_PER_HASH = {"blake256": 14 * 8 * 16, "sha256d": 2 * (64 * 25 + 48 * 13), "sia": 12 * 8 * 14 * 2}
LOGIC_OPS_PER_HASH = {"blake256": 14 * 8 * 8, "sha256d": 2 * (64 * 10 + 48 * 8), "sia": 12 * 8 * 14}


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,utilization.gpu,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.proc, self.path = gpu_index, None, None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.idx)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(5)
        except Exception:
            self.proc.kill()
        try:
            rows = [r.strip().split(", ") for r in open(self.path) if r.strip()]
            rows = [r for r in rows if len(r) >= 10]
            busy = [r for r in rows if r[4].strip().isdigit() and int(r[4]) >= 50] or rows   # samples under load
            if busy:
                out["sm_mhz"] = statistics.median(float(r[1]) for r in busy)
                out["sm_max_mhz"] = float(busy[0][2])
                names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
                out["reasons"] = [n for k, n in enumerate(names) if any(r[6 + k].startswith("Active") for r in busy)]
                out["samples"] = len(busy)
                out["power_w_max"] = max(float(r[3]) for r in busy)
        except Exception:
            pass
        finally:
            try:
                os.unlink(self.path)
            except OSError:
                pass
        return out


# ------------------------------------------------------------------------------------------
def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def time_region(torch, fn, steps, warmup, barrier):
    """Device time in ms of `steps` calls of fn(i) after `warmup` untimed calls."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for i in range(steps):
        fn(i)
    e.record()
    torch.cuda.synchronize()
    barrier()
    return s.elapsed_time(e)


def graph_region(torch, fn, nsets, steps, warmup):
    """Device time in ms per step with the launches replayed from a CUDA graph, so that no
    host launch overhead enters either side of the fused / back-to-back comparison."""
    for i in range(max(warmup, nsets)):
        fn(i)
    torch.cuda.synchronize()
    per_graph = 2 * nsets
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(per_graph):
            fn(i)
    replays = max(1, (steps + per_graph - 1) // per_graph)
    g.replay()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(replays):
        g.replay()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / (replays * per_graph)


def build_dl_sets(torch, ops, workloads, cfg, dev, nsets):
    """nsets independent (a, b) operator pairs for a DL configuration; returns (name, sets, bytes)."""
    sets = []
    if cfg == 0:
        w = workloads.config0()
        for _ in range(nsets):
            a = ops.Im2col(w["im"].to(dev), **w["im2col"])
            b = ops.MaxPool(w["pool"].to(dev), **w["maxpool"])
            sets.append((a, b))
        return "im2col_maxpool", sets, CFG0_BYTES
    if cfg == 1:
        w = workloads.config1()
        for _ in range(nsets):
            a = ops.Upsample(w["up"].to(dev), scale_factor=2)
            b = ops.BnStats(w["bn"].to(dev), w["eps"])
            sets.append((a, b))
        return "upsample_bnstats", sets, CFG1_BYTES
    w = workloads.config2()
    for _ in range(nsets):
        a = ops.Im2col(w["im"].to(dev), **w["im2col"])
        b = ops.Histc(w["hist"].to(dev), w["bins"], w["lo"], w["hi"])
        sets.append((a, b))
    return "im2col_histc", sets, CFG2_BYTES


def measure_dl_pair(torch, ops, sets, steps, warmup, barrier):
    n = len(sets)
    t_f = graph_region(torch, lambda i: ops.run_pair(*sets[i % n]), n, steps, warmup)
    t_v = vertical_time(torch, ops, sets, steps, warmup)
    t_b = graph_region(torch, lambda i: ops.run_back_to_back(*sets[i % n]), n, steps, warmup)
    t_a = graph_region(torch, lambda i: ops.run(sets[i % n][0]), n, steps, warmup)
    t_2 = graph_region(torch, lambda i: ops.run(sets[i % n][1]), n, steps, warmup)
    return t_f, t_b, t_a, t_2, t_v


def vertical_time(torch, ops, sets, steps, warmup):
    """Best of the vertical-fusion variants (same threads run both bodies), the reference's vfuse column."""
    from hfuse_b200 import _lib
    name = ops.pair_name(*sets[0])
    n, best = len(sets), None
    try:
        for v, d in enumerate(_lib.tune_variants(name)):
            if ":0:" not in d:
                continue
            _lib.tune_set(name, v, 0)
            t = graph_region(torch, lambda i: ops.run_pair(*sets[i % n]), n, steps, warmup)
            best = t if best is None else min(best, t)
    finally:
        _lib.tune_set(name, -1, 0)
    return best


def int32_peak(torch, dev):
    """Measured rate of independent 32-bit add/xor/rotate chains on every SM, in 10^12 lane
    operations per second, for the three mixes of hfuse_int32_probe; `peak` is the best of them."""
    import ctypes
    from hfuse_b200 import _lib
    sink = torch.zeros(1, dtype=torch.int32, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    out = {}
    for mix, name in ((0, "xor_rot"), (1, "add_xor_rot"), (2, "add_xor_rot_fma_add")):
        n = ctypes.c_uint64(0)
        best = 0.0
        for it in range(4):  # the first launch warms up
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            _lib.check(_lib.lib().hfuse_int32_probe(mix, 4096, sink.data_ptr(), ctypes.byref(n), st), "hfuse_int32_probe")
            e1.record()
            e1.synchronize()
            if it:
                best = max(best, n.value / (e0.elapsed_time(e1) * 1e-3) / 1e12)
        out[name + "_Tops"] = round(best, 2)
    out["peak_Tops"] = max(out.values())
    out["logic_pipe_peak_Tops"] = out["xor_rot_Tops"]
    return out


def extras(torch, ops, crypto, workloads, dev, steps, warmup, peak, barrier):
    """Fused vs back-to-back for every benchmark configuration (N = 1 only)."""
    out = {}
    for cfg in (0, 1, 2):
        name, sets, nbytes = build_dl_sets(torch, ops, workloads, cfg, dev, 4)
        tf, tb, ta, t2, tv = measure_dl_pair(torch, ops, sets, steps, warmup, barrier)
        out[f"cfg{cfg}_{name}"] = {
            "fused_us": round(tf * 1e3, 2), "back_to_back_us": round(tb * 1e3, 2),
            "vertical_fusion_us": round(tv * 1e3, 2),
            "first_alone_us": round(ta * 1e3, 2), "second_alone_us": round(t2 * 1e3, 2),
            "speedup_vs_back_to_back": round(tb / tf, 3), "GB_per_s": round(nbytes / tf / 1e6, 1),
            "frac_of_hbm_peak": round(nbytes / tf / 1e6 / peak, 3), "algorithmic_bytes": nbytes}
        del sets
        torch.cuda.empty_cache()
    # the three histc pairs the benchmark description names besides configuration 2
    w0, w1, w2 = workloads.config0(), workloads.config1(), workloads.config2()
    hist_bytes = w2["hist"].numel() * 4 + 1024

    def other(key):
        if key == "maxpool":
            return ops.MaxPool(w0["pool"].to(dev), **w0["maxpool"]), 89_915_392
        if key == "upsample":
            return ops.Upsample(w1["up"].to(dev), scale_factor=2), 128_450_560
        return ops.BnStats(w1["bn"].to(dev), w1["eps"]), 25_692_160
    for key in ("maxpool", "upsample", "bnstats"):
        sets, nbytes = [], 0
        for _ in range(4):
            b, ob = other(key)
            sets.append((ops.Histc(w2["hist"].to(dev), w2["bins"], w2["lo"], w2["hi"]), b))
            nbytes = hist_bytes + ob
        tf, tb, ta, t2, tv = measure_dl_pair(torch, ops, sets, steps, warmup, barrier)
        out[f"histc_{key}"] = {
            "fused_us": round(tf * 1e3, 2), "back_to_back_us": round(tb * 1e3, 2),
            "vertical_fusion_us": round(tv * 1e3, 2), "first_alone_us": round(ta * 1e3, 2),
            "second_alone_us": round(t2 * 1e3, 2), "speedup_vs_back_to_back": round(tb / tf, 3),
            "GB_per_s": round(nbytes / tf / 1e6, 1), "frac_of_hbm_peak": round(nbytes / tf / 1e6 / peak, 3),
            "algorithmic_bytes": nbytes}
        del sets
        torch.cuda.empty_cache()
    csteps = 2
    c3 = workloads.config3()
    a = crypto.Blake256(c3["blake_header"], c3["start"], c3["count"], c3["target"])
    b = crypto.Sha256d(c3["sha_header"], c3["start"], c3["count"], c3["target"])
    tf = time_region(torch, lambda i: crypto.run_pair(a, b), csteps, 1, barrier) / csteps
    hits_f = (a.result(), b.result())
    tb = time_region(torch, lambda i: crypto.run_back_to_back(a, b), csteps, 1, barrier) / csteps
    cpu3 = cpu_hash_rates(c3["blake_header"], c3["sha_header"], c3["target"])
    ipeak = int32_peak(torch, dev)
    out["int32_peak"] = ipeak
    ops3 = (SPEC_OPS_PER_HASH["blake256"] + SPEC_OPS_PER_HASH["sha256d"]) * c3["count"]
    lops3 = (LOGIC_OPS_PER_HASH["blake256"] + LOGIC_OPS_PER_HASH["sha256d"]) * c3["count"]
    out["cfg3_blake256_sha256d"] = {
        "spec_int32_ops_per_nonce_pair": SPEC_OPS_PER_HASH["blake256"] + SPEC_OPS_PER_HASH["sha256d"],
        "spec_Tops_fused": round(ops3 / tf / 1e9, 2),
        "logic_ops_per_nonce_pair": LOGIC_OPS_PER_HASH["blake256"] + LOGIC_OPS_PER_HASH["sha256d"],
        "logic_Tops_fused": round(lops3 / tf / 1e9, 2),
        "frac_of_logic_pipe_peak": round(lops3 / tf / 1e9 / ipeak["logic_pipe_peak_Tops"], 3),
        "nonces_each": c3["count"], "fused_ms": round(tf, 2), "back_to_back_ms": round(tb, 2),
        "speedup_vs_back_to_back": round(tb / tf, 3), "GH_per_s_each_fused": round(c3["count"] / tf / 1e6, 3),
        "hits": [hits_f[0][0], hits_f[1][0]], "fused_equals_unfused": hits_f == (a.result(), b.result()),
        "cpu_baseline": cpu3}
    c4 = workloads.config4(dev)
    s = crypto.Sia(c4["sia_header"], c4["start"], c4["count"], c4["target"])
    e = crypto.Ethash(c4["dag"], c4["header_hash"], c4["start"], c4["count"], c4["target"])
    tf = time_region(torch, lambda i: crypto.run_pair(s, e), csteps, 1, barrier) / csteps
    hits_f = (s.result(), e.result())
    tb = time_region(torch, lambda i: crypto.run_back_to_back(s, e), csteps, 1, barrier) / csteps
    te = time_region(torch, lambda i: crypto.run(e), 1, 1, barrier)
    out["cfg4_sia_ethash"] = {
        "nonces_each": c4["count"], "fused_ms": round(tf, 2), "back_to_back_ms": round(tb, 2),
        "speedup_vs_back_to_back": round(tb / tf, 3), "ethash_MH_per_s_fused": round(c4["count"] / tf / 1e3, 1),
        "ethash_MH_per_s_alone": round(c4["count"] / te / 1e3, 1),
        "ethash_frac_of_hbm_peak_fused": round(c4["count"] * ETHASH_BYTES_PER_HASH / tf / 1e6 / peak, 3),
        "hits": [hits_f[0][0], hits_f[1][0]], "fused_equals_unfused": hits_f == (s.result(), e.result()),
        "cpu_baseline": cpu_ethash_sia_rates(c4)}
    return out


def cpu_hash_rates(blake_header, sha_header, target, n=1 << 21):
    """CPU restatement (C, OpenMP over nonces, all host threads) on a bounded sample of 2^21 nonces."""
    from oracle import crypto as OC
    out = {"cores": OC.num_threads(), "kind": "port", "sample": f"{n} nonces per hash"}
    for kind, name, hdr in ((0, "blake256", blake_header), (1, "sha256d", sha_header)):
        t0 = time.perf_counter()
        OC.search(kind, hdr, 0, n, target)
        out[name + "_MH_per_s"] = round(n / (time.perf_counter() - t0) / 1e6, 2)
    return out


def cpu_ethash_sia_rates(c4, n_eth=1 << 17, n_sia=1 << 21):
    from oracle import crypto as OC
    dag = c4["dag"].cpu().numpy()
    out = {"cores": OC.num_threads(), "kind": "port", "sample": f"{n_eth} ethash nonces over the 1 GiB DAG, {n_sia} Sia nonces"}
    t0 = time.perf_counter()
    OC.search(3, c4["header_hash"], 0, n_eth, c4["target"], dag=dag)
    out["ethash_MH_per_s"] = round(n_eth / (time.perf_counter() - t0) / 1e6, 3)
    t0 = time.perf_counter()
    OC.search(2, c4["sia_header"], 0, n_sia, c4["target"])
    out["sia_MH_per_s"] = round(n_sia / (time.perf_counter() - t0) / 1e6, 2)
    return out


def cpu_pair_cfg1(torch, steps, warmup):
    """The CPU restatement of configuration 1 on all host cores; returns (ms per step, cores)."""
    from oracle import dl
    from hfuse_b200 import workloads
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    w = workloads.config1()
    for _ in range(warmup):
        dl.upsample_torch(w["up"], 112, 112)
        dl.bnstats_f32_torch(w["bn"], w["eps"])
    t0 = time.perf_counter()
    for _ in range(steps):
        dl.upsample_torch(w["up"], 112, 112)
        dl.bnstats_f32_torch(w["bn"], w["eps"])
    return (time.perf_counter() - t0) * 1e3 / steps, torch.get_num_threads()


def run_reference(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    import torch
    steps = args.steps
    ms, cores = cpu_pair_cfg1(torch, steps, args.warmup)
    val = CFG1_BYTES / ms / 1e6
    line = {
        "impl": "reference", "metric": METRIC,
        "value": round(val, 3), "unit": "GB/s", "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD},
        "cpu_baseline": {"value": round(val, 3), "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": f"{steps} full passes of configuration 1 with PyTorch CPU operators "
                                   "(F.interpolate bilinear + var_mean), all host threads"},
        "e2e": {"value": round(val, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def bind_near_gpu(local):
    """Best effort: run this rank on the host cores next to its GPU before any pinned buffer is
    allocated, so that the end-to-end copies do not cross sockets.  Returns a short description."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(local)
        allowed = os.sched_getaffinity(0)
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (max(allowed) // 64) + 1)
        ideal = {64 * i + b for i, w in enumerate(words) for b in range(64) if (int(w) >> b) & 1}
        near = sorted(ideal & allowed)
        if near and set(near) != allowed:
            os.sched_setaffinity(0, near)
            return f"bound to {len(near)} of {len(allowed)} allowed cores next to GPU {local}"
        return f"all {len(allowed)} allowed cores are next to GPU {local}" if near else "no allowed core is next to the GPU"
    except Exception as exc:       # NVML missing or refused: leave the affinity alone
        return f"not bound ({type(exc).__name__})"


def weak_seed(rank):
    """Seed of rank's batch shard of the headline workload (rank 0 = the single-GPU workload)."""
    return 1 + 1000 * rank


def check_headline(torch, sets, w, ex, dev, world):
    """Outside the timed region: the results the timed launches left in every buffer set against
    the oracle.  Upsample bit-exact with the NumPy restatement of this rank's input; mean / invstd
    within 1e-5 of float64 statistics over the batches of ALL ranks (their float64 moments summed
    with an NCCL all-reduce, a path that shares nothing with the in-kernel exchange); and all
    ranks must hold identical bits."""
    import numpy as np
    from oracle import dl
    out = {"upsample_bit_exact": True, "stats_within_1e-5": True, "ranks_identical": True}
    ref_up = dl.upsample_numpy(w["up"].numpy(), 112, 112)
    x = w["bn"].double()
    n = float(x.numel() // x.shape[1])
    mom = torch.stack([torch.full((x.shape[1],), n, dtype=torch.float64), x.sum(dim=(0, 2, 3)),
                       (x * x).sum(dim=(0, 2, 3))], dim=1).to(dev)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(mom, op=dist.ReduceOp.SUM)
    mom = mom.cpu()
    mean = mom[:, 1] / mom[:, 0]
    var = (mom[:, 2] / mom[:, 0] - mean * mean).clamp_min(0)
    invstd = 1.0 / torch.sqrt(var + w["eps"])
    worst = 0.0
    for a, b in sets:
        out["upsample_bit_exact"] &= bool(np.array_equal(a.out.cpu().numpy(), ref_up))
        em = ((b.mean.cpu().double() - mean).abs() / mean.abs()).max().item()
        es = ((b.invstd.cpu().double() - invstd).abs() / invstd.abs()).max().item()
        worst = max(worst, em, es)
    out["stats_within_1e-5"] = bool(worst <= 1e-5)
    out["stats_worst_rel_err"] = float(f"{worst:.3e}")
    if world > 1:
        import torch.distributed as dist
        bits = torch.cat([torch.cat([b.mean, b.invstd]) for _, b in sets]).view(torch.int32)
        lo, hi = bits.clone(), bits.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        out["ranks_identical"] = bool(torch.equal(lo, hi))
        flags = torch.tensor([int(out["upsample_bit_exact"]), int(out["stats_within_1e-5"])], device=dev)
        dist.all_reduce(flags, op=dist.ReduceOp.MIN)
        out["upsample_bit_exact"], out["stats_within_1e-5"] = bool(flags[0].item()), bool(flags[1].item())
    timed_out = bool(ex.timed_out()) if ex is not None else False
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([int(timed_out)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        timed_out = bool(t.item())
    ok = out["upsample_bit_exact"] and out["stats_within_1e-5"] and out["ranks_identical"] and not timed_out
    return ok, timed_out, out


# DRAM bytes (read + write) per launch of the kernel of the timed region, from one ncu capture of
# an isolated launch (dram__bytes_read.sum + dram__bytes_write.sum).  Both are below the
# algorithmic 154,142,720 B because about half of the output is still dirty in L2 when an
# isolated launch ends; the reads (51.4-51.7 MB for 51.4 MB of input) show that nothing is read twice.
NCU_TRAFFIC_BYTES = {"fused_kernel<UpsampleRole,BnStatsRole,896,128,1>": 98_881_792,
                     "fused_kernel<UpsampleRole,BnStatsRole,512,256,2>": 101_843_456,
                     "fused_pool_kernel<UpsampleRole,BnStatsXchgRole,896,128,1>": 98_200_000,
                     "fused_pool_kernel<UpsampleRole,BnStatsXchgRole,384,128,2>": None,
                     "fused_pool_kernel<UpsampleRole,BnStatsXchgRole,512,256,2>": 101_500_000,
                     "fused_pool_kernel<UpsampleRole,BnStatsXchgRole,384,256,2>": 100_000_000}


def run_ours(args):
    import torch
    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    use_dist = world > 1
    # rank 0 keeps all host cores: it also times the CPU baseline
    binding = bind_near_gpu(local) if use_dist and rank != 0 else "affinity left alone"
    if use_dist:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        barrier = lambda: dist.barrier(device_ids=[local])
    else:
        barrier = lambda: None
    from hfuse_b200 import _lib, crypto, ops, sharding, workloads
    _lib.lib()   # fail loudly if the CUDA library is missing
    peak, peak_kind = measured_peak_gbs()

    if args.im2col_path != "default":
        _lib.tune_option("im2col_store_path", 1 if args.im2col_path == "bulk" else 0)
    if args.histc_path != "default":
        _lib.tune_option("histc_load_path", 1 if args.histc_path == "bulk" else 0)
    if args.bnstats_path != "default":
        _lib.tune_option("bnstats_load_path", 1 if args.bnstats_path == "bulk" else 0)
    if args.only:
        return run_only(args, torch, ops, crypto, workloads, dev)
    if args.tune:
        return run_tune(args, torch, ops, crypto, workloads, dev)
    if args.study:
        return run_study(args, torch, ops, crypto, workloads, dev)

    NSETS = 6
    # weak scaling: every rank holds its own draw of the per-GPU configuration (its batch shard)
    w = workloads.config1(seed=weak_seed(rank))
    sets = []
    for _ in range(NSETS):
        sets.append((ops.Upsample(w["up"].to(dev), scale_factor=2), ops.BnStats(w["bn"].to(dev), w["eps"])))
    nbytes = CFG1_BYTES
    collective = "none"
    ex = None
    if use_dist and args.collective == "fused":
        # the cross-GPU sum of the moments happens inside the fused kernel, over peer memory;
        # if any rank cannot map its peers' buffers (CUDA IPC refused), every rank falls back to NCCL
        import torch.distributed as dist
        from hfuse_b200.exchange import BnExchange
        try:
            ex = BnExchange(256)
            ok_flag = torch.ones(1, device=dev)
        except Exception as exc:
            sys.stderr.write(f"rank {rank}: peer-memory exchange unavailable ({exc!r}); using NCCL\n")
            ok_flag = torch.zeros(1, device=dev)
        dist.all_reduce(ok_flag, op=dist.ReduceOp.MIN)
        if ok_flag.item() == 0:
            ex = None
    if args.pair_variant >= 0:
        _lib.tune_set("upsample_bnstats_allreduce" if ex is not None else "upsample_bnstats", args.pair_variant, 0)

    def shape_of(pair):      # "T1,T2,minBlocks" of the variant that will run
        wide = "_wide" if pair.endswith("_allreduce") and world > 4 else ""      # the exchange pair's default beyond four ranks
        d = _lib.tune_variants(pair)[args.pair_variant] if args.pair_variant >= 0 else _lib.tune_default(pair + wide)
        return d.replace(":", ",")
    if args.share_permille >= 0 and ex is not None:
        _lib.tune_set_share("upsample_bnstats_allreduce", args.share_permille)
    if args.tune_share:
        return run_tune_share(args, torch, _lib, ex, sets, NSETS, dev, rank, barrier, use_dist)
    stream = torch.cuda.Stream(dev)          # everything timed runs (and is captured) on this stream
    if ex is not None:
        collective = "in-kernel sum of the [256,3] f64 moments over NVLink peer stores"
        kernel_name = "fused_pool_kernel<UpsampleRole,BnStatsXchgRole,%s>" % shape_of("upsample_bnstats_allreduce")

        def step(i):
            ex.run_pair(*sets[i % NSETS])
        per_step_launches = 1
    elif use_dist:
        # per-GPU moments -> NCCL all-reduce -> finalize kernel, all on the timed stream
        collective = "NCCL all-reduce of the [256,3] f64 moments + finalize kernel"
        kernel_name = "fused_kernel<UpsampleRole,BnStatsRole,%s>" % shape_of("upsample_bnstats")
        for a, b in sets:
            b.moments = torch.empty((256, 3), dtype=torch.float64, device=dev)

        def step(i):
            a, b = sets[i % NSETS]
            ops.run_pair(a, b)
            sharding.allreduce_moments(b.moments)
            m, s_ = ops.bn_finalize(b.moments, b.eps)
            b.mean.copy_(m)
            b.invstd.copy_(s_)
        per_step_launches = 5
    else:
        kernel_name = "fused_kernel<UpsampleRole,BnStatsRole,%s>" % shape_of("upsample_bnstats")

        def step(i):
            ops.run_pair(*sets[i % NSETS])
        per_step_launches = 1

    # ---- warm-up, capture, timed region ------------------------------------------------------
    # The K steps of one pass are replayed from CUDA graphs (one graph of up to 240 consecutive
    # steps, plus a shorter one for what is left), so the host issues a handful of launches per
    # pass whatever K is.  A pass of K steps lasts well under a millisecond for small K, so the
    # timed region is R passes, R chosen so that the region lasts about a second (at least 50):
    # every pass is bracketed by CUDA events on the launching stream, each pass's time is the
    # maximum over ranks, and the figure reported is the median pass (min, max and mean beside
    # it).  The clock sampler runs over exactly that region.
    K = args.steps
    G = min(K, 240)
    graphs = []
    big = None                      # one graph holding P passes with an event between passes
    launch_mode = "direct launches"
    with torch.cuda.stream(stream):
        for i in range(max(args.warmup, NSETS)):
            step(i)
        stream.synchronize()
        if not args.no_graph:
            try:
                for n in ([G] if K % G == 0 else [G, K % G]):
                    g_ = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g_, stream=stream, capture_error_mode="thread_local"):
                        for i in range(n):
                            step(i)
                    graphs.append(g_)
                launch_mode = f"CUDA graph of {G} steps, replayed"
            except Exception as exc:          # capture unsupported here: time direct launches instead
                sys.stderr.write(f"CUDA graph capture failed ({exc!r}); timing direct launches\n")
                graphs = []
                torch.cuda.synchronize()

        def one_pass():
            if graphs:
                for _ in range(K // G):
                    graphs[0].replay()
                if K % G:
                    graphs[1].replay()
            else:
                for i in range(K):
                    step(i)

        for _ in range(3):                    # warm replays; the last one sizes the region
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            one_pass()
            e1.record()
            e1.synchronize()
        est = torch.tensor([max(e0.elapsed_time(e1), 1e-3)], dtype=torch.float64, device=dev)
        if use_dist:
            import torch.distributed as dist
            dist.all_reduce(est, op=dist.ReduceOp.MAX)       # every rank must choose the same R
        R = int(min(max(50, -(-args.region_ms // est.item())), 20000))
        # Short passes (small K) are chained: P passes go into ONE graph with an event-record node
        # between passes, so that a pass does not begin with the host's graph-launch latency (which
        # every rank would see at a slightly different moment).  The events are read after every
        # replay of that graph.
        P = max(1, min(50, 1000 // K)) if graphs and K % G == 0 and K == G else 1
        pass_ev = None
        if P > 1:
            try:
                pass_ev = [torch.cuda.Event(enable_timing=True, external=True) for _ in range(P + 1)]
                big = torch.cuda.CUDAGraph()
                with torch.cuda.graph(big, stream=stream, capture_error_mode="thread_local"):
                    pass_ev[0].record()
                    for p_ in range(P):
                        for i in range(K):
                            step(p_ * K + i)
                        pass_ev[p_ + 1].record()
                big.replay()
                stream.synchronize()
                pass_ev[0].elapsed_time(pass_ev[1])          # raises if such events cannot be timed
                R = -(-R // P) * P
                launch_mode = f"CUDA graph of {P} passes x {K} steps with an event node between passes, replayed"
            except Exception as exc:
                sys.stderr.write(f"event nodes inside a graph unavailable ({exc!r}); one graph launch per pass\n")
                big, pass_ev, P = None, None, 1
                torch.cuda.synchronize()
        sampler = ClockSampler(local)
        sampler.start()       # before the barrier: starting it takes a variable time on every rank
        torch.cuda.synchronize()
        barrier()
        pass_ms = []
        if big is not None:
            for _ in range(R // P):
                big.replay()
                stream.synchronize()
                pass_ms += [pass_ev[p_].elapsed_time(pass_ev[p_ + 1]) for p_ in range(P)]
        else:
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(R + 1)]
            ev[0].record()
            for r in range(R):
                one_pass()
                ev[r + 1].record()
            stream.synchronize()
            pass_ms = [ev[r].elapsed_time(ev[r + 1]) for r in range(R)]
    torch.cuda.synchronize()
    barrier()
    clocks = sampler.stop()
    # Every rank has the times of its own R passes.  Coupled ranks run at one common rate but a rank
    # that got ahead in one pass waits in the next, so its passes alternate around that rate: the
    # figure reported is each rank's MEDIAN pass, the maximum of those over the ranks (taking the
    # maximum pass by pass first would count every such alternation as a slow pass).  Beside it:
    # the mean (each rank's whole region, maximum over ranks) and the extreme passes of any rank.
    mine = torch.tensor(pass_ms, dtype=torch.float64, device=dev)
    stats = torch.stack([mine.median(), mine.mean(), mine.max(), -mine.min()])
    if use_dist:
        import torch.distributed as dist
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    stats = stats.cpu()
    ms = float(stats[0])                           # one pass of K steps
    ms_mean, ms_max, ms_min = float(stats[1]), float(stats[2]), -float(stats[3])
    launches = per_step_launches * K * R
    t_step = ms / K                                # ms per step = per launch of the fused kernel

    parity_ok, timed_out, parity = check_headline(torch, sets, w, ex, dev, world)

    # context for the roofline fraction: a device-to-device copy (tensor.copy_, i.e. cudaMemcpyAsync)
    # that moves the same number of bytes (half read, half written), timed the same way
    half = nbytes // 2 // 4
    csrc = [torch.empty(half, dtype=torch.float32, device=dev).normal_() for _ in range(NSETS)]
    cdst = [torch.empty(half, dtype=torch.float32, device=dev) for _ in range(NSETS)]
    t_copy = graph_region(torch, lambda i: cdst[i % NSETS].copy_(csrc[i % NSETS]), NSETS, 120, 3)
    del csrc, cdst
    # and a bare load/store kernel with the fused pair's own mix: 51,380,224 B read (both inputs), 102,762,496 B written
    rd, wr = 51_380_224, 102_762_496
    psrc = [torch.empty(rd // 4, dtype=torch.float32, device=dev).normal_() for _ in range(NSETS)]
    pdst = [torch.empty(wr // 4, dtype=torch.float32, device=dev) for _ in range(NSETS)]

    def probe(i):
        _lib.check(_lib.lib().hfuse_hbm_probe(psrc[i % NSETS].data_ptr(), rd, pdst[i % NSETS].data_ptr(), wr,
                                              torch.cuda.current_stream().cuda_stream), "hfuse_hbm_probe")
    t_mix = graph_region(torch, probe, NSETS, 120, 3)

    def probe_w(i):     # the same kernel writing only: what this memory sustains for pure stores
        _lib.check(_lib.lib().hfuse_hbm_probe(None, 0, pdst[i % NSETS].data_ptr(), wr,
                                              torch.cuda.current_stream().cuda_stream), "hfuse_hbm_probe")
    t_wr = graph_region(torch, probe_w, NSETS, 120, 3)
    # and both again with the writes issued as bulk (TMA) copies of 8 KB from shared memory
    wr_b = wr // 8192 * 8192

    def probe_b(i):
        _lib.check(_lib.lib().hfuse_hbm_probe_bulk(psrc[i % NSETS].data_ptr(), rd, pdst[i % NSETS].data_ptr(), wr_b,
                                                   torch.cuda.current_stream().cuda_stream), "hfuse_hbm_probe_bulk")
    t_mix_b = graph_region(torch, probe_b, NSETS, 120, 3)

    def probe_wb(i):
        _lib.check(_lib.lib().hfuse_hbm_probe_bulk(None, 0, pdst[i % NSETS].data_ptr(), wr_b,
                                                   torch.cuda.current_stream().cuda_stream), "hfuse_hbm_probe_bulk")
    t_wr_b = graph_region(torch, probe_wb, NSETS, 120, 3)
    del psrc, pdst

    # ---- end to end through the C ABI with host buffers (pinned), copies inside the timed region
    h_up, h_bn = w["up"].pin_memory(), w["bn"].pin_memory()
    # Two buffer sets and three streams (upload, kernel, download): the upload of step i+1 and
    # the download of step i-1 overlap the kernel of step i, so both PCIe directions are busy at
    # once.  Every step still uploads its own inputs and downloads its own outputs; the host
    # takes the results of a step as soon as its download event has completed.
    DEPTH = 2
    h_outs = [torch.empty(sets[0][0].out.shape, dtype=torch.float32).pin_memory() for _ in range(DEPTH)]
    h_stats = [torch.empty((2, 256), dtype=torch.float32).pin_memory() for _ in range(DEPTH)]
    s_in, s_k, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    e2e_steps = max(4, min(args.steps, 12))

    def e2e_run(with_kernel):
        """ms per step of the pipelined upload / kernel / download loop; without the kernel it is
        the same copies on the same streams and buffers: what the host link alone allows."""
        uploaded, computed, downloaded = [None] * DEPTH, [None] * DEPTH, [None] * DEPTH

        def e2e_step(i):
            k = i % DEPTH
            a0, b0 = sets[k]
            with torch.cuda.stream(s_in):
                if computed[k] is not None:
                    s_in.wait_event(computed[k])           # the previous kernel on this set has read its inputs
                a0.x.copy_(h_up, non_blocking=True)
                b0.x.copy_(h_bn, non_blocking=True)
                uploaded[k] = torch.cuda.Event()
                uploaded[k].record()
            with torch.cuda.stream(s_k):
                s_k.wait_event(uploaded[k])
                if downloaded[k] is not None:
                    s_k.wait_event(downloaded[k])          # the previous outputs of this set have left the device
                if with_kernel:
                    if ex is not None:
                        ex.run_pair(a0, b0)
                    else:
                        ops.run_pair(a0, b0)
                computed[k] = torch.cuda.Event()
                computed[k].record()
            with torch.cuda.stream(s_out):
                s_out.wait_event(computed[k])
                if downloaded[k] is not None:
                    downloaded[k].synchronize()            # the host has finished with this pinned buffer
                h_outs[k].copy_(a0.out, non_blocking=True)
                h_stats[k][0].copy_(b0.mean, non_blocking=True)
                h_stats[k][1].copy_(b0.invstd, non_blocking=True)
                downloaded[k] = torch.cuda.Event()
                downloaded[k].record()

        def e2e_drain():
            for evd in downloaded:
                if evd is not None:
                    evd.synchronize()                      # the caller holds every result
        for i in range(DEPTH):
            e2e_step(i)
        e2e_drain()
        torch.cuda.synchronize()
        barrier()
        t0 = time.perf_counter()
        for i in range(e2e_steps):
            e2e_step(i)
        e2e_drain()
        t_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps     # host clock: it ends when the results are on the host
        if use_dist:
            import torch.distributed as dist
            t = torch.tensor([t_ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            t_ms = float(t.item())
        return t_ms

    e2e_ms = e2e_run(True)
    copy_ms = e2e_run(False)
    h2d = h_up.numel() * 4 + h_bn.numel() * 4
    d2h = h_outs[0].numel() * 4 + h_stats[0].numel() * 4

    line = {
        "metric": METRIC,
        "value": round(world * nbytes * K / ms / 1e6, 1), "unit": "GB/s", "n_gpus": world,
        "steps": K, "warmup": args.warmup, "ms_per_step": round(t_step, 5),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "l2": f"steps rotate over {NSETS} independent buffer sets "
                               f"({NSETS * nbytes >> 20} MiB in total, L2 is 126 MB)",
                   "launch": launch_mode,
                   "timed": {"passes": R, "steps_per_pass": K, "region_ms": round(ms_mean * R, 2),
                             "us_per_step_median": round(t_step * 1e3, 3),
                             "us_per_step_min": round(ms_min / K * 1e3, 3),
                             "us_per_step_max": round(ms_max / K * 1e3, 3),
                             "us_per_step_mean": round(ms_mean / K * 1e3, 3),
                             "rule": "every pass = K steps between two CUDA events on the launching stream; "
                                     "per rank the median pass (and the mean of its region), max over ranks"},
                   "parallelism": f"batch-sharded x{world} (every rank its own draw of the per-GPU batch)",
                   "collective": collective, "host_binding": binding},
        "gpu_launches": launches,
        "parity_ok": parity_ok, "exchange_timed_out": timed_out, "parity": parity,
        "e2e": {"value": round(world * nbytes / e2e_ms / 1e6, 2), "unit": "GB/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": round(e2e_ms, 4),
                "copy_only_ms_per_step": round(copy_ms, 4), "frac_of_copy_only": round(copy_ms / e2e_ms, 3),
                "pipeline": "2 buffer sets, upload / kernel / download streams overlapped"},
        "roofline": {"bound": "hbm", "achieved": round(nbytes / t_step / 1e6, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(nbytes / t_step / 1e6 / peak, 4), "traffic": NCU_TRAFFIC_BYTES.get(kernel_name),
                     "peak_kind": peak_kind, "kernel": kernel_name,
                     "kernel_us": round(t_step * 1e3, 2),
                     "kernel_us_source": "the timed region: its only launches are this kernel",
                     "same_bytes_memcpy_d2d_us": round(t_copy * 1e3, 2),
                     "same_read_write_mix_bare_kernel_us": round(t_mix * 1e3, 2),
                     "write_only_bare_kernel_gbs": round(wr / t_wr / 1e6, 1),
                     "same_read_write_mix_bulk_store_kernel_us": round(t_mix_b * 1e3, 2),
                     "write_only_bulk_store_kernel_gbs": round(wr_b / t_wr_b / 1e6, 1)},
        "clocks": clocks,
    }
    if use_dist and not args.no_extras:
        line["dl_sharded"] = dl_sharded(torch, ops, sharding, workloads, dev, rank, world, barrier, peak)
        sharded = crypto_sharded(torch, crypto, sharding, workloads, dev, rank, world, barrier)
        if rank == 0:
            line["crypto_sharded"] = sharded
    if rank == 0:
        if not args.no_extras and world == 1:
            line["pairs"] = extras(torch, ops, crypto, workloads, dev, max(20, min(args.steps, 200)), 3, peak, barrier)
        torch.cuda.synchronize()
        cpu_ms, cores = cpu_pair_cfg1(torch, 5, 1)
        line["cpu_baseline"] = {"value": round(CFG1_BYTES / cpu_ms / 1e6, 3), "unit": "GB/s", "cores": cores,
                                "kind": "port", "sample": "5 full passes of configuration 1 with PyTorch CPU operators"}
        print(json.dumps(line), flush=True)
    if use_dist:
        wait_for_rank0(rank)
        shutdown(torch, (graphs, big))


def wait_for_rank0(rank):
    """Ranks other than 0 sleep on the rendezvous store until rank 0 has timed the CPU baseline
    and printed the line: a collective barrier here would have them spin on the host cores
    that the CPU baseline is being measured on."""
    import torch.distributed as dist
    store = dist.distributed_c10d._get_default_store()
    if rank == 0:
        store.set("hfuse_bench_line_printed", "1")
    else:
        store.wait(["hfuse_bench_line_printed"])


def dl_sharded(torch, ops, sharding, workloads, dev, rank, world, barrier, peak):
    """Configuration 2 split over the ranks (strong scaling: the total work is fixed): the im2col
    batch of 32 and the 2^24 histogram values are cut into one contiguous shard per GPU, every rank
    runs the fused im2col + histc pair on its shard, and the 256 counts are summed over ranks with
    an NCCL all-reduce on a side stream (it runs under the next step's kernel).  Time = max over
    ranks of the device time per step (replayed from a CUDA graph); the results are compared with the
    oracle on the unsplit inputs outside the timed region."""
    import numpy as np
    import torch.distributed as dist
    from oracle import dl
    w = workloads.config2()
    NS = 4
    im = sharding.shard_batch(w["im"], rank, world).contiguous()
    hv = sharding.shard_flat(w["hist"], rank, world).contiguous()
    sets = [(ops.Im2col(im.to(dev), **w["im2col"]), ops.Histc(hv.to(dev), w["bins"], w["lo"], w["hi"])) for _ in range(NS)]
    stream, side = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    summed = [None] * NS          # per buffer set: its counts have been summed (they may be cleared again)

    def step(i):
        # the all-reduce of step i runs on a side stream under the kernel of step i + 1
        k = i % NS
        a, b = sets[k]
        if summed[k] is not None:
            torch.cuda.current_stream().wait_event(summed[k])
        ops.run_pair(a, b)
        done = torch.cuda.Event()
        done.record()
        with torch.cuda.stream(side):
            side.wait_event(done)
            sharding.allreduce_counts(b.counts)
            summed[k] = torch.cuda.Event()
            summed[k].record()

    def join():
        torch.cuda.current_stream().wait_stream(side)
    with torch.cuda.stream(stream):
        for i in range(2 * NS):
            step(i)
        join()
        stream.synchronize()
        summed = [None] * NS
        G = 6 * NS
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
            for i in range(G):
                step(i)
            join()
        summed = [None] * NS      # events recorded during capture must not be waited on outside
        graph.replay()
        stream.synchronize()
        barrier()
        reps = 20
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(reps + 1)]
        ev[0].record()
        for r in range(reps):
            graph.replay()
            ev[r + 1].record()
        stream.synchronize()
    t = torch.tensor([ev[r].elapsed_time(ev[r + 1]) for r in range(reps)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    us = float(t.median()) / G * 1e3
    # parity, outside the timed region
    want_counts = dl.histc_torch(w["hist"], w["bins"], w["lo"], w["hi"])
    ok = True
    for a, b in sets:
        ok &= bool(np.array_equal(b.counts.cpu().numpy().view(np.uint32), want_counts))
    ok &= bool(torch.equal(sets[0][0].out.cpu(), dl.im2col_torch(im, 3, 3, 1, 1, 1, 1, 1, 1)))
    flag = torch.tensor([int(ok)], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    del graph
    return {"workload": f"config 2 split over {world} GPUs: im2col batch {im.shape[0]} and {hv.numel()} histogram values per GPU",
            "scaling": "strong", "us_per_step": round(us, 2), "GB_per_s_total": round(CFG2_BYTES / us / 1e3, 1),
            "frac_of_hbm_peak_per_gpu": round(CFG2_BYTES / world / us / 1e3 / peak, 3),
            "collective": "NCCL all-reduce of the 256 uint32 counts on a side stream, under the next step's kernel",
            "parity_ok": bool(flag.item())}


def run_tune_share(args, torch, _lib, ex, sets, nsets, dev, rank, barrier, use_dist):
    """Sweep of the exchange pair (upsample + statistics + in-kernel all-reduce) over thread splits
    and over the share of the upsample that the statistics range takes over, at the launched
    number of ranks; the time of a step is the maximum over ranks.  Rank 0 prints one JSON object."""
    from hfuse_b200.exchange import BnExchange
    if ex is None:
        ex = BnExchange(256)            # world of one (or NCCL fallback refused): the local buffer
    name = "upsample_bnstats_allreduce"
    descr = _lib.tune_variants(name)
    variants = [v for v, d in enumerate(descr) if ":0:" not in d]
    # "pool": items drawn from a cursor by both ranges; "pool_bulk": the same with the statistics read through bulk
    # copies; "0_bulk": no share (the upsample stays with its own range), statistics through bulk copies
    shares = (0, 100, 200, 300, 400, 500, "pool", "pool_bulk", "0_bulk")
    reps, gsteps = 6, 4 * nsets
    table = {}
    for v in variants:
        row = {}
        for share in shares:
            _lib.tune_set(name, v, 0)
            _lib.tune_option("bnstats_load_path", 1 if str(share).endswith("_bulk") else 0)
            if share in ("pool", "pool_bulk"):
                _lib.tune_set_share(name, -1)
                _lib.tune_option("exchange_pair_pool", 1)
            else:
                _lib.tune_set_share(name, 0 if share == "0_bulk" else share)
            for i in range(nsets):
                ex.run_pair(*sets[i])
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                for i in range(gsteps):
                    ex.run_pair(*sets[i % nsets])
            graph.replay()
            torch.cuda.synchronize()
            barrier()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(reps):
                graph.replay()
            e.record()
            torch.cuda.synchronize()
            t = torch.tensor([s.elapsed_time(e)], dtype=torch.float64, device=dev)
            if use_dist:
                import torch.distributed as dist
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            row[str(share)] = round(float(t.item()) / (reps * gsteps) * 1e3, 2)
            del graph
        table[descr[v]] = row
    _lib.tune_option("exchange_pair_pool", -1)
    _lib.tune_option("bnstats_load_path", -1)
    _lib.tune_set(name, -1, 0)
    _lib.tune_set_share(name, -1)
    timed_out = ex.timed_out()
    if rank == 0:
        best = min(((t, d, sh) for d, row in table.items() for sh, t in row.items()))
        print(json.dumps({"pair": name, "n_gpus": args.gpus, "unit": "us per step, max over ranks",
                          "best": {"variant": best[1], "index": descr.index(best[1]),
                                   "share_permille": -1 if best[2].startswith("pool") else int(best[2].split("_")[0]),
                                   "pool": best[2].startswith("pool"), "bnstats_bulk": int(best[2].endswith("_bulk")),
                                   "us": best[0]},
                          "exchange_timed_out": timed_out, "table": table}))
    if use_dist:
        shutdown(torch, None)
    ex.close()


def crypto_sharded(torch, crypto, sharding, workloads, dev, rank, world, barrier):
    """Configurations 3 and 4 with the nonce range cut into one contiguous shard per GPU (strong
    scaling: the total sweep is fixed), DAG replicated.  Time = max over ranks of the device time of
    the rank's fused launch; hit lists are gathered and merged on the host."""
    import torch.distributed as dist
    out = {}

    def timed(fn):
        fn()                                   # warm-up (also builds the occupancy cache)
        torch.cuda.synchronize()
        barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    c3 = workloads.config3()
    st, n = sharding.shard_nonces(c3["start"], c3["count"], rank, world)
    a = crypto.Blake256(c3["blake_header"], st, n, c3["target"])
    b = crypto.Sha256d(c3["sha_header"], st, n, c3["target"])
    ms = timed(lambda: crypto.run_pair(a, b))
    hits_a, hits_b = sharding.gather_hits(a.result()[1]), sharding.gather_hits(b.result()[1])
    out["cfg3_blake256_sha256d"] = {"nonces_each_total": c3["count"], "fused_ms": round(ms, 2),
                                    "GH_per_s_each": round(c3["count"] / ms / 1e6, 3),
                                    "hits": [len(hits_a), len(hits_b)], "blake256_nonces": [h[0] for h in hits_a]}
    c4 = workloads.config4(dev)
    st, n = sharding.shard_nonces(c4["start"], c4["count"], rank, world)
    s_ = crypto.Sia(c4["sia_header"], st, n, c4["target"])
    e_ = crypto.Ethash(c4["dag"], c4["header_hash"], st, n, c4["target"])
    ms = timed(lambda: crypto.run_pair(s_, e_))
    hits_s, hits_e = sharding.gather_hits(s_.result()[1]), sharding.gather_hits(e_.result()[1])
    out["cfg4_sia_ethash"] = {"nonces_each_total": c4["count"], "fused_ms": round(ms, 2),
                              "ethash_MH_per_s": round(c4["count"] / ms / 1e3, 1),
                              "sia_GH_per_s": round(c4["count"] / ms / 1e6, 3), "hits": [len(hits_s), len(hits_e)]}
    return out


def shutdown(torch, graph):
    """Leave a multi-rank run without waiting on NCCL teardown: with collectives captured in a
    CUDA graph, destroy_process_group() has been seen to block for minutes after all work was
    done.  Everything is synchronised and rank 0 has printed its line, so drop the graph, give
    the teardown a few seconds on a helper thread, and exit 0 either way."""
    import threading
    import torch.distributed as dist
    torch.cuda.synchronize()
    dist.barrier()
    del graph
    sys.stdout.flush()
    sys.stderr.flush()
    t = threading.Thread(target=dist.destroy_process_group, daemon=True)
    t.start()
    t.join(5.0)
    os._exit(0)


def run_only(args, torch, ops, crypto, workloads, dev):
    """One kernel or pair on its benchmark workload, for profiling and store-path comparisons:
    --only cfg0..cfg4 | any pair name (im2col_bnstats, histc_maxpool, sha256d_ethash, ...)
    --mode fused|b2b|a|b [--graph].  cfg0/1/2 = im2col_maxpool / upsample_bnstats / im2col_histc,
    cfg3/4 = blake256_sha256d / sia_ethash.  The halves of the other pairs take the shapes they
    have in the configuration that names them (im2col at batch 16 except beside histc).  cfg1 also
    takes --mode xchg: the exchange pair (send, share of the upsample, collect) over a world of one."""
    if "," in args.only or ":" in args.only:
        # several items in one process ("cfg0:a,cfg0:b,im2col_bnstats:fused"): one profiler run covers them all
        for item in args.only.split(","):
            sub = argparse.Namespace(**vars(args))
            sub.only, _, mode = item.partition(":")
            sub.mode = mode or args.mode
            run_only(sub, torch, ops, crypto, workloads, dev)
            torch.cuda.empty_cache()
        return
    from hfuse_b200 import _lib
    barrier = lambda: None
    alias = {"cfg0": "im2col_maxpool", "cfg1": "upsample_bnstats", "cfg2": "im2col_histc",
             "cfg3": "blake256_sha256d", "cfg4": "sia_ethash"}
    name = alias.get(args.only, args.only)
    if name in _lib.DL_PAIRS:
        w0, w1, w2 = workloads.config0(), workloads.config1(), workloads.config2()

        def mk(key):
            if key == "im2col":
                return ops.Im2col((w2 if name == "im2col_histc" else w0)["im"].to(dev), **w0["im2col"])
            if key == "maxpool":
                return ops.MaxPool(w0["pool"].to(dev), **w0["maxpool"])
            if key == "bnstats":
                return ops.BnStats(w1["bn"].to(dev), w1["eps"])
            if key == "upsample":
                return ops.Upsample(w1["up"].to(dev), scale_factor=2)
            return ops.Histc(w2["hist"].to(dev), w2["bins"], w2["lo"], w2["hi"])
        ka, kb = _lib.DL_PAIRS[name]
        sets = [(mk(ka), mk(kb)) for _ in range(2)]
        if args.mode == "xchg":
            from hfuse_b200.exchange import BnExchange
            ex = BnExchange(sets[0][1].x.shape[1])
            fn = lambda i: ex.run_pair(*sets[i % 2])
        else:
            fn = {"fused": lambda i: ops.run_pair(*sets[i % 2]), "b2b": lambda i: ops.run_back_to_back(*sets[i % 2]),
                  "a": lambda i: ops.run(sets[i % 2][0]), "b": lambda i: ops.run(sets[i % 2][1])}[args.mode]
        if args.graph:
            ms = graph_region(torch, fn, 2, args.steps, args.warmup)
        else:
            ms = time_region(torch, fn, args.steps, args.warmup, barrier) / args.steps
        print(json.dumps({"only": name, "mode": args.mode, "us_per_step": round(ms * 1e3, 2)}))
        return
    if name not in _lib.CRYPTO_PAIRS:
        raise SystemExit(f"--only {args.only}: not a configuration or a pair name")
    count = args.count
    c3 = workloads.config3()
    c4 = None
    if "ethash" in name or "sia" in name:      # the Sia header comes from configuration 4; only ethash needs its DAG
        c4 = workloads.config4(dev, dag_items=args.dag_items if "ethash" in name else 1024)

    def mkc(key):
        if key == "blake256":
            return crypto.Blake256(c3["blake_header"], 0, count, c3["target"])
        if key == "sha256d":
            return crypto.Sha256d(c3["sha_header"], 0, count, c3["target"])
        if key == "sia":
            return crypto.Sia(c4["sia_header"], 0, count, c4["target"])
        return crypto.Ethash(c4["dag"], c4["header_hash"], 0, count, c4["target"])
    ka, kb = _lib.CRYPTO_PAIRS[name]
    a, b = mkc(ka), mkc(kb)
    fn = {"fused": lambda i: crypto.run_pair(a, b), "b2b": lambda i: crypto.run_back_to_back(a, b),
          "a": lambda i: crypto.run(a), "b": lambda i: crypto.run(b)}[args.mode]
    ms = time_region(torch, fn, args.steps, args.warmup, barrier) / args.steps
    print(json.dumps({"only": name, "mode": args.mode, "count": count, "ms_per_step": round(ms, 3)}))


def run_tune(args, torch, ops, crypto, workloads, dev):
    """Sweep every compiled (T1, T2, blocks/SM) variant of every kernel and pair on the
    benchmark workloads and print the fastest per name as JSON (the reference's split /
    register-cap sweep, tools/llvm-smart-fuser/main.cpp:215-236 and
    scripts/profile_and_collect_data.py:40-57, done at run time instead of by recompiling).
    hfuse_b200/apply_tuning.py writes the result into the *_tuned.inc defaults."""
    from hfuse_b200 import _lib
    NS = 4
    w0, w1, w2 = workloads.config0(), workloads.config1(), workloads.config2()

    def mk(key, big_im2col=False):
        if key == "im2col":
            return ops.Im2col((w2 if big_im2col else w0)["im"].to(dev), **w0["im2col"])
        if key == "maxpool":
            return ops.MaxPool(w0["pool"].to(dev), **w0["maxpool"])
        if key == "bnstats":
            return ops.BnStats(w1["bn"].to(dev), w1["eps"])
        if key == "upsample":
            return ops.Upsample(w1["up"].to(dev), scale_factor=2)
        return ops.Histc(w2["hist"].to(dev), w2["bins"], w2["lo"], w2["hi"])

    result = {"solo": {}, "pair": {}}
    steps = 48

    def paths_of(name):
        """(store path of the im2col role, load path of the statistics role) combinations to sweep
        for this kernel or pair; None where the kernel has no such role."""
        ips = (0, 1) if "im2col" in name else (None,)
        bps = (0, 1) if "bnstats" in name else (None,)
        hps = (0, 1) if "histc" in name else (None,)
        return [(ip, bp, hp) for ip in ips for bp in bps for hp in hps]

    def label(d, path):
        ip, bp, hp = path
        return d + ("" if ip is None else f" path{ip}") + ("" if bp is None else f" bn{bp}") + ("" if hp is None else f" h{hp}")

    def sweep(name, run_one):
        """{((im2col path, statistics path), variant description): us} over every path and compiled variant."""
        times = {}
        try:
            for path in paths_of(name):
                if path[0] is not None:
                    _lib.tune_option("im2col_store_path", path[0])
                if path[1] is not None:
                    _lib.tune_option("bnstats_load_path", path[1])
                if path[2] is not None:
                    _lib.tune_option("histc_load_path", path[2])
                for v, d in enumerate(_lib.tune_variants(name)):
                    _lib.tune_set(name, v, 0)
                    times[(path, d)] = round(graph_region(torch, run_one, NS, steps, 3) * 1e3, 2)
        finally:
            _lib.tune_option("im2col_store_path", -1)
            _lib.tune_option("bnstats_load_path", -1)
            _lib.tune_option("histc_load_path", -1)
            _lib.tune_set(name, -1, 0)
        return times

    def describe(times, name, horizontal_only):
        descr = _lib.tune_variants(name)
        cand = {k: t for k, t in times.items() if not (horizontal_only and ":0:" in k[1])}
        (path, d), us = min(cand.items(), key=lambda kv: kv[1])
        out = {"best": descr.index(d), "variant": d, "us": us,
               "all": {label(d2, p): t for (p, d2), t in times.items()}}
        if path[0] is not None:
            out["im2col_bulk"] = path[0]
        if path[1] is not None:
            out["bnstats_bulk"] = path[1]
        if path[2] is not None:
            out["histc_bulk"] = path[2]
        return out, path

    for key in _lib.DL_SOLO:
        # im2col appears at two sizes in the benchmark (batch 16 and batch 32): its standalone
        # choice is made on the mean of both
        sets = [mk(key, big_im2col=(key == "im2col" and i % 2 == 1)) for i in range(NS)]
        times = sweep(key, lambda i: ops.run(sets[i % NS]))
        out, path = describe(times, key, False)
        result["solo"][key] = out
        _lib.tune_set(key, out["best"], 0)       # keep the best standalone for the b2b baseline
        if path[0] is not None:
            solo_im2col_path = path[0]
        if path[1] is not None:
            solo_bn_path = path[1]
        if path[2] is not None:
            solo_histc_path = path[2]
        del sets
        torch.cuda.empty_cache()
    for name, (ka, kb) in _lib.DL_PAIRS.items():
        big = name == "im2col_histc"
        sets = [(mk(ka, big), mk(kb, big)) for _ in range(NS)]
        if "im2col" in name:                     # the baseline's standalone im2col takes ITS best path
            _lib.tune_option("im2col_store_path", solo_im2col_path)
        if "bnstats" in name:                    # and so does the standalone statistics kernel
            _lib.tune_option("bnstats_load_path", solo_bn_path)
        if "histc" in name:                      # and the standalone histogram kernel
            _lib.tune_option("histc_load_path", solo_histc_path)
        t_b2b = graph_region(torch, lambda i: ops.run_back_to_back(*sets[i % NS]), NS, steps, 3) * 1e3
        times = sweep(name, lambda i: ops.run_pair(*sets[i % NS]))
        out, _ = describe(times, name, True)
        vert = {k: t for k, t in times.items() if ":0:" in k[1]}
        vbest = min(vert, key=vert.get)
        out.update({"back_to_back_us": round(t_b2b, 2), "speedup": round(t_b2b / out["us"], 3),
                    "vertical_best": vbest[1], "vertical_us": vert[vbest]})
        result["pair"][name] = out
        del sets
        torch.cuda.empty_cache()
    if args.tune_skip_crypto:
        print(json.dumps(result))
        return
    # crypto: reduced sweeps, 2^27 nonces (the benchmark configurations give both halves the same
    # count).  For ethash and its partners that is 0.2 s per launch: long enough for the board to reach
    # its power cap, under which the 2^30-nonce benchmark sweeps run; the best block shapes under the cap
    # are not the best ones of a few milliseconds.
    c3, c4 = workloads.config3(), workloads.config4(dev)
    NA, NE = 1 << 27, 1 << 27

    def mkc(key, n=None):
        if key == "blake256":
            return crypto.Blake256(c3["blake_header"], 0, n or NA, c3["target"])
        if key == "sha256d":
            return crypto.Sha256d(c3["sha_header"], 0, n or NA, c3["target"])
        if key == "sia":
            return crypto.Sia(c4["sia_header"], 0, n or NA, c4["target"])
        return crypto.Ethash(c4["dag"], c4["header_hash"], 0, NE, c4["target"])

    none = lambda: None
    for key in _lib.CRYPTO_SOLO:
        sobj = mkc(key)
        times = {}
        for v, d in enumerate(_lib.tune_variants(key)):
            _lib.tune_set(key, v, 0)
            times[d] = round(time_region(torch, lambda i: crypto.run(sobj), 2, 1, none) / 2, 3)
        best = min(times, key=times.get)
        _lib.tune_set(key, list(times).index(best), 0)
        result["solo"][key] = {"best": list(times).index(best), "variant": best, "ms": times[best], "all": times}
    for name, (ka, kb) in _lib.CRYPTO_PAIRS.items():
        n = NE if "ethash" in (ka, kb) else NA
        a, b = mkc(ka, n), mkc(kb, n)
        t_b2b = time_region(torch, lambda i: crypto.run_back_to_back(a, b), 2, 1, none) / 2
        times = {}
        for v, d in enumerate(_lib.tune_variants(name)):
            _lib.tune_set(name, v, 0)
            times[d] = round(time_region(torch, lambda i: crypto.run_pair(a, b), 2, 1, none) / 2, 3)
        _lib.tune_set(name, -1, 0)
        best = min(times, key=times.get)
        result["pair"][name] = {"best": list(times).index(best), "variant": best, "ms": times[best],
                                "back_to_back_ms": round(t_b2b, 3), "speedup": round(t_b2b / times[best], 3),
                                "all": times}
    print(json.dumps(result))


def run_study(args, torch, ops, crypto, workloads, dev):
    """Speedup of the fused pair over back-to-back as a function of the ratio of the two
    standalone times (the reference's Fig. 7 scatter, scripts/analyze_nvprof.py:272-273,483-648):
    one half keeps its benchmark size, the other half's batch (or nonce count) is scaled."""
    from hfuse_b200 import _lib
    NS, steps = 3, 36
    g = torch.Generator().manual_seed(7)

    def mk(key, scale):
        if key == "im2col":
            return ops.Im2col((torch.rand(max(1, int(16 * scale)), 64, 56, 56, generator=g) * 2 - 1).to(dev), 3, 1, 1, 1)
        if key == "maxpool":
            return ops.MaxPool((torch.rand(max(1, int(16 * scale)), 64, 112, 112, generator=g) * 2 - 1).to(dev), 2, 2)
        if key == "bnstats":
            return ops.BnStats((0.5 + 2 * torch.randn(max(1, int(32 * scale)), 256, 28, 28, generator=g)).to(dev), 1e-5)
        if key == "upsample":
            return ops.Upsample(torch.rand(max(1, int(16 * scale)), 128, 56, 56, generator=g).to(dev), scale_factor=2)
        return ops.Histc(torch.randn(int((1 << 24) * scale) // 4 * 4, generator=g).to(dev), 256, -4.0, 4.0)

    rows = []
    names = ("im2col_maxpool", "upsample_bnstats", "im2col_histc", "histc_maxpool", "maxpool_bnstats")
    scales = (0.25, 0.5, 1.0, 2.0, 4.0)
    if args.quick:          # a short form for tests: two pairs, three ratios, no crypto rows
        names, scales = ("upsample_bnstats", "histc_maxpool"), (0.5, 1.0, 2.0)
    for name in names:
        ka, kb = _lib.DL_PAIRS[name]
        for scale in scales:
            sets = [(mk(ka, 1.0), mk(kb, scale)) for _ in range(NS)]
            ta = graph_region(torch, lambda i: ops.run(sets[i % NS][0]), NS, steps, 3)
            tb = graph_region(torch, lambda i: ops.run(sets[i % NS][1]), NS, steps, 3)
            t2 = graph_region(torch, lambda i: ops.run_back_to_back(*sets[i % NS]), NS, steps, 3)
            best_h, best_v = (None, None), (None, None)
            for v, d in enumerate(_lib.tune_variants(name)):
                _lib.tune_set(name, v, 0)
                t = graph_region(torch, lambda i: ops.run_pair(*sets[i % NS]), NS, steps, 3)
                if ":0:" in d:
                    best_v = (t, d) if best_v[0] is None or t < best_v[0] else best_v
                else:
                    best_h = (t, d) if best_h[0] is None or t < best_h[0] else best_h
            _lib.tune_set(name, -1, 0)
            rows.append({"pair": name, "second_half_scale": scale, "first_us": round(ta * 1e3, 2),
                         "second_us": round(tb * 1e3, 2), "ratio_first_over_second": round(ta / tb, 3),
                         "back_to_back_us": round(t2 * 1e3, 2), "horizontal_us": round(best_h[0] * 1e3, 2),
                         "horizontal_variant": best_h[1], "vertical_us": round(best_v[0] * 1e3, 2),
                         "speedup_horizontal": round(t2 / best_h[0], 3), "speedup_vertical": round(t2 / best_v[0], 3)})
            del sets
            torch.cuda.empty_cache()
    if args.quick:
        print(json.dumps({"study": rows}))
        return
    c3, c4 = workloads.config3(), workloads.config4(dev)
    none = lambda: None
    NE = 1 << 22

    def med3(fn):   # a few milliseconds of random DAG reads move the board's clocks: median of three short regions
        return sorted(time_region(torch, fn, 2, 1, none) / 2 for _ in range(3))[1]

    for mult in (1, 4, 16, 64):
        a = crypto.Sia(c4["sia_header"], 0, NE * mult, c4["target"])
        b = crypto.Ethash(c4["dag"], c4["header_hash"], 0, NE, c4["target"])
        ta, tb, t2 = med3(lambda i: crypto.run(a)), med3(lambda i: crypto.run(b)), med3(lambda i: crypto.run_back_to_back(a, b))
        best = (None, None)
        for v, d in enumerate(_lib.tune_variants("sia_ethash")):
            _lib.tune_set("sia_ethash", v, 0)
            t = med3(lambda i: crypto.run_pair(a, b))
            best = (t, d) if best[0] is None or t < best[0] else best
        _lib.tune_set("sia_ethash", -1, 0)
        rows.append({"pair": "sia_ethash", "sia_nonces_per_ethash_nonce": mult, "first_ms": round(ta, 3),
                     "second_ms": round(tb, 3), "ratio_first_over_second": round(ta / tb, 3),
                     "back_to_back_ms": round(t2, 3), "horizontal_ms": round(best[0], 3), "horizontal_variant": best[1],
                     "speedup_horizontal": round(t2 / best[0], 3)})
    print(json.dumps({"study": rows}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--only", default="")
    ap.add_argument("--mode", default="fused", choices=["fused", "b2b", "a", "b", "xchg"])
    ap.add_argument("--count", type=int, default=1 << 24, help="nonces per step with --only cfg3|cfg4")
    ap.add_argument("--dag-items", type=int, default=8_388_608)
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--im2col-path", default="default", choices=["default", "registers", "bulk"],
                    help="store path of the im2col role: the compiled choice per kernel / pair, register tiles + "
                         "streaming stores, or shared-memory tile + bulk (TMA) stores")
    ap.add_argument("--histc-path", default="default", choices=["default", "registers", "bulk"],
                    help="load path of the histogram role: the compiled choice per kernel / pair, 16-byte loads into registers, or bulk (TMA) copies into a shared-memory ring")
    ap.add_argument("--bnstats-path", default="default", choices=["default", "registers", "bulk"],
                    help="load path of the statistics role: the compiled choice per kernel / pair, 16-byte loads into registers, or bulk (TMA) copies into shared memory")
    ap.add_argument("--pair-variant", type=int, default=-1,
                    help="force thread-range variant V of the headline pair (tuning aid; default: the compiled-in choice)")
    ap.add_argument("--tune-share", action="store_true",
                    help="sweep thread splits x upsample shares of the exchange pair at the launched number of ranks")
    ap.add_argument("--share-permille", type=int, default=-1,
                    help="N > 1, fused collective: share of the upsample that the statistics thread range takes over "
                         "while the moments travel (tuning aid; default: the compiled-in choice)")
    ap.add_argument("--collective", default="fused", choices=["fused", "nccl"],
                    help="N > 1: sum the batch-norm moments inside the fused kernel (peer memory) or with NCCL")
    ap.add_argument("--no-graph", action="store_true", help="time direct launches instead of CUDA-graph replays")
    ap.add_argument("--region-ms", type=float, default=1000.0,
                    help="length of the timed region: the K-step pass is repeated until it lasts about this long (at least 50 passes)")
    ap.add_argument("--tune", action="store_true", help="sweep all variants and print the best per kernel / pair")
    ap.add_argument("--tune-skip-crypto", action="store_true", help="with --tune: sweep the DL kernels and pairs only")
    ap.add_argument("--quick", action="store_true", help="with --study: two pairs and three ratios only")
    ap.add_argument("--study", action="store_true", help="speedup vs ratio of the standalone times, as JSON")
    ap.add_argument("--graph", action="store_true", help="with --only: replay the launches from a CUDA graph")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
