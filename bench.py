#!/usr/bin/env python3
"""Benchmark of the NVFP4 low-bit linear hot path on B200.

One "step" is one pass of the path over a Qwen3-8B-shaped decoder layer's
linears at M = 4096 tokens (synthetic data, random weights of that shape):

    producer(residual, hidden) -> QKV GEMM 4096->6144      O GEMM 4096->4096 (NVFP4 input resident)
    producer(residual, hidden) -> gate/up GEMM 4096->24576 down GEMM 12288->4096 (NVFP4 input resident)

`value` is GEMM TFLOP/s of the whole step (2*M*N*K summed over the four GEMMs,
divided by the step time including the two producer launches), inputs resident
in HBM.  `e2e` is the same metric through the torch operator API with the
step's bf16 inputs in pinned host memory and the step's result read back to
the host inside the timed region.

N > 1 (torchrun, one rank per GPU): the fixed M-token problem with the NVFP4
weights column-sharded over the ranks, activations replicated, outputs left
sharded (strong scaling; `--sharding columns`, the default).  The producer
runs on each rank's row shard and stores its NVFP4 rows into every rank's
activation buffer from inside the kernel (NVSwitch multicast stores over
symmetric memory), timed inside the step; the NCCL all-gather of the largest
output is timed separately.  The same line carries the step with every rank
running the whole producer (`replicated_producer`), with an NCCL all-gather
of the NVFP4 rows (`row_sharded_producer_nccl`), the Llama-3-70B FFN in the
same split (`c5_column_sharded`) and the token-sharded replicas
(`token_sharded`: every rank runs the whole step on its own tokens).

At N = 1 `detail` also holds: every GEMM timed back to back over rotating
buffers, a >= 2 s sustained run, the reference's own CUDA kernels on the same
buffers (`reference_cuda`, when oracle/_ref was built), the decode sweep on
rotating weight sets (`c3`), the grouped MoE GEMMs (`c4`) and the Llama-3-70B
FFN (`c5`).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c5|c4|model]
                    [--sharding columns|tokens] [--tokens M --graph] [--quick]
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "flashrt-hf-kernels_b200" / "torch-ext"))

import numpy as np  # noqa: E402
import torch  # noqa: E402

L2_BYTES = 126 << 20
EPS = 1e-6
# ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch, captured on the unsharded Qwen3-8B M=4096
# shapes (kernel -> bytes); reported as `traffic` only for a launch of exactly that shape
NCU_DRAM_TRAFFIC_BYTES = {("gemm", 4096, 6144, 4096): 29563904, ("gemm", 4096, 4096, 4096): 19248896,
                          ("gemm", 4096, 24576, 4096): 221514496, ("gemm", 4096, 4096, 12288): 70588160,
                          ("producer", 4096, 4096): 69002240}

WORKLOADS = {
    # name: (tokens, hidden, [(layer, N, K, fed_by_producer)])
    "c2": ("qwen3-8b-prefill-m4096", 4096, 4096,
           [("qkv", 6144, 4096, True), ("o", 4096, 4096, False), ("gate_up", 24576, 4096, True),
            ("down", 4096, 12288, False)]),
    "c5": ("llama3-70b-ffn-m8192", 8192, 8192,
           [("gate_up", 57344, 8192, True), ("down", 8192, 28672, False)]),
}
# Qwen3-30B-A3B-shaped grouped MoE (--workload c4): 128 experts, top-8, 4096 tokens
MOE = dict(name="qwen3-30b-a3b-moe-4096tok", experts=128, top_k=8, tokens=4096,
           layers=[("gate_up", 1536, 2048), ("down", 2048, 768)])


def measured_peaks():
    """Roofline denominators.  MEASURED_PEAKS.json holds a copy bandwidth and a cuBLAS bf16 rate (burst and
    sustained); it has no FP4 figure, so the FP4 tensor peak is ASSUMED to be 4 x the measured bf16 rate."""
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm_gbs=d["hbm_gbs"], fp4_burst=4.0 * d["bf16_tflops"], fp4_sustained=4.0 * d["bf16_tflops_sustained"],
                    source="of measured (MEASURED_PEAKS.json); FP4 peak assumed 4 x measured bf16")
    return dict(hbm_gbs=6650.0, fp4_burst=4.0 * 1590.0, fp4_sustained=4.0 * 1400.0,
                source="of fallback (6.65 TB/s, 1.59 PFLOP/s bf16); FP4 peak assumed 4 x bf16")


class ClockSampler:
    """Samples SM clock, power and throttle reasons through NVML (read-only) while a timed region runs."""

    def __init__(self, index: int, period=0.005):
        self.samples, self.power, self.reasons, self.max_mhz = [], [], set(), None
        self.period = period
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40,
                 "hw_power_brake": 0x80}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                self.power.append(nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0)
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["nvml unavailable"]}
        out = {"sm_mhz": int(statistics.median(self.samples)), "sm_max_mhz": self.max_mhz,
               "reasons": sorted(self.reasons), "samples": len(self.samples)}
        if self.power:
            out["power_w_max"] = round(max(self.power), 1)
        return out


def event_ms(fn, iters, warm=3, best_of=1):
    """mean milliseconds of fn() over `iters` back-to-back calls (CUDA events on the current stream); with
    best_of > 1 the region is timed that many times and the fastest is returned (the burst figure: the same
    convention as the measured bf16 / copy peaks the fractions are taken against)"""
    for _ in range(warm):
        fn()
    best = None
    for _ in range(best_of):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
        best = ms if best is None else min(best, ms)
    return best


def rotating_sets(bytes_per_call):
    """how many distinct buffer sets make one round of calls touch more than 4 x L2"""
    return max(1, min(8, math.ceil(4 * L2_BYTES / max(bytes_per_call, 1))))


# ----------------------------------------------------------------------------
# our arm
# ----------------------------------------------------------------------------
class Layer:
    """Device-resident tensors of one rank's shard of the workload."""

    def __init__(self, key, rank, world, dev, seed=1234, tokens=0, act_seed=None):
        """`world` column shards of the weights (1 = whole weights); `act_seed` draws this rank's own
        activations (token-sharded runs), the weights always come from `seed`."""
        import fp4_gemm
        from flashrt_b200_core import alloc_fp4
        self.name, self.M, self.H, layers = WORKLOADS[key]
        if tokens:
            self.name, self.M = f"{self.name.rsplit('-m', 1)[0]}-m{tokens}", tokens
        self.rank, self.world = rank, world
        g = torch.Generator(device=dev).manual_seed(seed)
        ga = torch.Generator(device=dev).manual_seed(seed + 1 if act_seed is None else act_seed)
        rn = lambda *s, scale=1.0: (torch.randn(*s, generator=g, device=dev) * scale).to(torch.bfloat16)
        rna = lambda *s: torch.randn(*s, generator=ga, device=dev).to(torch.bfloat16)
        self.hidden, self.residual0 = rna(self.M, self.H), rna(self.M, self.H)
        self.residual = self.residual0.clone()
        self.norm_w = (1.0 + 0.1 * torch.randn(self.H, generator=g, device=dev)).to(torch.bfloat16)
        self.act_packed, self.act_sf = alloc_fp4(self.M, self.H, dev)
        self.gemms = []
        self.flops_total = 0.0
        for lname, n, k, fed in layers:
            assert n % (world * 128) == 0, "column shard must keep whole 128-row scale groups"
            n_loc = n // world
            w = rn(n_loc, k, scale=0.02)
            wp, wsf = fp4_gemm.quantize_fp4_sfa_bf16(w, is_sfb=True)
            del w
            if fed:
                a_p, a_sf = self.act_packed, self.act_sf
            else:
                a_p, a_sf = fp4_gemm.quantize_fp4_sfa_bf16(rna(self.M, k))
            out = torch.empty(self.M, n_loc, device=dev, dtype=torch.bfloat16)
            self.gemms.append(dict(name=lname, n=n, n_loc=n_loc, k=k, fed=fed, wp=wp, wsf=wsf, a_p=a_p, a_sf=a_sf,
                                   out=out))
            self.flops_total += 2.0 * self.M * n * k
        self.bytes_streamed = sum(g_["wp"].numel() + g_["wsf"].numel() + g_["out"].numel() * 2 +
                                  g_["a_p"].numel() for g_ in self.gemms) + 2 * 3 * self.M * self.H * 2
        torch.cuda.synchronize()

    # -- the producer, whole or on this rank's row shard ------------------------------------------------
    def row_shard(self, world, rank):
        from flashrt_b200_core import sharding
        r0, r1 = sharding.row_shard_bounds(self.M, world, rank)
        per_group = ((self.H // 16 + 3) // 4) * 512
        return r0, r1, (r0 // 128) * per_group, ((r1 + 127) // 128) * per_group

    def producer_capi(self, capi, st, rows=None):
        L, P = capi.lib(), capi.ptr
        if rows is None:
            return L.frt_norm_quant_nvfp4(P(self.residual), P(self.hidden), P(self.norm_w), EPS, 1.0, None,
                                          P(self.act_packed), P(self.act_sf), self.M, self.H, 0, st)
        r0, r1, s0, s1 = rows
        return L.frt_norm_quant_nvfp4(P(self.residual[r0:r1]), P(self.hidden[r0:r1]), P(self.norm_w), EPS, 1.0, None,
                                      P(self.act_packed[r0:r1]), P(self.act_sf[s0:s1]), r1 - r0, self.H, 0, st)

    def gather_activations(self, dist, rows):
        """all-gather of the NVFP4 rows every rank produced for its row shard (in place: this rank's slice is
        already where the collective would put it)"""
        r0, r1, s0, s1 = rows
        dist.all_gather_into_tensor(self.act_packed, self.act_packed[r0:r1])
        dist.all_gather_into_tensor(self.act_sf, self.act_sf[s0:s1])

    def step_capi(self, capi, st, ev=None, dist=None, rows=None, shared=None):
        """one pass through the C ABI (resident inputs); optional (start,end) events per kernel.  With `rows` the
        producer runs on this rank's row shard and NCCL all-gathers the NVFP4 rows; with `shared` (a
        SharedActivations) the row-shard producer stores its rows into every rank's buffer from inside the kernel
        and a bounded wait kernel precedes the GEMM."""
        L = capi.lib()
        P = capi.ptr
        launches = 0
        n_fed = 0
        for i, g_ in enumerate(self.gemms):
            a_p, a_sf = g_["a_p"], g_["a_sf"]
            if g_["fed"]:
                pe = ev.get(("producer", i)) if ev is not None else None
                if pe:
                    pe[0].record()
                if shared is not None:
                    b = n_fed % shared.buffers
                    n_fed += 1
                    r0, r1 = shared.row0, shared.row0 + shared.rows_local
                    shared.produce(b, self.residual[r0:r1], self.hidden[r0:r1], self.norm_w, EPS, st)   # waits for the peers too
                    a_p, a_sf = shared.packed[b], shared.sf[b]
                    rc = 0
                    launches += 1
                else:
                    rc = self.producer_capi(capi, st, rows)
                    if rows is not None:
                        self.gather_activations(dist, rows)
                if pe:
                    pe[1].record()
                assert rc == 0, rc
                launches += 1
            ge = ev.get((g_["name"], i)) if ev is not None else None
            if ge:
                ge[0].record()
            rc = L.frt_nvfp4_gemm_bf16(P(a_p), P(a_sf), P(g_["wp"]), P(g_["wsf"]), None, None,
                                       P(g_["out"]), self.M, g_["n_loc"], g_["k"], 1.0, 0.0, st)
            if ge:
                ge[1].record()
            assert rc == 0, rc
            launches += 1
        return launches

    def step_ops(self, hidden, residual, dist=None, rows=None, shared=None):
        """one pass through the torch operator API; returns the last GEMM's output.  With `rows`, hidden and
        residual are this rank's row shard and the NVFP4 rows are exchanged: by the producer kernel itself when
        `shared` (a SharedActivations) is given, else by an NCCL all-gather."""
        import fp4_fused_ops
        import fp4_gemm
        from flashrt_b200_core import capi
        out = None
        n_fed = 0
        for g_ in self.gemms:
            if g_["fed"] and shared is not None:
                b = n_fed % shared.buffers
                n_fed += 1
                st = capi.stream_ptr()
                shared.produce(b, residual, hidden, self.norm_w, EPS, st)
                out = fp4_gemm.nvfp4_gemm_bf16(shared.packed[b], g_["wp"], shared.sf[b], g_["wsf"], out=g_["out"])
                continue
            if g_["fed"]:
                if rows is None:
                    fp4_fused_ops.residual_add_rms_norm_quant_nvfp4_swizzled_bf16(
                        residual, hidden, self.norm_w, EPS, packed=self.act_packed, sfa=self.act_sf)
                else:
                    r0, r1, s0, s1 = rows
                    fp4_fused_ops.residual_add_rms_norm_quant_nvfp4_swizzled_bf16(
                        residual, hidden, self.norm_w, EPS, packed=self.act_packed[r0:r1], sfa=self.act_sf[s0:s1])
                    self.gather_activations(dist, rows)
            out = fp4_gemm.nvfp4_gemm_bf16(g_["a_p"], g_["wp"], g_["a_sf"], g_["wsf"], out=g_["out"])
        return out


def gemm_back_to_back(layer, capi, st, peaks, iters=12):
    """Every GEMM of the layer alone, back to back over enough distinct buffer sets that one round of calls
    touches more than 4 x L2: no event inside the timed region, so no event cost in the number."""
    L, P = capi.lib(), capi.ptr
    out = {}
    for g_ in layer.gemms:
        torch.cuda.synchronize()
        time.sleep(0.5)            # each kernel is timed alone, from an idle GPU (the burst peaks are measured that way)
        per_call = g_["wp"].numel() + g_["wsf"].numel() + g_["a_p"].numel() + g_["a_sf"].numel() + g_["out"].numel() * 2
        sets = [g_] + [dict(g_, wp=g_["wp"].clone(), wsf=g_["wsf"].clone(), a_p=g_["a_p"].clone(),
                            a_sf=g_["a_sf"].clone(), out=torch.empty_like(g_["out"]))
                       for _ in range(rotating_sets(per_call) - 1)]

        def calls():
            for s_ in sets:
                L.frt_nvfp4_gemm_bf16(P(s_["a_p"]), P(s_["a_sf"]), P(s_["wp"]), P(s_["wsf"]), None, None, P(s_["out"]),
                                      layer.M, s_["n_loc"], s_["k"], 1.0, 0.0, st)
        ms = event_ms(calls, max(2, iters // len(sets)), best_of=3) / len(sets)
        tf = 2.0 * layer.M * g_["n_loc"] * g_["k"] / (ms * 1e-3) / 1e12
        out[g_["name"]] = {"shape": [layer.M, g_["n_loc"], g_["k"]], "us": round(ms * 1e3, 2), "tflops": round(tf, 1),
                           "frac_of_fp4_peak": round(tf / peaks["fp4_burst"], 4), "buffer_sets": len(sets),
                           "timing": "best of 3 regions"}
        del sets
    return out


def producer_back_to_back(layer, capi, st, peaks):
    """the fused producer alone, back to back over four input sets (larger than L2 together)"""
    from flashrt_b200_core import alloc_fp4
    L, P = capi.lib(), capi.ptr
    dev = layer.hidden.device
    psets = []
    for _ in range(4):
        pk, sfp_ = alloc_fp4(layer.M, layer.H, dev)
        psets.append((layer.hidden.clone(), layer.residual0.clone(), pk, sfp_))

    def producers():
        for hx, rx, pk, sfp_ in psets:
            L.frt_norm_quant_nvfp4(P(rx), P(hx), P(layer.norm_w), EPS, 1.0, None, P(pk), P(sfp_), layer.M, layer.H, 0, st)
    p_us = event_ms(producers, 10, best_of=3) / 4 * 1e3
    prod_bytes = layer.M * layer.H * 6.5625
    return psets, {"us": round(p_us, 2), "gbs": round(prod_bytes / p_us / 1e3, 1),
                   "frac_of_hbm_measured": round(prod_bytes / p_us / 1e3 / peaks["hbm_gbs"], 3),
                   "what": "fused residual+RMSNorm->NVFP4 on 4 rotating input sets, 40 launches, best of 3 regions"}


def reference_cuda_leg(layer, psets, capi, st, peaks):
    """The reference's own CUDA kernels, compiled unmodified into oracle/_ref (test infrastructure; this leg and
    the CPU baseline are the only places the benchmark touches it), on the same shapes and rotating buffers:
    its CUTLASS Sm100 NVFP4 GEMM with the default and the wide-N tile, its fused producer and its quantiser."""
    path = ROOT / "oracle" / "_ref" / "libflashrt_ref.so"
    if not path.exists():
        return {"unavailable": "oracle/_ref/libflashrt_ref.so was not built (no reference checkout at build time)"}
    ref = ctypes.CDLL(str(path))
    P = capi.ptr
    res = {}
    if ref.ref_has_cutlass():
        for g_ in layer.gemms:
            per_call = g_["wp"].numel() + g_["a_p"].numel() + g_["out"].numel() * 2
            sets = [g_] + [dict(g_, wp=g_["wp"].clone(), wsf=g_["wsf"].clone(), a_p=g_["a_p"].clone(),
                                a_sf=g_["a_sf"].clone(), out=torch.empty_like(g_["out"]))
                           for _ in range(rotating_sets(per_call) - 1)]
            row = {}
            for label, variant in (("default_tile_128x128x256", 0), ("widen_tile_128x256x128", 1)):
                torch.cuda.synchronize()
                time.sleep(0.5)    # same idle start as the per-GEMM leg of this library
                def calls():
                    for s_ in sets:
                        ref.ref_gemm_sm100_bf16(P(s_["a_p"]), P(s_["wp"]), P(s_["out"]), layer.M, s_["n_loc"], s_["k"],
                                                P(s_["a_sf"]), P(s_["wsf"]), ctypes.c_float(1.0), variant, st)
                ms = event_ms(calls, max(2, 12 // len(sets)), best_of=3) / len(sets)
                row[label] = round(2.0 * layer.M * g_["n_loc"] * g_["k"] / (ms * 1e-3) / 1e12, 1)
            row["best_tflops"] = max(row.values())
            row["reference_selects"] = "widen" if g_["n_loc"] >= 4 * g_["k"] else "default"
            res[g_["name"]] = row
            del sets
        hx, rx, pk, sfp_ = psets[0]

        def k10():
            for hx, rx, pk, sfp_ in psets:
                ref.ref_res_rms_fp4_bf16(P(rx), P(hx), P(layer.norm_w), P(pk), P(sfp_), layer.M, layer.H,
                                         ctypes.c_float(EPS), st)
        us = event_ms(k10, 10, best_of=3) / 4 * 1e3
        res["fused_producer"] = {"us": round(us, 2), "gbs": round(layer.M * layer.H * 6.5625 / us / 1e3, 1)}
    else:
        res["gemm"] = {"unavailable": "oracle/_ref was built without a CUTLASS header tree"}

    def k4():
        for hx, rx, pk, sfp_ in psets:
            ref.ref_quantize_bf16_vec(P(hx), P(pk), P(sfp_), layer.M, layer.H, st)
    us = event_ms(k4, 10, best_of=3) / 4 * 1e3
    res["quantizer"] = {"us": round(us, 2), "gbs": round(layer.M * layer.H * 2.5625 / us / 1e3, 1)}
    res["what"] = ("the reference's kernels compiled for sm_100a from its own sources (cluster 1x1x1 CUTLASS Sm100 GEMM, "
                   "fused residual+RMSNorm->NVFP4, vectorised quantiser), same shapes, same rotating buffers, CUDA events, best of 3 regions")
    return res


def sustained_leg(layer, capi, st, local_rank, ms_step, peaks, seconds=2.0):
    """the same step looped for >= `seconds`: clocks settle under the power cap, so this is the sustained figure"""
    n = max(10, int(seconds * 1e3 / ms_step) + 1)
    with ClockSampler(local_rank, period=0.02) as clocks:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(n):
            layer.step_capi(capi, st)
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / n
    c = clocks.summary()
    tf = layer.flops_total / (ms * 1e-3) / 1e12
    return {"steps": n, "seconds": round(ms * n / 1e3, 2), "ms_per_step": round(ms, 5), "tflops": round(tf, 1),
            "frac_of_fp4_sustained_peak": round(tf / peaks["fp4_sustained"], 4), "clocks": c,
            "ms_x_median_sm_mhz": round(ms * c["sm_mhz"], 2) if c.get("sm_mhz") else None}


def decode_leg(capi, dev, peaks, tokens=(1, 4, 16, 64), graph_replays=20):
    """Decode sweep on the Qwen3-8B linears: four distinct weight sets (434 MB, 3.4 x L2) visited in turn, so
    every weight byte comes from HBM; one CUDA graph holds the four steps; the weight stream is
    0.5625 * N * K bytes per GEMM."""
    import fp4_gemm
    from flashrt_b200_core import alloc_fp4
    L, P = capi.lib(), capi.ptr
    name, _, H, layers = WORKLOADS["c2"]
    g = torch.Generator(device=dev).manual_seed(77)
    wsets = []
    for _ in range(4):
        ws = []
        for lname, n, k, fed in layers:
            w = (torch.randn(n, k, generator=g, device=dev) * 0.02).to(torch.bfloat16)
            ws.append(fp4_gemm.quantize_fp4_sfa_bf16(w, is_sfb=True))
            del w
        wsets.append(ws)
    wbytes = sum(0.5625 * n * k for _, n, k, _ in layers)
    norm_w = torch.ones(H, device=dev, dtype=torch.bfloat16)
    out = {}
    for M in tokens:
        hidden = torch.randn(M, H, generator=g, device=dev).to(torch.bfloat16)
        residual = torch.randn(M, H, generator=g, device=dev).to(torch.bfloat16)
        act_p, act_sf = alloc_fp4(M, H, dev)
        res_in = [None if fed else fp4_gemm.quantize_fp4_sfa_bf16(torch.randn(M, k, generator=g, device=dev).to(torch.bfloat16))
                  for _, n, k, fed in layers]
        outs = [torch.empty(M, n, device=dev, dtype=torch.bfloat16) for _, n, k, _ in layers]
        torch.cuda.synchronize()

        def steps(st):
            n_l = 0
            for ws in wsets:
                for i, (lname, n, k, fed) in enumerate(layers):
                    if fed:
                        assert L.frt_norm_quant_nvfp4(P(residual), P(hidden), P(norm_w), EPS, 1.0, None, P(act_p), P(act_sf),
                                                      M, H, 0, st) == 0
                        n_l += 1
                    a_p, a_sf = (act_p, act_sf) if fed else res_in[i]
                    assert L.frt_nvfp4_gemm_bf16(P(a_p), P(a_sf), P(ws[i][0]), P(ws[i][1]), None, None, P(outs[i]),
                                                 M, n, k, 1.0, 0.0, st) == 0
                    n_l += 1
            return n_l
        steps(capi.stream_ptr())
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                steps(capi.stream_ptr())
        torch.cuda.synchronize()
        ms = event_ms(graph.replay, graph_replays) / len(wsets)
        gbs = wbytes / (ms * 1e-3) / 1e9
        out[f"m{M}"] = {"us_per_step": round(ms * 1e3, 2), "weight_stream_gbs": round(gbs, 1),
                        "frac_of_hbm_measured": round(gbs / peaks["hbm_gbs"], 3)}
        del graph
        # every GEMM of the step alone: the same launch over the four weight sets, four times, in one graph
        per = {}
        for i, (lname, n, k, fed) in enumerate(layers):
            a_p, a_sf = (act_p, act_sf) if fed else res_in[i]

            def calls(st):
                for _ in range(4):
                    for ws in wsets:
                        assert L.frt_nvfp4_gemm_bf16(P(a_p), P(a_sf), P(ws[i][0]), P(ws[i][1]), None, None, P(outs[i]),
                                                     M, n, k, 1.0, 0.0, st) == 0
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                g1 = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g1, stream=side):
                    calls(capi.stream_ptr())
            torch.cuda.synchronize()
            us = event_ms(g1.replay, 10) / 16 * 1e3
            per[lname] = {"us": round(us, 2), "gbs": round(0.5625 * n * k / us / 1e3, 1),
                          "frac_of_hbm_measured": round(0.5625 * n * k / us / 1e3 / peaks["hbm_gbs"], 3)}
            del g1
        out[f"m{M}"]["per_gemm_back_to_back"] = per
    out["what"] = (f"{name.rsplit('-m', 1)[0]} linears + 2 fused producers per step, 4 rotating weight sets "
                   f"({4 * wbytes / 1e6:.0f} MB), one CUDA graph of 4 steps replayed {graph_replays} times; "
                   f"{wbytes / 1e6:.1f} MB of weights per step")
    out["roofline"] = {"bound": "hbm", "kernel": "decode step (4 nvfp4_gemm_kernel + 2 norm_quant_kernel launches)",
                       "achieved": out["m1"]["weight_stream_gbs"] if "m1" in out else None, "peak": peaks["hbm_gbs"],
                       "unit": "GB/s", "frac": out["m1"]["frac_of_hbm_measured"] if "m1" in out else None}
    return out


def moe_setup(capi, dev):
    """routing of the synthetic workload: top-8 of seeded N(0,1) logits (= top-8 of their softmax), sorted by
    expert into per-expert offsets, with this library's router and routing-plan kernels"""
    L, P, st = capi.lib(), capi.ptr, capi.stream_ptr()
    experts = MOE["experts"]
    g0 = torch.Generator(device=dev).manual_seed(3)
    setup_logits = torch.randn(MOE["tokens"], experts, generator=g0, device=dev).to(torch.bfloat16)
    s_idx = torch.empty(MOE["tokens"], MOE["top_k"], dtype=torch.int32, device=dev)
    s_val = torch.empty(MOE["tokens"], MOE["top_k"], dtype=torch.float32, device=dev)
    offs_d = torch.empty(experts + 1, dtype=torch.int32, device=dev)
    s_rop = torch.empty(MOE["tokens"], MOE["top_k"], dtype=torch.int32, device=dev)
    s_tor = torch.empty(MOE["tokens"] * MOE["top_k"], dtype=torch.int32, device=dev)
    assert L.frt_router_topk_bf16(P(setup_logits), P(s_idx), P(s_val), MOE["tokens"], experts, MOE["top_k"], st) == 0
    assert L.frt_moe_route_plan(P(s_idx), MOE["tokens"], MOE["top_k"], experts, P(offs_d), P(s_rop), P(s_tor), st) == 0
    torch.cuda.synchronize()
    rows = int(offs_d[-1].item())
    alpha = torch.ones(experts, device=dev)
    work = torch.empty(int(L.frt_nvfp4_grouped_gemm_workspace_bytes(rows, experts)), dtype=torch.uint8, device=dev)
    sfb = lambda r, k: int(L.frt_nvfp4_sf_swizzled_bytes(r, k))
    layers, flops = [], 0.0
    for name, n, k in MOE["layers"]:
        ap = torch.randint(0, 256, (rows, k // 2), dtype=torch.uint8, device=dev)
        wp = torch.randint(0, 256, (experts, n, k // 2), dtype=torch.uint8, device=dev)
        asf = torch.randint(32, 80, (sfb(rows, k),), dtype=torch.uint8, device=dev)
        wsf = torch.randint(32, 80, (experts, sfb(n, k)), dtype=torch.uint8, device=dev)
        out = torch.empty(rows, n, dtype=torch.bfloat16, device=dev)
        layers.append((name, n, k, ap, wp, asf, wsf, out))
        flops += 2.0 * rows * n * k
    return dict(rows=rows, experts=experts, offs=offs_d, alpha=alpha, work=work, layers=layers, flops=flops, sfb=sfb)


def moe_measure(capi, dev, peaks, steps, warmup):
    L, P, st = capi.lib(), capi.ptr, capi.stream_ptr()
    S = moe_setup(capi, dev)
    rows, experts, layers = S["rows"], S["experts"], S["layers"]

    def one(layer_):
        name, n, k, ap, wp, asf, wsf, out = layer_
        rc = L.frt_nvfp4_grouped_gemm_bf16(P(ap), P(asf), P(wp), P(wsf), P(S["alpha"]), P(S["offs"]), None, 0, P(out), rows,
                                           n, k, experts, n * (k // 2), int(wsf.shape[1]), P(S["work"]), st)
        assert rc == 0, rc

    def step():
        for l_ in layers:
            one(l_)
    l0 = L.frt_launch_count()
    ms = event_ms(step, steps, warm=warmup)
    launches = int(L.frt_launch_count() - l0)
    per_layer = {}
    total_bytes = 0.0
    for l_ in layers:
        lms = event_ms(lambda: one(l_), max(5, steps // 2))
        fl = 2.0 * rows * l_[1] * l_[2]
        # algorithmic bytes: every expert's weights once, the routed activations once, the bf16 output once
        by = experts * l_[1] * l_[2] * 0.5625 + rows * l_[2] * 0.5625 + rows * l_[1] * 2.0
        total_bytes += by
        per_layer[l_[0]] = {"us": round(lms * 1e3, 1), "tflops": round(fl / (lms * 1e-3) / 1e12, 1),
                            "frac_of_fp4_peak": round(fl / (lms * 1e-3) / 1e12 / peaks["fp4_burst"], 4),
                            "algorithmic_mb": round(by / 1e6, 1), "flop_per_byte": round(fl / by, 1),
                            "gbs": round(by / (lms * 1e-3) / 1e9, 1),
                            "frac_of_hbm_measured": round(by / (lms * 1e-3) / 1e9 / peaks["hbm_gbs"], 3)}

    # ---- the whole routed layer through the C ABI: router -> plan -> quantise -> gather ->
    # grouped gate/up -> SwiGLU -> NVFP4 -> grouped down -> weighted un-permute
    T, E, topk = MOE["tokens"], experts, MOE["top_k"]
    (_, n1, k1, _, wp1, _, wsf1, out1), (_, n2, k2, _, wp2, _, wsf2, out2) = layers
    sfb = S["sfb"]
    g = torch.Generator(device=dev).manual_seed(11)
    hidden = torch.randn(T, k1, generator=g, device=dev).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g, device=dev).to(torch.bfloat16)
    idx = torch.empty(T, topk, dtype=torch.int32, device=dev)
    val = torch.empty(T, topk, dtype=torch.float32, device=dev)
    off = torch.empty(E + 1, dtype=torch.int32, device=dev)
    rop = torch.empty(T, topk, dtype=torch.int32, device=dev)
    tor = torch.empty(T * topk, dtype=torch.int32, device=dev)
    gp = torch.empty(T * topk, k1 // 2, dtype=torch.uint8, device=dev)
    gs = torch.zeros(sfb(T * topk, k1), dtype=torch.uint8, device=dev)
    hp = torch.empty(T * topk, k2 // 2, dtype=torch.uint8, device=dev)
    hs = torch.zeros(sfb(T * topk, k2), dtype=torch.uint8, device=dev)
    final = torch.empty(T, n2, dtype=torch.float32, device=dev)
    weights = torch.empty(T, topk, dtype=torch.float32, device=dev)
    R = T * topk
    alpha, work = S["alpha"], S["work"]

    def routed_layer():
        rcs = [L.frt_router_topk_softmax_bf16(P(logits), P(idx), P(val), P(weights), T, E, topk, st),
               L.frt_moe_route_plan(P(idx), T, topk, E, P(off), P(rop), P(tor), st),
               L.frt_moe_quantize_scatter_nvfp4(P(hidden), P(rop), P(gp), P(gs), T, topk, k1, st),
               L.frt_nvfp4_grouped_gemm_bf16(P(gp), P(gs), P(wp1), P(wsf1), P(alpha), P(off), None, 0, P(out1), R, n1,
                                             k1, E, n1 * (k1 // 2), int(wsf1.shape[1]), P(work), st),
               L.frt_silu_mul_quant_nvfp4(P(out1), P(hp), P(hs), R, n1 // 2, st),
               L.frt_nvfp4_grouped_gemm_bf16(P(hp), P(hs), P(wp2), P(wsf2), P(alpha), P(off), None, 0, P(out2), R, n2,
                                             k2, E, n2 * (k2 // 2), int(wsf2.shape[1]), P(work), st),
               L.frt_moe_weighted_sum_bf16(P(out2), P(rop), P(weights), P(final), T, topk, n2, n2, st)]
        assert not any(rcs), rcs

    routed_us = None
    if n1 // 2 == k2 and rows == R:
        routed_us = round(event_ms(routed_layer, max(5, min(50, steps))) * 1e3, 1)
    tf = S["flops"] / (ms * 1e-3) / 1e12
    return {"tflops": round(tf, 2), "ms_per_step": round(ms, 5), "routed_rows": rows, "experts": experts,
            "layers": per_layer, "routed_layer_us": routed_us, "gpu_launches": launches,
            "decode": moe_decode_leg(capi, dev, peaks, S),
            # 309 GFLOP over 620 MB of algorithmic traffic = 500 flop/byte, below the ridge of this GPU
            # (4 x measured bf16 / measured copy bandwidth = 1012 flop/byte): the bound is HBM
            "roofline": {"bound": "hbm", "kernel": "nvfp4_gemm_pair_kernel<grouped> (gate/up + down)",
                         "achieved": round(total_bytes / (ms * 1e-3) / 1e9, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": round(total_bytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4),
                         "algorithmic_bytes": int(total_bytes),
                         "peak_note": "of measured (MEASURED_PEAKS.json copy bandwidth); expert weights + routed activations "
                                      "+ bf16 outputs, each once",
                         "tensor_side": {"achieved": round(tf, 1), "peak": round(peaks["fp4_burst"], 1), "unit": "TFLOP/s",
                                         "frac": round(tf / peaks["fp4_burst"], 4)}},
            "what": "router top-k + softmax, routing plan, quantise into expert order, grouped gate/up, SwiGLU->NVFP4, "
                    "grouped down, weighted un-permute = routed_layer_us (11 launches of this library)"}


def moe_decode_leg(capi, dev, peaks, S, tokens=(1, 4, 16)):
    """The two grouped GEMMs at decode sizes: T tokens -> 8 T routed rows, a few rows per expert, so the job is a
    stream of the chosen experts' weights (the reference's decode-side counterpart is grouped-moe-gemv).  Several
    routings (different seeds) run in turn inside one CUDA graph so that the experts they touch exceed L2."""
    L, P = capi.lib(), capi.ptr
    experts, top_k = S["experts"], MOE["top_k"]
    out = {}
    for T in tokens:
        n_routes = max(4, 16 // T)
        rows = T * top_k
        routes = []
        for r in range(n_routes):
            g0 = torch.Generator(device=dev).manual_seed(100 + 17 * r + T)
            logits = torch.randn(T, experts, generator=g0, device=dev).to(torch.bfloat16)
            idx = torch.empty(T, top_k, dtype=torch.int32, device=dev)
            val = torch.empty(T, top_k, dtype=torch.float32, device=dev)
            offs = torch.empty(experts + 1, dtype=torch.int32, device=dev)
            rop = torch.empty(T, top_k, dtype=torch.int32, device=dev)
            tor = torch.empty(rows, dtype=torch.int32, device=dev)
            st = capi.stream_ptr()
            assert L.frt_router_topk_bf16(P(logits), P(idx), P(val), T, experts, top_k, st) == 0
            assert L.frt_moe_route_plan(P(idx), T, top_k, experts, P(offs), P(rop), P(tor), st) == 0
            routes.append(offs)
        torch.cuda.synchronize()
        touched = sum(int((o[1:] > o[:-1]).sum().item()) for o in routes) / n_routes     # experts with rows, per step
        work = torch.empty(int(L.frt_nvfp4_grouped_gemm_workspace_bytes(rows, experts)), dtype=torch.uint8, device=dev)
        bufs = []
        for name, n, k, _ap, wp, _asf, wsf, _out in S["layers"]:
            ap = torch.randint(0, 256, (rows, k // 2), dtype=torch.uint8, device=dev)
            asf = torch.randint(32, 80, (S["sfb"](rows, k),), dtype=torch.uint8, device=dev)
            bufs.append((n, k, ap, asf, wp, wsf, torch.empty(rows, n, dtype=torch.bfloat16, device=dev)))

        def steps(st):
            for offs in routes:
                for n, k, ap, asf, wp, wsf, o in bufs:
                    assert L.frt_nvfp4_grouped_gemm_bf16(P(ap), P(asf), P(wp), P(wsf), P(S["alpha"]), P(offs), None, 0, P(o), rows,
                                                         n, k, experts, n * (k // 2), int(wsf.shape[1]), P(work), st) == 0
        steps(capi.stream_ptr())
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                steps(capi.stream_ptr())
        torch.cuda.synchronize()
        us = event_ms(graph.replay, 20) / n_routes * 1e3
        wbytes = touched * sum(0.5625 * n * k for n, k, *_ in bufs)
        out[f"t{T}"] = {"routed_rows": rows, "experts_touched": round(touched, 1), "us_per_step": round(us, 2),
                        "weight_mb": round(wbytes / 1e6, 1), "weight_stream_gbs": round(wbytes / us / 1e3, 1),
                        "frac_of_hbm_measured": round(wbytes / us / 1e3 / peaks["hbm_gbs"], 3)}
        del graph
    out["what"] = ("grouped gate/up + down (plan + GEMM launches) for T tokens x top-8, several routings per CUDA graph so "
                   "that the touched experts' weights come from HBM; bytes = weights of the experts that have rows")
    return out


def run_ours(args, rank, world, local_rank):
    import torch.distributed as dist
    from flashrt_b200_core import capi, load
    load()
    if args.no_pdl:
        capi.lib().frt_set_option(4, 0)
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    peaks = measured_peaks()
    # N > 1: the fixed problem with column-sharded weights and replicated activations (strong scaling) unless
    # --sharding tokens: every rank runs the whole step on its OWN tokens (weights replicated, no collective).
    tokens_mode = world > 1 and args.sharding == "tokens"
    col_world = 1 if tokens_mode else world
    layer = Layer(args.workload, rank, col_world, dev, tokens=args.tokens,
                  act_seed=7000 + rank if tokens_mode else None)
    job_flops = layer.flops_total * (world if tokens_mode else 1)
    st = capi.stream_ptr()
    L = capi.lib()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        return ms

    def timed_steps(lay, n_steps, **kw):
        """barrier, n steps, barrier; milliseconds per step, max over ranks"""
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(n_steps):
            lay.step_capi(capi, st, **kw)
        t1.record()
        barrier()
        return max_over_ranks(t0.elapsed_time(t1) / n_steps)

    # N > 1, column-sharded: the producer runs on this rank's row shard and stores its NVFP4 rows into every
    # rank's activation buffer from inside the kernel (symmetric memory, NVSwitch multicast stores); where the
    # system has no symmetric memory every rank runs the whole producer instead.
    shared, shared_note = None, None
    if world > 1 and not tokens_mode and layer.M % (128 * world) == 0 and not args.graph and args.exchange != "none":
        try:
            from flashrt_b200_core.sharding import SharedActivations
            shared = SharedActivations(layer.M, layer.H, dev, multicast=args.exchange == "multicast")
        except Exception as e:
            shared_note = "symmetric memory unavailable: " + repr(e)[:160]
    step_kw = {"shared": shared} if shared is not None else {}

    for _ in range(args.warmup):
        layer.step_capi(capi, st, **step_kw)
    barrier()
    if args.graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                n_launch = layer.step_capi(capi, capi.stream_ptr())
        barrier()
        for _ in range(3):
            graph.replay()
        with ClockSampler(local_rank) as clocks:
            barrier()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(args.steps):
                graph.replay()
            t1.record()
            barrier()
        ms = t0.elapsed_time(t1) / args.steps
        wbytes = sum(0.5625 * g_["n_loc"] * g_["k"] for g_ in layer.gemms)
        if rank == 0:
            print(json.dumps({
                "metric": "nvfp4_linear_path_tflops", "value": round(job_flops / (ms * 1e-3) / 1e12, 3),
                "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": round(ms, 5), "higher_is_better": True, "data": "synthetic", "timing": "cuda graph replay",
                "config": {"workload": layer.name, "tokens": layer.M,
                           "l2": "ONE weight set replayed: partly L2-resident; detail.c3 of the default run rotates four"},
                "weight_stream_gbs_whole_step": round(wbytes / (ms * 1e-3) / 1e9, 1),
                "weight_stream_frac_of_hbm_measured": round(wbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 3),
                "gpu_launches": n_launch * args.steps, "clocks": clocks.summary()}), flush=True)
        return
    keys = [("producer", i) for i, g_ in enumerate(layer.gemms) if g_["fed"]] + \
           [(g_["name"], i) for i, g_ in enumerate(layer.gemms)]
    # Inside the timed region only the dominant kernel (the GEMM with the most flops) is bracketed by
    # events: a pair of event records costs a few microseconds of stream time, and twelve of them per
    # step would take ~8 % off `value`.  The per-kernel table comes from a second pass below.
    dom_i = max(range(len(layer.gemms)), key=lambda i: layer.gemms[i]["n_loc"] * layer.gemms[i]["k"])
    dom = (layer.gemms[dom_i]["name"], dom_i)
    events = [{dom: (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))}
              for _ in range(args.steps)]
    launches0 = L.frt_launch_count()
    with ClockSampler(local_rank) as clocks:
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for s in range(args.steps):
            layer.step_capi(capi, st, events[s], **step_kw)
        t1.record()
        barrier()
    ms_total = t0.elapsed_time(t1)
    launches = L.frt_launch_count() - launches0
    ms_step = max_over_ranks(ms_total) / args.steps
    value = job_flops / (ms_step * 1e-3) / 1e12

    dom_ms = statistics.mean(e[dom][0].elapsed_time(e[dom][1]) for e in events)
    # second pass (not part of `value`): every kernel bracketed by events
    n_detail = max(5, min(50, args.steps))
    ev2 = [{k: (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for k in keys}
           for _ in range(n_detail)]
    for s_ in range(n_detail):
        layer.step_capi(capi, st, ev2[s_], **step_kw)
    torch.cuda.synchronize()
    per_kernel = {}
    for k in keys:
        per_kernel[k] = statistics.mean(e[k][0].elapsed_time(e[k][1]) for e in ev2)
    gemm_ms = sum(v for k, v in per_kernel.items() if k[0] != "producer")
    prod_ms = [v for k, v in per_kernel.items() if k[0] == "producer"]
    dom_g = layer.gemms[dom[1]]
    dom_flops = 2.0 * layer.M * dom_g["n_loc"] * dom_g["k"]
    achieved = dom_flops / (dom_ms * 1e-3) / 1e12
    prod_bytes = layer.M * layer.H * 6.5625
    timed_region_s = ms_total * 1e-3
    detail = {
        "gemm_only_tflops": round(job_flops / (gemm_ms * 1e-3) / 1e12, 1),
        "in_step_us_with_event_overhead": {f"{k[0]}": round(v * 1e3, 2) for k, v in per_kernel.items()},
        "producer_in_step_gbs": round(prod_bytes / (statistics.mean(prod_ms) * 1e-3) / 1e9, 1) if prod_ms else None,
        "producer_frac_of_hbm_measured": round(prod_bytes / (statistics.mean(prod_ms) * 1e-3) / 1e9 /
                                               peaks["hbm_gbs"], 3) if prod_ms else None,
    }
    deep = world == 1 and not args.quick
    # ---- every GEMM alone, back to back over rotating buffers; the producer likewise --------------------
    psets = None
    if world == 1:
        detail["per_gemm"] = gemm_back_to_back(layer, capi, st, peaks)
        all_ms = sum(v["us"] for v in detail["per_gemm"].values()) * 1e-3
        detail["four_gemms_frac_of_fp4_peak" if len(layer.gemms) == 4 else "gemms_frac_of_fp4_peak"] = round(
            layer.flops_total / (all_ms * 1e-3) / 1e12 / peaks["fp4_burst"], 4)
    if any(g_["fed"] for g_ in layer.gemms) and world == 1:
        psets, detail["producer_back_to_back"] = producer_back_to_back(layer, capi, st, peaks)

    # ---- end to end through the torch operator API with host buffers ----------
    # N = 1: the step's two bf16 inputs (hidden, residual) sit in ONE pinned buffer and travel as one copy.
    # N > 1, column-sharded: each rank copies only ITS row shard of the inputs, runs the producer on those rows,
    # all-gathers the NVFP4 rows over NVLink (NCCL), runs its column shard of the GEMMs and reads back its
    # shard of the result; summed over ranks the job moves the same input rows once and the whole output once.
    rows = layer.row_shard(world, rank) if (world > 1 and not tokens_mode and layer.M % (128 * world) == 0) else None
    m_loc = layer.M if rows is None else rows[1] - rows[0]
    host_in = torch.empty(2, m_loc, layer.H, dtype=torch.bfloat16).pin_memory()
    sl = slice(None) if rows is None else slice(rows[0], rows[1])
    host_in[0].copy_(layer.hidden[sl].cpu())
    host_in[1].copy_(layer.residual0[sl].cpu())
    last = layer.gemms[-1]["out"]
    host_out = [torch.empty(last.shape, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    dev_in = [torch.empty(2, m_loc, layer.H, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    copy_s, comp_s, out_s = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    h2d = 2 * m_loc * layer.H * 2 * world            # whole job, every rank's copies
    d2h = last.numel() * 2 * world

    def e2e_steps(n):
        in_ready = [torch.cuda.Event(), torch.cuda.Event()]
        in_free = [torch.cuda.Event(), torch.cuda.Event()]
        out_ready, out_free = torch.cuda.Event(), torch.cuda.Event()
        for s in range(n):
            b = s & 1
            with torch.cuda.stream(copy_s):
                if s >= 2:
                    copy_s.wait_event(in_free[b])
                dev_in[b].copy_(host_in, non_blocking=True)
                in_ready[b].record(copy_s)
            with torch.cuda.stream(comp_s):
                comp_s.wait_event(in_ready[b])
                if s >= 1:
                    comp_s.wait_event(out_free)
                out = layer.step_ops(dev_in[b][0], dev_in[b][1], dist=dist, rows=rows, shared=shared)
                in_free[b].record(comp_s)
                out_ready.record(comp_s)
            with torch.cuda.stream(out_s):
                out_s.wait_event(out_ready)
                host_out[b].copy_(out, non_blocking=True)
                out_free.record(out_s)
        for s_ in (copy_s, comp_s, out_s):
            s_.synchronize()

    e2e_n = 0 if args.no_e2e else max(10, args.steps // 4)
    if e2e_n:
        e2e_steps(max(3, args.warmup // 4))
    barrier()
    w0 = time.perf_counter()
    e2e_steps(e2e_n)
    barrier()
    e2e_ms = max_over_ranks((time.perf_counter() - w0) * 1e3 / max(e2e_n, 1))
    e2e_val = job_flops / (e2e_ms * 1e-3) / 1e12

    # ---- all-gather of the sharded outputs, timed separately -------------------
    def time_allgather(lay):
        big = max(lay.gemms, key=lambda g_: g_["out"].numel())
        gathered = torch.empty((world * big["out"].shape[0], big["out"].shape[1]), device=dev, dtype=torch.bfloat16)
        for _ in range(3):
            dist.all_gather_into_tensor(gathered, big["out"])
        barrier()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for _ in range(10):
            dist.all_gather_into_tensor(gathered, big["out"])
        a1.record()
        barrier()
        ag_ms = max_over_ranks(a0.elapsed_time(a1) / 10)
        tot = gathered.numel() * 2
        del gathered
        return {"layer": big["name"], "ms": round(ag_ms, 4), "bytes_total": tot,
                "bus_gbs": round(tot * (world - 1) / world / (ag_ms * 1e-3) / 1e9, 1), "backend": "nccl"}

    def column_run(key, n_steps):
        """the workload `key` column-sharded over the ranks: replicated producer, and row-sharded producer +
        NCCL all-gather of the NVFP4 rows inside the step"""
        col = layer if key == args.workload and not tokens_mode else Layer(key, rank, world, dev)
        for _ in range(max(3, args.warmup // 2)):
            col.step_capi(capi, st)
        ms_rep = timed_steps(col, n_steps)
        res = {"value": round(col.flops_total / (ms_rep * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
               "ms_per_step": round(ms_rep, 5), "scaling": "strong",
               "what": f"{col.name}: fixed {col.M} tokens, weights column-sharded x{world}, activations replicated "
                       "(every rank runs the whole producer), outputs left sharded"}
        if col.M % (128 * world) == 0:
            rws = col.row_shard(world, rank)
            for _ in range(3):
                col.step_capi(capi, st, dist=dist, rows=rws)
            ms_row = timed_steps(col, n_steps, dist=dist, rows=rws)
            res["row_sharded_producer_nccl"] = {
                "value": round(col.flops_total / (ms_row * 1e-3) / 1e12, 2), "ms_per_step": round(ms_row, 5),
                "what": "producer on this rank's rows, NCCL all-gather of packed + scale bytes inside the step"}
            try:
                from flashrt_b200_core.sharding import SharedActivations
                legs = (("row_sharded_producer_peer_stores", False), ("row_sharded_producer_multicast", True))
                for label, mc in (legs if args.exchange_legs else ()):
                    sh = SharedActivations(col.M, col.H, dev, multicast=mc)
                    for _ in range(3):
                        col.step_capi(capi, st, shared=sh)
                    ms_sh = timed_steps(col, n_steps, shared=sh)
                    res[label] = {
                        "value": round(col.flops_total / (ms_sh * 1e-3) / 1e12, 2), "ms_per_step": round(ms_sh, 5),
                        "what": "producer on this rank's rows storing its NVFP4 rows into every rank's buffer from "
                                "inside the kernel (" + ("NVSwitch multicast stores" if sh.uses_multicast else
                                                         "peer stores over NVLink") + "), bounded flag wait before the GEMM"}
                    del sh
            except Exception as e:                          # no symmetric memory on this system
                res["row_sharded_producer_peer_stores"] = {"unavailable": repr(e)[:200]}
        res["allgather_separate"] = time_allgather(col)
        if col is not layer:
            del col
        return res

    allgather = column_sharded = token_sharded = c5_col = row_sharded = replicated = None
    if world > 1 and not tokens_mode:
        allgather = time_allgather(layer)
        if shared is not None:
            for _ in range(3):
                layer.step_capi(capi, st)
            ms_rep = timed_steps(layer, args.steps)
            replicated = {"value": round(layer.flops_total / (ms_rep * 1e-3) / 1e12, 2), "ms_per_step": round(ms_rep, 5),
                          "what": "the same step with every rank running the whole producer (no exchange)"}
        if layer.M % (128 * world) == 0:
            rws = layer.row_shard(world, rank)
            for _ in range(3):
                layer.step_capi(capi, st, dist=dist, rows=rws)
            ms_row = timed_steps(layer, args.steps, dist=dist, rows=rws)
            row_sharded = {"value": round(layer.flops_total / (ms_row * 1e-3) / 1e12, 2), "ms_per_step": round(ms_row, 5),
                           "what": "the same step with the producer on this rank's rows and an NCCL all-gather of the "
                                   "packed + scale bytes (M*K*0.5625 B per producer) inside the step"}
        if args.workload == "c2" and not args.tokens and not args.quick:
            # every rank runs the whole step on its own tokens: replicas, no collective (weak scaling)
            tok = Layer("c2", rank, 1, dev, act_seed=7000 + rank)
            for _ in range(3):
                tok.step_capi(capi, st)
            ms_tok = timed_steps(tok, args.steps)
            token_sharded = {"value": round(tok.flops_total * world / (ms_tok * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
                             "ms_per_step": round(ms_tok, 5), "scaling": "weak",
                             "what": f"every rank runs the whole step on its own {tok.M} tokens, weights replicated"}
            del tok
            torch.cuda.empty_cache()
            c5_col = column_run("c5", max(5, args.steps // 4))
    elif world > 1:
        column_sharded = column_run(args.workload, args.steps)
    # ---- the FFN as a connected chain: gate/up GEMM -> SwiGLU -> NVFP4 -> down GEMM ------
    # (not part of `value`: in the timed step above the down GEMM reads a resident NVFP4 input)
    names = [g_["name"] for g_ in layer.gemms]
    if world == 1 and "gate_up" in names and "down" in names:
        gu, dn = layer.gemms[names.index("gate_up")], layer.gemms[names.index("down")]
        Pc = capi.ptr
        hid = gu["n_loc"] // 2
        if dn["k"] == hid and hid % 128 == 0:
            def plain():
                L.frt_nvfp4_gemm_bf16(Pc(gu["a_p"]), Pc(gu["a_sf"]), Pc(gu["wp"]), Pc(gu["wsf"]), None, None,
                                      Pc(gu["out"]), layer.M, gu["n_loc"], gu["k"], 1.0, 0.0, st)
                L.frt_silu_mul_quant_nvfp4(Pc(gu["out"]), Pc(dn["a_p"]), Pc(dn["a_sf"]), layer.M, hid, st)
                L.frt_nvfp4_gemm_bf16(Pc(dn["a_p"]), Pc(dn["a_sf"]), Pc(dn["wp"]), Pc(dn["wsf"]), None, None,
                                      Pc(dn["out"]), layer.M, dn["n_loc"], dn["k"], 1.0, 0.0, st)

            def fused():
                L.frt_nvfp4_gemm_swiglu_nvfp4(Pc(gu["a_p"]), Pc(gu["a_sf"]), Pc(gu["wp"]), Pc(gu["wsf"]),
                                              Pc(dn["a_p"]), Pc(dn["a_sf"]), layer.M, gu["n_loc"], gu["k"], 1.0, st)
                L.frt_nvfp4_gemm_bf16(Pc(dn["a_p"]), Pc(dn["a_sf"]), Pc(dn["wp"]), Pc(dn["wsf"]), None, None,
                                      Pc(dn["out"]), layer.M, dn["n_loc"], dn["k"], 1.0, 0.0, st)
            n_it = max(5, min(50, args.steps))
            detail["ffn_chain"] = {"three_kernels_us": round(event_ms(plain, n_it) * 1e3, 1),
                                   "swiglu_in_gemm_epilogue_us": round(event_ms(fused, n_it) * 1e3, 1)}

    if deep:
        detail["sustained"] = sustained_leg(layer, capi, st, local_rank, ms_step, peaks)
        if psets is not None and args.workload == "c2" and not args.tokens:
            detail["reference_cuda"] = reference_cuda_leg(layer, psets, capi, st, peaks)
    del psets
    if deep and args.workload == "c2" and not args.tokens:
        torch.cuda.empty_cache()
        detail["c3"] = decode_leg(capi, dev, peaks)
        torch.cuda.empty_cache()
        detail["c4"] = moe_measure(capi, dev, peaks, steps=max(5, min(20, args.steps)), warmup=3)
        torch.cuda.empty_cache()
        c5 = Layer("c5", 0, 1, dev)
        for _ in range(3):
            c5.step_capi(capi, st)
        c5_ms = event_ms(lambda: c5.step_capi(capi, st), 5, warm=1)
        c5_tf = c5.flops_total / (c5_ms * 1e-3) / 1e12
        detail["c5"] = {"tflops": round(c5_tf, 1), "ms_per_step": round(c5_ms, 4), "config": c5.name,
                        "per_gemm": gemm_back_to_back(c5, capi, st, peaks, iters=4),
                        "roofline": {"bound": "tensor", "kernel": "nvfp4_gemm_pair_kernel (Llama-3-70B FFN, 8192 tokens)",
                                     "achieved": round(c5_tf, 1), "peak": round(peaks["fp4_burst"], 1), "unit": "TFLOP/s",
                                     "frac": round(c5_tf / peaks["fp4_burst"], 4), "peak_note": peaks["source"]}}
        del c5
        torch.cuda.empty_cache()

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu_baseline = run_cpu_port(args, steps=1, sample_rows=32)

    if rank == 0:
        # The timed region is a burst (milliseconds at boost clock) unless it runs for a second or more:
        # the burst bf16 figure x 4 is the denominator then, the sustained one otherwise.
        burst = timed_region_s < 1.0
        peak = peaks["fp4_burst"] if burst else peaks["fp4_sustained"]
        line = {
            "metric": "nvfp4_linear_path_tflops", "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 5), "higher_is_better": True,
            "scaling": "weak" if tokens_mode else "strong", "vs_baseline": None,
            "dtype": "nvfp4 (e2m1 x ue4m3, fp32 accumulate, bf16 out)",
            "data": "synthetic",
            "config": {"workload": layer.name, "tokens": layer.M, "hidden": layer.H,
                       "layers": {g_["name"]: [g_["n"], g_["k"]] for g_ in layer.gemms},
                       "global_tokens": layer.M * (world if tokens_mode else 1),
                       "parallelism": (f"token-sharded x{world}: every rank runs the step on its own {layer.M} tokens, "
                                       "weights replicated, no collective" if tokens_mode else
                                       f"column-sharded x{world}: NVFP4 weights partitioned by output columns, "
                                       "activations replicated, outputs left sharded" if world > 1 else "single GPU"),
                       "l2": f"inputs larger than L2: each step streams {layer.bytes_streamed >> 20} MiB "
                             f"({L2_BYTES >> 20} MiB L2), every tensor touched once per step"},
            "e2e": {"value": round(e2e_val, 2), "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": round(e2e_ms, 4),
                    "api": "torch ops fp4_fused_ops.residual_add_rms_norm_quant_nvfp4_swizzled_bf16 + "
                           "fp4_gemm.nvfp4_gemm_bf16; pinned host in/out, copies overlapped on side streams" +
                           ("; each rank copies its row shard of the inputs, the NVFP4 rows are all-gathered (NCCL)"
                            if rows is not None else "")},
            "gpu_launches": int(launches),
            "clocks": clocks.summary(),
            "roofline": {"bound": "tensor", "kernel": f"nvfp4_gemm_pair_kernel ({dom_g['name']} "
                         f"{layer.M}x{dom_g['n_loc']}x{dom_g['k']})", "achieved": round(achieved, 1),
                         "peak": round(peak, 1), "unit": "TFLOP/s",
                         "frac": round(achieved / peak, 4),
                         "peak_note": peaks["source"] + ("; burst figure: the timed region lasted "
                                                         f"{timed_region_s * 1e3:.1f} ms" if burst else
                                                         "; sustained figure: the timed region lasted "
                                                         f"{timed_region_s:.1f} s"),
                         "frac_of_sustained_peak": round(achieved / peaks["fp4_sustained"], 4),
                         "frac_of_nominal_9000": round(achieved / 9000.0, 4),
                         "algorithmic_flops_per_launch": dom_flops,
                         "traffic": NCU_DRAM_TRAFFIC_BYTES.get(("gemm", layer.M, dom_g["n_loc"], dom_g["k"]))},
            "detail": detail,
        }
        if "producer_back_to_back" in detail:
            pb = detail["producer_back_to_back"]
            line["roofline_producer"] = {
                "bound": "hbm", "kernel": f"norm_quant_kernel ({layer.M}x{layer.H} residual+RMSNorm->NVFP4)",
                "achieved": pb["gbs"], "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": pb["frac_of_hbm_measured"],
                "algorithmic_bytes": int(prod_bytes),
                # (at kernel end part of the output is still dirty in L2, so DRAM traffic is below the algorithmic bytes)
                "traffic": NCU_DRAM_TRAFFIC_BYTES.get(("producer", layer.M, layer.H))}
        if world > 1 and not tokens_mode:
            line["config"]["producer"] = (
                "row-sharded, NVFP4 rows stored into every rank's buffer by the producer kernel itself ("
                + ("NVSwitch multicast stores" if shared.uses_multicast else "peer stores") + "), bounded flag wait before "
                "each consumer GEMM; timed inside the step" if shared is not None else
                "replicated: every rank runs the whole producer" + (f" ({shared_note})" if shared_note else ""))
        for key, val in (("allgather_separate", allgather), ("replicated_producer", replicated),
                         ("row_sharded_producer_nccl", row_sharded),
                         ("column_sharded", column_sharded), ("token_sharded", token_sharded),
                         ("c5_column_sharded", c5_col), ("cpu_baseline", cpu_baseline)):
            if val:
                line[key] = val
        print(json.dumps(line), flush=True)


def run_moe(args, rank, world, local_rank):
    """Grouped NVFP4 GEMMs of one MoE layer (replicas only: every rank runs the whole workload)."""
    from flashrt_b200_core import capi, load
    load()
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    peaks = measured_peaks()
    with ClockSampler(local_rank) as clocks:
        r = moe_measure(capi, dev, peaks, args.steps, args.warmup)
    if rank == 0:
        print(json.dumps({
            "metric": "nvfp4_grouped_moe_tflops", "value": r["tflops"], "unit": "TFLOP/s",
            "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"],
            "higher_is_better": True, "scaling": "replicas only", "vs_baseline": None, "dtype": "nvfp4", "data": "synthetic",
            "config": {"workload": MOE["name"], "routed_rows": r["routed_rows"], "experts": r["experts"],
                       "layers": {l[0]: [l[1], l[2]] for l in MOE["layers"]},
                       "l2": "weights 340 MB + activations per step exceed the 126 MiB L2"},
            "roofline": r["roofline"],
            "detail": {"layers": r["layers"], "routed_layer_us": r["routed_layer_us"], "routed_layer": r["what"],
                       "decode": r.get("decode")},
            "gpu_launches": r["gpu_launches"], "clocks": clocks.summary()}), flush=True)


def model_measure(dev, layers=36, tokens=4096, reps=3):
    """A Qwen3-8B-shaped decoder (random weights, no checkpoint) through `transformers`: one prefill of `tokens`
    tokens in bf16 eager, with every projection swapped for an NVFP4 linear (what the reference's quantizer does),
    and with this library's fused conversion.  The attention kernel (torch SDPA) is the same in all three."""
    import copy
    import transformers
    from flashrt_layers.transformers_backend import convert_decoder_model
    cfg = transformers.Qwen3Config(hidden_size=4096, intermediate_size=12288, num_hidden_layers=layers,
                                   num_attention_heads=32, num_key_value_heads=8, head_dim=128, vocab_size=151936,
                                   max_position_embeddings=max(8192, tokens), initializer_range=0.006)
    cfg._attn_implementation = "sdpa"
    torch.manual_seed(0)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(dev):
            model = transformers.Qwen3Model(cfg).eval()
    finally:
        torch.set_default_dtype(prev)
    ids = torch.randint(0, cfg.vocab_size, (1, tokens), device=dev)

    def prefill_ms(m):
        with torch.no_grad():
            for _ in range(2):
                m(input_ids=ids, use_cache=False)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                out = m(input_ids=ids, use_cache=False).last_hidden_state
            e1.record()
            torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps, out

    res = {"config": f"qwen3-8b-shaped decoder, {layers} layers, hidden 4096, 32/8 heads x 128, FFN 12288, {tokens} tokens, "
                     "batch 1, random N(0, 0.006) weights (a projection then has gain ~0.4, so that 36 random layers do "
                     "not amplify rounding noise), transformers eager + SDPA attention"}
    res["bf16_eager_ms"], ref = prefill_ms(model)
    res["bf16_eager_ms"] = round(res["bf16_eager_ms"], 2)
    per_linear = copy.deepcopy(model)
    convert_decoder_model(per_linear, fuse=False)
    ms, out = prefill_ms(per_linear)
    res["nvfp4_per_linear_ms"] = round(ms, 2)
    cos = lambda a, b: round(torch.nn.functional.cosine_similarity(a.float().flatten(), b.float().flatten(), dim=0).item(), 4)
    res["cosine_vs_bf16_per_linear"] = cos(out, ref)
    out_per_linear = out
    del per_linear, out
    torch.cuda.empty_cache()
    convert_decoder_model(model, fuse=True)
    ms, out = prefill_ms(model)
    res["nvfp4_fused_ms"] = round(ms, 2)
    res["cosine_vs_bf16_fused"] = cos(out, ref)
    res["cosine_fused_vs_per_linear"] = cos(out, out_per_linear)
    res["speedup_vs_bf16_eager"] = round(res["bf16_eager_ms"] / ms, 2)
    res["what"] = ("fused = norm + quantise in one kernel with the residual additions inside it, q/k/v as one GEMM, "
                   "gate/up GEMM with the SwiGLU -> NVFP4 epilogue, down GEMM; per_linear = quantise + GEMM per nn.Linear")
    del model
    torch.cuda.empty_cache()
    return res


def run_model(args, rank, world, local_rank):
    from flashrt_b200_core import load
    load()
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    with ClockSampler(local_rank, period=0.02) as clocks:
        r = model_measure(dev)
    if rank == 0:
        print(json.dumps({
            "metric": "qwen3_8b_prefill_4096_ms", "value": r["nvfp4_fused_ms"], "unit": "ms", "n_gpus": 1,
            "steps": 3, "warmup": 2, "ms_per_step": r["nvfp4_fused_ms"], "higher_is_better": False,
            "scaling": "replicas only", "vs_baseline": None, "dtype": "nvfp4 linears, bf16 attention", "data": "synthetic",
            "config": {"workload": "qwen3-8b-shaped-decoder-prefill-4096"}, "detail": {"model": r},
            "clocks": clocks.summary()}), flush=True)


# ----------------------------------------------------------------------------
# CPU arm: the reference path restated for the host (oracle port)
# ----------------------------------------------------------------------------
def run_cpu_port(args, steps, sample_rows, warmup=0):
    """Times the pure-torch/numpy restatement of the reference path on the host
    cores for `sample_rows` tokens of the workload (weights dequantised once,
    as bind-time work)."""
    from oracle import nvfp4_oracle as O
    name, M, H, layers = WORKLOADS[args.workload]
    rng = np.random.default_rng(7)
    # every host thread this process may use (a launcher may have pinned OMP_NUM_THREADS to 1)
    threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(threads)
    bf = lambda a: O.f32_to_bf16_bits(a.astype(np.float32))
    hidden, residual = bf(rng.standard_normal((sample_rows, H))), bf(rng.standard_normal((sample_rows, H)))
    norm_w = bf(1 + 0.1 * rng.standard_normal(H))
    weights = []
    flops = 0.0
    for lname, n, k, fed in layers:
        # synthetic NVFP4 weight bytes (random codes, scales around N(0,.02) blocks), dequantised once
        wp = rng.integers(0, 256, (n, k // 2), dtype=np.uint8)
        wsf = rng.integers(20, 36, (n, k // 16), dtype=np.uint8)
        wdq = torch.from_numpy(O.dequantize_nvfp4(wp, wsf))
        act = None if fed else O.quantize_nvfp4(rng.standard_normal((sample_rows, k)).astype(np.float32))
        weights.append((lname, wdq, fed, act))
        flops += 2.0 * sample_rows * n * k

    def step(res):
        out = None
        for lname, wdq, fed, act in weights:
            if fed:
                q = O.fused_norm_quant(hidden, norm_w, EPS, res_bits=res)
                res = q["residual"]
                a = torch.from_numpy(O.dequantize_nvfp4(q["packed"], q["sf_linear"]))
            else:
                a = torch.from_numpy(O.dequantize_nvfp4(*act))
            out = (a @ wdq.T).to(torch.bfloat16)
        return out

    for _ in range(warmup):
        step(residual)
    t0 = time.perf_counter()
    for _ in range(steps):
        step(residual)
    dt = (time.perf_counter() - t0) / steps
    return {"value": round(flops / dt / 1e12, 5), "unit": "TFLOP/s", "cores": threads, "kind": "port",
            "ms_per_step_sample": round(dt * 1e3, 2),
            "sample": f"{sample_rows} of {M} tokens through all {len(layers)} linears of {name} "
                      f"(norm+quantise in numpy, dequantise + fp32 matmul in CPU torch, {threads} threads; "
                      f"weights dequantised once outside the timed region)"}


def run_reference(args, rank, world):
    """`--impl reference`: the reference's own CPU path for this metric.  The
    reference ships no CPU kernels; its CPU-runnable form of the path is the
    pure-torch oracle its tests use, restated under oracle/ (kind "port")."""
    if rank != 0:
        return
    if args.workload not in WORKLOADS:
        print(json.dumps({"impl": "reference", "unavailable": "the CPU arm covers the dense workloads (c2, c5)"}))
        return
    rows = 64
    steps_run = max(1, min(args.steps, 3))       # bounded: each step is a 64-token sample of the workload
    res = run_cpu_port(args, steps=steps_run, sample_rows=rows, warmup=min(args.warmup, 1))
    name, M, H, layers = WORKLOADS[args.workload]
    line = {"impl": "reference", "metric": "nvfp4_linear_path_tflops", "value": res["value"], "unit": "TFLOP/s",
            "n_gpus": world, "steps": steps_run, "warmup": min(args.warmup, 1),
            "ms_per_step": round(res["ms_per_step_sample"] * M / rows, 3), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "fp32 (dequantised NVFP4)", "data": "synthetic",
            "config": {"workload": name, "tokens": M, "hidden": H,
                       "layers": {l[0]: [l[1], l[2]] for l in layers}, "parallelism": "host CPU"},
            "cpu_baseline": {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": res["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS) + ["c4", "model"])
    ap.add_argument("--tokens", type=int, default=0, help="override the token count M (decode sweep: 1, 4, 16, 64)")
    ap.add_argument("--graph", action="store_true",
                    help="time CUDA-graph replays of the step (launch-bound decode shapes); prints a short line")
    ap.add_argument("--sharding", default="columns", choices=["columns", "tokens"],
                    help="N > 1: columns = column-sharded weights on the fixed problem (strong scaling, default); "
                         "tokens = data-parallel replicas over token rows (weak scaling)")
    ap.add_argument("--exchange", default="none", choices=["fused", "multicast", "none"],
                    help="N > 1, columns: fused = row-sharded producer that stores its rows into every rank's buffer "
                         "(peer stores; default); multicast = the same through NVSwitch multicast stores; "
                         "none = every rank runs the whole producer")
    ap.add_argument("--exchange-legs", action="store_true",
                    help="N > 1: also time the Llama-70B column-sharded step with the in-kernel exchange (peer stores "
                         "and multicast stores); needs torch symmetric memory")
    ap.add_argument("--no-pdl", action="store_true",
                    help="plain kernel launches instead of programmatic dependent launches (A/B)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--quick", action="store_true",
                    help="only the step itself: no sustained / reference-kernel / decode / MoE / Llama-70B legs")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (B200); there is no CPU fallback for the product path")
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        if args.workload == "c4":
            run_moe(args, rank, world, local_rank)
        elif args.workload == "model":
            run_model(args, rank, world, local_rank)
        else:
            run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
