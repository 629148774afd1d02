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
the host inside the timed region.  With N > 1 ranks (torchrun) every rank runs
the step on its own M tokens with replicated weights (token-sharded, no
collective: weak scaling, `value` = N ranks' flops / max time); the same line
carries `column_sharded`: the fixed M-token problem with the weights
column-sharded over the ranks, activations replicated, outputs left sharded
(strong scaling), and the NCCL all-gather of those outputs timed separately.
`--sharding columns` makes that form the headline instead.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c5|c4]
                    [--sharding tokens|columns] [--tokens M --graph]
"""
from __future__ import annotations

import argparse
import json
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
# measured DRAM traffic per launch of the four Qwen3-8B M=4096 GEMMs (ncu, bytes)
NCU_DRAM_TRAFFIC_BYTES = {"qkv": 29563904, "o": 19248896, "gate_up": 221514496, "down": 70588160}

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
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm_gbs=d["hbm_gbs"], fp4_tflops=4.0 * d["bf16_tflops_sustained"],
                    fp4_tflops_burst=4.0 * d["bf16_tflops"], source="measured (MEASURED_PEAKS.json; FP4 = 4 x bf16)")
    return dict(hbm_gbs=6650.0, fp4_tflops=4.0 * 1400.0, fp4_tflops_burst=4.0 * 1590.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
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
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.005)

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
        return {"sm_mhz": int(statistics.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


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
            # quantise the full-width weight in slabs so every rank derives the same bytes for its shard
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

    def step_capi(self, capi, st, ev=None):
        """one pass through the C ABI (resident inputs); optional (start,end) events per kernel"""
        L = capi.lib()
        P = capi.ptr
        launches = 0
        for i, g_ in enumerate(self.gemms):
            if g_["fed"]:
                pe = ev.get(("producer", i)) if ev is not None else None
                if pe:
                    pe[0].record()
                rc = L.frt_norm_quant_nvfp4(P(self.residual), P(self.hidden), P(self.norm_w), EPS, 1.0, None,
                                            P(self.act_packed), P(self.act_sf), self.M, self.H, 0, st)
                if pe:
                    pe[1].record()
                assert rc == 0, rc
                launches += 1
            ge = ev.get((g_["name"], i)) if ev is not None else None
            if ge:
                ge[0].record()
            rc = L.frt_nvfp4_gemm_bf16(P(g_["a_p"]), P(g_["a_sf"]), P(g_["wp"]), P(g_["wsf"]), None, None,
                                       P(g_["out"]), self.M, g_["n_loc"], g_["k"], 1.0, 0.0, st)
            if ge:
                ge[1].record()
            assert rc == 0, rc
            launches += 1
        return launches

    def step_ops(self, hidden, residual):
        """one pass through the torch operator API; returns the last GEMM's output"""
        import fp4_fused_ops
        import fp4_gemm
        out = None
        for g_ in self.gemms:
            if g_["fed"]:
                fp4_fused_ops.residual_add_rms_norm_quant_nvfp4_swizzled_bf16(
                    residual, hidden, self.norm_w, EPS, packed=self.act_packed, sfa=self.act_sf)
            out = fp4_gemm.nvfp4_gemm_bf16(g_["a_p"], g_["wp"], g_["a_sf"], g_["wsf"], out=g_["out"])
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
    # N > 1: by default every rank runs the whole step on its OWN tokens (weights replicated, no
    # collective: weak scaling); --sharding columns runs the fixed problem with column-sharded weights
    # and replicated activations (strong scaling), which the token-sharded run also reports beside it.
    tokens_mode = world > 1 and args.sharding != "columns"
    col_world = 1 if tokens_mode else world
    layer = Layer(args.workload, rank, col_world, dev, tokens=args.tokens,
                  act_seed=7000 + rank if tokens_mode else None)
    job_flops = layer.flops_total * (world if tokens_mode else 1)
    st = capi.stream_ptr()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        layer.step_capi(capi, st)
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
                "config": {"workload": layer.name, "tokens": layer.M},
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
    launches0 = capi.lib().frt_launch_count()
    with ClockSampler(local_rank) as clocks:
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for s in range(args.steps):
            layer.step_capi(capi, st, events[s])
        t1.record()
        barrier()
    ms_total = t0.elapsed_time(t1)
    launches = capi.lib().frt_launch_count() - launches0
    if world > 1:
        t = torch.tensor([ms_total], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    value = job_flops / (ms_step * 1e-3) / 1e12

    dom_ms = statistics.mean(e[dom][0].elapsed_time(e[dom][1]) for e in events)
    # second pass (not part of `value`): every kernel bracketed by events
    n_detail = max(5, min(50, args.steps))
    ev2 = [{k: (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for k in keys}
           for _ in range(n_detail)]
    for s_ in range(n_detail):
        layer.step_capi(capi, st, ev2[s_])
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
    detail = {
        "gemm_only_tflops": job_flops / (gemm_ms * 1e-3) / 1e12,
        "per_kernel_us": {f"{k[0]}": round(v * 1e3, 2) for k, v in per_kernel.items()},
        "per_gemm_tflops": {layer.gemms[k[1]]["name"]: round(2.0 * layer.M * layer.gemms[k[1]]["n_loc"] *
                            layer.gemms[k[1]]["k"] / (v * 1e-3) / 1e12, 1) for k, v in per_kernel.items()
                            if k[0] != "producer"},
        "weight_stream_gbs": round(sum(0.5625 * g_["n_loc"] * g_["k"] for g_ in layer.gemms) / (gemm_ms * 1e-3) / 1e9 * world, 1),
        "producer_gbs": round(prod_bytes / (statistics.mean(prod_ms) * 1e-3) / 1e9, 1) if prod_ms else None,
        "producer_frac_of_hbm_measured": round(prod_bytes / (statistics.mean(prod_ms) * 1e-3) / 1e9 /
                                               peaks["hbm_gbs"], 3) if prod_ms else None,
    }

    # ---- the producer alone, back to back over four input sets (292 MB: larger than L2) ----------------
    if any(g_["fed"] for g_ in layer.gemms):
        from flashrt_b200_core import alloc_fp4
        Lp, Pp = capi.lib(), capi.ptr
        psets = []
        for _ in range(4):
            pk, sfp_ = alloc_fp4(layer.M, layer.H, dev)
            psets.append((layer.hidden.clone(), layer.residual0.clone(), pk, sfp_))

        def producers():
            for hx, rx, pk, sfp_ in psets:
                Lp.frt_norm_quant_nvfp4(Pp(rx), Pp(hx), Pp(layer.norm_w), EPS, 1.0, None, Pp(pk), Pp(sfp_), layer.M,
                                        layer.H, 0, st)
        for _ in range(3):
            producers()
        torch.cuda.synchronize()
        q0, q1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        q0.record()
        for _ in range(10):
            producers()
        q1.record()
        torch.cuda.synchronize()
        p_us = q0.elapsed_time(q1) / 40 * 1e3
        detail["producer_back_to_back"] = {"us": round(p_us, 2), "gbs": round(prod_bytes / p_us / 1e3, 1),
                                           "frac_of_hbm_measured": round(prod_bytes / p_us / 1e3 / peaks["hbm_gbs"], 3),
                                           "what": "fused residual+RMSNorm->NVFP4 on 4 rotating input sets, 40 launches"}
        del psets

    # ---- end to end through the torch operator API with host buffers ----------
    # the step's two bf16 inputs (hidden, residual) sit in ONE pinned buffer and travel as one copy
    host_in = torch.empty(2, layer.M, layer.H, dtype=torch.bfloat16).pin_memory()
    host_in[0].copy_(layer.hidden.cpu())
    host_in[1].copy_(layer.residual0.cpu())
    last = layer.gemms[-1]["out"]
    host_out = [torch.empty(last.shape, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    dev_in = [torch.empty(2, layer.M, layer.H, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    copy_s, comp_s, out_s = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    h2d = 2 * layer.M * layer.H * 2 * world          # whole job: every rank copies its step inputs
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
                out = layer.step_ops(dev_in[b][0], dev_in[b][1])
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
    e2e_ms = (time.perf_counter() - w0) * 1e3 / max(e2e_n, 1)
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
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
        ag_ms = a0.elapsed_time(a1) / 10
        t = torch.tensor([ag_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ag_ms = float(t.item())
        tot = gathered.numel() * 2
        del gathered
        return {"layer": big["name"], "ms": round(ag_ms, 4), "bytes_total": tot,
                "bus_gbs": round(tot * (world - 1) / world / (ag_ms * 1e-3) / 1e9, 1), "backend": "nccl"}

    # ---- all-gather of the column-sharded outputs, timed separately; in a token-sharded run the
    # column-sharded form of the same (fixed-size) problem is measured here as well
    allgather = column_sharded = None
    if world > 1 and not tokens_mode:
        allgather = time_allgather(layer)
    elif world > 1:
        col = Layer(args.workload, rank, world, dev, tokens=args.tokens)
        for _ in range(args.warmup):
            col.step_capi(capi, st)
        barrier()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        for _ in range(args.steps):
            col.step_capi(capi, st)
        c1.record()
        barrier()
        t = torch.tensor([c0.elapsed_time(c1) / args.steps], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        col_ms = float(t.item())
        column_sharded = {"value": round(col.flops_total / (col_ms * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
                          "ms_per_step": round(col_ms, 5), "scaling": "strong",
                          "what": f"the same workload at a fixed {col.M} tokens, weights column-sharded x{world}, "
                                  "activations replicated, outputs left sharded",
                          "allgather_separate": time_allgather(col)}
        del col

    # ---- the FFN as a connected chain: gate/up GEMM -> SwiGLU -> NVFP4 -> down GEMM ------
    # (not part of `value`: in the timed step above the down GEMM reads a resident NVFP4 input)
    names = [g_["name"] for g_ in layer.gemms]
    if world == 1 and "gate_up" in names and "down" in names:
        gu, dn = layer.gemms[names.index("gate_up")], layer.gemms[names.index("down")]
        Lc, Pc = capi.lib(), capi.ptr
        hid = gu["n_loc"] // 2
        if dn["k"] == hid and hid % 128 == 0:
            def plain():
                Lc.frt_nvfp4_gemm_bf16(Pc(gu["a_p"]), Pc(gu["a_sf"]), Pc(gu["wp"]), Pc(gu["wsf"]), None, None,
                                       Pc(gu["out"]), layer.M, gu["n_loc"], gu["k"], 1.0, 0.0, st)
                Lc.frt_silu_mul_quant_nvfp4(Pc(gu["out"]), Pc(dn["a_p"]), Pc(dn["a_sf"]), layer.M, hid, st)
                Lc.frt_nvfp4_gemm_bf16(Pc(dn["a_p"]), Pc(dn["a_sf"]), Pc(dn["wp"]), Pc(dn["wsf"]), None, None,
                                       Pc(dn["out"]), layer.M, dn["n_loc"], dn["k"], 1.0, 0.0, st)

            def fused():
                Lc.frt_nvfp4_gemm_swiglu_nvfp4(Pc(gu["a_p"]), Pc(gu["a_sf"]), Pc(gu["wp"]), Pc(gu["wsf"]),
                                               Pc(dn["a_p"]), Pc(dn["a_sf"]), layer.M, gu["n_loc"], gu["k"], 1.0, st)
                Lc.frt_nvfp4_gemm_bf16(Pc(dn["a_p"]), Pc(dn["a_sf"]), Pc(dn["wp"]), Pc(dn["wsf"]), None, None,
                                       Pc(dn["out"]), layer.M, dn["n_loc"], dn["k"], 1.0, 0.0, st)

            chain = {}
            n_it = max(5, min(50, args.steps))
            for label, fn in (("three_kernels_us", plain), ("swiglu_in_gemm_epilogue_us", fused)):
                for _ in range(3):
                    fn()
                torch.cuda.synchronize()
                c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                c0.record()
                for _ in range(n_it):
                    fn()
                c1.record()
                torch.cuda.synchronize()
                chain[label] = round(c0.elapsed_time(c1) / n_it * 1e3, 1)
            detail["ffn_chain"] = chain

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu_baseline = run_cpu_port(args, steps=1, sample_rows=32)

    if rank == 0:
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
                                       f"column-sharded x{world}, activations replicated" if world > 1 else "single GPU"),
                       "l2": f"inputs larger than L2: each step streams {layer.bytes_streamed >> 20} MiB "
                             f"({L2_BYTES >> 20} MiB L2), every tensor touched once per step"},
            "e2e": {"value": round(e2e_val, 2), "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": round(e2e_ms, 4),
                    "api": "torch ops fp4_fused_ops.residual_add_rms_norm_quant_nvfp4_swizzled_bf16 + "
                           "fp4_gemm.nvfp4_gemm_bf16; pinned host in/out, copies overlapped on side streams"},
            "gpu_launches": int(launches),
            "clocks": clocks.summary(),
            "roofline": {"bound": "tensor", "kernel": f"nvfp4_gemm_pair_kernel ({dom_g['name']} "
                         f"{layer.M}x{dom_g['n_loc']}x{dom_g['k']})", "achieved": round(achieved, 1),
                         "peak": round(peaks["fp4_tflops"], 1), "unit": "TFLOP/s",
                         "frac": round(achieved / peaks["fp4_tflops"], 4),
                         "peak_note": peaks["source"] + ", sustained figure (kernel timed inside a long step)",
                         "frac_of_burst_peak": round(achieved / peaks["fp4_tflops_burst"], 4),
                         "frac_of_nominal_9000": round(achieved / 9000.0, 4),
                         "traffic": None},
            "detail": detail,
        }
        # ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel on this workload
        # (profiles/nvfp4_gemm_pair_and_producer_qwen3_8b_m4096.md); only meaningful for the unsharded default
        if args.workload == "c2" and not args.tokens and dom_g["n_loc"] == dom_g["n"]:
            line["roofline"]["traffic"] = NCU_DRAM_TRAFFIC_BYTES.get(dom_g["name"])
        if "producer_back_to_back" in detail:
            pb = detail["producer_back_to_back"]
            line["roofline_producer"] = {
                "bound": "hbm", "kernel": f"norm_quant_kernel ({layer.M}x{layer.H} residual+RMSNorm->NVFP4)",
                "achieved": pb["gbs"], "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": pb["frac_of_hbm_measured"],
                "algorithmic_bytes": int(prod_bytes),
                # ncu on this shape: 67.1 MB read + 1.9 MB written back by kernel end (the rest of the 46 MB of
                # output is still dirty in L2 then)
                "traffic": 69002240 if (layer.M, layer.H) == (4096, 4096) else None}
        if allgather:
            line["allgather_separate"] = allgather
        if column_sharded:
            line["column_sharded"] = column_sharded
        if cpu_baseline:
            line["cpu_baseline"] = cpu_baseline
        print(json.dumps(line), flush=True)


def run_moe(args, rank, world, local_rank):
    """Grouped NVFP4 GEMMs of one MoE layer (replicas only: every rank runs the whole workload)."""
    from flashrt_b200_core import capi, load
    load()
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    L, P, st = capi.lib(), capi.ptr, capi.stream_ptr()
    # routing of the synthetic workload: top-8 of seeded N(0,1) logits (= top-8 of their softmax), sorted by
    # expert into per-expert offsets, with this library's router and routing-plan kernels
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

    def step():
        for name, n, k, ap, wp, asf, wsf, out in layers:
            rc = L.frt_nvfp4_grouped_gemm_bf16(P(ap), P(asf), P(wp), P(wsf), P(alpha), P(offs_d), None, 0, P(out), rows,
                                               n, k, experts, n * (k // 2), int(wsf.shape[1]), P(work), st)
            assert rc == 0, rc

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    l0 = L.frt_launch_count()
    with ClockSampler(local_rank) as clocks:
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(args.steps):
            step()
        t1.record()
        torch.cuda.synchronize()
    ms = t0.elapsed_time(t1) / args.steps
    launches = int(L.frt_launch_count() - l0)

    # ---- the whole routed layer through the C ABI: router -> plan -> quantise -> gather ->
    # grouped gate/up -> SwiGLU -> NVFP4 -> grouped down -> weighted un-permute
    T, E, topk = MOE["tokens"], experts, MOE["top_k"]
    (_, n1, k1, _, wp1, _, wsf1, out1), (_, n2, k2, _, wp2, _, wsf2, out2) = layers
    g = torch.Generator(device=dev).manual_seed(11)
    hidden = torch.randn(T, k1, generator=g, device=dev).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g, device=dev).to(torch.bfloat16)
    idx = torch.empty(T, topk, dtype=torch.int32, device=dev)
    val = torch.empty(T, topk, dtype=torch.float32, device=dev)
    off = torch.empty(E + 1, dtype=torch.int32, device=dev)
    rop = torch.empty(T, topk, dtype=torch.int32, device=dev)
    tor = torch.empty(T * topk, dtype=torch.int32, device=dev)
    xp = torch.empty(T, k1 // 2, dtype=torch.uint8, device=dev)
    xs = torch.zeros(sfb(T, k1), dtype=torch.uint8, device=dev)
    gp = torch.empty(T * topk, k1 // 2, dtype=torch.uint8, device=dev)
    gs = torch.zeros(sfb(T * topk, k1), dtype=torch.uint8, device=dev)
    hp = torch.empty(T * topk, k2 // 2, dtype=torch.uint8, device=dev)
    hs = torch.zeros(sfb(T * topk, k2), dtype=torch.uint8, device=dev)
    final = torch.empty(T, n2, dtype=torch.float32, device=dev)
    weights = torch.empty(T, topk, dtype=torch.float32, device=dev)
    R = T * topk

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
        for _ in range(3):
            routed_layer()
        torch.cuda.synchronize()
        r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_it = max(5, min(50, args.steps))
        r0.record()
        for _ in range(n_it):
            routed_layer()
        r1.record()
        torch.cuda.synchronize()
        routed_us = round(r0.elapsed_time(r1) / n_it * 1e3, 1)
    if rank == 0:
        print(json.dumps({
            "metric": "nvfp4_grouped_moe_tflops", "value": round(flops / (ms * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
            "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 5),
            "higher_is_better": True, "scaling": "replicas only", "vs_baseline": None, "dtype": "nvfp4", "data": "synthetic",
            "config": {"workload": MOE["name"], "routed_rows": rows, "experts": experts,
                       "layers": {l[0]: [l[1], l[2]] for l in layers},
                       "l2": "weights 340 MB + activations per step exceed the 126 MiB L2"},
            "detail": {"routed_layer_us": routed_us,
                       "routed_layer": "router top-k + softmax, routing plan, quantise into expert order, grouped gate/up, "
                                       "SwiGLU->NVFP4, grouped down, weighted un-permute (11 launches of this library)"},
            "gpu_launches": launches, "clocks": clocks.summary()}), flush=True)


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
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS) + ["c4"])
    ap.add_argument("--tokens", type=int, default=0, help="override the token count M (decode sweep: 1, 4, 16, 64)")
    ap.add_argument("--graph", action="store_true",
                    help="time CUDA-graph replays of the step (launch-bound decode shapes); prints a short line")
    ap.add_argument("--sharding", default="tokens", choices=["tokens", "columns"],
                    help="N > 1: tokens = data-parallel over token rows (weak scaling, default); columns = "
                         "column-sharded weights on the fixed problem (strong scaling)")
    ap.add_argument("--no-pdl", action="store_true",
                    help="plain kernel launches instead of programmatic dependent launches (A/B)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
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
        else:
            run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
