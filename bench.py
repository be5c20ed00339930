#!/usr/bin/env python
"""Headline benchmark: MoE-FFN tokens/s and HBM GB/s, Qwen3.5-35B-A3B expert shape,
40 stacked MoE layers with all 40 x 256 experts resident in the HBM slot pool.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--tokens T] [--impl ours|reference]

A step is one pass of T tokens (default 1) through all layers: router -> top-8 ->
residency lookup -> shared + routed expert FFN -> combine, hidden += y feeding the
next layer. Prints ONE JSON line. With N > 1 (torchrun) every rank runs an
independent replica of the workload on its own GPU (the single-GPU workloads do
not shard; no collective on the data path) and the value is the aggregate.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
sys.path.insert(1, str(ROOT / "tests"))   # fixtures, the oracle bindings and the GPU harness (test infrastructure)

SEED = 20240
LAYERS = 40
METRIC = "MoE-FFN tokens/s and HBM GB/s vs 8 TB/s peak at 1/2/4/8 B200"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--tokens", type=int, default=1, help="decode batch: 1, 4 or 16")
    ap.add_argument("--layers", type=int, default=LAYERS)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=["decode", "prefill", "ep", "gptoss"], default="decode",
                    help="decode: the 40-layer sweep (headline); prefill: one layer, 4096 rows, Zipf(1.1)-skewed routing")
    ap.add_argument("--rows", type=int, default=4096, help="rows of the prefill workload")
    ap.add_argument("--no-sweep", action="store_true", help="skip the T=4 / T=16 lines of the sweep")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    return ap.parse_args()


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


def router_weights(layer: int, ne: int, d: int) -> np.ndarray:
    return np.random.default_rng(SEED * 1000 + layer).normal(0, 0.02, (ne, d)).astype(np.float32)


def gate_weights(layer: int, d: int) -> np.ndarray:
    return np.random.default_rng(SEED * 1000 + 500 + layer).normal(0, 0.02, d).astype(np.float32)


def input_tokens(T: int, d: int) -> np.ndarray:
    import fixtures as fx
    return fx.round_bf16(np.random.default_rng(SEED).normal(0, 1, (T, d)).astype(np.float32))


# ------------------------------------------------------------------ clocks

class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except ValueError:
                continue
            for name, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------ CPU arm (oracle / reference GEMV)

def cpu_reference_run(T: int, layers: int, steps: int, warmup: int, budget_s: float):
    """The reference's CPU implementation of the path on the host cores: its own compiled
    int4 GEMV (oracle/_ref) under the restated expert FFN, router and combine (oracle/)."""
    sys.path.insert(0, str(ROOT / "tests"))
    import oracle_lib as O
    import fixtures as fx

    cfg = fx.qwen_config(max_tokens=16)
    kind = "reference" if O.use_reference_gemv(True) else "port"
    cores = os.cpu_count() or 1
    ecfg = O.expert_cfg(cfg.d, cfg.f)
    lcfg = O.layer_cfg(ecfg, O.expert_cfg(cfg.d, cfg.shared_f), True)
    x0 = input_tokens(T, cfg.d)
    routers = [router_weights(l, cfg.num_experts, cfg.d) for l in range(layers)]
    gates = [gate_weights(l, cfg.d) for l in range(layers)]
    shared = [O.synth_block(O.expert_cfg(cfg.d, cfg.shared_f), SEED, l, 100000) for l in range(layers)]
    cache: dict = {}

    def block(l, e):
        if (l, e) not in cache:
            cache[(l, e)] = O.synth_block(ecfg, SEED, l, e)
        return cache[(l, e)]

    def step():
        h = x0.copy()
        for l in range(layers):
            ids = np.zeros((T, cfg.top_k), np.uint32)
            w = np.zeros((T, cfg.top_k), np.float32)
            for t in range(T):
                ids[t], w[t] = O.router_select(O.router_logits_f32(routers[l], h[t]), cfg.top_k, round_f16=True)
            blocks = {int(e): block(l, int(e)) for e in np.unique(ids)}
            y = O.moe_layer(lcfg, blocks, shared[l], gates[l], h, ids, w, threads=cores)
            h = fx.round_bf16(h + fx.round_bf16(y))
        return h

    step()  # generates and caches the blocks the routing touches; not timed
    for _ in range(max(0, warmup - 1)):
        step()
    times = []
    t_begin = time.perf_counter()
    for _ in range(steps):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - t_begin > budget_s:
            break
    O.use_reference_gemv(False)
    ms = 1e3 * sum(times) / len(times)
    return {"value": T / (ms / 1e3), "unit": "tokens/s", "cores": cores, "kind": kind,
            "sample": f"{len(times)} steps of {T} token(s) x {layers} layers (router + 8 routed + 1 shared expert per layer), "
                      f"{cores} threads over experts", "ms_per_step": ms, "steps": len(times)}


# ------------------------------------------------------------------ our arm

class Workload:
    """All layers resident on one GPU; per-layer handles so that every layer keeps its own work lists."""

    def __init__(self, T: int, layers: int, device_index: int, cfg=None):
        import torch
        from shrike_b200 import capi
        import fixtures as fx
        from shrike_b200.moe import ExpertCellArena, MoE, RouterOperands, expert_offsets, round_up

        self.torch = torch
        self.T, self.L = T, layers
        torch.cuda.set_device(device_index)
        self.dev = torch.device("cuda", device_index)
        self.cfg = cfg = cfg if cfg is not None else fx.qwen_config(max_tokens=16)
        self.moes = [MoE(cfg, device_index) for _ in range(layers)]
        self.off, self.block_bytes = expert_offsets(cfg)
        self.soff, self.sblock_bytes = expert_offsets(cfg, shared=True) if cfg.has_shared else (None, 0)
        stride = round_up(max(self.block_bytes, self.sblock_bytes), 256)
        ne = cfg.num_experts
        self.pool = ExpertCellArena(self.moes[0], layers * (ne + 1), stride, chunks=8)
        self.routers, self.shared, self._keep = [], [], []
        for l in range(layers):
            self.pool.fill_synthetic(l * ne, ne, SEED, l)
            if cfg.has_shared:
                self.pool.fill_synthetic(layers * ne + l, 1, SEED, l, first_expert=100000, shared=True)
            m = self.moes[l]
            m.create_residency(1)
            m.residency_set_layer_identity(0, l * ne)
            rw = torch.from_numpy(router_weights(l, ne, cfg.d)).to(self.dev)
            gw = torch.from_numpy(gate_weights(l, cfg.d)).to(self.dev) if cfg.shared_gated else None
            self._keep += [rw, gw]
            self.routers.append(RouterOperands(weights=rw, shared_gate=gw))
            self.shared.append(capi.SharedExpert(self.pool.cell_address(layers * ne + l), self.soff)
                               if cfg.has_shared else None)
        k = cfg.top_k
        self.ids = [torch.zeros((T, k), dtype=torch.int32, device=self.dev) for _ in range(layers)]
        self.slots = [torch.zeros((T, k), dtype=torch.int32, device=self.dev) for _ in range(layers)]
        self.w = [torch.zeros((T, k), dtype=torch.float32, device=self.dev) for _ in range(layers)]
        self.gate = [torch.zeros(T, dtype=torch.float32, device=self.dev) for _ in range(layers)]
        self.x_host = torch.from_numpy(input_tokens(T, cfg.d)).to(torch.bfloat16).pin_memory()
        self.out_host = torch.empty_like(self.x_host).pin_memory()
        self.x0 = self.x_host.to(self.dev)
        self.hidden = torch.zeros_like(self.x0)
        self.y = torch.zeros_like(self.x0)
        self.launches_per_step = layers * 3
        torch.cuda.synchronize()

    def layers_on_device(self):
        """router -> classification -> plan -> phase 1 -> phase 2 for every layer; hidden carries on."""
        for l in range(self.L):
            self.moes[l].encode_decode_layer(self.pool, self.off, 0, self.routers[l], self.hidden, self.y,
                                             self.hidden, self.shared[l], self.ids[l], self.w[l])

    def step_resident(self):
        self.hidden.copy_(self.x0)
        self.layers_on_device()

    def step_e2e(self):
        self.hidden.copy_(self.x_host, non_blocking=True)
        self.layers_on_device()
        self.out_host.copy_(self.hidden, non_blocking=True)

    def build_work_lists(self):
        """The per-phase graphs run the expert kernels from work lists; the one-row layer call routes inside the
        expert kernels and leaves none, so the route kernel builds them here (outside any timed region)."""
        for l in range(self.L):
            self.moes[l].encode_route_decode(self.routers[l], 0, self.pool, self.hidden, self.ids[l], self.w[l],
                                             self.gate[l] if self.cfg.shared_gated else None)
        self.torch.cuda.synchronize()

    def phase1_only(self):
        for l in range(self.L):
            self.moes[l].encode_phase1(self.pool, self.off, self.T, self.shared[l])

    def phase2_only(self):
        for l in range(self.L):
            self.moes[l].encode_phase2_reduce(self.pool, self.off, self.w[l], self.y, self.T, None, self.shared[l],
                                              self.gate[l] if self.cfg.shared_gated else None)

    def capture(self, fn):
        torch = self.torch
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            fn()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        return g

    def time_graph(self, g, steps: int, warmup: int) -> float:
        """Mean ms per replay, CUDA events on the launching stream."""
        torch = self.torch
        for _ in range(warmup):
            g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    def distinct_experts(self):
        return [int(self.torch.unique(self.ids[l]).numel()) for l in range(self.L)]

    def check_status(self):
        for m in self.moes:
            m.status()

    def close(self):
        self.pool.close()
        for m in self.moes:
            m.close()


def run_ours(args, rank: int, world: int, local_rank: int):
    import torch
    import torch.distributed as dist

    T, L, K, W = args.tokens, args.layers, args.steps, max(3, args.warmup)
    wl = Workload(T, L, local_rank)
    g_step = wl.capture(wl.step_resident)
    g_e2e = wl.capture(wl.step_e2e)
    wl.check_status()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    barrier()
    ms = wl.time_graph(g_step, K, W)
    barrier()
    ms_e2e = wl.time_graph(g_e2e, K, W)
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([ms, ms_e2e], dtype=torch.float64, device=wl.dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(t[0]), float(t[1])
    wl.check_status()

    # roofline of the dominant kernel (phase 1: gate/up dequant-GEMV + GLU), timed alone:
    # one launch per layer, each on a different layer's cold expert blocks
    cfg = wl.cfg
    o = wl.off
    gate_up_bytes = o.down_w                      # gate + up sub-tensors of one block
    down_bytes = wl.block_bytes - o.down_w
    distinct = wl.distinct_experts()
    wl.build_work_lists()
    g_p1 = wl.capture(wl.phase1_only)
    g_p2 = wl.capture(wl.phase2_only)
    ms_p1 = wl.time_graph(g_p1, max(10, K // 2), 3) / L
    ms_p2 = wl.time_graph(g_p2, max(10, K // 2), 3) / L
    units = [u + 1 for u in distinct]             # + the shared expert
    mean_units = sum(units) / L
    peak, peak_src = measured_peaks()
    # dram__bytes_read + dram__bytes_write of one phase-1 launch from the ncu capture summarised in
    # profiles/phase1_kernel_qwen_batch1.md: 10,654,848 B for 9 experts, i.e. 1.0036 x the algorithmic bytes;
    # traffic grows with the experts a launch touches, so it is scaled by the units of this run.
    traffic = mean_units * 10_654_848 / 9.0
    p1_gbs = mean_units * gate_up_bytes / (ms_p1 * 1e-3) / 1e9
    p2_gbs = mean_units * down_bytes / (ms_p2 * 1e-3) / 1e9
    layer_gbs = mean_units * wl.block_bytes / (ms / L * 1e-3) / 1e9

    line = None
    if rank == 0:
        tokens = T * world
        line = {
            "metric": METRIC, "value": tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int4 weights x fp16 operands, fp32 accumulate", "data": "synthetic",
            "config": {
                "workload": f"qwen3.5-35b-a3b expert shape, {L}-layer decode sweep, batch {T} "
                            f"(D 2048, 256 experts top-8 + gated shared, F 512, int4 g64 bf16 meta)",
                "tokens_per_step_per_gpu": T, "layers": L, "parallelism": "replicas" if world > 1 else "single",
                "l2": "inputs larger than L2: every step streams "
                      f"{mean_units * wl.block_bytes * L / 1e6:.0f} MB of distinct expert blocks (L2 126 MB)",
                "pool_gb": wl.pool.cells * wl.pool.cell_stride / 1e9,
            },
            "hbm_gbs_per_layer": layer_gbs,
            "roofline": {"bound": "hbm", "kernel": "phase1_kernel<4,64,bf16>", "achieved": p1_gbs, "peak": peak,
                         "unit": "GB/s", "frac": p1_gbs / peak, "peak_source": peak_src, "traffic": traffic,
                         "algorithmic_bytes_per_launch": mean_units * gate_up_bytes, "us_per_launch": ms_p1 * 1e3,
                         "phase2": {"achieved": p2_gbs, "frac": p2_gbs / peak, "us_per_launch": ms_p2 * 1e3,
                                    "algorithmic_bytes_per_launch": mean_units * down_bytes},
                         "whole_layer": {"achieved": layer_gbs, "frac": layer_gbs / peak,
                                         "us_per_layer": ms / L * 1e3}},
            "e2e": {"value": tokens / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": T * cfg.d * 2, "d2h_bytes_per_step": T * cfg.d * 2},
            "gpu_launches": wl.launches_per_step * K,
            "distinct_experts_per_layer": sum(distinct) / L,
            "clocks": clocks,
        }
    wl.close()
    return line


def run_prefill(args, local_rank: int):
    """Ragged prefill through one Qwen-shape int4 layer: rows routed top-8 of 256 with a Zipf(1.1) prior on the
    expert ids, permuted by expert on the device, expert-grouped GEMM on the tcgen05 tensor cores."""
    import torch
    from shrike_b200 import capi
    import fixtures as fx
    from shrike_b200.moe import ExpertCellArena, MoE, RouterOperands, expert_offsets, round_up
    sys.path.insert(0, str(ROOT / "tests"))
    from gpu_harness import bf16_tensor

    T, K, W = args.rows, args.steps, max(3, args.warmup)
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    cfg = fx.qwen_config(max_tokens=T)
    moe = MoE(cfg, local_rank)
    off, block_bytes = expert_offsets(cfg)
    soff, sbytes = expert_offsets(cfg, shared=True)
    pool = ExpertCellArena(moe, cfg.num_experts + 1, round_up(max(block_bytes, sbytes), 256))
    pool.fill_synthetic(0, cfg.num_experts, SEED, 0)
    pool.fill_synthetic(cfg.num_experts, 1, SEED, 0, first_expert=100000, shared=True)
    moe.create_residency(1)
    moe.residency_set_layer_identity(0, 0)
    shared = capi.SharedExpert(pool.cell_address(cfg.num_experts), soff)
    ops = RouterOperands(weights=torch.from_numpy(router_weights(0, cfg.num_experts, cfg.d)).to(dev),
                         shared_gate=torch.from_numpy(gate_weights(0, cfg.d)).to(dev),
                         logit_bias=bf16_tensor(fx.zipf_logit_bias(cfg.num_experts, 1.1), dev))
    x_host = torch.from_numpy(input_tokens(T, cfg.d)).to(torch.bfloat16).pin_memory()
    y_host = torch.empty_like(x_host).pin_memory()
    x = x_host.to(dev)
    y = torch.empty_like(x)
    ids = torch.zeros((T, cfg.top_k), dtype=torch.int32, device=dev)
    slots = torch.zeros_like(ids)
    w = torch.zeros((T, cfg.top_k), dtype=torch.float32, device=dev)
    gate = torch.zeros(T, dtype=torch.float32, device=dev)

    def route():
        moe.encode_router(ops, x, ids, w, gate)
        moe.encode_residency_classification(ids, 0, slots)

    def experts():
        moe.encode_prefill(pool, off, ids, slots, w, x, y, None, shared, gate)

    def step():
        route()
        experts()

    def step_e2e():
        x.copy_(x_host, non_blocking=True)
        step()
        y_host.copy_(y, non_blocking=True)

    def timed(fn, steps, warm):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    sampler = ClockSampler(local_rank)
    sampler.start()
    ms = timed(step, K, W)
    ms_experts = timed(experts, K, 2)
    ms_e2e = timed(step_e2e, K, 2)
    clocks = sampler.stop()
    moe.status()
    counts = torch.bincount(ids.flatten().long(), minlength=cfg.num_experts).cpu().numpy()
    flops = 6.0 * cfg.d * cfg.f * T * cfg.top_k + 6.0 * cfg.d * cfg.shared_f * T
    peak = 1590.0
    src = "fallback (1.59 PFLOP/s)"
    pk = ROOT / "MEASURED_PEAKS.json"
    if pk.exists():
        peak = float(json.loads(pk.read_text())["bf16_tflops"])
        src = "measured (MEASURED_PEAKS.json bf16_tflops, burst)"
    tf = flops / (ms_experts * 1e-3) / 1e12
    line = {
        "metric": METRIC, "value": T / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int4 weights dequantised to fp16 operands, fp32 accumulate (TMEM)", "data": "synthetic",
        "config": {"workload": f"ragged prefill, one qwen3.5-35b-a3b-shape int4 layer, {T} rows, top-8 of 256, "
                               "Zipf(1.1) prior on the router logits, gated shared expert",
                   "rows_per_expert_max": int(counts.max()), "rows_per_expert_median": float(np.median(counts)),
                   "experts_hit": int((counts > 0).sum()),
                   "l2": "inputs larger than L2: 453 MB of expert blocks + 268 MB of per-pair rows per step"},
        "roofline": {"bound": "tensor", "kernel": "umma_expert_kernel<4,64,bf16,{0,1}> (+ plan, combine)",
                     "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak, "peak_source": src,
                     "traffic": None, "algorithmic_flops": flops, "ms_experts": ms_experts},
        "e2e": {"value": T / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": T * cfg.d * 2, "d2h_bytes_per_step": T * cfg.d * 2},
        "gpu_launches": K * 12, "clocks": clocks,
    }
    pool.close()
    moe.close()
    return line



def run_gptoss(args, local_rank: int):
    """gpt-oss-20B-shape layers (D = F = 2880, 32 experts top-4, int4 g32, additive biases, clamped SwiGLU, no
    shared expert) at --tokens rows (1 or 64): 8 independently seeded layers chained like the decode sweep, so
    every layer call streams its own cold expert blocks."""
    import torch
    import fixtures as fx
    T, L, K, W = args.tokens, min(args.layers, 8), args.steps, max(3, args.warmup)
    cfg = fx.gpt_oss_config(max_tokens=128)
    wl = Workload(T, L, local_rank, cfg)
    g_step = wl.capture(wl.step_resident)
    g_e2e = wl.capture(wl.step_e2e)
    sampler = ClockSampler(local_rank)
    sampler.start()
    ms = wl.time_graph(g_step, K, W)
    ms_e2e = wl.time_graph(g_e2e, K, W)
    clocks = sampler.stop()
    wl.check_status()
    distinct = wl.distinct_experts()
    mean_units = sum(distinct) / L
    peak, peak_src = measured_peaks()
    gbs = mean_units * wl.block_bytes / (ms / L * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": T / (ms / 1e3) , "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int4 weights x fp16 operands, fp32 accumulate", "data": "synthetic",
        "config": {"workload": f"gpt-oss-20b expert shape, {L} chained layers, batch {T} (D 2880, F 2880, 32 experts top-4, "
                               "int4 g32, bf16 additive biases, clamped SwiGLU)",
                   "layers": L, "distinct_experts_per_layer": mean_units,
                   "l2": f"inputs larger than L2: {mean_units * L * wl.block_bytes / 1e6:.0f} MB of distinct expert "
                         "blocks per step"},
        "roofline": {"bound": "hbm", "kernel": "whole layer call (one row: route + phase 1 + phase 2; more than 16 rows: router + expert-grouped tcgen05 path)", "achieved": gbs, "peak": peak,
                     "unit": "GB/s", "frac": gbs / peak, "peak_source": peak_src, "traffic": None,
                     "us_per_layer": ms / L * 1e3},
        "e2e": {"value": T / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": wl.x_host.numel() * 2, "d2h_bytes_per_step": wl.out_host.numel() * 2},
        "gpu_launches": (K + W) * wl.launches_per_step, "clocks": clocks,
    }
    wl.close()
    return line


def run_ep(args, rank: int, world: int, local_rank: int):
    """Expert-parallel Kimi-Linear-shape layer (int8 g64, 256 experts top-8 sigmoid, shared expert): every rank
    holds 256/N experts and its own mixed batch of 16 decode rows + one 2048-row prefill chunk; rows are
    dispatched and combined with all-to-all over NCCL. Weak scaling: N x 2064 rows per step."""
    import torch
    import torch.distributed as dist
    from shrike_b200 import capi
    import fixtures as fx
    from shrike_b200.ep import ExpertParallelLayer
    from shrike_b200.moe import RouterOperands, expert_offsets

    rows, K, W = 16 + 2048, args.steps, max(3, args.warmup)
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    cfg = fx.kimi_config(max_tokens=rows)
    group = None
    layer = ExpertParallelLayer(cfg, rank, world, local_rank, rows, group)
    layer.pool.fill_synthetic(0, layer.epr, SEED, 0, first_expert=layer.lo)
    soff, sbytes = expert_offsets(cfg, shared=True)
    sh = torch.from_numpy(fx.synth_block(cfg, SEED, 0, 100000, shared=True).copy()).to(dev)
    layer.set_shared(capi.SharedExpert(sh.data_ptr(), soff))
    sys.path.insert(0, str(ROOT / "tests"))
    from gpu_harness import bf16_tensor
    correction = np.random.default_rng(SEED + 7).uniform(-0.1, 0.1, cfg.num_experts).astype(np.float32)
    ops = RouterOperands(weights=torch.from_numpy(router_weights(0, cfg.num_experts, cfg.d)).to(dev),
                         logit_bias=bf16_tensor(correction, dev))
    # every rank routes its own rows
    xr = np.random.default_rng(SEED + 1000 + rank).normal(0, 1, (rows, cfg.d)).astype(np.float32)
    x_host = torch.from_numpy(xr).to(torch.bfloat16).pin_memory()
    y_host = torch.empty_like(x_host).pin_memory()
    x = x_host.to(dev)
    y = torch.empty_like(x)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    def step():
        layer.forward(ops, x, y)

    def step_e2e():
        x.copy_(x_host, non_blocking=True)
        layer.forward(ops, x, y)
        y_host.copy_(y, non_blocking=True)

    for _ in range(W):
        step()
    layer.home.status()
    layer.routed.status()
    sampler = ClockSampler(local_rank)
    sampler.start()
    ms = timed(step, K)
    clocks = sampler.stop()
    ms_e2e = timed(step_e2e, K)
    sent = int(layer.send_counts.sum().item())
    line = {
        "metric": METRIC, "value": world * rows * K / (ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": K,
        "warmup": W, "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 weights dequantised to fp16 operands, fp32 accumulate (TMEM)", "data": "synthetic",
        "config": {"workload": "kimi-linear-48b-shape layer, expert parallel: 256 experts top-8 sigmoid + shared "
                               "expert, D 2304, F 1024, int8 g64; 16 decode rows + one 2048-row prefill chunk per "
                               "rank; all-to-all dispatch and combine over NCCL",
                   "rows_per_rank": rows, "experts_per_rank": layer.epr, "parallelism": f"ep{world}",
                   "rows_sent_by_rank0": sent,
                   "l2": f"inputs larger than L2: {layer.epr * layer.block_bytes / 1e6:.0f} MB of expert blocks per rank"},
        "e2e": {"value": world * rows * K / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e / K,
                "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": y_host.numel() * 2},
        "gpu_launches": None, "clocks": clocks,
    }
    layer.close()
    return line


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if rank != 0:
            return
        budget = 120.0
        r = cpu_reference_run(args.tokens, args.layers, args.steps, args.warmup, budget)
        print(json.dumps({
            "impl": "reference", "metric": METRIC, "value": r["value"], "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": r["steps"], "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "int4 weights, fp32 arithmetic", "data": "synthetic",
            "config": {"workload": f"qwen3.5-35b-a3b expert shape, {args.layers}-layer decode sweep, batch {args.tokens}, "
                                   "CPU path on the host cores"},
            "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": r["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }))
        return

    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU path in this library); "
                         "use --impl reference for the CPU arm")
    if args.workload == "prefill":
        if rank == 0:
            print(json.dumps(run_prefill(args, local_rank)))
        return
    if args.workload == "gptoss":
        if rank == 0:
            print(json.dumps(run_gptoss(args, local_rank)))
        return
    if args.workload == "ep":
        import torch.distributed as dist
        if world > 1:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        line = run_ep(args, rank, world, local_rank)
        if rank == 0:
            print(json.dumps(line))
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    line = run_ours(args, rank, world, local_rank)
    if rank == 0:
        if world == 1 and not args.no_sweep and args.tokens == 1:
            sweep = {}
            for T in (4, 16):
                a2 = argparse.Namespace(**vars(args))
                a2.tokens, a2.steps = T, max(10, args.steps // 2)
                l2 = run_ours(a2, 0, 1, local_rank)
                sweep[f"batch_{T}"] = {"tokens_per_s": l2["value"], "ms_per_step": l2["ms_per_step"],
                                       "hbm_gbs_per_layer": l2["hbm_gbs_per_layer"],
                                       "distinct_experts_per_layer": l2["distinct_experts_per_layer"],
                                       "phase1_gbs": l2["roofline"]["achieved"], "phase1_frac": l2["roofline"]["frac"],
                                       "phase2_gbs": l2["roofline"]["phase2"]["achieved"]}
            line["sweep"] = sweep
        if world == 1 and not args.no_cpu_baseline:
            r = cpu_reference_run(args.tokens, args.layers, 1000, 2, 15.0)
            line["cpu_baseline"] = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
