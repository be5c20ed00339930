#!/usr/bin/env python
"""Headline benchmark: MoE-FFN tokens/s and HBM GB/s, Qwen3.5-35B-A3B expert shape,
40 stacked MoE layers with all 40 x 256 experts resident in the HBM slot pool.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--tokens T] [--impl ours|reference]

A step is one pass of T tokens (default 1) through all layers: router -> top-8 ->
residency lookup -> shared + routed expert FFN -> combine; the output joins the residual stream that feeds the
next layer (stream_rows). Prints ONE JSON line.

N = 1: the line also carries compact blocks for the other workloads -- `sweep` (batch 4 and 16),
`prefill` (4096 ragged rows on the tensor cores), `gptoss` (1 and 64 rows) -- and the CPU baseline.
N > 1 (torchrun): `value` is N independent replicas of the decode sweep (the single-GPU workloads do
not shard; no collective on their data path), and the `ep` block is the expert-parallel workload
(Kimi-Linear shape, experts sharded over the N ranks, rows dispatched and combined over NVLink)
measured in the same job, with the same rank's one-GPU time measured first.
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
# dram__bytes_read.sum + dram__bytes_write.sum of one decode_layer_kernel launch over its algorithmic bytes,
# from an ncu capture of the layer kernel on 8 layers: 18.15 MB of DRAM reads per launch, no writes
TRAFFIC_RATIO = 1.14   # DRAM bytes per launch over the algorithmic bytes (15.93 MB of expert blocks + 2.1 MB of fp32 router rows)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--tokens", type=int, default=1, help="decode batch: 1, 4 or 16")
    ap.add_argument("--layers", type=int, default=LAYERS)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=["all", "decode", "prefill", "ep", "gptoss"], default="all",
                    help="all: the headline decode sweep plus the compact blocks of the other workloads; "
                         "one name: that workload alone (decode = the headline line without the extra blocks)")
    ap.add_argument("--rows", type=int, default=4096, help="rows of the prefill workload")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    return ap.parse_args()


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured (MEASURED_PEAKS.json: hbm_gbs, bf16_tflops burst)"
    return 6650.0, 1590.0, "fallback (6.65 TB/s, 1.59 PFLOP/s: earlier measurements on this pool)"


def router_weights(layer: int, ne: int, d: int) -> np.ndarray:
    return np.random.default_rng(SEED * 1000 + layer).normal(0, 0.02, (ne, d)).astype(np.float32)


def gate_weights(layer: int, d: int) -> np.ndarray:
    return np.random.default_rng(SEED * 1000 + 500 + layer).normal(0, 0.02, d).astype(np.float32)


def input_tokens(T: int, d: int, seed: int = SEED) -> np.ndarray:
    import fixtures as fx
    return fx.round_bf16(np.random.default_rng(seed).normal(0, 1, (T, d)).astype(np.float32))


def stream_rows(L: int, T: int, d: int) -> np.ndarray:
    """The residual stream of the stacked workload, [(L + 1) x T x d] bf16 N(0,1): block 0 enters layer 0, block
    l stands for what the rest of transformer block l (attention + normalisation, not part of this path) adds
    between MoE layer l-1 and MoE layer l. Layer l's input is block l + y of layer l-1, so every layer's routing
    depends on the layer before it, and the stream keeps unit scale (fed back unnormalised, the quadratic
    SwiGLU of 40 synthetic layers overflows fp16 within 8 layers)."""
    return np.stack([input_tokens(T, d, SEED + 17 * l) for l in range(L + 1)])


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
    import oracle_lib as O
    import fixtures as fx

    cfg = fx.qwen_config(max_tokens=16)
    kind = "reference" if O.use_reference_gemv(True) else "port"
    cores = os.cpu_count() or 1
    ecfg = O.expert_cfg(cfg.d, cfg.f)
    lcfg = O.layer_cfg(ecfg, O.expert_cfg(cfg.d, cfg.shared_f), True)
    rows = stream_rows(layers, T, cfg.d)
    routers = [router_weights(l, cfg.num_experts, cfg.d) for l in range(layers)]
    gates = [gate_weights(l, cfg.d) for l in range(layers)]
    shared = [O.synth_block(O.expert_cfg(cfg.d, cfg.shared_f), SEED, l, 100000) for l in range(layers)]
    cache: dict = {}

    def block(l, e):
        if (l, e) not in cache:
            cache[(l, e)] = O.synth_block(ecfg, SEED, l, e)
        return cache[(l, e)]

    def step():
        h = rows[0].copy()
        for l in range(layers):
            ids = np.zeros((T, cfg.top_k), np.uint32)
            w = np.zeros((T, cfg.top_k), np.float32)
            for t in range(T):
                ids[t], w[t] = O.router_select(O.router_logits_f32(routers[l], h[t]), cfg.top_k, round_f16=True)
            blocks = {int(e): block(l, int(e)) for e in np.unique(ids)}
            y = O.moe_layer(lcfg, blocks, shared[l], gates[l], h, ids, w, threads=cores)
            h = fx.round_bf16(rows[l + 1] + y)
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
    tasks = T * cfg.top_k + T
    return {"value": T / (ms / 1e3), "unit": "tokens/s", "cores": cores, "kind": kind,
            "sample": f"{len(times)} steps of {T} token(s) x {layers} layers (router + 8 routed + 1 shared expert per layer); "
                      f"one thread per expert task: {min(tasks, cores)} of {cores} host threads busy, "
                      f"{max(0, cores - tasks)} idle", "ms_per_step": ms, "steps": len(times)}


# ------------------------------------------------------------------ the decode stack

class Workload:
    """All layers resident on one GPU; per-layer handles so that every layer keeps its own work lists."""

    def __init__(self, T: int, layers: int, device_index: int, cfg=None):
        import torch
        from shrike_b200 import capi
        import fixtures as fx
        from shrike_b200.moe import DecodeStack, ExpertCellArena, MoE, RouterOperands, expert_offsets, round_up

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
        self.w = [torch.zeros((T, k), dtype=torch.float32, device=self.dev) for _ in range(layers)]
        self.rows_host = torch.from_numpy(stream_rows(layers, T, cfg.d)).to(torch.bfloat16).pin_memory()
        self.out_host = torch.empty((T, cfg.d), dtype=torch.bfloat16).pin_memory()
        self.rows0 = self.rows_host.to(self.dev)
        self.stream = torch.zeros_like(self.rows0)
        self.y = torch.zeros((T, cfg.d), dtype=cfg.torch_y_dtype, device=self.dev)
        self.stack = DecodeStack([(self.moes[l], self.pool, self.off, 0, self.routers[l], self.shared[l])
                                  for l in range(layers)], T)
        # kernels of this library per layer call: one row = the single fused launch; up to 16 rows = route +
        # phase 1 + phase 2; more (on a handle that owns the prefill operands) = the expert-grouped path
        self.launches_per_step = layers * (1 if T == 1 else 3 if T <= 16 else 14)
        torch.cuda.synchronize()

    def step_resident(self):
        """Inputs already in HBM: one device copy re-arms the residual stream, then every layer call."""
        self.stream.copy_(self.rows0)
        for l in range(self.L):
            self.moes[l].encode_decode_layer(self.pool, self.off, 0, self.routers[l], self.stream[l], self.y,
                                             self.stream[l + 1], self.shared[l], self.ids[l], self.w[l])

    def step_host(self):
        """One step through the C-ABI entry point for host buffers: H2D of the rows, every layer, D2H, sync."""
        self.stack.forward_host(self.rows_host, self.out_host)

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

    def time_host(self, steps: int, warmup: int) -> float:
        """Mean ms per host-buffer step (every call ends with a stream synchronise)."""
        for _ in range(warmup):
            self.step_host()
        t0 = time.perf_counter()
        for _ in range(steps):
            self.step_host()
        return 1e3 * (time.perf_counter() - t0) / steps

    def distinct_experts(self):
        return [int(self.torch.unique(self.ids[l]).numel()) for l in range(self.L)]

    def check_status(self):
        for m in self.moes:
            m.status()

    def close(self):
        self.stack.close()
        self.pool.close()
        for m in self.moes:
            m.close()


def run_decode(T: int, L: int, K: int, W: int, rank: int, world: int, local_rank: int, cfg=None):
    """The stacked decode sweep on this rank's GPU: (ms per device-resident step, ms per host-buffer step,
    bytes of distinct expert blocks a layer streams, the workload)."""
    import torch
    import torch.distributed as dist
    wl = Workload(T, L, local_rank, cfg)
    g_step = wl.capture(wl.step_resident)
    wl.check_status()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    barrier()
    ms = wl.time_graph(g_step, K, W)
    barrier()
    ms_host = wl.time_host(K, W)
    barrier()
    if world > 1:
        t = torch.tensor([ms, ms_host], dtype=torch.float64, device=wl.dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_host = float(t[0]), float(t[1])
    wl.check_status()
    units = [u + (1 if wl.cfg.has_shared else 0) for u in wl.distinct_experts()]
    return ms, ms_host, sum(units) / L * wl.block_bytes, wl


def decode_line(args, rank: int, world: int, local_rank: int):
    T, L, K, W = args.tokens, args.layers, args.steps, max(3, args.warmup)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms, ms_host, layer_bytes, wl = run_decode(T, L, K, W, rank, world, local_rank)
    clocks = sampler.stop() if rank == 0 else None
    cfg = wl.cfg
    hbm, _, src = measured_peaks()
    gbs = layer_bytes / (ms / L * 1e-3) / 1e9
    kernel = ("decode_layer_kernel<4,64,bf16> (router + top-8 + lookup + gate/up + GLU + down + combine of one row, one launch)"
              if T == 1 else "route_fused_kernel + phase1_kernel<4,64,bf16> + phase2_kernel<4,64,bf16>")
    line = None
    if rank == 0:
        tokens = T * world
        line = {
            "metric": METRIC, "value": tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int4 weights x fp16 operands, fp32 accumulate; bf16 x in, fp32 y out", "data": "synthetic",
            "config": {
                "workload": f"qwen3.5-35b-a3b expert shape, {L}-layer decode sweep, batch {T} "
                            f"(D 2048, 256 experts top-8 + gated shared, F 512, int4 g64 bf16 meta)",
                "tokens_per_step_per_gpu": T, "layers": L, "parallelism": "replicas" if world > 1 else "single",
                "l2": f"inputs larger than L2: every step streams {layer_bytes * L / 1e6:.0f} MB of distinct expert "
                      "blocks (L2 126 MB)",
                "stream": "layer l's input = seeded N(0,1) row l (standing for attention + norm) + y of layer l-1",
                "launch": "one stream per GPU, SHRIKE_SINGLE_STREAM=1 (no cooperative launch; the library's default is cooperative)"
                          if os.environ.get("SHRIKE_SINGLE_STREAM") else "cooperative",
                "pool_gb": round(wl.pool.cells * wl.pool.cell_stride / 1e9, 2),
            },
            "roofline": {"bound": "hbm", "kernel": kernel, "achieved": gbs, "peak": hbm, "unit": "GB/s",
                         "frac": gbs / hbm, "whole_layer_frac": gbs / hbm, "peak_source": src,
                         "traffic": layer_bytes * TRAFFIC_RATIO if (TRAFFIC_RATIO and T == 1) else None,
                         "algorithmic_bytes_per_launch": layer_bytes, "us_per_launch": ms / L * 1e3,
                         "note": "a launch is a whole layer; its time is the step's CUDA-event time / layers, "
                                 "launch hand-over included"},
            "e2e": {"value": tokens / (ms_host * 1e-3), "unit": "tokens/s", "ms_per_step": ms_host,
                    "h2d_bytes_per_step": (L + 1) * T * cfg.d * 2, "d2h_bytes_per_step": T * cfg.d * 2,
                    "api": "shrike_decode_stack_forward_host (pinned host rows in, every layer call, host rows out, sync)"},
            "gpu_launches": wl.launches_per_step * K,
            "distinct_experts_per_layer": layer_bytes / wl.block_bytes - 1,
            "clocks": clocks,
        }
    wl.close()
    return line


# ------------------------------------------------------------------ compact blocks of the other workloads

def sweep_block(args, local_rank: int) -> dict:
    out = {}
    hbm, _, _ = measured_peaks()
    for T in (4, 16):
        K = max(10, args.steps // 4)
        ms, ms_host, layer_bytes, wl = run_decode(T, args.layers, K, 3, 0, 1, local_rank)
        L = args.layers
        gbs = layer_bytes / (ms / L * 1e-3) / 1e9
        out[f"batch_{T}"] = {"tokens_per_s": round(T / (ms * 1e-3), 1), "e2e_tokens_per_s": round(T / (ms_host * 1e-3), 1),
                             "us_per_layer": round(ms / L * 1e3, 2), "hbm_gbs": round(gbs, 1), "frac": round(gbs / hbm, 4),
                             "distinct_experts_per_layer": round(layer_bytes / wl.block_bytes - 1, 1)}
        wl.close()
    return out


def prefill_block(args, local_rank: int) -> dict:
    """Ragged prefill through one Qwen-shape int4 layer: rows routed top-8 of 256 with a Zipf(1.1) prior on the
    expert ids, permuted by expert on the device, expert-grouped GEMM on the tcgen05 tensor cores."""
    import torch
    from shrike_b200 import capi
    import fixtures as fx
    from shrike_b200.moe import ExpertCellArena, MoE, RouterOperands, expert_offsets, round_up
    from gpu_harness import bf16_tensor

    T, K, W = args.rows, max(10, args.steps // 4), 3
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
    y_host = torch.empty(x_host.shape, dtype=cfg.torch_y_dtype).pin_memory()
    x = x_host.to(dev)
    y = torch.empty(x.shape, dtype=cfg.torch_y_dtype, device=dev)
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

    ms = timed(step, K, W)
    ms_router = timed(route, K, 2)
    ms_experts = timed(experts, K, 2)
    # end to end through the host-buffer entry point: H2D of the rows, router, classification, experts, D2H, sync
    for _ in range(2):
        moe.layer_forward_host(pool, off, 0, ops, x_host, y_host, shared)
    t0 = time.perf_counter()
    for _ in range(K):
        moe.layer_forward_host(pool, off, 0, ops, x_host, y_host, shared)
    ms_e2e = 1e3 * (time.perf_counter() - t0) / K
    moe.status()
    counts = torch.bincount(ids.flatten().long(), minlength=cfg.num_experts).cpu().numpy()
    flops = 6.0 * cfg.d * cfg.f * T * cfg.top_k + 6.0 * cfg.d * cfg.shared_f * T
    _, peak, src = measured_peaks()
    tf = flops / (ms_experts * 1e-3) / 1e12
    out = {"workload": f"ragged prefill, one qwen-shape int4 layer, {T} rows, top-8 of 256, Zipf(1.1) router prior",
           "rows_per_s": round(T / (ms * 1e-3)), "ms_per_step": round(ms, 4), "ms_router": round(ms_router, 4),
           "ms_experts": round(ms_experts, 4), "tflops": round(tf, 1), "peak_tflops": peak, "frac": round(tf / peak, 4),
           "bound": "tensor", "kernel": "umma_expert_kernel<4,64,bf16,{0,1}> (+ plan, combine)",
           "e2e_rows_per_s": round(T / (ms_e2e * 1e-3)), "h2d_bytes": T * cfg.d * 2, "d2h_bytes": T * cfg.d * 4,
           "experts_hit": int((counts > 0).sum()), "rows_per_expert_max": int(counts.max())}
    pool.close()
    moe.close()
    return out


def gptoss_block(args, local_rank: int) -> dict:
    """gpt-oss-20B-shape layers (D = F = 2880, 32 experts top-4, int4 g32, additive biases, clamped SwiGLU, no
    shared expert) at 1 and 64 rows: 8 independently seeded layers chained like the decode sweep."""
    import fixtures as fx
    hbm, _, _ = measured_peaks()
    out = {"workload": "gpt-oss-20b expert shape, 8 chained layers (D 2880, F 2880, 32 experts top-4, int4 g32, "
                       "bf16 additive biases, clamped SwiGLU)"}
    for T in (1, 64):
        cfg = fx.gpt_oss_config(max_tokens=128)
        K = max(10, args.steps // 4)
        ms, ms_host, layer_bytes, wl = run_decode(T, 8, K, 3, 0, 1, local_rank, cfg)
        gbs = layer_bytes / (ms / 8 * 1e-3) / 1e9
        out[f"rows_{T}"] = {"tokens_per_s": round(T / (ms * 1e-3), 1), "e2e_tokens_per_s": round(T / (ms_host * 1e-3), 1),
                            "us_per_layer": round(ms / 8 * 1e3, 2), "hbm_gbs": round(gbs, 1), "frac": round(gbs / hbm, 4),
                            "distinct_experts_per_layer": round(layer_bytes / wl.block_bytes, 1)}
        wl.close()
    return out


def ep_block(args, rank: int, world: int, local_rank: int) -> dict:
    """Expert-parallel Kimi-Linear-shape layer (int8 g64, 256 experts top-8 sigmoid, shared expert): every rank
    brings its own mixed batch of 16 decode rows + one 2048-row prefill chunk (weak scaling: N x 2064 rows per
    step). Measured twice in this process: with all 256 experts on this rank alone (world 1, no exchange), then
    with the experts sharded over the N ranks and the rows dispatched and combined over NVLink."""
    import torch
    import torch.distributed as dist
    from shrike_b200 import capi
    import fixtures as fx
    from shrike_b200.ep import ExpertParallelLayer
    from shrike_b200.moe import RouterOperands, expert_offsets
    from gpu_harness import bf16_tensor

    rows, K, W = 16 + 2048, max(10, args.steps // 4), 3
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    cfg = fx.kimi_config(max_tokens=rows)
    soff, _ = expert_offsets(cfg, shared=True)
    sh = torch.from_numpy(fx.synth_block(cfg, SEED, 0, 100000, shared=True).copy()).to(dev)
    correction = np.random.default_rng(SEED + 7).uniform(-0.1, 0.1, cfg.num_experts).astype(np.float32)
    ops = RouterOperands(weights=torch.from_numpy(router_weights(0, cfg.num_experts, cfg.d)).to(dev),
                         logit_bias=bf16_tensor(correction, dev))
    xr = input_tokens(rows, cfg.d, SEED + 1000 + rank)
    x = torch.from_numpy(xr).to(torch.bfloat16).to(dev)
    y = torch.empty(x.shape, dtype=cfg.torch_y_dtype, device=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def measure(layer):
        for _ in range(W):
            layer.forward(ops, x, y)
        layer.status()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(K):
            layer.forward(ops, x, y)
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1) / K], dtype=torch.float64, device=dev)
        if layer.world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        layer.status()
        return float(ms.item())

    def build(r, n):
        layer = ExpertParallelLayer(cfg, r, n, local_rank, rows)
        layer.pool.fill_synthetic(0, layer.epr, SEED, 0, first_expert=layer.lo)
        layer.set_shared(capi.SharedExpert(sh.data_ptr(), soff))
        return layer

    single = build(0, 1)
    ms1 = measure(single)
    single.close()
    layer = build(rank, world)
    ms_n = measure(layer)
    stats = layer.exchange_stats(ops, x, y, K)
    # parity of this rank's rows against the CPU oracle on a seeded sample (rank 0 only; the oracle is the checker)
    parity = None
    if rank == 0:
        import oracle_lib as O
        sample = np.sort(np.random.default_rng(3).choice(rows, 48, replace=False))
        layer.forward(ops, x, y)
        torch.cuda.synchronize()
        got = y.float().cpu().numpy()[sample]
        ids_d, w_d = layer.routing(ops, x)
        ids = ids_d.cpu().numpy().astype(np.uint32)[sample]
        wts = w_d.cpu().numpy()[sample]
        ecfg = O.expert_cfg(cfg.d, cfg.f, bits=8)
        lcfg = O.layer_cfg(ecfg, O.expert_cfg(cfg.d, cfg.shared_f, bits=8), False)
        blocks = {int(e): fx.synth_block(cfg, SEED, 0, int(e)) for e in np.unique(ids)}
        ref = O.moe_layer(lcfg, blocks, fx.synth_block(cfg, SEED, 0, 100000, shared=True), None, xr[sample], ids, wts,
                          threads=os.cpu_count() or 8)
        parity = float(np.linalg.norm(got - ref) / np.linalg.norm(ref))
    recv = torch.tensor([stats["rows_received"]], dtype=torch.float64, device=dev)
    recv_max, recv_sum = recv.clone(), recv.clone()
    if world > 1:
        dist.all_reduce(recv_max, op=dist.ReduceOp.MAX)
        dist.all_reduce(recv_sum, op=dist.ReduceOp.SUM)
    layer.close()
    rows_s_1, rows_s_n = rows / (ms1 * 1e-3), world * rows / (ms_n * 1e-3)
    return {"workload": "kimi-linear-48b-shape layer, expert parallel: 256 experts top-8 sigmoid + shared expert, D 2304, "
                        "F 1024, int8 g64; 16 decode rows + one 2048-row prefill chunk per rank",
            "world": world, "rows_per_rank": rows, "rows_per_s": round(rows_s_n), "ms_per_step": round(ms_n, 4),
            "rows_per_s_one_gpu": round(rows_s_1), "ms_per_step_one_gpu": round(ms1, 4),
            "efficiency": round(rows_s_n / (world * rows_s_1), 4),
            # the exchange is fused into the layer (rows stored into the peers' buffers by the dispatch kernels, partial
            # rows returned by the combine of the local call): what it and the imbalance between ranks cost is the
            # step's time over the same rank's one-GPU step on the same rows
            "ms_exchange_and_imbalance": round(ms_n - ms1, 4),
            "bytes_sent_per_rank": stats["bytes_sent"], "rows_received_max_over_mean": round(
                float(recv_max.item()) / (float(recv_sum.item()) / world), 4),
            "exchange": stats["exchange"], "parity_rel_l2": parity}


def main():
    args = parse_args()
    # The benchmark drives one stream per GPU: the one-launch decode layer may give up its cooperative launch
    # (read once, when a handle is created), which lets a layer's prologue overlap the previous layer's tail.
    os.environ.setdefault("SHRIKE_SINGLE_STREAM", "1")
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if rank != 0:
            return
        r = cpu_reference_run(args.tokens, args.layers, args.steps, args.warmup, 120.0)
        print(json.dumps({
            "impl": "reference", "metric": METRIC, "value": r["value"], "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": r["steps"], "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "int4 weights, fp32 arithmetic", "data": "synthetic",
            "config": {"workload": f"qwen3.5-35b-a3b expert shape, {args.layers}-layer decode sweep, batch {args.tokens} "
                                   "(D 2048, 256 experts top-8 + gated shared, F 512, int4 g64 bf16 meta)",
                       "arm": "the reference's CPU path on the host cores"},
            "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": r["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }))
        return

    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU path in this library); "
                         "use --impl reference for the CPU arm")
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    only = args.workload
    line = None
    if only in ("all", "decode"):
        line = decode_line(args, rank, world, local_rank)
    if world == 1:
        blocks = {}
        if only == "all" and args.tokens == 1:
            blocks["sweep"] = sweep_block(args, local_rank)
        if only in ("all", "prefill"):
            blocks["prefill"] = prefill_block(args, local_rank)
        if only in ("all", "gptoss"):
            blocks["gptoss"] = gptoss_block(args, local_rank)
        if only == "ep":
            blocks["ep"] = ep_block(args, 0, 1, local_rank)
        if line is None:
            line = {"metric": METRIC, "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup)}
        line.update(blocks)
        if only in ("all", "decode") and not args.no_cpu_baseline:
            r = cpu_reference_run(args.tokens, args.layers, 1000, 2, 15.0)
            line["cpu_baseline"] = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")}
    else:
        if only in ("all", "ep"):
            ep = ep_block(args, rank, world, local_rank)
            if rank == 0:
                if line is None:
                    line = {"metric": METRIC, "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup)}
                line["ep"] = ep
    if rank == 0 and line is not None:
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
