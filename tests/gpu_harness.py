"""Builds one synthetic MoE layer on the device through the C ABI and the same
layer for the CPU oracle, so that parity tests read: run both, compare."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np
import torch

import oracle_lib as O
from shrike_b200 import capi
import fixtures as fx
from shrike_b200.moe import ExpertCellArena, MoE, MoEConfig, RouterOperands, expert_offsets, round_up


def rel_l2(a: np.ndarray, b: np.ndarray) -> float:
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def to_act_tensor(x: np.ndarray, act_dtype: int, device) -> torch.Tensor:
    t = torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32))
    return t.to(device=device, dtype={capi.DTYPE_BF16: torch.bfloat16, capi.DTYPE_FP16: torch.float16,
                                      capi.DTYPE_FP32: torch.float32}[act_dtype]).contiguous()


def bf16_tensor(values: np.ndarray, device) -> torch.Tensor:
    """bf16 operand vector (bit patterns in an int16 tensor)."""
    return torch.from_numpy(fx.bf16_bits(values).view(np.int16).copy()).to(device)


def oracle_expert_cfg(cfg: MoEConfig, shared: bool = False) -> O.ExpertCfg:
    return O.expert_cfg(cfg.d, cfg.shared_f if shared else cfg.f, cfg.weight_bits, cfg.group_size, cfg.meta_dtype,
                        cfg.activation, cfg.expert_bias)


class Layer:
    """One layer: `num_experts` blocks in pool cells [first_cell, ...), optional shared expert, router."""

    def __init__(self, cfg: MoEConfig, seed: int = 1, device_fill: bool = False, layer: int = 0,
                 first_cell: int = 0, extra_cells: int = 0, chunks: int = 1, logit_bias: np.ndarray | None = None,
                 per_expert_scale: np.ndarray | None = None, router_sigma: float = 0.02):
        self.cfg = cfg
        self.seed = seed
        self.layer = layer
        self.first_cell = first_cell
        self.device = torch.device("cuda:0")
        self.moe = MoE(cfg)
        self.offsets, self.block_bytes = expert_offsets(cfg)
        stride = round_up(self.block_bytes, 256)
        self.pool = ExpertCellArena(self.moe, first_cell + cfg.num_experts + extra_cells, stride, chunks)
        self._blocks: dict[int, np.ndarray] = {}
        self.device_fill = device_fill
        if device_fill:
            self.pool.fill_synthetic(first_cell, cfg.num_experts, seed, layer)
        else:
            for e in range(cfg.num_experts):
                self.pool.upload(first_cell + e, self.block(e))
        self.moe.create_residency(layer + 1)
        self.moe.residency_set_layer_identity(layer, first_cell)
        self.shared = None
        self.shared_block_host = None
        if cfg.has_shared:
            so, sbytes = expert_offsets(cfg, shared=True)
            self.shared_block_host = fx.synth_block(cfg, seed, layer, 100000, shared=True)
            assert self.shared_block_host.nbytes == sbytes
            self._shared_dev = torch.from_numpy(self.shared_block_host.copy()).to(self.device)
            self.shared = capi.SharedExpert(self._shared_dev.data_ptr(), so)
        rng = np.random.default_rng(seed * 7919 + layer)
        self.router_w = rng.normal(0, router_sigma, (cfg.num_experts, cfg.d)).astype(np.float32)
        self.gate_w = rng.normal(0, 0.02, cfg.d).astype(np.float32) if cfg.shared_gated else None
        self.logit_bias = None if logit_bias is None else fx.round_bf16(logit_bias)
        self.per_expert_scale = None if per_expert_scale is None else fx.round_bf16(per_expert_scale)
        self.router_packed = None
        if cfg.router_weight_bits:
            self.router_packed = fx.quantize_affine(self.router_w, cfg.router_weight_bits)
            self._rw = torch.from_numpy(self.router_packed[0].copy()).to(self.device)
            self._rs = torch.from_numpy(self.router_packed[1].view(np.int16).copy()).to(self.device)
            self._rb = torch.from_numpy(self.router_packed[2].view(np.int16).copy()).to(self.device)
        else:
            self._rw = torch.from_numpy(self.router_w).to(self.device)
            self._rs = self._rb = None
        self.router_ops = RouterOperands(
            weights=self._rw, scales=self._rs, biases=self._rb,
            logit_bias=None if self.logit_bias is None else bf16_tensor(self.logit_bias, self.device),
            per_expert_scale=None if self.per_expert_scale is None else bf16_tensor(self.per_expert_scale, self.device),
            shared_gate=None if self.gate_w is None else torch.from_numpy(self.gate_w).to(self.device))
        torch.cuda.synchronize()

    def close(self):
        self.pool.close()
        self.moe.close()

    # -- host copies of the blocks -------------------------------------------
    def block(self, e: int) -> np.ndarray:
        if e not in self._blocks:
            self._blocks[e] = fx.synth_block(self.cfg, self.seed, self.layer, e)
        return self._blocks[e]

    # -- device path ----------------------------------------------------------
    def route(self, x_dev: torch.Tensor, stride: int | None = None, rows: int | None = None):
        T = x_dev.shape[0] if rows is None else rows
        k = self.cfg.top_k
        ids = torch.empty((T, k), dtype=torch.int32, device=self.device)
        w = torch.empty((T, k), dtype=torch.float32, device=self.device)
        gate = torch.empty(T, dtype=torch.float32, device=self.device) if self.cfg.shared_gated else None
        self.moe.encode_router(self.router_ops, x_dev, ids, w, gate, query_count=T, hidden_stride_elements=stride)
        return ids, w, gate

    def classify(self, ids: torch.Tensor):
        slots = torch.empty_like(ids)
        counts = torch.zeros(2, dtype=torch.int32, device=self.device)
        self.moe.encode_residency_classification(ids, self.layer, slots, counts)
        return slots, counts

    def forward(self, x: np.ndarray, prefill: bool | None = None, hidden: np.ndarray | None = None,
                io_status: int | None = None, fused: bool = False):
        """router -> classification -> decode/prefill. Returns (y fp32, ids, weights, hidden_out).
        fused=True takes the one-call decode layer (three dependent launches) instead."""
        cfg = self.cfg
        x_dev = to_act_tensor(x, cfg.act_dtype, self.device)
        T = x_dev.shape[0]
        if fused:
            ids = torch.empty((T, cfg.top_k), dtype=torch.int32, device=self.device)
            w = torch.empty((T, cfg.top_k), dtype=torch.float32, device=self.device)
            y = torch.empty(x_dev.shape, dtype=cfg.torch_y_dtype, device=self.device)
            h = None if hidden is None else to_act_tensor(hidden, cfg.act_dtype, self.device)
            st = None if io_status is None else torch.tensor([io_status], dtype=torch.int32, device=self.device)
            self.moe.encode_decode_layer(self.pool, self.offsets, self.layer, self.router_ops, x_dev, y, h,
                                         self.shared, ids, w, st)
            self.moe.status()
            return (y.float().cpu().numpy(), ids.cpu().numpy().astype(np.uint32), w.cpu().numpy(),
                    None if h is None else h.float().cpu().numpy())
        ids, w, gate = self.route(x_dev)
        slots, _ = self.classify(ids)
        y = torch.empty(x_dev.shape, dtype=cfg.torch_y_dtype, device=self.device)
        h = None if hidden is None else to_act_tensor(hidden, cfg.act_dtype, self.device)
        if prefill is None:
            prefill = T > capi.MAX_DECODE_TOKENS
        if prefill:
            self.moe.encode_prefill(self.pool, self.offsets, ids, slots, w, x_dev, y, h, self.shared, gate)
        else:
            st = None if io_status is None else torch.tensor([io_status], dtype=torch.int32, device=self.device)
            self.moe.encode_decode(self.pool, self.offsets, slots, w, x_dev, y, h, self.shared, gate, st)
        self.moe.status()
        return (y.float().cpu().numpy(), ids.cpu().numpy().astype(np.uint32), w.cpu().numpy(),
                None if h is None else h.float().cpu().numpy())

    # -- oracle ------------------------------------------------------------------
    def act_round(self, x: np.ndarray) -> np.ndarray:
        """The values the device sees after x is stored in the activation dtype."""
        x = np.asarray(x, dtype=np.float32)
        if self.cfg.act_dtype == capi.DTYPE_BF16:
            return fx.round_bf16(x)
        if self.cfg.act_dtype == capi.DTYPE_FP16:
            return x.astype(np.float16).astype(np.float32)
        return x

    def oracle_route(self, x: np.ndarray):
        cfg = self.cfg
        xr = self.act_round(x)
        ids = np.zeros((xr.shape[0], cfg.top_k), dtype=np.uint32)
        w = np.zeros((xr.shape[0], cfg.top_k), dtype=np.float32)
        logits_all = []
        for t in range(xr.shape[0]):
            if cfg.router_weight_bits:
                p, s, b = self.router_packed
                logits = O.router_logits_affine(p, s, b, cfg.router_weight_bits, xr[t])
            else:
                logits = O.router_logits_f32(self.router_w, xr[t])
            logits_all.append(logits)
            ids[t], w[t] = O.router_select(logits, cfg.top_k, bias=self.logit_bias,
                                           per_expert_scale=self.per_expert_scale,
                                           sigmoid=cfg.router_kind == capi.ROUTER_SIGMOID,
                                           scaling=cfg.routed_scaling, round_f16=cfg.round_route_weights_f16)
        return ids, w, np.stack(logits_all)

    def oracle_forward(self, x: np.ndarray, ids: np.ndarray | None = None, weights: np.ndarray | None = None,
                       threads: int | None = None, skip_experts: set | None = None, rows: np.ndarray | None = None):
        """The oracle's y for all rows, or for the sample `rows` (full-size workloads: the CPU FFN costs
        about 10 ms per row at the Qwen shape)."""
        cfg = self.cfg
        threads = threads or min(32, os.cpu_count() or 8)
        xr = self.act_round(x)
        if ids is None:
            ids, weights, _ = self.oracle_route(x)
        weights = np.array(weights, dtype=np.float32)
        if rows is not None:
            xr, ids, weights = xr[rows], ids[rows], weights[rows]
        if skip_experts:
            weights = np.where(np.isin(ids, list(skip_experts)), np.float32(0), weights)
        needed = sorted(set(int(e) for e in ids.ravel()))
        if self.device_fill:
            blocks = {e: self.pool.download(self.first_cell + e, self.block_bytes) for e in needed}
        else:
            blocks = {e: self.block(e) for e in needed}
        lcfg = O.layer_cfg(oracle_expert_cfg(cfg), oracle_expert_cfg(cfg, True) if cfg.has_shared else None,
                           cfg.shared_gated)
        return O.moe_layer(lcfg, blocks, self.shared_block_host, self.gate_w, xr, ids, weights, threads=threads)


def small_config(**kw) -> MoEConfig:
    base = dict(d=128, f=64, num_experts=16, top_k=4, weight_bits=4, group_size=64, act_dtype=capi.DTYPE_FP32,
                has_shared=True, shared_gated=True, shared_f=64, max_tokens=64)
    base.update(kw)
    return MoEConfig(**base)


def inputs(T: int, d: int, seed: int = 0) -> np.ndarray:
    """bf16-representable N(0,1) activations, as the benchmark configs specify."""
    return fx.round_bf16(np.random.default_rng(seed).normal(0, 1, (T, d)).astype(np.float32))
