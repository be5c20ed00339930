"""Seeded synthetic inputs and the test-side quantiser, in numpy.

Mirrors the reference's fixture helpers: SplitMix64 / SeedTree
(sources/ShrikeValidation/Support/PRNG), bf16 helpers and the min/max affine
quantisers (sources/Shrike/Infrastructure/ModelIO/Quantization.swift:16-191),
and the packed expert block order (RepackPlanner.swift:735-826). The shapes of
the five benchmark workloads live here too: activations bf16 (the default of
MoEConfig) in, fp32 y out, which is the configuration the 1e-3 parity bar is
stated for.
"""
from __future__ import annotations

import numpy as np

from shrike_b200 import capi
from shrike_b200.moe import MoEConfig

MASK64 = (1 << 64) - 1
GOLDEN = 0x9E3779B97F4A7C15


class SplitMix64:
    """SplitMix64.swift: state += golden; z = mix(state)."""

    def __init__(self, seed: int):
        self.state = seed & MASK64

    def next(self) -> int:
        self.state = (self.state + GOLDEN) & MASK64
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
        return z ^ (z >> 31)

    def uniform(self, lo: float, hi: float) -> np.float32:
        """Uniform float in [lo, hi), 24-bit mantissa (SplitMix64.swift:22-25)."""
        u = np.float32(self.next() >> 40) / np.float32(1 << 24)
        return np.float32(lo) + (np.float32(hi) - np.float32(lo)) * u

    def uniform_array(self, n: int, lo: float, hi: float) -> np.ndarray:
        return np.array([self.uniform(lo, hi) for _ in range(n)], dtype=np.float32)


class SeedTree:
    """SeedTree.swift: child stream = SplitMix64(root ^ fnv1a(label))."""

    def __init__(self, root: int):
        self.root = root & MASK64

    def key(self, label: str) -> SplitMix64:
        h = 0xCBF29CE484222325
        for byte in label.encode("utf-8"):
            h ^= byte
            h = (h * 0x100000001B3) & MASK64
        return SplitMix64(self.root ^ h)


def splitmix64_stream(key: int, n: int) -> np.ndarray:
    """First n outputs of SplitMix64(seed=key), vectorised (counter mode)."""
    with np.errstate(over="ignore"):
        z = np.uint64(key) + (np.arange(1, n + 1, dtype=np.uint64) * np.uint64(GOLDEN))
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


# ---- bf16 / fp16 ---------------------------------------------------------------

def bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-half-to-even fp32 -> bf16 bit patterns (Quantization.swift:16-23)."""
    u = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    return (((u + 0x7FFF + lsb) >> 16) & 0xFFFF).astype(np.uint16)


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def round_bf16(x: np.ndarray) -> np.ndarray:
    return bf16_to_f32(bf16_bits(x))


def meta_bits(x: np.ndarray, meta_dtype: int) -> np.ndarray:
    if meta_dtype == capi.DTYPE_FP16:
        return np.asarray(x, dtype=np.float32).astype(np.float16).view(np.uint16)
    return bf16_bits(x)


def meta_to_f32(bits: np.ndarray, meta_dtype: int) -> np.ndarray:
    if meta_dtype == capi.DTYPE_FP16:
        return np.asarray(bits, dtype=np.uint16).view(np.float16).astype(np.float32)
    return bf16_to_f32(bits)


# ---- quantiser (test fixtures only) ---------------------------------------------

def quantize_affine(rows: np.ndarray, bits: int, group: int = 64, meta_dtype: int = capi.DTYPE_BF16):
    """`Quantization.quantizeInt4Affine` / `quantizeInt8Affine` for a [rows, n] matrix.

    Returns (packed uint8 [rows, n*bits/8], scales uint16 [rows, n/group], biases uint16 [...]).
    scale = (max-min)/(2^bits-1), bias = min, both rounded to the meta dtype
    before q is computed; a constant group gets scale 1.
    """
    rows = np.asarray(rows, dtype=np.float32)
    r, n = rows.shape
    assert n % group == 0
    g = rows.reshape(r, n // group, group)
    wmin = g.min(axis=2)
    wmax = g.max(axis=2)
    qmax = np.float32((1 << bits) - 1)
    const = wmax == wmin
    scale_f = np.where(const, np.float32(1), (wmax - wmin) / qmax).astype(np.float32)
    bias_f = wmin.astype(np.float32)
    s_bits = meta_bits(scale_f, meta_dtype)
    b_bits = meta_bits(bias_f, meta_dtype)
    scale = meta_to_f32(s_bits, meta_dtype)
    bias = meta_to_f32(b_bits, meta_dtype)
    inv = np.where(scale == 0, np.float32(0), np.float32(1) / scale).astype(np.float32)
    qf = ((g - bias[..., None]) * inv[..., None]).astype(np.float32)
    # Swift's .rounded() is half away from zero
    q = np.where(qf >= 0, np.floor(qf + np.float32(0.5)), np.ceil(qf - np.float32(0.5)))
    q = np.clip(q, 0, float(qmax)).astype(np.uint8).reshape(r, n)
    if bits == 4:
        packed = (q[:, 0::2] | (q[:, 1::2] << 4)).astype(np.uint8)
    else:
        packed = q
    return packed, s_bits, b_bits


def dequantize_affine(packed: np.ndarray, scales: np.ndarray, biases: np.ndarray, bits: int, group: int = 64,
                      meta_dtype: int = capi.DTYPE_BF16) -> np.ndarray:
    """`dequantizeInt4Affine` / `dequantizeInt8Affine`: w = q*scale + bias in fp32."""
    packed = np.asarray(packed, dtype=np.uint8)
    if bits == 4:
        q = np.empty((packed.shape[0], packed.shape[1] * 2), dtype=np.float32)
        q[:, 0::2] = packed & 0x0F
        q[:, 1::2] = packed >> 4
    else:
        q = packed.astype(np.float32)
    s = np.repeat(meta_to_f32(scales, meta_dtype), group, axis=1)
    b = np.repeat(meta_to_f32(biases, meta_dtype), group, axis=1)
    return (q * s + b).astype(np.float32)


def pack_expert_block(gate, up, down, gate_ab=None, up_ab=None, down_ab=None) -> np.ndarray:
    """Lays (packed, scales, biases) triples out in the packer's order:
    gate, gate_scales, gate_biases, [gate_bias], up..., down... ."""
    parts = []
    for (w, s, b), ab in ((gate, gate_ab), (up, up_ab), (down, down_ab)):
        parts += [np.ascontiguousarray(w).view(np.uint8).ravel(),
                  np.ascontiguousarray(s, dtype=np.uint16).view(np.uint8).ravel(),
                  np.ascontiguousarray(b, dtype=np.uint16).view(np.uint8).ravel()]
        if ab is not None:
            parts.append(bf16_bits(ab).view(np.uint8).ravel())
    return np.concatenate(parts)


# ---- synthetic blocks (same function as the library's device fill) ----------------

def _mix64(z: int) -> int:
    z &= MASK64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
    return z ^ (z >> 31)


def synth_block_key(seed: int, layer: int, expert: int) -> int:
    return _mix64(seed ^ _mix64(((layer << 32) | expert) + GOLDEN))


def synth_block(config: MoEConfig, seed: int, layer: int, expert: int, shared: bool = False) -> np.ndarray:
    """The packed block `shrike_pool_fill_synthetic` writes for (seed, layer, expert)."""
    f = config.shared_f if shared else config.f
    d = config.d
    key = synth_block_key(seed, layer, expert)
    base = np.float32(0.02) / np.float32(7.5) if config.weight_bits == 4 else np.float32(0.02) / np.float32(127.5)
    zp = np.float32(-8.0 if config.weight_bits == 4 else -128.0)
    parts = []
    for p, (rows, cols) in enumerate(((f, d), (f, d), (d, f))):
        wwords = rows * (cols * config.weight_bits // 8) // 8
        parts.append(splitmix64_stream(key ^ (0x1000 + p), wwords).view(np.uint8))
        n_meta = rows * (cols // config.group_size)
        r = splitmix64_stream(key ^ (0x2000 + p), n_meta)
        u = (r >> np.uint64(40)).astype(np.float32) * np.float32(1.0 / 16777216.0)
        sc = base * (np.float32(0.5) + u)
        sb = meta_bits(sc, config.meta_dtype)
        bb = meta_bits(zp * meta_to_f32(sb, config.meta_dtype), config.meta_dtype)
        parts += [sb.view(np.uint8), bb.view(np.uint8)]
        if config.expert_bias:
            r = splitmix64_stream(key ^ (0x3000 + p), rows)
            s = ((r & np.uint64(0xFFFF)) + ((r >> np.uint64(16)) & np.uint64(0xFFFF))
                 + ((r >> np.uint64(32)) & np.uint64(0xFFFF)) + ((r >> np.uint64(48)) & np.uint64(0xFFFF)))
            v = (s.astype(np.float32) - np.float32(131070.0)) * np.float32(2.6429e-6)
            parts.append(bf16_bits(v).view(np.uint8))
    return np.concatenate(parts)


# ---- workload shapes ----------------------------------------------------------------

def qwen_config(max_tokens: int = 16, **kw) -> MoEConfig:
    """Qwen3.5-35B-A3B MoE layer: D 2048, 256 experts top-8, F 512, int4 g64, gated shared expert."""
    base = dict(d=2048, f=512, num_experts=256, top_k=8, weight_bits=4, group_size=64,
                activation=capi.ACT_SILU, has_shared=True, shared_gated=True, shared_f=512,
                max_tokens=max_tokens, y_dtype=capi.DTYPE_FP32)
    base.update(kw)
    return MoEConfig(**base)


def gpt_oss_config(max_tokens: int = 64, group_size: int = 32, **kw) -> MoEConfig:
    """gpt-oss-20B MoE layer: D = F = 2880, 32 experts top-4, additive biases, clamped SwiGLU, no shared expert."""
    base = dict(d=2880, f=2880, num_experts=32, top_k=4, weight_bits=4, group_size=group_size,
                activation=capi.ACT_CLAMPED_SWIGLU, expert_bias=True, has_shared=False,
                max_tokens=max_tokens, y_dtype=capi.DTYPE_FP32)
    base.update(kw)
    return MoEConfig(**base)


def kimi_config(max_tokens: int = 2064, **kw) -> MoEConfig:
    """Kimi-Linear-48B MoE layer: D 2304, 256 experts top-8 sigmoid x2.446, F 1024, int8 g64, ungated shared."""
    base = dict(d=2304, f=1024, num_experts=256, top_k=8, weight_bits=8, group_size=64,
                activation=capi.ACT_SILU, router_kind=capi.ROUTER_SIGMOID, routed_scaling=2.446,
                has_shared=True, shared_gated=False, shared_f=1024, max_tokens=max_tokens,
                y_dtype=capi.DTYPE_FP32)
    base.update(kw)
    return MoEConfig(**base)


def zipf_logit_bias(num_experts: int, s: float = 1.1) -> np.ndarray:
    """log p_e with p_e proportional to (e+1)^-s: the skew prior of the ragged prefill workload."""
    p = (np.arange(1, num_experts + 1, dtype=np.float64)) ** (-s)
    p /= p.sum()
    return np.log(p).astype(np.float32)
