"""ctypes access to the CPU oracle (oracle/shrike_oracle.c) for the test-suite.

The oracle is the checker, never the thing under test: nothing under
shrike_b200/ imports this module.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
ORACLE_DIR = ROOT / "oracle"
ORACLE_LIB = ORACLE_DIR / "_build" / "libshrike_oracle.so"
REF_LIB = ORACLE_DIR / "_ref" / "libshrike_ref_gemv.so"


class ExpertCfg(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("d", "f", "bits", "group", "meta_dtype", "activation", "expert_bias")]


class Offsets(C.Structure):
    _fields_ = [("w", C.c_uint32 * 3), ("s", C.c_uint32 * 3), ("b", C.c_uint32 * 3), ("ab", C.c_uint32 * 3),
                ("stride", C.c_uint32)]


class RouterCfg(C.Structure):
    _fields_ = [("num_experts", C.c_uint32), ("top_k", C.c_uint32), ("kind", C.c_uint32),
                ("weight_kind", C.c_uint32), ("scaling", C.c_float), ("round_weights_f16", C.c_uint32)]


class LayerCfg(C.Structure):
    _fields_ = [("expert", ExpertCfg), ("has_shared", C.c_uint32), ("shared_gated", C.c_uint32),
                ("shared", ExpertCfg)]


_lib = None
_ref = None


def build() -> None:
    subprocess.run(["make", "-C", str(ORACLE_DIR)], check=True, capture_output=True)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not ORACLE_LIB.exists():
            build()
        _lib = C.CDLL(str(ORACLE_LIB))
        _lib.so_bf16_to_f32.restype = C.c_float
        _lib.so_bf16_to_f32.argtypes = [C.c_uint16]
        _lib.so_f16_to_f32.restype = C.c_float
        _lib.so_f16_to_f32.argtypes = [C.c_uint16]
        _lib.so_f32_to_bf16.restype = C.c_uint16
        _lib.so_f32_to_bf16.argtypes = [C.c_float]
        _lib.so_f32_to_f16.restype = C.c_uint16
        _lib.so_f32_to_f16.argtypes = [C.c_float]
        _lib.so_exp_det.restype = C.c_float
        _lib.so_exp_det.argtypes = [C.c_float]
        _lib.so_glu.restype = C.c_float
        _lib.so_glu.argtypes = [C.c_float, C.c_float, C.c_uint32]
        _lib.so_splitmix64_at.restype = C.c_uint64
        _lib.so_splitmix64_at.argtypes = [C.c_uint64, C.c_uint64]
        _lib.so_synth_block_key.restype = C.c_uint64
        _lib.so_synth_block_key.argtypes = [C.c_uint64, C.c_uint32, C.c_uint32]
        _lib.so_classify_residency.restype = C.c_uint32
        _lib.so_group_pairs.restype = C.c_int
        _lib.so_plan_expert_waves.restype = C.c_int
    return _lib


def ref_lib():
    """The reference's own compiled int4 GEMV, or None when it was not built."""
    global _ref
    if _ref is None and REF_LIB.exists():
        _ref = C.CDLL(str(REF_LIB))
    return _ref


def use_reference_gemv(enable: bool) -> bool:
    """Routes the oracle's int4/g64/bf16 GEMV through the reference's compiled code."""
    r = ref_lib()
    if enable and r is None:
        return False
    fn = C.cast(r.shrike_int4_affine_gemv, C.c_void_p) if enable else C.c_void_p(None)
    lib().so_set_reference_int4_gemv(fn)
    return True


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def expert_cfg(d, f, bits=4, group=64, meta_dtype=0, activation=0, expert_bias=False) -> ExpertCfg:
    return ExpertCfg(d, f, bits, group, meta_dtype, activation, int(expert_bias))


def offsets(cfg: ExpertCfg) -> Offsets:
    o = Offsets()
    lib().so_offsets_make(C.byref(cfg), C.byref(o))
    return o


def affine_gemv(weights, scales, biases, x, rows, n, bits=4, group=64, meta_dtype=0) -> np.ndarray:
    w = np.ascontiguousarray(weights, dtype=np.uint8)
    s = np.ascontiguousarray(scales, dtype=np.uint16)
    b = np.ascontiguousarray(biases, dtype=np.uint16)
    xx = np.ascontiguousarray(x, dtype=np.float32)
    out = np.zeros(rows, dtype=np.float32)
    lib().so_affine_gemv(_p(w), _p(s), _p(b), _p(xx), C.c_size_t(rows), C.c_size_t(n), C.c_uint32(bits),
                         C.c_uint32(group), C.c_uint32(meta_dtype), _p(out))
    return out


def reference_int4_gemv(weights, scales, biases, x, rows, n) -> np.ndarray:
    r = ref_lib()
    assert r is not None
    w = np.ascontiguousarray(weights, dtype=np.uint8)
    s = np.ascontiguousarray(scales, dtype=np.uint16)
    b = np.ascontiguousarray(biases, dtype=np.uint16)
    xx = np.ascontiguousarray(x, dtype=np.float32)
    out = np.zeros(rows, dtype=np.float32)
    r.shrike_int4_affine_gemv(_p(w), _p(s), _p(b), _p(xx), C.c_size_t(rows), C.c_size_t(n), _p(out))
    return out


def expert_ffn_accumulate(block, cfg: ExpertCfg, x, route_weight, out) -> None:
    blk = np.ascontiguousarray(block, dtype=np.uint8)
    xx = np.ascontiguousarray(x, dtype=np.float32)
    o = offsets(cfg)
    scratch = np.zeros(2 * cfg.f + cfg.d, dtype=np.float32)
    assert out.dtype == np.float32 and out.flags.c_contiguous
    lib().so_expert_ffn_accumulate(_p(blk), C.byref(cfg), C.byref(o), _p(xx), C.c_float(route_weight),
                                   _p(scratch), _p(out))


def router_logits_f32(w, x) -> np.ndarray:
    w = np.ascontiguousarray(w, dtype=np.float32)
    x = np.ascontiguousarray(x, dtype=np.float32)
    ne, d = w.shape
    out = np.zeros(ne, dtype=np.float32)
    lib().so_router_logits_f32(_p(w), _p(x), C.c_uint32(ne), C.c_uint32(d), _p(out))
    return out


def router_logits_affine(w, scales, biases, bits, x, effective_scale=None) -> np.ndarray:
    w = np.ascontiguousarray(w, dtype=np.uint8)
    s = np.ascontiguousarray(scales, dtype=np.uint16)
    b = np.ascontiguousarray(biases, dtype=np.uint16)
    x = np.ascontiguousarray(x, dtype=np.float32)
    ne = w.shape[0]
    d = x.shape[0]
    es = None if effective_scale is None else np.ascontiguousarray(effective_scale, dtype=np.float32)
    out = np.zeros(ne, dtype=np.float32)
    lib().so_router_logits_affine(_p(w), _p(s), _p(b), C.c_uint32(bits), _p(x),
                                  _p(es) if es is not None else None, C.c_uint32(ne), C.c_uint32(d), _p(out))
    return out


def router_select(logits, top_k, bias=None, per_expert_scale=None, sigmoid=False, scaling=1.0, round_f16=True):
    lg = np.ascontiguousarray(logits, dtype=np.float32)
    ne = lg.shape[0]
    cfg = RouterCfg(ne, top_k, 1 if sigmoid else 0, 0, scaling, int(round_f16))
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    pes = None if per_expert_scale is None else np.ascontiguousarray(per_expert_scale, dtype=np.float32)
    ids = np.zeros(top_k, dtype=np.uint32)
    w = np.zeros(top_k, dtype=np.float32)
    lib().so_router_select(_p(lg), _p(b) if b is not None else None, _p(pes) if pes is not None else None,
                           C.byref(cfg), _p(ids), _p(w))
    return ids, w


def classify_residency(topk, table, num_experts):
    topk = np.ascontiguousarray(topk, dtype=np.uint32)
    table = np.ascontiguousarray(table, dtype=np.uint64)
    k = topk.shape[0]
    slots = np.zeros(k, dtype=np.uint32)
    hp = np.zeros(k, dtype=np.uint32)
    mp = np.zeros(k, dtype=np.uint32)
    me = np.zeros(k, dtype=np.uint32)
    misses = lib().so_classify_residency(_p(topk), _p(table), C.c_uint32(k), C.c_uint32(num_experts), _p(slots),
                                         _p(hp), _p(mp), _p(me))
    return slots, int(misses), mp[:misses], me[:misses]


def layer_cfg(expert: ExpertCfg, shared: ExpertCfg | None = None, shared_gated=False) -> LayerCfg:
    return LayerCfg(expert, 1 if shared is not None else 0, int(shared_gated),
                    shared if shared is not None else ExpertCfg())


def moe_layer(cfg: LayerCfg, blocks: dict, shared_block, shared_gate_w, x, ids, weights, threads=1) -> np.ndarray:
    """blocks: {expert id: uint8 array}. x [T, d] fp32; ids/weights [T, K]."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    ids = np.ascontiguousarray(ids, dtype=np.uint32)
    weights = np.ascontiguousarray(weights, dtype=np.float32)
    T, d = x.shape
    K = ids.shape[1]
    n = max(blocks.keys()) + 1 if blocks else 1
    arr = (C.c_void_p * n)()
    keep = []
    for e, blk in blocks.items():
        b = np.ascontiguousarray(blk, dtype=np.uint8)
        keep.append(b)
        arr[e] = b.ctypes.data
    sb = None if shared_block is None else np.ascontiguousarray(shared_block, dtype=np.uint8)
    gw = None if shared_gate_w is None else np.ascontiguousarray(shared_gate_w, dtype=np.float32)
    y = np.zeros((T, d), dtype=np.float32)
    lib().so_moe_layer(C.byref(cfg), arr, _p(sb) if sb is not None else None, _p(gw) if gw is not None else None,
                       _p(x), C.c_uint32(T), _p(ids), _p(weights), C.c_uint32(K), _p(y), C.c_uint32(threads))
    return y


def reduce_token_major(partials, weights, tokens, top_k, d) -> np.ndarray:
    p = np.ascontiguousarray(partials, dtype=np.float32)
    w = np.ascontiguousarray(weights, dtype=np.float32)
    out = np.zeros((tokens, d), dtype=np.float32)
    lib().so_reduce_token_major(_p(p), _p(w), C.c_uint32(tokens), C.c_uint32(top_k), C.c_uint32(d), _p(out))
    return out


def group_pairs(pairs, tokens, top_k, num_experts):
    """pairs: uint32 [n, 4] (token, expert, rank, weight bits). Returns (rc, sorted, offsets, counts)."""
    p = np.ascontiguousarray(pairs, dtype=np.uint32)
    n = p.shape[0]
    out = np.zeros_like(p)
    off = np.zeros(num_experts, dtype=np.uint32)
    cnt = np.zeros(num_experts, dtype=np.uint32)
    rc = lib().so_group_pairs(_p(p), C.c_uint32(n), C.c_uint32(tokens), C.c_uint32(top_k), C.c_uint32(num_experts),
                              _p(out), _p(off), _p(cnt))
    return rc, out, off, cnt


def plan_expert_waves(slots, pair_starts, pair_counts, staging_rows, row_tile=64, max_blocks=4096):
    s = np.ascontiguousarray(slots, dtype=np.uint32)
    ps = np.ascontiguousarray(pair_starts, dtype=np.uint32)
    pc = np.ascontiguousarray(pair_counts, dtype=np.uint32)
    blocks = np.zeros((max_blocks, 5), dtype=np.uint32)
    wave_of = np.zeros(max_blocks, dtype=np.uint32)
    padded = np.zeros(max_blocks, dtype=np.uint32)
    n = lib().so_plan_expert_waves(_p(s), _p(ps), _p(pc), C.c_uint32(len(s)), C.c_uint32(staging_rows),
                                   C.c_uint32(row_tile), _p(blocks), _p(wave_of), _p(padded), C.c_uint32(max_blocks))
    if n < 0:
        return n, None, None, None
    n_waves = int(wave_of[:n].max()) + 1 if n else 0
    return n, blocks[:n], wave_of[:n], padded[:n_waves]


def synth_block(cfg: ExpertCfg, seed: int, layer: int, expert: int) -> np.ndarray:
    o = offsets(cfg)
    blk = np.zeros(o.stride, dtype=np.uint8)
    key = lib().so_synth_block_key(C.c_uint64(seed), C.c_uint32(layer), C.c_uint32(expert))
    lib().so_synth_fill_block(C.byref(cfg), C.byref(o), C.c_uint64(key), _p(blk))
    return blk
