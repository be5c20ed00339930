"""Pins the CPU oracle against the known-answer cases of the reference's own
tests (restated from their formulas; the reference ships no binary fixtures)
and against the reference's compiled int4 GEMV."""
import math

import numpy as np
import pytest

import oracle_lib as O
from shrike_b200 import capi
import fixtures as fx
from shrike_b200.moe import MoEConfig


def lcg_rows(count, n, seed):
    """CPUExpertFFNTests.rows (CPUExpertFFNTests.swift:17-28): LCG floats in [-1, 1]."""
    state = seed
    out = np.empty((count, n), dtype=np.float32)
    for r in range(count):
        for c in range(n):
            state = (state * 6364136223846793005 + 1442695040888963407) & fx.MASK64
            v = (state >> 33) & 0xFFFFFFFF
            if v >= 1 << 31:
                v -= 1 << 32
            out[r, c] = np.float32(v) / np.float32(2147483647)
    return out


def dequant_then_dot(packed, s, b, x, bits=4, group=64):
    """DequantInt4GemvRef.apply: bulk dequantise, then a dot product per row."""
    w = fx.dequantize_affine(packed, s, b, bits, group)
    return (w.astype(np.float64) @ np.asarray(x, dtype=np.float64)).astype(np.float32)


# K1 -- CPUExpertFFNTests.offsetsCoverTheBlockExactlyWithNoOverlap
def test_k1_block_geometry():
    o = O.offsets(O.expert_cfg(2048, 512))
    assert o.stride == 1_769_472
    assert o.w[0] == 0 and o.s[0] == 524_288 and o.w[1] == 589_824 and o.w[2] == 1_179_648
    bounds = [o.w[0], o.s[0], o.b[0], o.w[1], o.s[1], o.b[1], o.w[2], o.s[2], o.b[2]]
    assert bounds == sorted(bounds)
    # the other two workload shapes (sizes quoted in the survey of the reference's layouts)
    assert O.offsets(O.expert_cfg(2304, 1024, bits=8)).stride == 7_520_256
    assert O.offsets(O.expert_cfg(2880, 2880, group=64, expert_bias=True)).stride == 14_014_080
    assert O.offsets(O.expert_cfg(2880, 2880, group=32, expert_bias=True)).stride == 15_569_280


# K2 -- CPUExpertFFNTests.matchesTheReferenceFFN
@pytest.mark.parametrize("use_ref", [False, True])
def test_k2_ffn_matches_dequant_reference(use_ref):
    if use_ref and O.ref_lib() is None:
        pytest.skip("reference GEMV not built")
    d, f = 128, 64
    gate = fx.quantize_affine(lcg_rows(f, d, 1), 4)
    up = fx.quantize_affine(lcg_rows(f, d, 2), 4)
    down = fx.quantize_affine(lcg_rows(d, f, 3), 4)
    blob = fx.pack_expert_block(gate, up, down)
    state = 99
    x = np.empty(d, dtype=np.float32)
    for i in range(d):
        state = (state * 6364136223846793005 + 1) & fx.MASK64
        v = (state >> 33) & 0xFFFFFFFF
        if v >= 1 << 31:
            v -= 1 << 32
        x[i] = np.float32(v) / np.float32(2147483647)
    g = dequant_then_dot(*gate, x)
    u = dequant_then_dot(*up, x)
    act = (g / (1 + np.exp(-g))) * u
    expected = dequant_then_dot(*down, act)
    out = np.zeros(d, dtype=np.float32)
    O.use_reference_gemv(use_ref)
    try:
        O.expert_ffn_accumulate(blob, O.expert_cfg(d, f), x, 1.0, out)
    finally:
        O.use_reference_gemv(False)
    scale = max(float(np.abs(expected).max()), 1.0)
    assert np.abs(out - expected).max() <= 2e-4 * scale


# K3 -- CPUExpertFFNTests.accumulatesScaledByRouteWeight
def test_k3_route_weight_accumulates():
    d, f = 128, 64
    blob = fx.pack_expert_block(fx.quantize_affine(lcg_rows(f, d, 7), 4), fx.quantize_affine(lcg_rows(f, d, 8), 4),
                                fx.quantize_affine(lcg_rows(d, f, 9), 4))
    x = np.full(d, 0.05, dtype=np.float32)
    cfg = O.expert_cfg(d, f)
    once = np.zeros(d, dtype=np.float32)
    O.expert_ffn_accumulate(blob, cfg, x, 1.0, once)
    twice = np.zeros(d, dtype=np.float32)
    O.expert_ffn_accumulate(blob, cfg, x, 0.75, twice)
    O.expert_ffn_accumulate(blob, cfg, x, 0.25, twice)
    assert np.abs(once - twice).max() <= 1e-4 * max(float(np.abs(once).max()), 1.0)


def constant_blob(bits, d=128, f=64):
    """MoEFusedFFNTests.makeConstantBlob: q = 0, scale = 0, biases 1/64, 0.5/64, 1/64."""
    def proj(rows, cols, bias):
        return (np.zeros((rows, cols * bits // 8), np.uint8), np.zeros((rows, cols // 64), np.uint16),
                np.full((rows, cols // 64), fx.bf16_bits(np.float32(bias))[()], np.uint16))
    return fx.pack_expert_block(proj(f, d, 1 / 64), proj(f, d, 0.5 / 64), proj(d, f, 1 / 64))


# K4 -- MoEFusedFFNTests.affineRoutedPipelineSupportsQwenBits
@pytest.mark.parametrize("bits", [4, 8])
def test_k4_constant_block(bits):
    d, f = 128, 64
    blob = constant_blob(bits)
    cfg = O.layer_cfg(O.expert_cfg(d, f, bits=bits))
    x = np.ones((1, d), dtype=np.float32)
    ids = np.arange(8, dtype=np.uint32)[None]
    w = np.full((1, 8), 0.125, dtype=np.float32)
    y = O.moe_layer(cfg, {e: blob for e in range(8)}, None, None, x, ids, w)
    assert np.abs(y - 2 / (1 + math.exp(-2))).max() < 0.01


# K5 -- MoEFusedFFNTests.productionRoutedPipelineSpecHitsAndFixupMissesMatchReference: eight int4 experts
# drawn from SeedTree(0x2D3)/"production-routed-moe" (weights U(-0.4, 0.4) quantised by the fixture
# quantiser, x and residual U(-0.5, 0.5) rounded to fp16, route weights fp16(0.04 + 0.015 k)), the
# routed-only pipeline y = residual + sum_k w_k * down_k(gelu_tanh(gate_k x) * up_k x) of
# MoeRef.applyStreamedRouted, at the reference's chained-reduction tolerance 1e-2 (max abs / max abs ref).
def k5_fixture():
    d, f, k = 128, 64, 8
    rng = fx.SeedTree(0x2D3).key("production-routed-moe")
    def mat(rows, cols):
        return np.array([[rng.uniform(-0.4, 0.4) for _ in range(cols)] for _ in range(rows)], dtype=np.float32)
    experts = []
    for _ in range(k):
        g, u, dn = mat(f, d), mat(f, d), mat(d, f)
        experts.append(tuple(fx.quantize_affine(m, 4) for m in (g, u, dn)))
    x = np.array([rng.uniform(-0.5, 0.5) for _ in range(d)], np.float32).astype(np.float16).astype(np.float32)
    residual = np.array([rng.uniform(-0.5, 0.5) for _ in range(d)], np.float32).astype(np.float16).astype(np.float32)
    w = np.array([0.04 + 0.015 * i for i in range(k)], np.float32).astype(np.float16).astype(np.float32)
    expected = residual.astype(np.float64)
    for (gate, up, down), wk in zip(experts, w):
        gv = dequant_then_dot(*gate, x).astype(np.float64)
        uv = dequant_then_dot(*up, x).astype(np.float64)
        act = 0.5 * gv * (1 + np.tanh(0.7978845608028654 * (gv + 0.044715 * gv ** 3))) * uv
        expected = expected + float(wk) * dequant_then_dot(*down, act.astype(np.float32))
    blobs = [fx.pack_expert_block(*e) for e in experts]
    return d, f, k, blobs, x, residual, w, expected.astype(np.float32)


def test_k5_routed_pipeline_matches_the_streamed_reference():
    d, f, k, blobs, x, residual, w, expected = k5_fixture()
    out = residual.copy()
    cfg = O.expert_cfg(d, f, activation=capi.ACT_GELU_TANH)
    for blob, wk in zip(blobs, w):
        O.expert_ffn_accumulate(blob, cfg, x, float(wk), out)
    assert np.abs(out - expected).max() / np.abs(expected).max() < 1e-2
    # far inside it: the oracle is fp32 throughout, the reference's own kernels round to fp16
    assert np.abs(out - expected).max() / np.abs(expected).max() < 1e-4


def test_router_never_selects_nan_or_minus_infinity():
    """router_topk_select_body's insertion scan (moe.metal:436-456): a NaN score fails every comparison and
    -inf is not greater than the initial -inf, so neither is ever inserted; with fewer candidates than top_k
    the remaining picks keep the initial id 0 and, under softmax, weight exp(-inf - max) = 0."""
    logits = np.linspace(1.0, 2.0, 16, dtype=np.float32)
    bias = np.zeros(16, np.float32)
    bias[15] = -np.inf      # the best score, masked
    bias[14] = np.nan
    ids, w = O.router_select(logits, 4, bias=bias, round_f16=False)
    assert list(ids) == [13, 12, 11, 10] and abs(float(w.sum()) - 1) < 1e-6
    bias[:] = -np.inf
    bias[3] = 0.0
    bias[9] = 0.0
    ids, w = O.router_select(logits, 4, bias=bias, round_f16=False)
    assert list(ids) == [9, 3, 0, 0] and w[2] < 1e-30 and w[3] < 1e-30 and abs(float(w[:2].sum()) - 1) < 1e-6


# K6 -- gpt-oss expert: additive biases + clamped SwiGLU (MoeRef.runFFNGptOss)
def test_k6_gpt_oss_expert():
    d, f = 128, 64
    rng = fx.SeedTree(0x6F55)
    def mat(label, rows, cols):
        k = rng.key(label)
        return np.array([[k.uniform(-0.4, 0.4) for _ in range(cols)] for _ in range(rows)], dtype=np.float32)
    gate, up, down = (fx.quantize_affine(mat(n, r, c), 4) for n, r, c in
                      (("gate", f, d), ("up", f, d), ("down", d, f)))
    gb = fx.round_bf16(rng.key("gate_bias").uniform_array(f, -0.5, 0.5))
    ub = fx.round_bf16(rng.key("up_bias").uniform_array(f, -0.5, 0.5))
    db = fx.round_bf16(rng.key("down_bias").uniform_array(d, -0.5, 0.5))
    x = rng.key("x").uniform_array(d, -0.5, 0.5) * np.float32(6)
    blob = fx.pack_expert_block(gate, up, down, gb, ub, db)
    g = np.minimum(dequant_then_dot(*gate, x) + gb, 7.0)
    u = np.clip(dequant_then_dot(*up, x) + ub, -7.0, 7.0)
    act = (g / (1 + np.exp(-1.702 * g))) * (u + 1)
    expected = dequant_then_dot(*down, act.astype(np.float32)) + db
    out = np.zeros(d, dtype=np.float32)
    O.expert_ffn_accumulate(blob, O.expert_cfg(d, f, activation=2, expert_bias=True), x, 1.0, out)
    assert np.abs(out - expected).max() <= 1e-2 * max(float(np.abs(expected).max()), 1.0)
    assert np.abs(g).max() > 0  # the clamp path is reachable at this input scale


def sort_reference(scores, k):
    """RouterTopKTests.reference: sort by score descending, ties to the lower id."""
    order = sorted(range(len(scores)), key=lambda e: (-float(scores[e]), e))
    return order[:k]


def router_fixture(seed, experts=16, dim=128, hidden_lo=-1.0, with_eff=False):
    rng = fx.SplitMix64(seed)
    w = np.array([[rng.uniform(-0.05, 0.05) + np.float32(e) * np.float32(0.01) for _ in range(dim)]
                  for e in range(experts)], dtype=np.float32)
    hidden = rng.uniform_array(dim, hidden_lo, hidden_lo + 2.0 if hidden_lo < 0 else 1.5)
    eff = None
    if with_eff:
        inv = np.float32(1.0) / np.sqrt(np.float32(dim))
        eff = np.array([rng.uniform(0.5, 1.5) * inv for _ in range(dim)], dtype=np.float32)
    pes = rng.uniform_array(experts, 0.6, 1.4)
    return w, hidden, eff, pes


# K7 -- RouterTopKTests.productionRouterMatchesReference / topFourRouterMatchesReference
@pytest.mark.parametrize("seed,k,with_eff", [(0xA5B6_1234, 8, True), (0xB44D_5678, 4, False)])
def test_k7_router_matches_sort_reference(seed, k, with_eff):
    w, hidden, eff, pes = router_fixture(seed, with_eff=with_eff)
    packed, s, b = fx.quantize_affine(w, 8)
    x = hidden if eff is None else hidden * eff
    ref_logits = dequant_then_dot(packed, s, b, x, bits=8)
    logits = O.router_logits_affine(packed, s, b, 8, hidden, eff)
    assert np.abs(logits - ref_logits).max() < 1e-4
    ids, weights = O.router_select(logits, k, per_expert_scale=pes, round_f16=True)
    expect_ids = sort_reference(ref_logits, k)
    assert list(ids) == expect_ids
    e = np.exp(ref_logits[expect_ids] - ref_logits[expect_ids[0]])
    assert np.abs(weights - e / e.sum() * pes[expect_ids]).max() < 5e-3


# K7 -- additiveLogitBiasShiftsSelectionAndWeights
def test_k7_logit_bias_moves_selection():
    rng = fx.SplitMix64(0x0B1A_5EED)
    w = np.array([[rng.uniform(-0.05, 0.05) + np.float32(e) * np.float32(0.01) for _ in range(128)]
                  for e in range(16)], dtype=np.float32)
    hidden = rng.uniform_array(128, 0.5, 1.5)
    packed, s, b = fx.quantize_affine(w, 8)
    logits = O.router_logits_affine(packed, s, b, 8, hidden)
    ids0, _ = O.router_select(logits, 4)
    bias = np.zeros(16, dtype=np.float32)
    bias[0] = 100.0
    ids1, w1 = O.router_select(logits, 4, bias=bias)
    assert 0 not in ids0 and ids1[0] == 0 and w1[0] > 0.99


# K7 -- productionRouterResolvesNearTieLikeReference
def test_k7_near_tie():
    rng = fx.SplitMix64(0x71E_0F4A)
    pattern = rng.uniform_array(128, 0.2, 1.0)
    hidden = rng.uniform_array(128, 0.5, 1.5)
    gains = np.zeros(16, dtype=np.float32)
    gains[:7] = 1.0 - np.arange(7, dtype=np.float32) * np.float32(0.05)
    gains[7] = 0.5
    gains[8] = np.float32(0.5) * (np.float32(1.0) + np.float32(1e-4))
    gains[9:] = 0.4 - np.arange(7, dtype=np.float32) * np.float32(0.02)
    w = gains[:, None] * pattern[None, :]
    packed, s, b = fx.quantize_affine(w.astype(np.float32), 8)
    ref_logits = dequant_then_dot(packed, s, b, hidden, bits=8)
    logits = O.router_logits_affine(packed, s, b, 8, hidden)
    ids, _ = O.router_select(logits, 8)
    assert list(ids) == sort_reference(ref_logits, 8)


def test_exact_ties_go_to_the_lower_expert():
    logits = np.array([1.0, 3.0, 3.0, 2.0, 3.0, 0.5], dtype=np.float32)
    ids, w = O.router_select(logits, 4, round_f16=False)
    assert list(ids) == [1, 2, 4, 3]
    assert abs(float(w.sum()) - 1.0) < 1e-6


# K8 -- sigmoid router: NE=256, K=8, scaling 2.446, bias moves selection not weight
@pytest.mark.parametrize("seed", [0x516_0001, 0x516_0002, 0x516_0003, 0x516_0004])
def test_k8_sigmoid_router(seed):
    rng = fx.SplitMix64(seed)
    ne, dim, k = 256, 128, 8
    w = np.array([[rng.uniform(-0.05, 0.05) + np.float32(e % 37) * np.float32(0.003) for _ in range(dim)]
                  for e in range(ne)], dtype=np.float32)
    hidden = rng.uniform_array(dim, -1.0, 1.0)
    bias = fx.round_bf16(rng.uniform_array(ne, -0.1, 0.1))
    packed, s, b = fx.quantize_affine(w, 8)
    ref_logits = dequant_then_dot(packed, s, b, hidden, bits=8).astype(np.float64)
    sig = 1 / (1 + np.exp(-ref_logits))
    expect = sort_reference(sig + bias, k)
    logits = O.router_logits_affine(packed, s, b, 8, hidden)
    ids, weights = O.router_select(logits, k, bias=bias, sigmoid=True, scaling=2.446, round_f16=True)
    assert list(ids) == expect
    orig = sig[expect]
    assert np.abs(weights - orig / (orig.sum() + 1e-20) * 2.446).max() < 5e-3


def test_router_f32_order_is_close_to_exact():
    rng = np.random.default_rng(5)
    w = rng.normal(0, 0.02, (256, 2048)).astype(np.float32)
    x = fx.round_bf16(rng.normal(0, 1, 2048).astype(np.float32))
    logits = O.router_logits_f32(w, x)
    exact = w.astype(np.float64) @ x.astype(np.float64)
    assert np.abs(logits - exact).max() < 2e-5


def test_exp_det_accuracy():
    xs = np.linspace(-30, 30, 2001, dtype=np.float32)
    got = np.array([O.lib().so_exp_det(float(v)) for v in xs])
    assert np.abs(got / np.exp(xs.astype(np.float64)) - 1).max() < 4e-7


def test_half_conversions_match_numpy():
    rng = np.random.default_rng(1)
    vals = np.concatenate([rng.normal(0, 1, 2000), rng.normal(0, 1e-5, 500), rng.normal(0, 3e4, 500),
                           [0.0, -0.0, 65504.0, 65519.9, 65520.0, 6e-8, 2.98e-8, 2.99e-8]]).astype(np.float32)
    L = O.lib()
    for v in vals:
        assert L.so_f32_to_f16(float(v)) == int(np.float32(v).astype(np.float16).view(np.uint16)), v
    halves = rng.integers(0, 0x7C00, 2000).astype(np.uint16)
    for h in halves:
        assert L.so_f16_to_f32(int(h)) == float(np.uint16(h).view(np.float16))
    assert all(L.so_f32_to_bf16(float(v)) == int(fx.bf16_bits(np.float32(v))) for v in vals[:1000])


# the restated GEMV against the reference's own compiled code
@pytest.mark.parametrize("rows,n", [(64, 128), (512, 2048), (2048, 512)])
def test_restated_gemv_equals_reference_binary(rows, n):
    if O.ref_lib() is None:
        pytest.skip("reference GEMV not built")
    rng = np.random.default_rng(rows + n)
    w = rng.integers(0, 256, (rows, n // 2)).astype(np.uint8)
    s = fx.bf16_bits(rng.uniform(0.001, 0.004, (rows, n // 64)).astype(np.float32))
    b = fx.bf16_bits((-8 * fx.bf16_to_f32(s)).astype(np.float32))
    x = rng.normal(0, 1, n).astype(np.float32)
    ours = O.affine_gemv(w, s, b, x, rows, n)
    theirs = O.reference_int4_gemv(w, s, b, x, rows, n)
    # same algorithm; the two builds may vectorise the inner sums differently
    assert np.abs(ours - theirs).max() <= 2e-5 * max(float(np.abs(theirs).max()), 1.0)
    exact = fx.dequantize_affine(w, s, b, 4).astype(np.float64) @ x.astype(np.float64)
    assert np.abs(theirs - exact).max() <= 1e-4 * max(float(np.abs(exact).max()), 1.0)


# K14 -- quantiser round trip bound
@pytest.mark.parametrize("bits", [4, 8])
def test_k14_quantiser_round_trip(bits):
    rng = np.random.default_rng(bits)
    w = rng.uniform(-0.4, 0.4, (32, 256)).astype(np.float32)
    packed, s, b = fx.quantize_affine(w, bits)
    back = fx.dequantize_affine(packed, s, b, bits)
    scale = np.repeat(fx.bf16_to_f32(s), 64, axis=1)
    assert (np.abs(back - w) <= scale + 1e-4).all()


# K12 -- closed-form synthetic pool, int4 and int8, generic GEMV vs dequantised reference
@pytest.mark.parametrize("bits", [4, 8])
def test_k12_closed_form_pool(bits):
    d = f = 192
    x = ((np.arange(d) % 17) - 8).astype(np.float32)
    for e in range(3):
        def w(role, rows, cols):
            r = np.arange(rows)[:, None]
            c = np.arange(cols)[None, :]
            return ((e + 1) * 0.001 + (role + 1) * 0.003 + ((r % 7) - 3) * 0.0004 + ((c % 11) - 5) * 0.0002).astype(np.float32)
        gate, up, down = (fx.quantize_affine(w(i, r, c), bits) for i, (r, c) in enumerate(((f, d), (f, d), (d, f))))
        blob = fx.pack_expert_block(gate, up, down)
        g = dequant_then_dot(*gate, x, bits=bits)
        u = dequant_then_dot(*up, x, bits=bits)
        act = ((g / (1 + np.exp(-g.astype(np.float64)))) * u).astype(np.float32)
        expected = dequant_then_dot(*down, act, bits=bits)
        out = np.zeros(d, dtype=np.float32)
        O.expert_ffn_accumulate(blob, O.expert_cfg(d, f, bits=bits), x, 1.0, out)
        assert np.abs(out - expected).max() <= 1e-4 * max(1.0, float(np.abs(expected).max()))


# K13 -- token-major reduce
def test_k13_reduce_token_major():
    rng = np.random.default_rng(13)
    T, K, D = 5, 8, 96
    p = rng.normal(0, 1, (T * K, D)).astype(np.float32)
    w = rng.uniform(0, 0.3, (T, K)).astype(np.float32)
    got = O.reduce_token_major(p, w, T, K, D)
    ref = np.einsum("tk,tkd->td", w.astype(np.float64), p.reshape(T, K, D).astype(np.float64))
    assert np.abs(got - ref).max() < 2e-3


# K10 -- PrefillMoEGroupingTests
def test_k10_grouping_sorts_and_counts():
    pairs = [(0, 3, 0, 10), (0, 1, 1, 11), (0, 4, 2, 12), (1, 1, 0, 13), (1, 3, 1, 14), (1, 2, 2, 15),
             (2, 4, 0, 16), (2, 3, 1, 17), (2, 1, 2, 18), (3, 5, 0, 19), (3, 1, 1, 20), (3, 4, 2, 21)][::-1]
    rc, out, off, cnt = O.group_pairs(np.array(pairs, dtype=np.uint32), 4, 3, 6)
    assert rc == 0
    assert list(out[:, 1]) == [1, 1, 1, 1, 2, 3, 3, 3, 4, 4, 4, 5]
    assert [list(r) for r in out[:, [0, 2]]] == [[0, 1], [1, 0], [2, 2], [3, 1], [1, 2], [0, 0], [1, 1], [2, 1],
                                                 [0, 2], [2, 0], [3, 2], [3, 0]]
    assert list(off) == [0xFFFFFFFF, 0, 4, 5, 8, 11]
    assert list(cnt) == [0, 4, 1, 3, 3, 1]


def test_k10_grouping_is_order_independent_and_keeps_weight_bits():
    token_major = [(0, 2, 0, 101), (0, 1, 1, 102), (1, 2, 0, 103), (1, 0, 1, 104), (2, 1, 0, 105), (2, 2, 1, 106)]
    shuffled = [token_major[i] for i in (5, 1, 3, 0, 4, 2)]
    a = O.group_pairs(np.array(token_major, dtype=np.uint32), 3, 2, 3)
    b = O.group_pairs(np.array(shuffled, dtype=np.uint32), 3, 2, 3)
    assert a[0] == 0 and b[0] == 0 and (a[1] == b[1]).all()
    assert list(a[1][:, 3]) == [104, 102, 105, 101, 103, 106]


def test_k10_grouping_rejects_bad_pairs():
    ok = [(0, 0, 0, 0), (0, 1, 1, 0)]
    assert O.group_pairs(np.array(ok, dtype=np.uint32), 1, 2, 2)[0] == 0
    assert O.group_pairs(np.array([(1, 0, 0, 0), (0, 1, 1, 0)], dtype=np.uint32), 1, 2, 2)[0] == -2
    assert O.group_pairs(np.array([(0, 0, 2, 0), (0, 1, 1, 0)], dtype=np.uint32), 1, 2, 2)[0] == -3
    assert O.group_pairs(np.array([(0, 2, 0, 0), (0, 1, 1, 0)], dtype=np.uint32), 1, 2, 2)[0] == -4
    assert O.group_pairs(np.array([(0, 0, 1, 0), (0, 1, 1, 0)], dtype=np.uint32), 1, 2, 2)[0] == -5
    assert O.group_pairs(np.array(ok[:1], dtype=np.uint32), 1, 2, 2)[0] == -1


# K11 -- wave planner (PrefillGroupedRoutedMoETests+Execution.swift:382-432)
def test_k11_wave_planner():
    n, blocks, wave_of, padded = O.plan_expert_waves([0, 1, 2, 3], [0, 40, 72, 77], [40, 32, 5, 3], 1024)
    assert n == 4 and list(blocks[:, 3]) == [0, 64, 128, 192] and list(padded) == [256]
    assert list(blocks[:, 4]) == [0, 1, 2, 3] and set(wave_of) == {0}
    # a 600-row expert in 512-row waves splits 512 + 88
    n, blocks, wave_of, padded = O.plan_expert_waves([7], [100], [600], 512)
    assert n == 2 and list(blocks[:, 2]) == [512, 88] and list(blocks[:, 1]) == [100, 612]
    assert list(wave_of) == [0, 1] and list(padded) == [512, 128]
    # experts spill across waves at tile boundaries
    n, blocks, wave_of, padded = O.plan_expert_waves([0, 1], [0, 100], [100, 100], 128)
    assert [list(b) for b in blocks] == [[0, 0, 100, 0, 0], [1, 100, 100, 0, 0]] and list(wave_of) == [0, 1]
    assert O.plan_expert_waves([0], [0], [10], 100)[0] == -1  # staging not a multiple of the tile


def test_classification_follows_the_table():
    table = np.zeros(16, dtype=np.uint64)
    for e in range(16):
        table[e] = (2 << 32) | (100 + e)
    table[5] = (1 << 32) | 105        # loading, not resident
    table[9] = (2 << 32) | 0xFFFFFFFF  # resident flag without a slot
    slots, misses, mp, me = O.classify_residency([3, 5, 9, 40], table, 16)
    assert list(slots) == [103, 0xFFFFFFFF, 0xFFFFFFFF, 115] and misses == 2
    assert list(mp) == [1, 2] and list(me) == [5, 9]


@pytest.mark.parametrize("bits,group,meta,bias", [(4, 64, 0, False), (4, 32, 1, True), (8, 64, 0, False)])
def test_synthetic_block_is_the_same_function_in_numpy_and_c(bits, group, meta, bias):
    cfg = MoEConfig(d=256, f=128, num_experts=8, top_k=2, weight_bits=bits, group_size=group, meta_dtype=meta,
                    expert_bias=bias)
    a = fx.synth_block(cfg, 0x5EED, 3, 5)
    b = O.synth_block(O.expert_cfg(256, 128, bits, group, meta, 0, bias), 0x5EED, 3, 5)
    assert a.shape == b.shape and (a == b).all()
    off = O.offsets(O.expert_cfg(256, 128, bits, group, meta, 0, bias))
    s = fx.meta_to_f32(a[off.s[0]:off.b[0]].view(np.uint16), meta)
    z = fx.meta_to_f32(a[off.b[0]:off.b[0] + (off.b[0] - off.s[0])].view(np.uint16), meta)
    base = 0.02 / (7.5 if bits == 4 else 127.5)
    assert s.min() >= base * 0.49 and s.max() <= base * 1.51
    assert (z == -(8 if bits == 4 else 128) * s).all()


def test_moe_layer_threads_agree():
    d, f = 128, 64
    cfg = O.layer_cfg(O.expert_cfg(d, f), O.expert_cfg(d, f), shared_gated=True)
    ecfg = O.expert_cfg(d, f)
    blocks = {e: O.synth_block(ecfg, 1, 0, e) for e in range(6)}
    shared = O.synth_block(ecfg, 1, 0, 1000)
    rng = np.random.default_rng(0)
    x = rng.normal(0, 1, (3, d)).astype(np.float32)
    ids = np.array([[0, 1], [2, 3], [4, 5]], dtype=np.uint32)
    w = rng.uniform(0.1, 0.9, (3, 2)).astype(np.float32)
    gw = rng.normal(0, 0.1, d).astype(np.float32)
    a = O.moe_layer(cfg, blocks, shared, gw, x, ids, w, threads=1)
    b = O.moe_layer(cfg, blocks, shared, gw, x, ids, w, threads=4)
    assert (a == b).all() and np.abs(a).max() > 0
