// Top-k selection shared by the router kernels and the self-routing decode kernels.
//
//   router_topk_select_body     moe.metal:419-491
//   moe_classify_residency_body moe.metal:121-151
//
// The helpers are templates over the argument block: it must carry ne, top_k, logit_bias,
// per_expert_scale, sigmoid_scores, scaling and round_f16.
#pragma once

#include "internal.h"

namespace shrike {

// exp(x) as a fixed sequence of IEEE fp32 operations: identical results on the
// host restatement and on the device.
__host__ __device__ __forceinline__ float exp_det(float x) {
#ifdef __CUDA_ARCH__
#define SHRIKE_FMA(a, b, c) __fmaf_rn((a), (b), (c))
#define SHRIKE_MUL(a, b) __fmul_rn((a), (b))
#else
#define SHRIKE_FMA(a, b, c) fmaf((a), (b), (c))
#define SHRIKE_MUL(a, b) ((a) * (b))
#endif
    x = fminf(88.0f, fmaxf(-87.0f, x));
    const float n = rintf(SHRIKE_MUL(x, 1.4426950408889634f));
    float r = SHRIKE_FMA(n, -0.693145751953125f, x);
    r = SHRIKE_FMA(n, -1.428606765330187e-06f, r);
    float p = 1.0f / 720.0f;
    p = SHRIKE_FMA(p, r, 1.0f / 120.0f);
    p = SHRIKE_FMA(p, r, 1.0f / 24.0f);
    p = SHRIKE_FMA(p, r, 1.0f / 6.0f);
    p = SHRIKE_FMA(p, r, 0.5f);
    p = SHRIKE_FMA(p, r, 1.0f);
    p = SHRIKE_FMA(p, r, 1.0f);
    const int e = (int)n + 127;
#ifdef __CUDA_ARCH__
    const float scale = __uint_as_float((uint32_t)e << 23);
#else
    union { uint32_t u; float f; } c; c.u = (uint32_t)e << 23; const float scale = c.f;
#endif
    return SHRIKE_MUL(p, scale);
#undef SHRIKE_FMA
#undef SHRIKE_MUL
}

__device__ __forceinline__ float sigmoid_det(float x) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, exp_det(-x))); }

// Order-preserving key of a selection score; 0 = not a candidate. The reference's insertion scan
// (moe.metal:436-456) never inserts a NaN score (every comparison is false) nor -inf (not greater than the
// initial -inf, and the tie-break wants an id below 0): both map to 0 here.
__device__ __forceinline__ uint32_t key_of_score(float s) {
    s = __fadd_rn(s, 0.0f);  // -0 -> +0
    if (!(s > -INFINITY)) return 0u;
    const uint32_t b = __float_as_uint(s);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
// The score a key stands for; a pick that found no candidate keeps the scan's initial -inf (and id 0).
__device__ __forceinline__ float score_of_key(uint32_t k) {
    if (k == 0u) return -INFINITY;
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// Key of expert e's selection score; the same arithmetic as select_row.
template <class A>
__device__ __forceinline__ uint32_t selection_key_of(float raw, float bias, const A& a) {
    return key_of_score(__fadd_rn(a.sigmoid_scores ? sigmoid_det(raw) : raw, bias));
}

template <bool CG, class A>
__device__ __forceinline__ uint32_t selection_key(const float* lg, const A& a, uint32_t e) {
    if (e >= a.ne) return 0u;
    const float raw = CG ? __ldcg(lg + e) : lg[e];
    const float bias = a.logit_bias ? bf16_bits_to_f32(a.logit_bias[e]) : 0.0f;
    return selection_key_of(raw, bias, a);
}

// Route weights of the picks (lane r holds the r-th pick): moe.metal:458-490, sums in rank order.
template <bool CG, class A>
__device__ __forceinline__ float selection_weight(const float* lg, const A& a, uint32_t lane, float my_score,
                                                  uint32_t my_id) {
    const uint32_t top_k = a.top_k;
    float val;
    if (a.sigmoid_scores) {
        val = lane < top_k ? sigmoid_det(CG ? __ldcg(lg + my_id) : lg[my_id]) : 0.f;
    } else {
        const float mx = __shfl_sync(0xffffffffu, my_score, 0);
        val = lane < top_k ? exp_det(__fsub_rn(my_score, mx)) : 0.f;
    }
    float sum = 0.f;
    for (uint32_t r = 0; r < top_k; ++r) sum = __fadd_rn(sum, __shfl_sync(0xffffffffu, val, r));
    float w;
    if (a.sigmoid_scores) w = __fmul_rn(val, __fdiv_rn(a.scaling, __fadd_rn(sum, 1e-20f)));
    else w = __fdiv_rn(val, sum);
    const float pes = a.per_expert_scale ? bf16_bits_to_f32(a.per_expert_scale[my_id]) : 1.0f;
    w = __fmul_rn(w, pes);
    if (a.round_f16) w = __half2float(__float2half_rn(w));
    return w;
}

struct alignas(16) SelectSmem {
    uint32_t keys[SHRIKE_MAX_EXPERTS];   // read back 16 bytes at a time
    uint32_t cand_key[32], cand_id[32];
    uint32_t sel_key[SHRIKE_MAX_TOP_K], sel_id[SHRIKE_MAX_TOP_K];
};

// The same picks as select_row, by the whole block (4 warps) for one row, without the K serial
// rounds: every expert counts the experts that beat it ((score desc, id asc) is a total order, so
// the count is its rank). Warp w ranks its 64 experts among themselves and keeps the best 8;
// warp 0 ranks the 32 survivors. Lane r of warp 0 returns the r-th pick; call from all threads.
// CG: read the logits past L1 (they were written by other blocks of this launch); false for a
// copy that already sits in shared memory.
template <bool CG = true, class A>
__device__ __forceinline__ void select_row_block(const float* lg, const A& a, SelectSmem& ss, uint32_t& out_id,
                                                 float& out_w) {
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // the first four warps do the work; larger blocks only join the barriers
    if (tid < 128) {
        // both logits (and biases) are requested before either is used: one L2 round trip, not two
        const uint32_t e0 = tid, e1 = tid + 128;
        const float raw0 = e0 < a.ne ? (CG ? __ldcg(lg + e0) : lg[e0]) : 0.f;
        const float raw1 = e1 < a.ne ? (CG ? __ldcg(lg + e1) : lg[e1]) : 0.f;
        uint16_t lb0 = 0, lb1 = 0;
        if (a.logit_bias) {
            if (e0 < a.ne) lb0 = a.logit_bias[e0];
            if (e1 < a.ne) lb1 = a.logit_bias[e1];
        }
        ss.keys[e0] = e0 < a.ne ? selection_key_of(raw0, bf16_bits_to_f32(lb0), a) : 0u;
        ss.keys[e1] = e1 < a.ne ? selection_key_of(raw1, bf16_bits_to_f32(lb1), a) : 0u;
    }
    if (tid < 32) { ss.cand_key[tid] = 0u; ss.cand_id[tid] = 0u; }
    if (tid < SHRIKE_MAX_TOP_K) { ss.sel_key[tid] = 0u; ss.sel_id[tid] = 0u; }
    __syncthreads();
    if (warp < 4) {
        const uint32_t base = warp * 64;
        const uint32_t k0 = ss.keys[base + lane], k1 = ss.keys[base + 32 + lane];
        uint32_t r0a = 0, r0b = 0, r1a = 0, r1b = 0;
        const uint4* kv = (const uint4*)(ss.keys + base);
#pragma unroll
        for (uint32_t j4 = 0; j4 < 16; ++j4) {
            const uint4 v = kv[j4];
            const uint32_t kj[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (uint32_t q = 0; q < 4; ++q) {
                const uint32_t j = 4 * j4 + q;
                const uint32_t b0 = (kj[q] > k0 || (kj[q] == k0 && j < lane)) ? 1u : 0u;
                const uint32_t b1 = (kj[q] > k1 || (kj[q] == k1 && j < lane + 32u)) ? 1u : 0u;
                if (q & 1) { r0b += b0; r1b += b1; } else { r0a += b0; r1a += b1; }
            }
        }
        const uint32_t r0 = r0a + r0b, r1 = r1a + r1b;
        if (k0 != 0u && r0 < 8u) { ss.cand_key[warp * 8 + r0] = k0; ss.cand_id[warp * 8 + r0] = base + lane; }
        if (k1 != 0u && r1 < 8u) { ss.cand_key[warp * 8 + r1] = k1; ss.cand_id[warp * 8 + r1] = base + 32 + lane; }
    }
    __syncthreads();
    out_id = 0;
    out_w = 0.f;
    if (warp == 0) {
        const uint32_t ck = ss.cand_key[lane], ci = ss.cand_id[lane];
        uint32_t rank = 0;
#pragma unroll
        for (uint32_t j = 0; j < 32; ++j) {
            const uint32_t okey = __shfl_sync(0xffffffffu, ck, j), oid = __shfl_sync(0xffffffffu, ci, j);
            rank += (okey > ck || (okey == ck && oid < ci)) ? 1u : 0u;
        }
        if (ck != 0u && rank < a.top_k) { ss.sel_key[rank] = ck; ss.sel_id[rank] = ci; }
        __syncwarp();
        float my_score = 0.f;
        uint32_t my_id = 0;
        if (lane < a.top_k) {
            my_score = score_of_key(ss.sel_key[lane]);
            my_id = ss.sel_id[lane];
        }
        out_w = selection_weight<CG>(lg, a, lane, my_score, my_id);
        out_id = my_id;
    }
    __syncthreads();   // the scratch is reused by the next row
}


}  // namespace shrike
