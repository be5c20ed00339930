// Router: logits, top-k selection with renormalisation, residency lookup.
//
//   router_gemv_body            moe.metal:324-364   (affine rows)
//   router_topk_select_body     moe.metal:419-491
//   prefill_router_tiled_body   prefill.metal:446-563 (same arithmetic per row)
//   moe_classify_residency_body moe.metal:121-151
//
// Selection must agree with the CPU restatement bit for bit, so the logits are
// summed in one fixed order: a warp owns an expert row, lane l accumulates its
// elements sequentially with fused multiply-adds, and the 32 lane sums are
// combined by a butterfly (xor 16, 8, 4, 2, 1). fp32 rows: lane l takes the
// float4 chunks l, l+32, ... ; affine rows: lane l takes elements 64g+2l,
// 64g+2l+1 of every group g, as the shader does. exp() is a fixed sequence of
// fp32 operations (exp_det) instead of the library routine for the same reason.
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

__device__ __forceinline__ float butterfly_sum(float v) {
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, m));
    return v;
}

__device__ __forceinline__ void load_act4(const void* row, uint32_t c, uint32_t dt, float (&x)[4]) {
    if (dt == SHRIKE_DTYPE_FP32) {
        const float4 v = __ldg((const float4*)row + c);
        x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
    } else {
        const uint2 v = __ldg((const uint2*)row + c);
        if (dt == SHRIKE_DTYPE_FP16) {
            x[0] = f16_bits_to_f32(v.x & 0xffff); x[1] = f16_bits_to_f32(v.x >> 16);
            x[2] = f16_bits_to_f32(v.y & 0xffff); x[3] = f16_bits_to_f32(v.y >> 16);
        } else {
            x[0] = __uint_as_float(v.x << 16); x[1] = __uint_as_float(v.x & 0xffff0000u);
            x[2] = __uint_as_float(v.y << 16); x[3] = __uint_as_float(v.y & 0xffff0000u);
        }
    }
}

constexpr int kRouterMaxChunks = 23;  // d <= 2944 (the reference stages at most 2880, moe.metal:11)
constexpr int kRouterWarps = 4;       // rows per block, as router_gemv_r4

// grid (ceil((ne + has_gate)/4), token blocks); fp32 rows kept in registers and
// reused for every token of the block.
__global__ void __launch_bounds__(kRouterWarps * 32)
router_logits_f32_kernel(const float* __restrict__ w, const float* __restrict__ gate_row,
                         const uint16_t* __restrict__ eff_scale, const void* __restrict__ hidden,
                         uint32_t T, uint32_t stride, uint32_t dt, uint32_t ne, uint32_t d,
                         uint32_t tokens_per_block, float* __restrict__ logits,
                         float* __restrict__ gate_out) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t e = blockIdx.x * kRouterWarps + warp;
    const bool is_gate = gate_row != nullptr && e == ne;
    if (e >= ne && !is_gate) return;
    const float4* row = (const float4*)(is_gate ? gate_row : w + (size_t)e * d);
    const uint32_t chunks = d / 4;
    float4 wr[kRouterMaxChunks];
#pragma unroll
    for (int i = 0; i < kRouterMaxChunks; ++i) {
        const uint32_t c = lane + 32 * i;
        if (c < chunks) wr[i] = __ldg(row + c);
    }
    const uint32_t t0 = blockIdx.y * tokens_per_block;
    const uint32_t t1 = min(T, t0 + tokens_per_block);
    const size_t esz = dt == SHRIKE_DTYPE_FP32 ? 4 : 2;
    for (uint32_t tk = t0; tk < t1; ++tk) {
        const void* xrow = (const uint8_t*)hidden + (size_t)tk * stride * esz;
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < kRouterMaxChunks; ++i) {
            const uint32_t c = lane + 32 * i;
            if (c < chunks) {
                float x[4];
                load_act4(xrow, c, dt, x);
                if (eff_scale && !is_gate) {
                    const uint2 s = __ldg((const uint2*)eff_scale + c);
                    x[0] = __fmul_rn(x[0], __uint_as_float(s.x << 16));
                    x[1] = __fmul_rn(x[1], __uint_as_float(s.x & 0xffff0000u));
                    x[2] = __fmul_rn(x[2], __uint_as_float(s.y << 16));
                    x[3] = __fmul_rn(x[3], __uint_as_float(s.y & 0xffff0000u));
                }
                acc = __fmaf_rn(wr[i].x, x[0], acc);
                acc = __fmaf_rn(wr[i].y, x[1], acc);
                acc = __fmaf_rn(wr[i].z, x[2], acc);
                acc = __fmaf_rn(wr[i].w, x[3], acc);
            }
        }
        acc = butterfly_sum(acc);
        if (lane == 0) {
            if (is_gate) gate_out[tk] = sigmoid_det(acc);
            else logits[(size_t)tk * ne + e] = acc;
        }
    }
}

__device__ __forceinline__ uint32_t affine_value(const uint8_t* packed, uint32_t element, uint32_t bits) {
    const uint32_t bit = element * bits, byte = bit >> 3, shift = bit & 7u;
    uint32_t word = packed[byte];
    if (shift + bits > 8u) word |= ((uint32_t)packed[byte + 1u]) << 8;
    return (word >> shift) & ((1u << bits) - 1u);
}

// Affine int8/int4 rows, group 64, bf16 scales/biases: router_gemv_body.
__global__ void __launch_bounds__(kRouterWarps * 32)
router_logits_affine_kernel(const uint8_t* __restrict__ w, const uint16_t* __restrict__ scales,
                            const uint16_t* __restrict__ biases, uint32_t bits,
                            const float* __restrict__ gate_row,
                            const uint16_t* __restrict__ eff_scale, const void* __restrict__ hidden,
                            uint32_t T, uint32_t stride, uint32_t dt, uint32_t ne, uint32_t d,
                            uint32_t tokens_per_block, float* __restrict__ logits,
                            float* __restrict__ gate_out) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t e = blockIdx.x * kRouterWarps + warp;
    const bool is_gate = gate_row != nullptr && e == ne;
    if (e >= ne && !is_gate) return;
    const uint32_t groups = d / 64;
    const uint32_t t0 = blockIdx.y * tokens_per_block;
    const uint32_t t1 = min(T, t0 + tokens_per_block);
    const size_t esz = dt == SHRIKE_DTYPE_FP32 ? 4 : 2;
    for (uint32_t tk = t0; tk < t1; ++tk) {
        const void* xrow = (const uint8_t*)hidden + (size_t)tk * stride * esz;
        float acc = 0.f;
        if (is_gate) {
            // the scalar gate row is fp32: lane-strided float4 chunks as above
            for (uint32_t c = lane; c < d / 4; c += 32) {
                float x[4];
                load_act4(xrow, c, dt, x);
                const float4 g4 = __ldg((const float4*)gate_row + c);
                acc = __fmaf_rn(g4.x, x[0], acc); acc = __fmaf_rn(g4.y, x[1], acc);
                acc = __fmaf_rn(g4.z, x[2], acc); acc = __fmaf_rn(g4.w, x[3], acc);
            }
        } else {
            const uint8_t* row = w + (size_t)e * (d * bits / 8);
            for (uint32_t gi = 0; gi < groups; ++gi) {
                const float s = bf16_bits_to_f32(scales[e * groups + gi]);
                const float b = bf16_bits_to_f32(biases[e * groups + gi]);
                const uint32_t idx = gi * 64 + lane * 2;
                const float q0 = (float)affine_value(row, idx, bits);
                const float q1 = (float)affine_value(row, idx + 1, bits);
                float x0 = load_act(xrow, idx, dt), x1 = load_act(xrow, idx + 1, dt);
                if (eff_scale) {
                    x0 = __fmul_rn(x0, bf16_bits_to_f32(eff_scale[idx]));
                    x1 = __fmul_rn(x1, bf16_bits_to_f32(eff_scale[idx + 1]));
                }
                acc = __fmaf_rn(s, __fadd_rn(__fmul_rn(q0, x0), __fmul_rn(q1, x1)), acc);
                acc = __fmaf_rn(b, __fadd_rn(x0, x1), acc);
            }
        }
        acc = butterfly_sum(acc);
        if (lane == 0) {
            if (is_gate) gate_out[tk] = sigmoid_det(acc);
            else logits[(size_t)tk * ne + e] = acc;
        }
    }
}

// One warp per row. The (score desc, expert asc) order is total, so K rounds
// of a warp arg-max give exactly the list the reference's insertion scan
// builds (moe.metal:436-456).
__global__ void __launch_bounds__(128)
router_select_kernel(const float* __restrict__ logits, const uint16_t* __restrict__ logit_bias,
                     const uint16_t* __restrict__ per_expert_scale, uint32_t T, uint32_t ne,
                     uint32_t top_k, uint32_t sigmoid_scores, float scaling, uint32_t round_f16,
                     uint32_t* __restrict__ out_ids, float* __restrict__ out_w) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t row = blockIdx.x * 4 + warp;
    if (row >= T) return;
    const float* lg = logits + (size_t)row * ne;
    float sc[8];
    uint32_t taken = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t e = lane + 32 * i;
        float s = -INFINITY;
        if (e < ne) {
            const float raw = lg[e];
            const float b = logit_bias ? bf16_bits_to_f32(logit_bias[e]) : 0.0f;
            s = __fadd_rn(sigmoid_scores ? sigmoid_det(raw) : raw, b);
        } else {
            taken |= 1u << i;
        }
        sc[i] = s;
    }
    float my_score = 0.f;   // lane r keeps the r-th selection
    uint32_t my_id = 0;
    for (uint32_t r = 0; r < top_k; ++r) {
        float best = -INFINITY;
        uint32_t best_e = 0xffffffffu;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t e = lane + 32 * i;
            if (!(taken & (1u << i)) && (best_e == 0xffffffffu || sc[i] > best)) {
                best = sc[i];
                best_e = e;   // ascending e within a lane: ties keep the lower id
            }
        }
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) {
            const float os = __shfl_xor_sync(0xffffffffu, best, m);
            const uint32_t oe = __shfl_xor_sync(0xffffffffu, best_e, m);
            if (oe != 0xffffffffu && (best_e == 0xffffffffu || os > best || (os == best && oe < best_e))) {
                best = os;
                best_e = oe;
            }
        }
        if (best_e != 0xffffffffu && (best_e & 31u) == lane) taken |= 1u << (best_e >> 5);
        if (lane == r) { my_score = best; my_id = best_e == 0xffffffffu ? 0u : best_e; }
    }
    // weights (moe.metal:458-490), sums in rank order
    float val;
    if (sigmoid_scores) val = lane < top_k ? sigmoid_det(lg[my_id]) : 0.f;
    else {
        const float mx = __shfl_sync(0xffffffffu, my_score, 0);
        val = lane < top_k ? exp_det(__fsub_rn(my_score, mx)) : 0.f;
    }
    float sum = 0.f;
    for (uint32_t r = 0; r < top_k; ++r) sum = __fadd_rn(sum, __shfl_sync(0xffffffffu, val, r));
    if (lane < top_k) {
        float w;
        if (sigmoid_scores) w = __fmul_rn(val, __fdiv_rn(scaling, __fadd_rn(sum, 1e-20f)));
        else w = __fdiv_rn(val, sum);
        const float pes = per_expert_scale ? bf16_bits_to_f32(per_expert_scale[my_id]) : 1.0f;
        w = __fmul_rn(w, pes);
        if (round_f16) w = __half2float(__float2half_rn(w));
        out_ids[(size_t)row * top_k + lane] = my_id;
        out_w[(size_t)row * top_k + lane] = w;
    }
}

// moe_classify_residency_body for T rows; one thread walks the pairs in order
// so that the miss lists keep router order.
__global__ void classify_kernel(const uint32_t* __restrict__ ids, const uint64_t* __restrict__ table,
                                uint32_t n_pairs, uint32_t ne, uint32_t* __restrict__ slots,
                                uint32_t* __restrict__ counts, uint32_t* __restrict__ miss_pos,
                                uint32_t* __restrict__ miss_exp) {
    __shared__ uint32_t s_miss[1024];
    uint32_t base = 0;
    for (uint32_t p0 = 0; p0 < n_pairs; p0 += blockDim.x) {
        const uint32_t p = p0 + threadIdx.x;
        bool miss = false;
        uint32_t e = 0;
        if (p < n_pairs) {
            e = min(ids[p], ne - 1u);
            const uint64_t word = table[e];
            const uint32_t slot = (uint32_t)(word & 0xffffffffu), state = (uint32_t)(word >> 32);
            const bool hit = state == 2u && slot != SHRIKE_SLOT_MISS;
            slots[p] = hit ? slot : SHRIKE_SLOT_MISS;
            miss = !hit;
        }
        s_miss[threadIdx.x] = miss ? 1u : 0u;
        const uint32_t chunk = __syncthreads_count(miss);
        if (miss && (miss_pos || miss_exp)) {
            uint32_t before = 0;
            for (uint32_t j = 0; j < threadIdx.x; ++j) before += s_miss[j];
            if (miss_pos) miss_pos[base + before] = p;
            if (miss_exp) miss_exp[base + before] = e;
        }
        base += chunk;
        __syncthreads();
    }
    if (threadIdx.x == 0 && counts) {
        counts[0] = n_pairs - base;
        counts[1] = base;
    }
}

cudaError_t launch_router(const shrike_moe* m, cudaStream_t st, const shrike_router_operands& ops,
                          const void* hidden, uint32_t T, uint32_t stride, uint32_t* ids,
                          float* weights, float* shared_gate) {
    const shrike_moe_config& c = m->cfg;
    const bool gate = ops.shared_gate != nullptr && shared_gate != nullptr;
    const uint32_t rows = c.num_experts + (gate ? 1u : 0u);
    uint32_t tpb = 1;
    if (T > 64) tpb = 32;
    else if (T > 8) tpb = 4;
    const dim3 grid((rows + kRouterWarps - 1) / kRouterWarps, (T + tpb - 1) / tpb);
    if (c.router_weight_bits == 0) {
        router_logits_f32_kernel<<<grid, kRouterWarps * 32, 0, st>>>(
            (const float*)ops.weights, gate ? ops.shared_gate : nullptr, ops.effective_scale, hidden, T,
            stride, c.act_dtype, c.num_experts, c.d, tpb, m->ws.logits, shared_gate);
    } else {
        router_logits_affine_kernel<<<grid, kRouterWarps * 32, 0, st>>>(
            (const uint8_t*)ops.weights, ops.scales, ops.biases, c.router_weight_bits,
            gate ? ops.shared_gate : nullptr, ops.effective_scale, hidden, T, stride, c.act_dtype,
            c.num_experts, c.d, tpb, m->ws.logits, shared_gate);
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    router_select_kernel<<<(T + 3) / 4, 128, 0, st>>>(
        m->ws.logits, ops.logit_bias, ops.per_expert_scale, T, c.num_experts, c.top_k,
        c.router_kind == SHRIKE_ROUTER_SIGMOID, c.routed_scaling, c.round_route_weights_f16, ids, weights);
    return cudaGetLastError();
}

cudaError_t launch_classify(const shrike_moe* m, cudaStream_t st, const uint32_t* ids,
                            const uint64_t* table, uint32_t T, uint32_t* slots, uint32_t* counts,
                            uint32_t* miss_pos, uint32_t* miss_exp) {
    classify_kernel<<<1, 1024, 0, st>>>(ids, table, T * m->cfg.top_k, m->cfg.num_experts, slots, counts,
                                        miss_pos, miss_exp);
    return cudaGetLastError();
}

}  // namespace shrike
