// The router's dot products, shared by the router kernels and the fused decode-layer kernel.
//
// Selection must agree with the CPU restatement bit for bit, so every logit is summed in one fixed
// order: a warp owns an expert row, lane l accumulates its elements sequentially with fused
// multiply-adds, and the 32 lane sums are combined by a butterfly (xor 16, 8, 4, 2, 1). fp32 rows:
// lane l takes the float4 chunks l, l+32, ...; affine rows (router_gemv_body, moe.metal:324-364):
// lane l takes elements 64g+2l, 64g+2l+1 of every group g, as the shader does.
#pragma once

#include "internal.h"

namespace shrike {

constexpr int kRouterMaxChunks = 23;  // d <= 2944 (the reference stages at most 2880, moe.metal:11)

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

// N chunks per lane; PRED: the row may be shorter than 32*N chunks.
template <int N, bool PRED>
__device__ __forceinline__ void load_row_f32(const float* row, uint32_t chunks, uint32_t lane, float4 (&wr)[N]) {
#pragma unroll
    for (int i = 0; i < N; ++i) {
        const uint32_t c = lane + 32 * i;
        if (!PRED || c < chunks) {
            // a volatile load: it must stay ahead of the dependency wait that follows the prefetch
            const uint4 v = ldg_stream_u128((const float4*)row + c);
            wr[i] = make_float4(__uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z), __uint_as_float(v.w));
        }
    }
}

// One lane's share of an fp32 row against one activation row: float4 chunks
// lane, lane+32, ... in order, four fused multiply-adds each. The activation
// chunks are fetched eight at a time ahead of the arithmetic: issued one by
// one between the dependent multiply-adds they cost one L2 round trip each.
template <int N, bool PRED>
__device__ __forceinline__ float lane_dot_f32(const float4 (&wr)[N], uint32_t chunks, uint32_t lane,
                                              const void* xrow, uint32_t dt, const uint16_t* eff_scale) {
    float acc = 0.f;
    constexpr int kBatch = 8;
#pragma unroll
    for (int i0 = 0; i0 < N; i0 += kBatch) {
        uint4 raw[kBatch];
        uint2 es[kBatch];
#pragma unroll
        for (int j = 0; j < kBatch; ++j) {
            const int i = i0 + j;
            const uint32_t c = lane + 32 * i;
            raw[j] = make_uint4(0, 0, 0, 0);
            es[j] = make_uint2(0x3f803f80u, 0x3f803f80u);   // bf16 ones
            if (i < N && (!PRED || c < chunks)) {
                if (dt == SHRIKE_DTYPE_FP32) {
                    raw[j] = __ldg((const uint4*)xrow + c);
                } else {
                    const uint2 v = __ldg((const uint2*)xrow + c);
                    raw[j].x = v.x; raw[j].y = v.y;
                }
                if (eff_scale) es[j] = __ldg((const uint2*)eff_scale + c);
            }
        }
#pragma unroll
        for (int j = 0; j < kBatch; ++j) {
            const int i = i0 + j;
            const uint32_t c = lane + 32 * i;
            if (i < N && (!PRED || c < chunks)) {
                float x[4];
                if (dt == SHRIKE_DTYPE_FP32) {
                    x[0] = __uint_as_float(raw[j].x); x[1] = __uint_as_float(raw[j].y);
                    x[2] = __uint_as_float(raw[j].z); x[3] = __uint_as_float(raw[j].w);
                } else if (dt == SHRIKE_DTYPE_FP16) {
                    x[0] = f16_bits_to_f32(raw[j].x & 0xffff); x[1] = f16_bits_to_f32(raw[j].x >> 16);
                    x[2] = f16_bits_to_f32(raw[j].y & 0xffff); x[3] = f16_bits_to_f32(raw[j].y >> 16);
                } else {
                    x[0] = __uint_as_float(raw[j].x << 16); x[1] = __uint_as_float(raw[j].x & 0xffff0000u);
                    x[2] = __uint_as_float(raw[j].y << 16); x[3] = __uint_as_float(raw[j].y & 0xffff0000u);
                }
                if (eff_scale) {
                    x[0] = __fmul_rn(x[0], __uint_as_float(es[j].x << 16));
                    x[1] = __fmul_rn(x[1], __uint_as_float(es[j].x & 0xffff0000u));
                    x[2] = __fmul_rn(x[2], __uint_as_float(es[j].y << 16));
                    x[3] = __fmul_rn(x[3], __uint_as_float(es[j].y & 0xffff0000u));
                }
                acc = __fmaf_rn(wr[i].x, x[0], acc);
                acc = __fmaf_rn(wr[i].y, x[1], acc);
                acc = __fmaf_rn(wr[i].z, x[2], acc);
                acc = __fmaf_rn(wr[i].w, x[3], acc);
            }
        }
    }
    return acc;
}

// router_gemv_body (moe.metal:324-364): lane l takes elements 64g+2l, 64g+2l+1 of every group g.
// The operands of eight groups are requested before the first is used (one memory round trip per
// eight groups instead of one per group); the arithmetic and its order are the shader's.
__device__ __forceinline__ float lane_dot_affine(const uint8_t* row, const uint16_t* s_row,
                                                 const uint16_t* b_row, uint32_t bits, uint32_t groups,
                                                 uint32_t lane, const void* xrow, uint32_t dt,
                                                 const uint16_t* eff_scale) {
    float acc = 0.f;
    constexpr uint32_t kBatch = 8;
    for (uint32_t g0 = 0; g0 < groups; g0 += kBatch) {
        uint16_t sr[kBatch], br[kBatch];
        uint32_t qr[kBatch], er[kBatch];
        float x0r[kBatch], x1r[kBatch];
#pragma unroll
        for (uint32_t j = 0; j < kBatch; ++j) {
            const uint32_t gi = g0 + j;
            if (gi < groups) {
                const uint32_t idx = gi * 64 + lane * 2;
                sr[j] = s_row[gi];
                br[j] = b_row[gi];
                // both elements: one byte (int4) or two bytes (int8), the low one first
                qr[j] = bits == 4 ? (uint32_t)row[idx >> 1] : (uint32_t)*(const uint16_t*)(row + idx);
                if (dt == SHRIKE_DTYPE_FP32) {
                    const float2 v = *(const float2*)((const float*)xrow + idx);
                    x0r[j] = v.x; x1r[j] = v.y;
                } else {
                    const uint32_t v = *(const uint32_t*)((const uint16_t*)xrow + idx);
                    if (dt == SHRIKE_DTYPE_FP16) {
                        x0r[j] = f16_bits_to_f32(v & 0xffff); x1r[j] = f16_bits_to_f32(v >> 16);
                    } else {
                        x0r[j] = __uint_as_float(v << 16); x1r[j] = __uint_as_float(v & 0xffff0000u);
                    }
                }
                er[j] = eff_scale ? *(const uint32_t*)(eff_scale + idx) : 0x3f803f80u;
            }
        }
#pragma unroll
        for (uint32_t j = 0; j < kBatch; ++j) {
            const uint32_t gi = g0 + j;
            if (gi < groups) {
                const float sc = bf16_bits_to_f32(sr[j]);
                const float bi = bf16_bits_to_f32(br[j]);
                const float q0 = (float)(bits == 4 ? (qr[j] & 0xfu) : (qr[j] & 0xffu));
                const float q1 = (float)(bits == 4 ? (qr[j] >> 4) : (qr[j] >> 8));
                float x0 = x0r[j], x1 = x1r[j];
                if (eff_scale) {
                    x0 = __fmul_rn(x0, __uint_as_float(er[j] << 16));
                    x1 = __fmul_rn(x1, __uint_as_float(er[j] & 0xffff0000u));
                }
                acc = __fmaf_rn(sc, __fadd_rn(__fmul_rn(q0, x0), __fmul_rn(q1, x1)), acc);
                acc = __fmaf_rn(bi, __fadd_rn(x0, x1), acc);
            }
        }
    }
    return acc;
}

}  // namespace shrike
