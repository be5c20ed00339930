// Shared device helpers: dtype conversion, PTX wrappers (mma.sync, bulk copy,
// mbarrier with bounded waits, streaming loads) and the handle's internals.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/shrike_b200.h"

namespace shrike {

// ---- status word ------------------------------------------------------------
// Kernels never trap or spin without bound: a wait that runs out records a
// code here and the kernel carries on to its exit.
enum : uint32_t { kStatusOk = 0, kStatusWaitTimeout = 1, kStatusBadIndex = 2, kStatusOperandRange = 3 };

__device__ __forceinline__ void report_status(uint32_t* status, uint32_t code) {
    if (status) atomicMax(status, code);
}

// ---- dtypes -----------------------------------------------------------------
__device__ __forceinline__ float bf16_bits_to_f32(uint16_t b) {
    return __uint_as_float(((uint32_t)b) << 16);
}
__device__ __forceinline__ float f16_bits_to_f32(uint16_t b) {
    return __half2float(__ushort_as_half(b));
}
template <int META>
__device__ __forceinline__ float meta_to_f32(uint16_t b) {
    return META == SHRIKE_DTYPE_FP16 ? f16_bits_to_f32(b) : bf16_bits_to_f32(b);
}

// Element `i` of an activation row of dtype `dt`, widened to fp32 exactly.
__device__ __forceinline__ float load_act(const void* p, size_t i, uint32_t dt) {
    if (dt == SHRIKE_DTYPE_FP32) return ((const float*)p)[i];
    if (dt == SHRIKE_DTYPE_FP16) return f16_bits_to_f32(((const uint16_t*)p)[i]);
    return bf16_bits_to_f32(((const uint16_t*)p)[i]);
}
__device__ __forceinline__ void store_act(void* p, size_t i, uint32_t dt, float v) {
    if (dt == SHRIKE_DTYPE_FP32) ((float*)p)[i] = v;
    else if (dt == SHRIKE_DTYPE_FP16) ((__half*)p)[i] = __float2half_rn(v);
    else ((__nv_bfloat16*)p)[i] = __float2bfloat16_rn(v);
}
// The value an activation store would leave behind (hidden += y adds the
// rounded y, as moe_phase2_finish does, moe.metal:889-893).
__device__ __forceinline__ float round_act(uint32_t dt, float v) {
    if (dt == SHRIKE_DTYPE_FP32) return v;
    if (dt == SHRIKE_DTYPE_FP16) return __half2float(__float2half_rn(v));
    return __bfloat162float(__float2bfloat16_rn(v));
}

// ---- loads ------------------------------------------------------------------
// Weight bytes are read exactly once per call: keep them out of L1.
__device__ __forceinline__ uint32_t ldg_stream_u32(const void* p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg_stream_u64(const void* p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];"
                 : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 ldg_stream_u128(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// ---- tensor core (legacy path used for the skinny decode tiles) -------------
// D(16x8,f32) += A(16x16,f16,row) * B(16x8,f16,col)
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;  // (a & b) | c
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

// ---- mbarrier + 1-D bulk copy (TMA engine, no tensor map, no multicast) ------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;"
                 ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// global -> shared; dst, src 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// Bounded wait: returns false (and the caller reports a timeout) instead of
// spinning forever if the copy never lands.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t it = 0; it < (1u << 20); ++it) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
        if (ok) return true;
        if (it > 4) __nanosleep(64);  // a waiting warp should not eat issue slots
    }
    return false;
}

// ---- cp.async (16-byte global -> shared copies issued by every lane) ---------
__device__ __forceinline__ void cp_async_16(uint32_t smem_addr, const void* gptr) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr), "l"(gptr) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

#ifdef SHRIKE_TRACE   // debug builds only: per-block timestamps
__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#endif

// ---- programmatic dependent launch ---------------------------------------
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// moe_hidden_activation / moe_glu, moe.metal:233-238, 280-288.
__device__ __forceinline__ float glu(float gate, float up, uint32_t activation) {
    if (activation == SHRIKE_ACT_CLAMPED_SWIGLU) {
        const float gc = fminf(gate, 7.0f);
        const float uc = fmaxf(-7.0f, fminf(up, 7.0f));
        return (gc / (1.0f + expf(-1.702f * gc))) * (uc + 1.0f);
    }
    if (activation == SHRIKE_ACT_GELU_TANH) {
        const float x3 = gate * gate * gate;
        float inner = 0.7978845608028654f * (gate + 0.044715f * x3);
        inner = fmaxf(-20.0f, fminf(inner, 20.0f));
        return (0.5f * gate * (1.0f + tanhf(inner))) * up;
    }
    return (gate / (1.0f + expf(-gate))) * up;
}

// ---- layout of the fp16 operand copies ------------------------------------
// The B operand of the skinny MMA tiles is a copy of the activation row in fp16
// whose aligned blocks of 8 elements are stored in the order the nibble
// unpacking produces them: position p of a block holds element kPerm8[p].
// int8 weights unpack in natural order and use the identity.
__host__ __device__ __forceinline__ uint32_t perm_index(uint32_t i, bool int4) {
    // inverse of {0,4,1,5,2,6,3,7}: element e sits at position kInv8[e]
    const uint32_t e = i & 7u;
    const uint32_t pos = int4 ? (((e & 3u) << 1) | (e >> 2)) : e;
    return (i & ~7u) | pos;
}


// Converts the aligned block of 8 activations `blk` of a row to the fp16
// operand layout and returns the sum of the 8 rounded values. Thread-to-block
// assignment is up to the caller; group sums are formed with xprep_group_sum.
// The tiles take fp16 operands: an activation whose magnitude exceeds the largest fp16 value is
// clamped to it and reported through the status word (kStatusOperandRange) instead of turning
// into an infinity.
constexpr float kHalfMax = 65504.0f;

// fp16 bits of an inter-phase activation (the reference keeps them in fp16 too, moe.metal:829): a magnitude
// beyond the fp16 range saturates and is reported like an out-of-range input.
__device__ __forceinline__ uint16_t act_to_half_bits(float v, uint32_t* status) {
    if (fabsf(v) > kHalfMax) {
        report_status(status, kStatusOperandRange);
        v = copysignf(kHalfMax, v);
    }
    return __half_as_ushort(__float2half_rn(v));
}

__device__ __forceinline__ float xprep_block8(const void* xrow, uint32_t blk, uint32_t dt, bool int4,
                                              uint16_t* xh_row, uint32_t* status) {
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = load_act(xrow, (size_t)blk * 8 + j, dt);
    if (dt != SHRIKE_DTYPE_FP16) {
        bool over = false;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (fabsf(v[j]) > kHalfMax) {   // false for NaN, which passes through
                over = true;
                v[j] = copysignf(kHalfMax, v[j]);
            }
        }
        if (over) report_status(status, kStatusOperandRange);
    }
    __half h[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) h[j] = __float2half_rn(v[j]);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) sum += __half2float(h[j]);
    uint16_t o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[perm_index(j, int4)] = __half_as_ushort(h[j]);
    uint4 pk;
    pk.x = o[0] | ((uint32_t)o[1] << 16); pk.y = o[2] | ((uint32_t)o[3] << 16);
    pk.z = o[4] | ((uint32_t)o[5] << 16); pk.w = o[6] | ((uint32_t)o[7] << 16);
    *(uint4*)(xh_row + (size_t)blk * 8) = pk;
    return sum;
}

// All rows' blocks, block index i = row * (d/8) + blk handled by consecutive
// threads [lo, hi) of the calling kernel (lo a multiple of 32 per warp), and
// the per-group sums: the group/8 consecutive lanes of a group add up with
// shuffles. Every lane of a warp must call this together.
__device__ __forceinline__ void xprep_item(const void* x, size_t row_stride_bytes, uint32_t d, uint32_t group,
                                           uint32_t dt, bool int4, uint32_t item, bool valid, uint16_t* xh,
                                           float* xsum, uint32_t* status, const uint32_t* row_map = nullptr,
                                           uint32_t n_rows = 0xffffffffu) {
    // row_map: row r of the call is row row_map[r] of x; rows from n_rows on carry no work
    const uint32_t per_row = d / 8;
    float sum = 0.f;
    uint32_t row = 0, blk = 0;
    if (valid) {
        row = item / per_row;
        blk = item - row * per_row;
        valid = row < n_rows;
    }
    if (valid) {
        const uint32_t src = row_map ? row_map[row] : row;
        sum = xprep_block8((const uint8_t*)x + (size_t)src * row_stride_bytes, blk, dt, int4, xh + (size_t)row * d,
                           status);
    }
    const uint32_t lanes = group / 8;  // 8 or 4 lanes per group
    for (uint32_t o = 1; o < lanes; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (valid && (blk & (lanes - 1)) == 0) xsum[(size_t)row * (d / group) + blk / lanes] = sum;
}

}  // namespace shrike
