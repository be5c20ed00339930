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
#include "plan.cuh"
#include "router_math.cuh"
#include "select.cuh"

namespace shrike {

constexpr int kRouterWarps = 8;       // expert rows per block (router_gemv_r4 has four); the block that finishes last
                                      // selects with as many warps

struct RouterArgs {
    const void* w;                 // fp32 rows, or packed affine rows
    const uint16_t* scales;        // affine only
    const uint16_t* biases;        // affine only
    uint32_t bits;                 // 0 = fp32
    const float* gate_row;         // shared expert scalar gate row or NULL
    const uint16_t* eff_scale;
    const uint16_t* logit_bias;
    const uint16_t* per_expert_scale;
    const void* hidden;
    uint32_t T, stride, dt, ne, d, top_k;
    uint32_t sigmoid_scores;
    float scaling;
    uint32_t round_f16;
    float* logits;
    uint32_t* ids;
    float* weights;
    float* gate_out;
    uint32_t tokens_per_block;
    uint32_t no_tail;              // fused decode: stop after the logits and the operand copy (the expert kernels route)
    uint32_t row_base;             // first row of this launch (the tiled prefill router leaves only the gate row)
    // fused decode tail (route_fused_kernel only)
    const uint64_t* table;
    uint32_t pool_cells;
    const uint32_t* io_status;
    uint32_t with_shared, int4, group;
    uint32_t* slots;
    uint32_t* counts;
    Instance* inst;
    uint32_t* n_inst;
    uint32_t* sorted;
    uint16_t* xh;
    float* xsum;
    uint32_t* done_counter;
    uint32_t* status;
    uint32_t max_inst;
};

// Logits (and the shared expert's scalar gate as row `ne`) of this warp's row
// for the block's tokens. `pre` runs between the weight-row prefetch and the
// first read of the activations.
template <int N, bool PRED, typename Pre>
__device__ __forceinline__ void logits_rows(const RouterArgs& a, Pre pre) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t e = a.row_base + blockIdx.x * kRouterWarps + warp;
    const bool is_gate = a.gate_row != nullptr && e == a.ne;
    const bool active = e < a.ne || is_gate;
    const bool f32row = a.bits == 0 || is_gate;
    const uint32_t chunks = a.d / 4, groups = a.d / 64;
    float4 wr[N];
    if (active && f32row)
        load_row_f32<N, PRED>(is_gate ? a.gate_row : (const float*)a.w + (size_t)e * a.d, chunks, lane, wr);
    pre();
    if (!active) return;
    const uint32_t t0 = blockIdx.y * a.tokens_per_block;
    const uint32_t t1 = min(a.T, t0 + a.tokens_per_block);
    const size_t esz = a.dt == SHRIKE_DTYPE_FP32 ? 4 : 2;
    for (uint32_t tk = t0; tk < t1; ++tk) {
        const void* xrow = (const uint8_t*)a.hidden + (size_t)tk * a.stride * esz;
        float acc;
        if (f32row) {
            acc = lane_dot_f32<N, PRED>(wr, chunks, lane, xrow, a.dt, is_gate ? nullptr : a.eff_scale);
        } else {
            acc = lane_dot_affine((const uint8_t*)a.w + (size_t)e * (a.d * a.bits / 8), a.scales + (size_t)e * groups,
                                  a.biases + (size_t)e * groups, a.bits, groups, lane, xrow, a.dt, a.eff_scale);
        }
        acc = butterfly_sum(acc);
        if (lane == 0) {
            if (is_gate) a.gate_out[tk] = sigmoid_det(acc);
            else a.logits[(size_t)tk * a.ne + e] = acc;
        }
    }
}

// The common hidden sizes get straight-line code without bounds checks.
template <typename Pre>
__device__ __forceinline__ void logits_body(const RouterArgs& a, Pre pre) {
    if (a.d == 2048) logits_rows<16, false>(a, pre);
    else if (a.d == 2304) logits_rows<18, false>(a, pre);
    else logits_rows<kRouterMaxChunks, true>(a, pre);
}

// Top-k of one row by one warp. The (score desc, expert asc) order is total,
// so K rounds of a warp arg-max give exactly the list the reference's
// insertion scan builds (moe.metal:436-456). Lane r returns the r-th pick.
// CG: read the logits past L1 (they were written by other blocks of this launch).
template <bool CG>
__device__ __forceinline__ void select_row(const float* lg, const RouterArgs& a, uint32_t lane,
                                           uint32_t& out_id, float& out_w) {
    const uint32_t ne = a.ne, top_k = a.top_k;
    // order-preserving integer keys (0 = not a candidate): one warp-wide max and one warp-wide min per pick
    uint32_t key[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) key[i] = selection_key<CG>(lg, a, lane + 32 * i);
    float my_score = 0.f;
    uint32_t my_id = 0;
    for (uint32_t r = 0; r < top_k; ++r) {
        uint32_t bestk = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) bestk = max(bestk, key[i]);
        const uint32_t wmax = __reduce_max_sync(0xffffffffu, bestk);
        uint32_t cand = 0xffffffffu;
#pragma unroll
        for (int i = 7; i >= 0; --i) cand = (key[i] == wmax && wmax != 0u) ? lane + 32u * i : cand;
        const uint32_t win = __reduce_min_sync(0xffffffffu, cand);  // ties: the lower expert id
        if (win != 0xffffffffu && (win & 31u) == lane) {
#pragma unroll
            for (int i = 0; i < 8; ++i) key[i] = (win >> 5) == (uint32_t)i ? 0u : key[i];
        }
        if (lane == r) {
            my_score = score_of_key(wmax);
            my_id = win == 0xffffffffu ? 0u : win;
        }
    }
    // weights (moe.metal:458-490), sums in rank order
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
    out_id = my_id;
    out_w = w;
}

// grid (ceil((ne + has_gate)/4), token blocks)
__global__ void __launch_bounds__(kRouterWarps * 32) router_logits_kernel(const RouterArgs a) {
    logits_body(a, [] {});
}

// ---- prefill router: register-tiled logits ---------------------------------------
//
// Hundreds of rows against the same fp32 router matrix: the warp-per-row kernel
// above re-reads every activation row once per expert row and stalls on those
// loads. Here a block owns 32 expert rows x 32 tokens, stages both operands in
// shared memory (activations converted to fp32 once per block), and a warp
// accumulates an 8 x 16 register tile. Lane l still owns the float4 chunks
// l, l+32, ... of every row and walks them in order with one fused multiply-add
// per element, and the 32 lane sums still meet in the xor 16..1 butterfly, so
// each logit is the same sequence of roundings as in the warp-per-row kernel.
// Chunks past the end of a row are staged as zeros: adding +0 changes nothing.
constexpr int kTileRows = 32, kTileTokens = 32, kTileStage = 256;   // 256 elements of K per stage
constexpr int kTileWarpRows = 8, kTileWarpTokens = 16;
constexpr size_t kTileSmemBytes = 2 * (size_t)(kTileRows + kTileTokens) * kTileStage * sizeof(float);

__device__ __forceinline__ void cp_async_16_zfill(uint32_t smem_addr, const void* gptr, bool valid) {
    const uint32_t n = valid ? 16u : 0u;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr), "l"(gptr), "r"(n) : "memory");
}

__global__ void __launch_bounds__(256, 1) router_logits_tiled_kernel(const RouterArgs a) {
    extern __shared__ __align__(16) float tile_smem[];
    float* const w_s = tile_smem;                                           // [2][32][256]
    float* const x_s = tile_smem + 2 * kTileRows * kTileStage;              // [2][32][256]
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t e0 = blockIdx.x * kTileRows, t0 = blockIdx.y * kTileTokens;
    const uint32_t chunks = a.d / 4;
    const uint32_t stages = (a.d + kTileStage - 1) / kTileStage;
    const size_t esz = a.dt == SHRIKE_DTYPE_FP32 ? 4 : 2;

    // staging roles: thread -> (row, 8 chunks of 4 floats) of each operand tile
    const uint32_t srow = tid >> 3, sc0 = (tid & 7) * 8;                    // 32 rows x 8 threads x 8 chunks
    const uint32_t wrow = min(e0 + srow, a.ne - 1), xtok = min(t0 + srow, a.T - 1);
    const float* const wsrc = (const float*)a.w + (size_t)wrow * a.d;
    const uint8_t* const xsrc = (const uint8_t*)a.hidden + (size_t)xtok * a.stride * esz;

    uint4 xr[8];   // the next stage's activations: 32 elements (16-bit) or 2 x 16 (fp32)
    auto fetch_w = [&](uint32_t s, uint32_t buf) {
        const uint32_t dst = (uint32_t)__cvta_generic_to_shared(w_s + ((size_t)buf * kTileRows + srow) * kTileStage);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t c = s * (kTileStage / 4) + sc0 + j;
            cp_async_16_zfill(dst + (sc0 + j) * 16, wsrc + (size_t)min(c, chunks - 1) * 4, c < chunks);
        }
        cp_async_commit();
    };
    auto fetch_x = [&](uint32_t s) {
        if (a.dt == SHRIKE_DTYPE_FP32) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t c = s * (kTileStage / 4) + sc0 + j;
                xr[j] = c < chunks ? __ldg((const uint4*)xsrc + c) : make_uint4(0, 0, 0, 0);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t c = s * (kTileStage / 4) + sc0 + 2 * j;       // two chunks per 16 bytes
                xr[j] = c < chunks ? __ldg((const uint4*)xsrc + c / 2) : make_uint4(0, 0, 0, 0);
            }
        }
    };
    auto store_x = [&](uint32_t s, uint32_t buf) {
        float4* const dst = (float4*)(x_s + ((size_t)buf * kTileTokens + srow) * kTileStage) + sc0;
        const uint2* const es = a.eff_scale ? (const uint2*)a.eff_scale + s * (kTileStage / 4) + sc0 : nullptr;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float4 v;
            if (a.dt == SHRIKE_DTYPE_FP32) {
                v = make_float4(__uint_as_float(xr[j].x), __uint_as_float(xr[j].y), __uint_as_float(xr[j].z),
                                __uint_as_float(xr[j].w));
            } else {
                const uint32_t lo = (j & 1) ? xr[j / 2].z : xr[j / 2].x, hi = (j & 1) ? xr[j / 2].w : xr[j / 2].y;
                if (a.dt == SHRIKE_DTYPE_FP16)
                    v = make_float4(f16_bits_to_f32(lo & 0xffff), f16_bits_to_f32(lo >> 16), f16_bits_to_f32(hi & 0xffff),
                                    f16_bits_to_f32(hi >> 16));
                else
                    v = make_float4(__uint_as_float(lo << 16), __uint_as_float(lo & 0xffff0000u),
                                    __uint_as_float(hi << 16), __uint_as_float(hi & 0xffff0000u));
            }
            if (es && s * (kTileStage / 4) + sc0 + j < chunks) {
                const uint2 q = __ldg(es + j);
                v.x = __fmul_rn(v.x, __uint_as_float(q.x << 16));
                v.y = __fmul_rn(v.y, __uint_as_float(q.x & 0xffff0000u));
                v.z = __fmul_rn(v.z, __uint_as_float(q.y << 16));
                v.w = __fmul_rn(v.w, __uint_as_float(q.y & 0xffff0000u));
            }
            dst[j] = v;
        }
    };

    float acc[kTileWarpRows][kTileWarpTokens];
#pragma unroll
    for (int r = 0; r < kTileWarpRows; ++r)
#pragma unroll
        for (int t = 0; t < kTileWarpTokens; ++t) acc[r][t] = 0.f;

    fetch_w(0, 0);
    fetch_x(0);
    store_x(0, 0);
    cp_async_wait<0>();
    __syncthreads();

    const uint32_t rg = warp & 3, tg = warp >> 2;
    for (uint32_t s = 0; s < stages; ++s) {
        const uint32_t buf = s & 1;
        const bool more = s + 1 < stages;
        if (more) {
            fetch_w(s + 1, buf ^ 1);
            fetch_x(s + 1);
        }
        const float4* const wb = (const float4*)(w_s + ((size_t)buf * kTileRows + rg * kTileWarpRows) * kTileStage);
        const float4* const xb = (const float4*)(x_s + ((size_t)buf * kTileTokens + tg * kTileWarpTokens) * kTileStage);
#pragma unroll
        for (int ii = 0; ii < kTileStage / 128; ++ii) {
            float4 wv[kTileWarpRows];
#pragma unroll
            for (int r = 0; r < kTileWarpRows; ++r) wv[r] = wb[r * (kTileStage / 4) + ii * 32 + lane];
#pragma unroll
            for (int t = 0; t < kTileWarpTokens; ++t) {
                const float4 xv = xb[t * (kTileStage / 4) + ii * 32 + lane];
#pragma unroll
                for (int r = 0; r < kTileWarpRows; ++r) {
                    float v = acc[r][t];
                    v = __fmaf_rn(wv[r].x, xv.x, v);
                    v = __fmaf_rn(wv[r].y, xv.y, v);
                    v = __fmaf_rn(wv[r].z, xv.z, v);
                    v = __fmaf_rn(wv[r].w, xv.w, v);
                    acc[r][t] = v;
                }
            }
        }
        if (more) {
            store_x(s + 1, buf ^ 1);
            cp_async_wait<0>();
        }
        __syncthreads();
    }

    // butterfly, then lane 2t + (r / 4) stores the four logits (r & ~3 .. +3) of token t
    float4 out = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int t = 0; t < kTileWarpTokens; ++t)
#pragma unroll
        for (int r = 0; r < kTileWarpRows; ++r) {
            const float v = butterfly_sum(acc[r][t]);
            if (lane == (uint32_t)(2 * t + r / 4)) {
                if ((r & 3) == 0) out.x = v;
                else if ((r & 3) == 1) out.y = v;
                else if ((r & 3) == 2) out.z = v;
                else out.w = v;
            }
        }
    const uint32_t tok = t0 + tg * kTileWarpTokens + (lane >> 1);
    const uint32_t e = e0 + rg * kTileWarpRows + (lane & 1) * 4;
    if (tok < a.T) {
        float* const dst = a.logits + (size_t)tok * a.ne + e;
        if (e + 4 <= a.ne && (a.ne & 3u) == 0) {
            *(float4*)dst = out;
        } else {
            if (e + 0 < a.ne) dst[0] = out.x;
            if (e + 1 < a.ne) dst[1] = out.y;
            if (e + 2 < a.ne) dst[2] = out.z;
            if (e + 3 < a.ne) dst[3] = out.w;
        }
    }
}

// The same tile for 16-bit activations without a per-column scale (the common case): both operands go to
// shared memory by cp.async, three stages deep, the activations as they are (half the bytes), and are widened
// where they are multiplied -- exact, so the logits are unchanged. Thread t of a row's eight copies 16-byte
// units t, t + 8, ...: a warp's copies land 128 bytes a row, free of bank conflicts. (The kernel above holds
// the next stage's activations in registers across the multiply loop; the compiler sinks those loads to their
// use, and a block of 8 warps then waits for L2 once per stage.)
constexpr uint32_t kTile16WBytes = kTileRows * kTileStage * 4, kTile16XBytes = kTileTokens * kTileStage * 2;
constexpr uint32_t kTile16Buf = kTile16WBytes + kTile16XBytes, kTile16Bufs = 3;
constexpr size_t kTile16SmemBytes = (size_t)kTile16Bufs * kTile16Buf;

template <bool FP16>
__global__ void __launch_bounds__(256, 1) router_logits_tiled16_kernel(const RouterArgs a) {
    extern __shared__ __align__(16) uint8_t tile16_smem[];
    const uint32_t smem0 = (uint32_t)__cvta_generic_to_shared(tile16_smem);
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t e0 = blockIdx.x * kTileRows, t0 = blockIdx.y * kTileTokens;
    const uint32_t chunks = a.d / 4, units = a.d / 8;   // float4 chunks of a weight row, 16-byte units of an activation row
    const uint32_t stages = (a.d + kTileStage - 1) / kTileStage;
    const uint32_t srow = tid >> 3, l8 = tid & 7;
    const float* const wsrc = (const float*)a.w + (size_t)min(e0 + srow, a.ne - 1) * a.d;
    const uint8_t* const xsrc = (const uint8_t*)a.hidden + (size_t)min(t0 + srow, a.T - 1) * a.stride * 2;

    auto fetch = [&](uint32_t s, uint32_t buf) {
        const uint32_t wdst = smem0 + buf * kTile16Buf + srow * (kTileStage * 4);
#pragma unroll
        for (uint32_t j = 0; j < 8; ++j) {
            const uint32_t u = j * 8 + l8, c = s * (kTileStage / 4) + u;
            cp_async_16_zfill(wdst + u * 16, wsrc + (size_t)min(c, chunks - 1) * 4, c < chunks);
        }
        const uint32_t xdst = smem0 + buf * kTile16Buf + kTile16WBytes + srow * (kTileStage * 2);
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) {
            const uint32_t u = j * 8 + l8, c = s * (kTileStage / 8) + u;
            cp_async_16_zfill(xdst + u * 16, xsrc + (size_t)min(c, units - 1) * 16, c < units);
        }
        cp_async_commit();
    };

    float acc[kTileWarpRows][kTileWarpTokens];
#pragma unroll
    for (int r = 0; r < kTileWarpRows; ++r)
#pragma unroll
        for (int t = 0; t < kTileWarpTokens; ++t) acc[r][t] = 0.f;

    fetch(0, 0);
    if (stages > 1) fetch(1, 1);
    const uint32_t rg = warp & 3, tg = warp >> 2;
    for (uint32_t s = 0; s < stages; ++s) {
        const uint32_t buf = s % kTile16Bufs;
        if (s + 1 < stages) cp_async_wait<1>();
        else cp_async_wait<0>();
        __syncthreads();   // stage s has landed for every thread, and every warp is done with stage s - 1
        if (s + 2 < stages) fetch(s + 2, (s + 2) % kTile16Bufs);
        const float4* const wb = (const float4*)(tile16_smem + (size_t)buf * kTile16Buf) + rg * kTileWarpRows * (kTileStage / 4);
        const uint2* const xb = (const uint2*)(tile16_smem + (size_t)buf * kTile16Buf + kTile16WBytes) + tg * kTileWarpTokens * (kTileStage / 4);
#pragma unroll
        for (int ii = 0; ii < kTileStage / 128; ++ii) {
            float4 wv[kTileWarpRows];
#pragma unroll
            for (int r = 0; r < kTileWarpRows; ++r) wv[r] = wb[r * (kTileStage / 4) + ii * 32 + lane];
#pragma unroll
            for (int t = 0; t < kTileWarpTokens; ++t) {
                const uint2 q = xb[t * (kTileStage / 4) + ii * 32 + lane];
                float4 xv;
                if (FP16)
                    xv = make_float4(f16_bits_to_f32(q.x & 0xffff), f16_bits_to_f32(q.x >> 16), f16_bits_to_f32(q.y & 0xffff),
                                     f16_bits_to_f32(q.y >> 16));
                else
                    xv = make_float4(__uint_as_float(q.x << 16), __uint_as_float(q.x & 0xffff0000u), __uint_as_float(q.y << 16),
                                     __uint_as_float(q.y & 0xffff0000u));
#pragma unroll
                for (int r = 0; r < kTileWarpRows; ++r) {
                    float v = acc[r][t];
                    v = __fmaf_rn(wv[r].x, xv.x, v);
                    v = __fmaf_rn(wv[r].y, xv.y, v);
                    v = __fmaf_rn(wv[r].z, xv.z, v);
                    v = __fmaf_rn(wv[r].w, xv.w, v);
                    acc[r][t] = v;
                }
            }
        }
    }

    // butterfly, then lane 2t + (r / 4) stores the four logits (r & ~3 .. +3) of token t
    float4 out = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int t = 0; t < kTileWarpTokens; ++t)
#pragma unroll
        for (int r = 0; r < kTileWarpRows; ++r) {
            const float v = butterfly_sum(acc[r][t]);
            if (lane == (uint32_t)(2 * t + r / 4)) {
                if ((r & 3) == 0) out.x = v;
                else if ((r & 3) == 1) out.y = v;
                else if ((r & 3) == 2) out.z = v;
                else out.w = v;
            }
        }
    const uint32_t tok = t0 + tg * kTileWarpTokens + (lane >> 1);
    const uint32_t e = e0 + rg * kTileWarpRows + (lane & 1) * 4;
    if (tok < a.T) {
        float* const dst = a.logits + (size_t)tok * a.ne + e;
        if (e + 4 <= a.ne && (a.ne & 3u) == 0) {
            *(float4*)dst = out;
        } else {
            if (e + 0 < a.ne) dst[0] = out.x;
            if (e + 1 < a.ne) dst[1] = out.y;
            if (e + 2 < a.ne) dst[2] = out.z;
            if (e + 3 < a.ne) dst[3] = out.w;
        }
    }
}

// The shared expert's scalar gate for many rows (the tiled router covers the expert rows only): one
// warp per row of activations at a time, the gate row held in registers, the same lane order, fused
// multiply-adds and butterfly as everywhere else. grid ceil(T / 32), block 256: a warp takes 4 rows.
__global__ void __launch_bounds__(256) router_gate_rows_kernel(const RouterArgs a) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t chunks = a.d / 4;
    const size_t esz = a.dt == SHRIKE_DTYPE_FP32 ? 4 : 2;
    float4 wr[kRouterMaxChunks];
    load_row_f32<kRouterMaxChunks, true>(a.gate_row, chunks, lane, wr);
    for (uint32_t j = 0; j < 4; ++j) {
        const uint32_t tk = blockIdx.x * 32 + warp * 4 + j;
        if (tk >= a.T) break;
        const void* xrow = (const uint8_t*)a.hidden + (size_t)tk * a.stride * esz;
        const float acc = butterfly_sum(lane_dot_f32<kRouterMaxChunks, true>(wr, chunks, lane, xrow, a.dt, nullptr));
        if (lane == 0) a.gate_out[tk] = sigmoid_det(acc);
    }
}

__global__ void __launch_bounds__(128) router_select_kernel(const RouterArgs a) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t row = blockIdx.x * 4 + warp;
    if (row >= a.T) return;
    uint32_t id;
    float w;
    select_row<false>(a.logits + (size_t)row * a.ne, a, lane, id, w);
    if (lane < a.top_k) {
        a.ids[(size_t)row * a.top_k + lane] = id;
        a.weights[(size_t)row * a.top_k + lane] = w;
    }
}

// Decode (T <= 64) in one launch: logits by all blocks; the block that
// finishes last then selects, looks the experts up in the residency table and
// builds the work lists -- no wait on another block anywhere. Every block also
// converts its slice of the activation rows to the fp16 operand layout.
// grid (ceil((ne + has_gate)/4), 1..4 token groups).
__global__ void __launch_bounds__(kRouterWarps * 32) route_fused_kernel(const RouterArgs a) {
    __shared__ PlanSmem sm;
    __shared__ uint32_t ids_sm[kPlanMaxPairs];
    __shared__ SelectSmem sel;
    __shared__ uint32_t s_last, s_miss;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // the weight rows do not depend on the previous kernel: fetch them first
    logits_body(a, [&] {
        pdl_wait();
        pdl_launch_dependents();
    });

    // every block converts its share of the activation rows (blocks of 8 elements)
    {
        const uint32_t items = a.T * (a.d / 8);
        const size_t esz = a.dt == SHRIKE_DTYPE_FP32 ? 4 : 2;
        const uint32_t n_blocks = gridDim.x * gridDim.y, block = blockIdx.y * gridDim.x + blockIdx.x;
        for (uint32_t i0 = block * blockDim.x; i0 < items; i0 += n_blocks * blockDim.x)
            xprep_item(a.hidden, (size_t)a.stride * esz, a.d, a.group, a.dt, a.int4 != 0, i0 + tid, i0 + tid < items,
                       a.xh, a.xsum, a.status);
    }

    if (a.no_tail) return;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const uint32_t ticket = atomicAdd(a.done_counter, 1u);
        s_last = ticket == gridDim.x * gridDim.y - 1 ? 1u : 0u;
        if (s_last) *a.done_counter = 0;
        s_miss = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();

    if (a.T == 1) {
        // one row: the whole block ranks it (no serial rounds)
        uint32_t id;
        float w;
        select_row_block(a.logits, a, sel, id, w);
        if (warp == 0 && lane < a.top_k) {
            a.ids[lane] = id;
            a.weights[lane] = w;
            ids_sm[lane] = id;
        }
    } else {
        // several rows: a warp per row, the rows side by side (the same picks and weights: both forms build the
        // list of the reference's insertion scan)
        for (uint32_t row = warp; row < a.T; row += kRouterWarps) {
            uint32_t id;
            float w;
            select_row<true>(a.logits + (size_t)row * a.ne, a, lane, id, w);
            if (lane < a.top_k) {
                a.ids[(size_t)row * a.top_k + lane] = id;
                a.weights[(size_t)row * a.top_k + lane] = w;
                ids_sm[row * a.top_k + lane] = id;
            }
        }
    }
    __syncthreads();
    bool ready = true;
    if (a.io_status) {
        const uint32_t s = *a.io_status;
        ready = s == 1u || s == 3u;
    }
    const uint32_t n_pairs = a.T * a.top_k;
    uint32_t misses = 0;
    for (uint32_t p = tid; p < n_pairs; p += blockDim.x) {
        const uint32_t e = min(ids_sm[p], a.ne - 1u);
        const uint64_t word = a.table[e];
        uint32_t slot = (uint32_t)(word & 0xffffffffu);
        const bool hit = (uint32_t)(word >> 32) == 2u && slot != SHRIKE_SLOT_MISS;
        if (!hit) { slot = SHRIKE_SLOT_MISS; ++misses; }
        if (a.slots) a.slots[p] = slot;
        if (slot != SHRIKE_SLOT_MISS && slot >= a.pool_cells) {
            report_status(a.status, kStatusBadIndex);
            slot = SHRIKE_SLOT_MISS;
        }
        sm.key[p] = ready ? slot : SHRIKE_SLOT_MISS;
    }
    if (misses) atomicAdd(&s_miss, misses);
    __syncthreads();
    if (tid == 0 && a.counts) {
        a.counts[0] = n_pairs - s_miss;
        a.counts[1] = s_miss;
    }
    // One row: every pair is its own instance; order them by cell as plan_body
    // would, with eight shuffles instead of the block-wide sort.
    bool fast = false;
    if (a.T == 1) {
        const uint32_t my = lane < n_pairs ? sm.key[lane] : SHRIKE_SLOT_MISS;
        uint32_t rank = 0;
        bool dup = false;
        for (uint32_t j = 0; j < n_pairs; ++j) {
            const uint32_t o = __shfl_sync(0xffffffffu, my, j);
            if (my != SHRIKE_SLOT_MISS && o != SHRIKE_SLOT_MISS) {
                rank += (o < my || (o == my && j < lane)) ? 1u : 0u;
                dup |= (o == my && j != lane);
            }
        }
        fast = !__any_sync(0xffffffffu, dup);  // same answer in every warp
        if (fast && warp == 0) {
            const uint32_t n_routed = __popc(__ballot_sync(0xffffffffu, my != SHRIKE_SLOT_MISS));
            if (my != SHRIKE_SLOT_MISS) {
                Instance in;
                in.kind = 0; in.slot = my; in.first = rank; in.count = 1;
                for (int q = 0; q < 8; ++q) in.pair[q] = lane;
                a.inst[rank] = in;
                a.sorted[rank] = lane;
            }
            if (lane == 0) {
                if (a.with_shared) {
                    Instance in;
                    in.kind = 1; in.slot = 0; in.first = 0; in.count = 1;
                    for (int q = 0; q < 8; ++q) in.pair[q] = 0;
                    a.inst[n_routed] = in;
                }
                *a.n_inst = n_routed + (a.with_shared ? 1u : 0u);
            }
        }
    }
    if (!fast) plan_body(sm, n_pairs, a.T, a.with_shared, a.inst, a.n_inst, a.sorted, a.max_inst, a.status);
}

// moe_classify_residency_body for T rows. The miss lists keep router order: block b takes pairs
// [1024 b, 1024 b + 1024) and first counts the misses of all the pairs before them itself (independent loads,
// no hand-over between blocks), so its misses go to their final places.
__global__ void __launch_bounds__(1024) classify_kernel(const uint32_t* __restrict__ ids, const uint64_t* __restrict__ table,
                                                        uint32_t n_pairs, uint32_t ne, uint32_t* __restrict__ slots,
                                                        uint32_t* __restrict__ counts, uint32_t* __restrict__ miss_pos,
                                                        uint32_t* __restrict__ miss_exp) {
    __shared__ uint32_t s_miss[1024];
    __shared__ uint32_t s_base;
    auto lookup = [&](uint32_t p, uint32_t& e, uint32_t& slot) {
        e = min(ids[p], ne - 1u);
        const uint64_t word = table[e];
        slot = (uint32_t)(word & 0xffffffffu);
        return (uint32_t)(word >> 32) == 2u && slot != SHRIKE_SLOT_MISS;
    };
    if (threadIdx.x == 0) s_base = 0;
    __syncthreads();
    uint32_t before_me = 0;
#pragma unroll 4
    for (uint32_t j = 0; j < blockIdx.x; ++j) {
        uint32_t e, slot;
        before_me += lookup(j * 1024u + threadIdx.x, e, slot) ? 0u : 1u;
    }
    for (int o = 16; o; o >>= 1) before_me += __shfl_xor_sync(0xffffffffu, before_me, o);
    if ((threadIdx.x & 31u) == 0 && before_me) atomicAdd(&s_base, before_me);
    const uint32_t p = blockIdx.x * 1024u + threadIdx.x;
    bool miss = false;
    uint32_t e = 0;
    if (p < n_pairs) {
        uint32_t slot;
        const bool hit = lookup(p, e, slot);
        slots[p] = hit ? slot : SHRIKE_SLOT_MISS;
        miss = !hit;
    }
    s_miss[threadIdx.x] = miss ? 1u : 0u;
    const uint32_t chunk = __syncthreads_count(miss);
    const uint32_t base = s_base;
    if (miss && (miss_pos || miss_exp)) {
        uint32_t before = 0;
        for (uint32_t j = 0; j < threadIdx.x; ++j) before += s_miss[j];
        if (miss_pos) miss_pos[base + before] = p;
        if (miss_exp) miss_exp[base + before] = e;
    }
    if (threadIdx.x == 0 && counts && blockIdx.x == gridDim.x - 1) {
        counts[0] = n_pairs - (base + chunk);
        counts[1] = base + chunk;
    }
}

static RouterArgs make_router_args(const shrike_moe* m, const shrike_router_operands& ops, const void* hidden,
                                   uint32_t T, uint32_t stride, uint32_t* ids, float* weights,
                                   float* shared_gate) {
    const shrike_moe_config& c = m->cfg;
    RouterArgs a = {};
    a.w = ops.weights; a.scales = ops.scales; a.biases = ops.biases; a.bits = c.router_weight_bits;
    a.gate_row = (ops.shared_gate && shared_gate) ? ops.shared_gate : nullptr;
    a.eff_scale = ops.effective_scale; a.logit_bias = ops.logit_bias; a.per_expert_scale = ops.per_expert_scale;
    a.hidden = hidden; a.T = T; a.stride = stride; a.dt = c.act_dtype; a.ne = c.num_experts; a.d = c.d;
    a.top_k = c.top_k; a.sigmoid_scores = c.router_kind == SHRIKE_ROUTER_SIGMOID; a.scaling = c.routed_scaling;
    a.round_f16 = c.round_route_weights_f16; a.logits = m->ws.logits; a.ids = ids; a.weights = weights;
    a.gate_out = shared_gate; a.tokens_per_block = T;
    return a;
}

cudaError_t launch_router(const shrike_moe* m, cudaStream_t st, const shrike_router_operands& ops,
                          const void* hidden, uint32_t T, uint32_t stride, uint32_t* ids,
                          float* weights, float* shared_gate) {
    RouterArgs a = make_router_args(m, ops, hidden, T, stride, ids, weights, shared_gate);
    const uint32_t rows = a.ne + (a.gate_row ? 1u : 0u);
    cudaError_t e;
    if (T > 256 && a.bits == 0 && a.d % 8 == 0 && stride % 8 == 0 && ((uintptr_t)hidden & 15u) == 0 &&
        ((uintptr_t)a.w & 15u) == 0) {
        // tiled logits for the expert rows; the warp-per-row kernel keeps the gate row
        static bool attr_set[64] = {};
        int dev = 0;
        cudaGetDevice(&dev);
        if (dev < 64 && !attr_set[dev]) {
            e = cudaFuncSetAttribute(router_logits_tiled_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)kTileSmemBytes);
            if (e != cudaSuccess) return e;
            attr_set[dev] = true;
        }
        const dim3 grid((a.ne + kTileRows - 1) / kTileRows, (T + kTileTokens - 1) / kTileTokens);
        if (a.dt != SHRIKE_DTYPE_FP32 && !a.eff_scale) {
            static bool attr16_set[64] = {};
            if (dev < 64 && !attr16_set[dev]) {
                e = cudaFuncSetAttribute(router_logits_tiled16_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kTile16SmemBytes);
                if (e == cudaSuccess)
                    e = cudaFuncSetAttribute(router_logits_tiled16_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)kTile16SmemBytes);
                if (e != cudaSuccess) return e;
                attr16_set[dev] = true;
            }
            if (a.dt == SHRIKE_DTYPE_FP16) router_logits_tiled16_kernel<true><<<grid, 256, kTile16SmemBytes, st>>>(a);
            else router_logits_tiled16_kernel<false><<<grid, 256, kTile16SmemBytes, st>>>(a);
        } else {
            router_logits_tiled_kernel<<<grid, 256, kTileSmemBytes, st>>>(a);
        }
        e = cudaGetLastError();
        if (e != cudaSuccess) return e;
        if (a.gate_row) {
            router_gate_rows_kernel<<<(T + 31) / 32, 256, 0, st>>>(a);
            e = cudaGetLastError();
            if (e != cudaSuccess) return e;
        }
    } else {
        uint32_t tpb = 1;
        if (T > 64) tpb = 32;
        else if (T > 8) tpb = 4;
        a.tokens_per_block = tpb;
        const dim3 grid((rows + kRouterWarps - 1) / kRouterWarps, (T + tpb - 1) / tpb);
        router_logits_kernel<<<grid, kRouterWarps * 32, 0, st>>>(a);
        e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    router_select_kernel<<<(T + 3) / 4, 128, 0, st>>>(a);
    return cudaGetLastError();
}

cudaError_t launch_route_fused(const shrike_moe* m, cudaStream_t st, const shrike_router_operands& ops,
                               const void* hidden, uint32_t T, uint32_t stride, const uint64_t* table,
                               uint32_t pool_cells, const uint32_t* io_status, uint32_t* ids, float* weights,
                               float* shared_gate, uint32_t* slots, uint32_t* counts, bool pdl, bool no_tail) {
    RouterArgs a = make_router_args(m, ops, hidden, T, stride, ids, weights, shared_gate);
    a.no_tail = no_tail ? 1u : 0u;
    a.table = table; a.pool_cells = pool_cells; a.io_status = io_status;
    a.with_shared = m->cfg.has_shared; a.int4 = m->cfg.weight_bits == 4; a.group = m->cfg.group_size;
    a.xsum = m->ws.xsum;
    a.slots = slots; a.counts = counts; a.inst = m->ws.inst; a.n_inst = m->ws.n_inst; a.sorted = m->ws.sorted;
    a.xh = m->ws.xh; a.done_counter = m->ws.done_counter; a.status = m->ws.status; a.max_inst = max_instances(m->cfg, T);
    const uint32_t rows = a.ne + (a.gate_row ? 1u : 0u);
    cudaLaunchConfig_t cfg = {};
    // several rows: up to four blocks share an expert row's tokens (65 blocks would leave half of the SMs idle)
    const uint32_t gy = T < 4 ? (T ? T : 1u) : 4u;
    a.tokens_per_block = (T + gy - 1) / gy;
    cfg.gridDim = dim3((rows + kRouterWarps - 1) / kRouterWarps, gy);
    cfg.blockDim = dim3(kRouterWarps * 32);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = pdl ? attr : nullptr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, route_fused_kernel, a);
}

cudaError_t launch_classify(const shrike_moe* m, cudaStream_t st, const uint32_t* ids,
                            const uint64_t* table, uint32_t T, uint32_t* slots, uint32_t* counts,
                            uint32_t* miss_pos, uint32_t* miss_exp) {
    const uint32_t n_pairs = T * m->cfg.top_k;
    classify_kernel<<<n_pairs > 1024u ? (n_pairs + 1023u) / 1024u : 1u, 1024, 0, st>>>(ids, table, n_pairs, m->cfg.num_experts, slots, counts,
                                                                              miss_pos, miss_exp);
    return cudaGetLastError();
}

}  // namespace shrike

// ---- router entry point that allocates nothing --------------------------------
//
// Some hosts cannot let this library call cudaMalloc at all: a decode loop that
// has handed every free byte of HBM to the expert pool, a process whose memory
// plan is fixed before the first token, or a latency-critical thread that must
// not take cudaMalloc's device-wide synchronisation. shrike_moe_create sizes a
// workspace with cudaMalloc, so those hosts cannot own a handle. This entry
// point runs the router (logits + top-k + weights, and the shared expert's
// scalar gate) without one: its only scratch, the logits of up to
// SHRIKE_STATIC_ROUTER_MAX_ROWS rows by SHRIKE_MAX_EXPERTS experts, lives in
// the file-scope device array below (64 KiB on every GPU that loads the
// library, until the process exits).
#include <mutex>

namespace shrike {

static __device__ __align__(256) float g_static_router_logits[SHRIKE_STATIC_ROUTER_MAX_ROWS * SHRIKE_MAX_EXPERTS];

// Device address of the array, per device ordinal. The array's name is only a
// host-side stand-in in host code; the address the kernels need comes from
// cudaGetSymbolAddress, asked once per device with that device current.
static float* g_static_logits_ptr[64] = {};
static std::mutex g_static_logits_mutex;

static cudaError_t static_logits_for_current_device(float** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_static_logits_mutex);
    if (!g_static_logits_ptr[dev]) {
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_static_router_logits);
        if (e != cudaSuccess) return e;
        g_static_logits_ptr[dev] = p;
    }
    *out = g_static_logits_ptr[dev];
    return cudaSuccess;
}

static int static_router_fail(char* text, size_t bytes, int code, const char* msg) {
    if (text && bytes) {
        size_t i = 0;
        for (; msg[i] && i + 1 < bytes; ++i) text[i] = msg[i];
        text[i] = 0;
    }
    return code;
}


// Affine rows -> fp32 (load-time utility for operands a packed file holds quantised): one thread per element.
__global__ void __launch_bounds__(256)
dequant_affine_rows_kernel(const uint8_t* __restrict__ packed, const uint16_t* __restrict__ scales,
                           const uint16_t* __restrict__ biases, uint32_t bits, uint32_t group, uint32_t meta_f16,
                           uint32_t rows, uint32_t cols, float* __restrict__ out) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)rows * cols) return;
    const uint32_t r = (uint32_t)(i / cols), c = (uint32_t)(i - (size_t)r * cols);
    const uint8_t byte = packed[(size_t)r * (cols * bits / 8) + (bits == 4 ? c / 2 : c)];
    const uint32_t q = bits == 4 ? ((c & 1u) ? (uint32_t)(byte >> 4) : (uint32_t)(byte & 15u)) : (uint32_t)byte;
    const size_t g = (size_t)r * (cols / group) + c / group;
    const float sc = meta_f16 ? f16_bits_to_f32(scales[g]) : bf16_bits_to_f32(scales[g]);
    const float bi = meta_f16 ? f16_bits_to_f32(biases[g]) : bf16_bits_to_f32(biases[g]);
    out[i] = __fmaf_rn((float)q, sc, bi);
}

cudaError_t launch_dequant_affine_rows(cudaStream_t st, const void* packed, const void* scales, const void* biases,
                                       uint32_t bits, uint32_t group, uint32_t meta_dtype, uint32_t rows, uint32_t cols,
                                       float* out) {
    const size_t n = (size_t)rows * cols;
    dequant_affine_rows_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(
        (const uint8_t*)packed, (const uint16_t*)scales, (const uint16_t*)biases, bits, group,
        meta_dtype == SHRIKE_DTYPE_FP16 ? 1u : 0u, rows, cols, out);
    return cudaGetLastError();
}

}  // namespace shrike

extern "C" int shrike_encode_router_static(const shrike_moe_config* config, void* stream,
                                           const shrike_router_operands* ops, const void* hidden,
                                           uint32_t query_count, uint32_t hidden_stride_elements,
                                           uint32_t* out_indices, float* out_weights, float* out_shared_gate,
                                           char* error_text, size_t error_text_bytes) {
    using namespace shrike;
    auto bad = [&](int code, const char* msg) { return static_router_fail(error_text, error_text_bytes, code, msg); };
    if (!config) return bad(SHRIKE_EINVAL, "static router: config is null");
    if (query_count == 0) return SHRIKE_OK;
    const shrike_moe_config& c = *config;
    if (query_count > SHRIKE_STATIC_ROUTER_MAX_ROWS)
        return bad(SHRIKE_ERANGE, "static router: query_count exceeds SHRIKE_STATIC_ROUTER_MAX_ROWS (64); "
                                  "the built-in scratch holds 64 rows of logits");
    if (c.num_experts == 0 || c.num_experts > SHRIKE_MAX_EXPERTS)
        return bad(SHRIKE_ERANGE, "static router: num_experts must be 1..256 (the built-in scratch is 64 x 256 floats)");
    if (c.top_k == 0 || c.top_k > SHRIKE_MAX_TOP_K || c.top_k > c.num_experts)
        return bad(SHRIKE_EINVAL, "static router: top_k must be 1..8 and at most num_experts");
    if (c.d == 0 || c.d % 64 != 0 || c.d > 2944) return bad(SHRIKE_EINVAL, "static router: d must be a multiple of 64, at most 2944");
    if (c.act_dtype > SHRIKE_DTYPE_FP32 || c.router_kind > SHRIKE_ROUTER_SIGMOID ||
        (c.router_weight_bits != 0 && c.router_weight_bits != 4 && c.router_weight_bits != 8))
        return bad(SHRIKE_EINVAL, "static router: unknown act_dtype, router_kind or router_weight_bits");
    if (!ops || !ops->weights || !hidden || !out_indices || !out_weights)
        return bad(SHRIKE_EINVAL, "static router: null operand");
    if (c.router_weight_bits != 0 && (!ops->scales || !ops->biases))
        return bad(SHRIKE_EINVAL, "static router: affine weights need scales and biases");
    if (hidden_stride_elements < c.d || hidden_stride_elements % 4 != 0)
        return bad(SHRIKE_EINVAL, "static router: hidden stride must be >= d and a multiple of 4 elements");
    if (c.shared_gated && (!ops->shared_gate || !out_shared_gate))
        return bad(SHRIKE_EINVAL, "static router: a shared_gated config needs shared_gate and out_shared_gate");
    const char* why = nullptr;
    if (!router_operands_aligned(c, *ops, hidden, &why)) return bad(SHRIKE_EINVAL, why);
    float* logits = nullptr;
    cudaError_t e = static_logits_for_current_device(&logits);
    if (e != cudaSuccess) return bad(SHRIKE_EIO, cudaGetErrorString(e));

    RouterArgs a = {};
    a.w = ops->weights; a.scales = ops->scales; a.biases = ops->biases; a.bits = c.router_weight_bits;
    a.gate_row = (ops->shared_gate && out_shared_gate) ? ops->shared_gate : nullptr;
    a.eff_scale = ops->effective_scale; a.logit_bias = ops->logit_bias; a.per_expert_scale = ops->per_expert_scale;
    a.hidden = hidden; a.T = query_count; a.stride = hidden_stride_elements; a.dt = c.act_dtype;
    a.ne = c.num_experts; a.d = c.d; a.top_k = c.top_k;
    a.sigmoid_scores = c.router_kind == SHRIKE_ROUTER_SIGMOID; a.scaling = c.routed_scaling;
    a.round_f16 = c.round_route_weights_f16; a.logits = logits; a.ids = out_indices; a.weights = out_weights;
    a.gate_out = out_shared_gate;
    const uint32_t rows = a.ne + (a.gate_row ? 1u : 0u);
    const uint32_t tpb = query_count > 8 ? 4 : 1;
    a.tokens_per_block = tpb;
    cudaStream_t st = (cudaStream_t)stream;
    router_logits_kernel<<<dim3((rows + kRouterWarps - 1) / kRouterWarps, (query_count + tpb - 1) / tpb),
                           kRouterWarps * 32, 0, st>>>(a);
    e = cudaGetLastError();
    if (e != cudaSuccess) return bad(SHRIKE_EIO, cudaGetErrorString(e));
    router_select_kernel<<<(query_count + 3) / 4, 128, 0, st>>>(a);
    e = cudaGetLastError();
    if (e != cudaSuccess) return bad(SHRIKE_EIO, cudaGetErrorString(e));
    return SHRIKE_OK;
}

