// Device-side routing plans: which rows go to which expert block.
//
// Decode (few rows): the (row, rank) pairs are ordered by pool slot with a
// rank sort inside one block, cut into instances of at most 8 rows that share
// a block, and the activation rows are copied to the fp16 operand layout.
//
// Prefill: PrefillMoEGrouping.groupTokenExpertPairs
// (PrefillMoEGrouping.swift:269-370) as a three-step counting sort by expert
// id that keeps (token, rank) order inside an expert, in place of the host
// sort the reference runs between two GPU syncs (RealForwardRunner.swift:4305).
#include "plan.cuh"

namespace shrike {

constexpr uint32_t kPlanThreads = 512;

__device__ __forceinline__ uint32_t block_exclusive_scan(uint32_t v, uint32_t* warp_sums, uint32_t& total) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= (uint32_t)o) inc += n;
    }
    if (lane == 31) warp_sums[warp] = inc;
    __syncthreads();
    uint32_t base = 0, tot = 0;
    const uint32_t nw = blockDim.x >> 5;
    for (uint32_t w = 0; w < nw; ++w) {
        const uint32_t s = warp_sums[w];
        if (w < warp) base += s;
        tot += s;
    }
    __syncthreads();
    total = tot;
    return base + inc - v;
}

__global__ void __launch_bounds__(kPlanThreads)
decode_plan_kernel(const uint32_t* __restrict__ slots, uint32_t T, uint32_t top_k,
                   const uint32_t* __restrict__ io_status, uint32_t with_shared, uint32_t pool_cells,
                   Instance* __restrict__ inst, uint32_t* __restrict__ n_inst,
                   uint32_t* __restrict__ sorted, const void* __restrict__ x, uint32_t act_dtype,
                   uint32_t d, uint32_t int4, uint32_t group, uint16_t* __restrict__ xh,
                   float* __restrict__ xsum, uint32_t* status, uint32_t max_inst) {
    __shared__ PlanSmem sm;
    const uint32_t tid = threadIdx.x;
    const uint32_t n_pairs = T * top_k;

    // moe_io_ready (moe.metal:36-39): a pending or failed batch leaves only the
    // shared term.
    bool ready = true;
    if (io_status) {
        const uint32_t s = *io_status;
        ready = s == 1u || s == 3u;
    }
    for (uint32_t p = tid; p < n_pairs; p += kPlanThreads) {
        uint32_t s = ready ? slots[p] : SHRIKE_SLOT_MISS;
        if (s != SHRIKE_SLOT_MISS && s >= pool_cells) {
            report_status(status, kStatusBadIndex);
            s = SHRIKE_SLOT_MISS;
        }
        sm.key[p] = s;
    }
    __syncthreads();
    plan_body(sm, n_pairs, T, with_shared, inst, n_inst, sorted, max_inst, status);

    // fp16 operand copy of the activation rows and their per-group sums
    const uint32_t items = T * (d / 8);
    const size_t row_bytes = (size_t)d * (act_dtype == SHRIKE_DTYPE_FP32 ? 4 : 2);
    for (uint32_t i0 = 0; i0 < items; i0 += kPlanThreads)
        xprep_item(x, row_bytes, d, group, act_dtype, int4 != 0, i0 + tid, i0 + tid < items, xh, xsum, status);
}

cudaError_t launch_decode_plan(const shrike_moe* m, cudaStream_t st, const uint32_t* slots,
                               const void* x, uint32_t T, const uint32_t* io_status, bool with_shared,
                               uint32_t pool_cells) {
    decode_plan_kernel<<<1, kPlanThreads, 0, st>>>(
        slots, T, m->cfg.top_k, io_status, with_shared ? 1u : 0u, pool_cells,
        m->ws.inst, m->ws.n_inst, m->ws.sorted, x, m->cfg.act_dtype, m->cfg.d,
        m->cfg.weight_bits == 4 ? 1u : 0u, m->cfg.group_size, m->ws.xh, m->ws.xsum, m->ws.status, max_instances(m->cfg, T));
    return cudaGetLastError();
}

// ---- prefill grouping -------------------------------------------------------

constexpr uint32_t kGroupTokens = 128;  // rows per block

// Step 1: per block, a bitmap of the rows that chose each expert; writes the
// per-(block, expert) counts.
__global__ void __launch_bounds__(256)
group_hist_kernel(const uint32_t* __restrict__ ids, uint32_t T, uint32_t top_k, uint32_t ne,
                  uint32_t* __restrict__ block_hist, uint32_t* status) {
    __shared__ uint32_t bits[SHRIKE_MAX_EXPERTS][kGroupTokens / 32];
    const uint32_t t0 = blockIdx.x * kGroupTokens;
    for (uint32_t i = threadIdx.x; i < SHRIKE_MAX_EXPERTS * (kGroupTokens / 32); i += blockDim.x)
        (&bits[0][0])[i] = 0;
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < kGroupTokens * top_k; i += blockDim.x) {
        const uint32_t tl = i / top_k, t = t0 + tl;
        if (t < T) {
            const uint32_t e = ids[(size_t)t * top_k + (i - tl * top_k)];
            if (e < ne) {
                // a row that names one expert twice (no top-k router does) is counted once and reported
                const uint32_t bit = 1u << (tl & 31);
                if (atomicOr(&bits[e][tl >> 5], bit) & bit) report_status(status, kStatusBadIndex);
            } else if (e != 0xffffffffu) {
                // out of range: the pair is dropped and reported (0xffffffff is the expert-parallel layer's
                // "this pick lives on another rank" and is dropped silently)
                report_status(status, kStatusBadIndex);
            }
        }
    }
    __syncthreads();
    for (uint32_t e = threadIdx.x; e < ne; e += blockDim.x) {
        uint32_t c = 0;
#pragma unroll
        for (int w = 0; w < (int)(kGroupTokens / 32); ++w) c += __popc(bits[e][w]);
        block_hist[(size_t)blockIdx.x * ne + e] = c;
    }
}

// Step 2 (one block): per-expert totals, exclusive scan over experts, and the
// running base of every (block, expert) cell.
__global__ void __launch_bounds__(256)
group_scan_kernel(uint32_t* __restrict__ block_hist, uint32_t n_blocks, uint32_t ne,
                  uint32_t* __restrict__ offsets, uint32_t* __restrict__ counts) {
    __shared__ uint32_t warp_sums[8];
    const uint32_t e = threadIdx.x;
    uint32_t total = 0;
    if (e < ne)
        for (uint32_t b = 0; b < n_blocks; ++b) total += block_hist[(size_t)b * ne + e];
    uint32_t all;
    const uint32_t base = block_exclusive_scan(e < ne ? total : 0u, warp_sums, all);
    if (e < ne) {
        counts[e] = total;
        offsets[e] = total ? base : 0xffffffffu;
        uint32_t run = base;
        for (uint32_t b = 0; b < n_blocks; ++b) {
            const uint32_t c = block_hist[(size_t)b * ne + e];
            block_hist[(size_t)b * ne + e] = run;
            run += c;
        }
    }
}

// Step 3: place every pair at base(block, expert) + number of earlier rows of
// the block that chose the same expert.
__global__ void __launch_bounds__(256)
group_place_kernel(const uint32_t* __restrict__ ids, const float* __restrict__ weights, uint32_t T,
                   uint32_t top_k, uint32_t ne, const uint32_t* __restrict__ block_base,
                   uint32_t* __restrict__ sorted_pairs, uint32_t* __restrict__ sorted_ids) {
    __shared__ uint32_t bits[SHRIKE_MAX_EXPERTS][kGroupTokens / 32];
    const uint32_t t0 = blockIdx.x * kGroupTokens;
    for (uint32_t i = threadIdx.x; i < SHRIKE_MAX_EXPERTS * (kGroupTokens / 32); i += blockDim.x)
        (&bits[0][0])[i] = 0;
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < kGroupTokens * top_k; i += blockDim.x) {
        const uint32_t tl = i / top_k, t = t0 + tl;
        if (t < T) {
            const uint32_t e = ids[(size_t)t * top_k + (i - tl * top_k)];
            if (e < ne) atomicOr(&bits[e][tl >> 5], 1u << (tl & 31));
        }
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < kGroupTokens * top_k; i += blockDim.x) {
        const uint32_t tl = i / top_k, t = t0 + tl, r = i - tl * top_k;
        if (t >= T) continue;
        const uint32_t e = ids[(size_t)t * top_k + r];
        if (e >= ne) continue;
        uint32_t before = 0;
        const uint32_t word = tl >> 5;
        for (uint32_t w = 0; w < word; ++w) before += __popc(bits[e][w]);
        before += __popc(bits[e][word] & ((1u << (tl & 31)) - 1u));
        const uint32_t pos = block_base[(size_t)blockIdx.x * ne + e] + before;
        if (sorted_pairs) {
            uint4 p;
            p.x = t; p.y = e; p.z = r;
            // weight bits as the reference stores them: fp16 in the low half
            p.w = weights ? (uint32_t)__half_as_ushort(__float2half_rn(weights[(size_t)t * top_k + r])) : 0u;
            ((uint4*)sorted_pairs)[pos] = p;
        }
        if (sorted_ids) sorted_ids[pos] = t * top_k + r;
    }
}

cudaError_t launch_group_pairs(const shrike_moe* m, cudaStream_t st, const uint32_t* ids,
                               const float* weights, uint32_t T, uint32_t* sorted_pairs,
                               uint32_t* offsets, uint32_t* counts) {
    const uint32_t nb = (T + kGroupTokens - 1) / kGroupTokens;
    const uint32_t ne = m->cfg.num_experts, k = m->cfg.top_k;
    if (nb == 0) {
        cudaError_t e = cudaMemsetAsync(counts, 0, ne * 4, st);
        if (e != cudaSuccess) return e;
        return cudaMemsetAsync(offsets, 0xff, ne * 4, st);
    }
    group_hist_kernel<<<nb, 256, 0, st>>>(ids, T, k, ne, m->ws.block_hist, m->ws.status);
    group_scan_kernel<<<1, 256, 0, st>>>(m->ws.block_hist, nb, ne, offsets, counts);
    group_place_kernel<<<nb, 256, 0, st>>>(ids, weights, T, k, ne, m->ws.block_hist, sorted_pairs,
                                           m->ws.sorted);
    return cudaGetLastError();
}

}  // namespace shrike
