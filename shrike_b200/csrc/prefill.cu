// Prefill path for ragged batches: rows are permuted by expert on the device
// (plan.cu), every expert's rows run through the expert-grouped GEMM (or, for
// shapes it does not take, the dequant-fused tiles in instances of 8), the
// down projection's epilogue multiplies each row by its route weight and adds
// it into one fp32 accumulator row per token (the weighted reduce of
// prefill_moe_reduce_token_major, prefill.metal:624-645, without the
// per-(row, rank) partial rows), and a last pass converts and does the two
// residual adds of RealForwardRunner.swift:4658-4665.
#include "internal.h"

namespace shrike {

// One thread per expert: ceil(count/8) instances each, in expert order.
__global__ void __launch_bounds__(256)
prefill_instances_kernel(const uint32_t* __restrict__ offsets, const uint32_t* __restrict__ counts,
                         const uint32_t* __restrict__ slot_of_expert, uint32_t ne, uint32_t T,
                         uint32_t with_shared, uint32_t pool_cells,
                         const uint32_t* __restrict__ sorted, Instance* __restrict__ inst,
                         uint32_t* __restrict__ n_inst, uint32_t* status) {
    __shared__ uint32_t warp_sums[8];
    const uint32_t e = threadIdx.x;
    uint32_t n = 0, slot = SHRIKE_SLOT_MISS, c = 0;
    if (e < ne && counts[e] > 0) {
        c = counts[e];
        slot = slot_of_expert[e];
        if (slot != SHRIKE_SLOT_MISS && slot >= pool_cells) {
            report_status(status, kStatusBadIndex);
            slot = SHRIKE_SLOT_MISS;
        }
        if (slot != SHRIKE_SLOT_MISS) n = (c + 7) / 8;
    }
    // exclusive scan over 256 threads
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t inc = n;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t v = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= (uint32_t)o) inc += v;
    }
    if (lane == 31) warp_sums[warp] = inc;
    __syncthreads();
    uint32_t base = 0, total = 0;
    for (uint32_t w = 0; w < 8; ++w) {
        if (w < warp) base += warp_sums[w];
        total += warp_sums[w];
    }
    base += inc - n;
    for (uint32_t j = 0; j < n; ++j) {
        Instance in;
        in.kind = 0; in.slot = slot; in.first = offsets[e] + 8 * j; in.count = min(8u, c - 8 * j);
        for (uint32_t q = 0; q < 8; ++q) in.pair[q] = sorted[in.first + (q < in.count ? q : 0)];
        inst[base + j] = in;
    }
    const uint32_t n_shared = with_shared ? (T + 7) / 8 : 0;
    for (uint32_t j = threadIdx.x; j < n_shared; j += blockDim.x) {
        Instance in;
        in.kind = 1; in.slot = 0; in.first = 8 * j; in.count = min(8u, T - 8 * j);
        for (uint32_t q = 0; q < 8; ++q) in.pair[q] = 8 * j + (q < in.count ? q : 0);
        inst[total + j] = in;
    }
    if (threadIdx.x == 0) *n_inst = total + n_shared;
}

// x -> fp16 operand layout and per-group sums, all rows.
__global__ void __launch_bounds__(256)
prefill_xprep_kernel(const void* __restrict__ x, uint32_t T, uint32_t d, uint32_t group, uint32_t act_dtype,
                     uint32_t int4, uint16_t* __restrict__ xh, float* __restrict__ xsum, uint32_t* status,
                     const uint32_t* __restrict__ row_map, const uint32_t* __restrict__ n_rows_dev) {
    const uint32_t items = T * (d / 8);
    const size_t row_bytes = (size_t)d * (act_dtype == SHRIKE_DTYPE_FP32 ? 4 : 2);
    const uint32_t n_rows = n_rows_dev ? *n_rows_dev : T;
    for (uint32_t i0 = blockIdx.x * blockDim.x; i0 < items; i0 += gridDim.x * blockDim.x)
        xprep_item(x, row_bytes, d, group, act_dtype, int4 != 0, i0 + threadIdx.x, i0 + threadIdx.x < items, xh,
                   xsum, status, row_map, n_rows);
}

// slot_of_expert[e] = the cell every pair of expert e resolved to.
// A streamed batch whose status word is not READY (moe_io_ready, moe.metal:36-39) leaves every expert
// without a cell: only the shared term remains.
__global__ void __launch_bounds__(256)
prefill_slot_of_expert_kernel(const uint32_t* __restrict__ ids, const uint32_t* __restrict__ slots,
                              uint32_t n_pairs, uint32_t ne, const uint32_t* __restrict__ io_status,
                              uint32_t* __restrict__ slot_of_expert) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (io_status) {
        const uint32_t s = *io_status;
        if (s != 1u && s != 3u) return;
    }
    if (i < n_pairs) {
        const uint32_t e = ids[i];
        if (e < ne) slot_of_expert[e] = slots[i];
    }
}

// y[t] = the accumulated row (shared term and weighted expert rows, fp32); hidden += y.
__global__ void __launch_bounds__(256)
prefill_combine_kernel(const float* __restrict__ yacc, uint32_t n, uint32_t act_dtype, uint32_t y_dtype,
                       void* __restrict__ y, void* __restrict__ hidden) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float acc = yacc[i];
    store_act(y, i, y_dtype, acc);
    if (hidden) {
        const float h = load_act(hidden, i, act_dtype) + round_act(y_dtype, acc);
        store_act(hidden, i, act_dtype, h);
    }
}

cudaError_t launch_prefill_plan(const shrike_moe* m, cudaStream_t st, const uint32_t* ids,
                                const uint32_t* slots, const void* x, uint32_t T, bool with_shared,
                                uint32_t pool_cells, bool warp_mma_instances, const uint32_t* io_status,
                                const uint32_t* row_map, const uint32_t* n_rows, float* accumulator) {
    const shrike_moe_config& c = m->cfg;
    const Workspace& ws = m->ws;
    cudaError_t e = cudaMemsetAsync(ws.slot_of_expert, 0xff, c.num_experts * 4, st);
    if (e != cudaSuccess) return e;
    // the rows the down epilogue adds into: the workspace's, or the caller's fp32 output itself
    e = cudaMemsetAsync(accumulator ? accumulator : ws.yacc, 0, (size_t)T * c.d * 4, st);
    if (e != cudaSuccess) return e;
    const uint32_t n_pairs = T * c.top_k;
    prefill_slot_of_expert_kernel<<<(n_pairs + 255) / 256, 256, 0, st>>>(ids, slots, n_pairs, c.num_experts,
                                                                         io_status, ws.slot_of_expert);
    e = launch_group_pairs(m, st, ids, nullptr, T, nullptr, ws.expert_offsets, ws.expert_counts);
    if (e != cudaSuccess) return e;
    if (warp_mma_instances)   // the tensor-core path builds its own 256-row instances
        prefill_instances_kernel<<<1, 256, 0, st>>>(ws.expert_offsets, ws.expert_counts, ws.slot_of_expert,
                                                    c.num_experts, T, with_shared ? 1u : 0u, pool_cells, ws.sorted,
                                                    ws.inst, ws.n_inst, ws.status);
    const uint32_t items = T * (c.d / 8);
    prefill_xprep_kernel<<<min(2048u, (items + 255) / 256), 256, 0, st>>>(
        x, T, c.d, c.group_size, c.act_dtype, c.weight_bits == 4 ? 1u : 0u, ws.xh, ws.xsum, ws.status, row_map, n_rows);
    return cudaGetLastError();
}

cudaError_t launch_prefill_combine(const shrike_moe* m, cudaStream_t st, uint32_t T, void* y, void* hidden) {
    const shrike_moe_config& c = m->cfg;
    const uint32_t n = T * c.d;
    prefill_combine_kernel<<<(n + 255) / 256, 256, 0, st>>>(m->ws.yacc, n, c.act_dtype, c.y_dtype, y, hidden);
    return cudaGetLastError();
}

}  // namespace shrike
