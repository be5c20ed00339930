// Expert parallelism: dispatch and combine around the all-to-all.
//
// The reference runs on one device; sharding the routed experts over the GPUs
// of one box is this build's addition. Rank r owns experts
// [r*experts_per_rank, (r+1)*experts_per_rank) of every layer. The router is
// replicated, so a token's home rank knows which ranks need its row:
//
//   dispatch  one copy of the row per destination RANK (not per expert), with
//             the expert ids local to that rank and the route weights; rows
//             are packed per destination in token order, at a fixed capacity
//             so that the exchange needs no size negotiation and no host sync
//   (all-to-all over NVLink; NCCL, issued by the host)
//   local     every rank runs its experts on the rows it received through the
//             ordinary prefill/decode calls; ids of other ranks' experts and
//             padding rows resolve to SHRIKE_SLOT_MISS and contribute nothing
//   (all-to-all back: one weighted partial-sum row per (token, rank))
//   combine   y = shared(x) + sum over ranks of the returned rows, in rank
//             order; hidden += y (moe_phase2_finish, moe.metal:889-893)
#include "internal.h"

namespace shrike {

constexpr uint32_t kEpInvalid = 0xffffffffu;

// grid = world blocks of 1024 threads. Block g: which tokens have an expert on
// rank g, their row index at g (exclusive prefix in token order), ids/weights.
__global__ void __launch_bounds__(1024)
ep_plan_kernel(const uint32_t* __restrict__ ids, const float* __restrict__ weights, uint32_t T, uint32_t top_k,
               uint32_t world, uint32_t experts_per_rank, uint32_t cap, uint32_t* __restrict__ send_ids,
               float* __restrict__ send_w, uint32_t* __restrict__ send_counts, int32_t* __restrict__ row_of) {
    __shared__ uint32_t warp_counts[32];
    const uint32_t g = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint32_t base = 0;
    for (uint32_t t0 = 0; t0 < T; t0 += 1024) {
        const uint32_t t = t0 + tid;
        bool mine = false;
        if (t < T) {
            for (uint32_t k = 0; k < top_k; ++k) mine |= ids[(size_t)t * top_k + k] / experts_per_rank == g;
        }
        const uint32_t ballot = __ballot_sync(0xffffffffu, mine);
        if (lane == 0) warp_counts[warp] = __popc(ballot);
        __syncthreads();
        uint32_t before = 0, total = 0;
        for (uint32_t w = 0; w < 32; ++w) {
            if (w < warp) before += warp_counts[w];
            total += warp_counts[w];
        }
        if (t < T) {
            int32_t row = -1;
            if (mine) {
                const uint32_t r = base + before + __popc(ballot & ((1u << lane) - 1u));
                if (r < cap) {
                    row = (int32_t)r;
                    for (uint32_t k = 0; k < top_k; ++k) {
                        const uint32_t e = ids[(size_t)t * top_k + k];
                        const bool here = e / experts_per_rank == g;
                        const size_t o = ((size_t)g * cap + r) * top_k + k;
                        send_ids[o] = here ? e - g * experts_per_rank : kEpInvalid;
                        send_w[o] = here ? weights[(size_t)t * top_k + k] : 0.0f;
                    }
                }
            }
            row_of[(size_t)t * world + g] = row;
        }
        base += total;
        __syncthreads();
    }
    if (tid == 0) send_counts[g] = base < cap ? base : cap;
}

// grid (T, world): copy the token's row into its slot at every destination.
__global__ void __launch_bounds__(256)
ep_copy_rows_kernel(const void* __restrict__ x, const int32_t* __restrict__ row_of, uint32_t world, uint32_t cap,
                    uint32_t row_bytes, void* __restrict__ send_x) {
    const uint32_t t = blockIdx.x, g = blockIdx.y;
    const int32_t row = row_of[(size_t)t * world + g];
    if (row < 0) return;
    const uint4* src = (const uint4*)((const uint8_t*)x + (size_t)t * row_bytes);
    uint4* dst = (uint4*)((uint8_t*)send_x + ((size_t)g * cap + row) * row_bytes);
    for (uint32_t i = threadIdx.x; i < row_bytes / 16; i += blockDim.x) dst[i] = src[i];
}

// Received ids -> pool cells through the local residency table; invalid ids miss.
__global__ void __launch_bounds__(256)
ep_local_slots_kernel(const uint32_t* __restrict__ recv_ids, const uint64_t* __restrict__ table, uint32_t n,
                      uint32_t ne_local, uint32_t* __restrict__ slots) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint32_t e = recv_ids[i];
    uint32_t slot = SHRIKE_SLOT_MISS;
    if (e < ne_local) {
        const uint64_t word = table[e];
        const uint32_t s = (uint32_t)(word & 0xffffffffu);
        if ((uint32_t)(word >> 32) == 2u && s != SHRIKE_SLOT_MISS) slot = s;
    }
    slots[i] = slot;
}

// grid (ceil(d/256), T)
__global__ void __launch_bounds__(256)
ep_combine_kernel(const void* __restrict__ recv_y, const int32_t* __restrict__ row_of,
                  const void* __restrict__ y_home, uint32_t T, uint32_t world, uint32_t cap, uint32_t d,
                  uint32_t act_dtype, uint32_t y_dtype, void* __restrict__ y, void* __restrict__ hidden) {
    const uint32_t t = blockIdx.y, i = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T || i >= d) return;
    const size_t o = (size_t)t * d + i;
    float acc = y_home ? load_act(y_home, o, y_dtype) : 0.0f;
    for (uint32_t g = 0; g < world; ++g) {
        const int32_t row = row_of[(size_t)t * world + g];
        if (row >= 0) acc += load_act(recv_y, ((size_t)g * cap + row) * d + i, y_dtype);
    }
    store_act(y, o, y_dtype, acc);
    if (hidden) {
        const float h = load_act(hidden, o, act_dtype) + round_act(y_dtype, acc);
        store_act(hidden, o, act_dtype, h);
    }
}

cudaError_t launch_ep_dispatch(const shrike_moe* m, cudaStream_t st, const void* x, const uint32_t* ids,
                               const float* weights, uint32_t T, uint32_t world, uint32_t experts_per_rank,
                               uint32_t cap, void* send_x, uint32_t* send_ids, float* send_w,
                               uint32_t* send_counts, int32_t* row_of) {
    const shrike_moe_config& c = m->cfg;
    cudaError_t e = cudaMemsetAsync(send_ids, 0xff, (size_t)world * cap * c.top_k * 4, st);
    if (e != cudaSuccess) return e;
    ep_plan_kernel<<<world, 1024, 0, st>>>(ids, weights, T, c.top_k, world, experts_per_rank, cap, send_ids, send_w,
                                           send_counts, row_of);
    const uint32_t row_bytes = c.d * (uint32_t)act_bytes(c.act_dtype);
    ep_copy_rows_kernel<<<dim3(T, world), 256, 0, st>>>(x, row_of, world, cap, row_bytes, send_x);
    return cudaGetLastError();
}

cudaError_t launch_ep_local_slots(const shrike_moe* m, cudaStream_t st, const uint32_t* recv_ids,
                                  const uint64_t* table, uint32_t rows, uint32_t* slots) {
    const uint32_t n = rows * m->cfg.top_k;
    ep_local_slots_kernel<<<(n + 255) / 256, 256, 0, st>>>(recv_ids, table, n, m->cfg.num_experts, slots);
    return cudaGetLastError();
}

cudaError_t launch_ep_combine(const shrike_moe* m, cudaStream_t st, const void* recv_y, const int32_t* row_of,
                              const void* y_home, uint32_t T, uint32_t world, uint32_t cap, void* y, void* hidden) {
    const shrike_moe_config& c = m->cfg;
    ep_combine_kernel<<<dim3((c.d + 255) / 256, T), 256, 0, st>>>(recv_y, row_of, y_home, T, world, cap, c.d,
                                                                 c.act_dtype, c.y_dtype, y, hidden);
    return cudaGetLastError();
}

}  // namespace shrike
