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

// ---- the exchange over peer memory (NVLink loads/stores, no collective library) -------------------------
//
// Every rank owns one exchange buffer that its peers can address (one process per GPU: opened through a
// CUDA IPC handle; one process driving several GPUs: the pointer itself). The sending kernels store rows
// straight into the destination's receive area -- only the rows that were routed there move, nothing is
// padded to a fixed capacity -- and then publish {epoch, row count} with a release store at system scope;
// the receiver's wait is a bounded poll of its own memory that, when it gives up, reports through the
// status word and lets the call run on with zero rows from that source. Plain stores only: no multicast,
// no multimem, no TMA from or to another GPU's memory.
//
//   buffer of rank g:  recv_x [world][cap][d]   rows sent by rank s land in block s
//                      recv_ids / recv_w [world][cap][top_k]
//                      ret [world][cap][d]      partial rows returned by rank s (y dtype)
//                      arrive [world], ret_arrive [world]   64-bit {epoch, count} words

struct EpPeers {
    uint8_t* base[SHRIKE_EP_MAX_WORLD];
};

__device__ __forceinline__ void st_release_sys_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// As ep_plan_kernel, with the ids and weights written into the destination's receive area.
__global__ void __launch_bounds__(1024)
ep_plan_peer_kernel(const uint32_t* __restrict__ ids, const float* __restrict__ weights, uint32_t T, uint32_t top_k,
                    uint32_t world, uint32_t rank, uint32_t experts_per_rank, uint32_t cap, EpPeers peers,
                    EpLayout lay, uint32_t* __restrict__ send_counts, int32_t* __restrict__ row_of) {
    __shared__ uint32_t warp_counts[32];
    const uint32_t g = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint32_t* dst_ids = (uint32_t*)(peers.base[g] + lay.off_recv_ids) + (size_t)rank * cap * top_k;
    float* dst_w = (float*)(peers.base[g] + lay.off_recv_w) + (size_t)rank * cap * top_k;
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
                        dst_ids[(size_t)r * top_k + k] = here ? e - g * experts_per_rank : kEpInvalid;
                        dst_w[(size_t)r * top_k + k] = here ? weights[(size_t)t * top_k + k] : 0.0f;
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

// grid (T, world): the row, straight into its slot in the destination's receive area.
__global__ void __launch_bounds__(256)
ep_copy_rows_peer_kernel(const void* __restrict__ x, const int32_t* __restrict__ row_of, uint32_t world, uint32_t rank,
                         uint32_t cap, uint32_t row_bytes, EpPeers peers, EpLayout lay) {
    const uint32_t t = blockIdx.x, g = blockIdx.y;
    const int32_t row = row_of[(size_t)t * world + g];
    if (row < 0) return;
    const uint4* src = (const uint4*)((const uint8_t*)x + (size_t)t * row_bytes);
    uint4* dst = (uint4*)(peers.base[g] + lay.off_recv_x + ((size_t)rank * cap + row) * row_bytes);
    for (uint32_t i = threadIdx.x; i < row_bytes / 16; i += blockDim.x) dst[i] = src[i];
}

// One thread per destination: everything this rank stored there is ordered before the word that says so.
// what = 0: rows dispatched (count = send_counts[g]); 1: partial rows returned.
__global__ void ep_signal_kernel(EpPeers peers, EpLayout lay, uint32_t world, uint32_t rank, uint32_t epoch,
                                 uint32_t what, const uint32_t* __restrict__ send_counts) {
    const uint32_t g = threadIdx.x;
    if (g >= world) return;
    __threadfence_system();
    unsigned long long* flag = (unsigned long long*)(peers.base[g] + (what ? lay.off_ret_arrive : lay.off_arrive)) + rank;
    const unsigned long long count = what ? 0ull : (unsigned long long)send_counts[g];
    st_release_sys_u64(flag, ((unsigned long long)epoch << 32) | count);
}

// Bounded wait for every source's word of this epoch (about a second, then the status word says so and the
// source counts as having sent nothing). what = 0: also the prefix of the row counts and their total.
__global__ void ep_wait_kernel(const uint8_t* __restrict__ mine, EpLayout lay, uint32_t world, uint32_t epoch,
                               uint32_t what, uint32_t cap, uint32_t* __restrict__ prefix, uint32_t* __restrict__ n_rows,
                               uint32_t* status, uint32_t max_polls) {
    __shared__ uint32_t counts[SHRIKE_EP_MAX_WORLD];
    const uint32_t s = threadIdx.x;
    if (s < world) {
        const unsigned long long* flag = (const unsigned long long*)(mine + (what ? lay.off_ret_arrive : lay.off_arrive)) + s;
        uint32_t count = 0;
        bool ok = false;
        for (uint32_t it = 0; it < max_polls; ++it) {
            const unsigned long long v = ld_acquire_sys_u64(flag);
            if ((uint32_t)(v >> 32) == epoch) {
                count = (uint32_t)v;
                ok = true;
                break;
            }
            __nanosleep(it < 64 ? 100 : 1000);
        }
        if (!ok) report_status(status, kStatusWaitTimeout);
        counts[s] = count < cap ? count : cap;
    }
    __syncthreads();
    if (what == 0 && s == 0) {
        uint32_t run = 0;
        for (uint32_t i = 0; i < world; ++i) {
            prefix[i] = run;
            run += counts[i];
        }
        prefix[world] = run;
        *n_rows = run;
    }
}

// Received rows, compact: row t of the local call is row (t - prefix[s]) of source s. Local expert ids ->
// pool cells through the residency table; rows past the total carry no work.
__global__ void __launch_bounds__(256)
ep_compact_kernel(const uint8_t* __restrict__ mine, EpLayout lay, uint32_t world, uint32_t cap, uint32_t top_k,
                  uint32_t ne_local, const uint64_t* __restrict__ table, const uint32_t* __restrict__ prefix,
                  uint32_t t_max, uint32_t* __restrict__ c_ids, float* __restrict__ c_w,
                  uint32_t* __restrict__ c_slots, uint32_t* __restrict__ row_map) {
    const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= t_max) return;
    const uint32_t total = prefix[world];
    if (t >= total) {
        row_map[t] = 0;
        for (uint32_t k = 0; k < top_k; ++k) {
            c_ids[(size_t)t * top_k + k] = kEpInvalid;
            c_w[(size_t)t * top_k + k] = 0.0f;
            c_slots[(size_t)t * top_k + k] = SHRIKE_SLOT_MISS;
        }
        return;
    }
    uint32_t s = 0;
    while (s + 1 < world && t >= prefix[s + 1]) ++s;
    const uint32_t g_row = s * cap + (t - prefix[s]);
    row_map[t] = g_row;
    const uint32_t* ids = (const uint32_t*)(mine + lay.off_recv_ids) + (size_t)g_row * top_k;
    const float* w = (const float*)(mine + lay.off_recv_w) + (size_t)g_row * top_k;
    for (uint32_t k = 0; k < top_k; ++k) {
        const uint32_t e = ids[k];
        uint32_t slot = SHRIKE_SLOT_MISS;
        if (e < ne_local) {
            const uint64_t word = table[e];
            const uint32_t c = (uint32_t)(word & 0xffffffffu);
            if ((uint32_t)(word >> 32) == 2u && c != SHRIKE_SLOT_MISS) slot = c;
        }
        c_ids[(size_t)t * top_k + k] = e < ne_local ? e : kEpInvalid;
        c_w[(size_t)t * top_k + k] = w[k];
        c_slots[(size_t)t * top_k + k] = slot;
    }
}

// The accumulated partial row of every received row goes back to its home rank's return area (y dtype):
// the weighted combine of the local call and the return exchange in one pass.
__global__ void __launch_bounds__(256)
ep_return_kernel(const float* __restrict__ yacc, const uint32_t* __restrict__ row_map,
                 const uint32_t* __restrict__ n_rows, uint32_t rank, uint32_t cap, uint32_t d, uint32_t y_dtype,
                 EpPeers peers, EpLayout lay) {
    // grid (column blocks, a fixed number of row walkers): the number of received rows is only known on the device
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= d) return;
    const uint32_t n = *n_rows;
    for (uint32_t t = blockIdx.y; t < n; t += gridDim.y) {
        const uint32_t g_row = row_map[t], s = g_row / cap, row = g_row - s * cap;
        void* dst = peers.base[s] + lay.off_ret;
        store_act(dst, ((size_t)rank * cap + row) * d + i, y_dtype, yacc[(size_t)t * d + i]);
    }
}

EpLayout ep_layout(const shrike_moe_config& c, uint32_t world, uint32_t cap) {
    EpLayout l;
    auto up = [](size_t v) { return (v + 255) / 256 * 256; };
    size_t cur = 0;
    l.off_recv_x = cur; cur = up(cur + (size_t)world * cap * c.d * act_bytes(c.act_dtype));
    l.off_recv_ids = cur; cur = up(cur + (size_t)world * cap * c.top_k * 4);
    l.off_recv_w = cur; cur = up(cur + (size_t)world * cap * c.top_k * 4);
    l.off_ret = cur; cur = up(cur + (size_t)world * cap * c.d * act_bytes(c.y_dtype));
    l.off_arrive = cur; cur = up(cur + (size_t)world * 8);
    l.off_ret_arrive = cur; cur = up(cur + (size_t)world * 8);
    l.bytes = cur;
    return l;
}

static EpPeers make_peers(uint8_t* const* base, uint32_t world) {
    EpPeers p;
    for (uint32_t i = 0; i < SHRIKE_EP_MAX_WORLD; ++i) p.base[i] = i < world ? base[i] : nullptr;
    return p;
}

cudaError_t launch_ep_dispatch_peer(const shrike_moe* m, cudaStream_t st, const void* x, const uint32_t* ids,
                                    const float* weights, uint32_t T, uint32_t world, uint32_t rank,
                                    uint32_t experts_per_rank, uint32_t cap, uint8_t* const* peer_base,
                                    const EpLayout& lay, uint32_t epoch, uint32_t* send_counts, int32_t* row_of) {
    const shrike_moe_config& c = m->cfg;
    const EpPeers peers = make_peers(peer_base, world);
    if (T > 0) {
        ep_plan_peer_kernel<<<world, 1024, 0, st>>>(ids, weights, T, c.top_k, world, rank, experts_per_rank, cap, peers, lay,
                                                    send_counts, row_of);
        const uint32_t row_bytes = c.d * (uint32_t)act_bytes(c.act_dtype);
        ep_copy_rows_peer_kernel<<<dim3(T, world), 256, 0, st>>>(x, row_of, world, rank, cap, row_bytes, peers, lay);
    } else {
        cudaError_t e = cudaMemsetAsync(send_counts, 0, world * 4, st);
        if (e != cudaSuccess) return e;
    }
    ep_signal_kernel<<<1, SHRIKE_EP_MAX_WORLD, 0, st>>>(peers, lay, world, rank, epoch, 0, send_counts);
    return cudaGetLastError();
}

cudaError_t launch_ep_receive(const shrike_moe* routed, cudaStream_t st, const uint8_t* mine, const EpLayout& lay,
                              uint32_t world, uint32_t cap, uint32_t epoch, const uint64_t* table, uint32_t t_max,
                              uint32_t* prefix, uint32_t* n_rows, uint32_t* c_ids, float* c_w, uint32_t* c_slots,
                              uint32_t* row_map, uint32_t max_polls) {
    ep_wait_kernel<<<1, SHRIKE_EP_MAX_WORLD, 0, st>>>(mine, lay, world, epoch, 0, cap, prefix, n_rows, routed->ws.status,
                                                      max_polls);
    ep_compact_kernel<<<(t_max + 255) / 256, 256, 0, st>>>(mine, lay, world, cap, routed->cfg.top_k,
                                                           routed->cfg.num_experts, table, prefix, t_max, c_ids, c_w,
                                                           c_slots, row_map);
    return cudaGetLastError();
}

cudaError_t launch_ep_return(const shrike_moe* routed, cudaStream_t st, const uint32_t* row_map, const uint32_t* n_rows,
                             uint32_t t_max, uint32_t world, uint32_t rank, uint32_t cap, uint8_t* const* peer_base,
                             const EpLayout& lay, uint32_t epoch) {
    const shrike_moe_config& c = routed->cfg;
    const EpPeers peers = make_peers(peer_base, world);
    ep_return_kernel<<<dim3((c.d + 255) / 256, t_max < 1024u ? t_max : 1024u), 256, 0, st>>>(routed->ws.yacc, row_map, n_rows, rank, cap, c.d,
                                                                     c.y_dtype, peers, lay);
    ep_signal_kernel<<<1, SHRIKE_EP_MAX_WORLD, 0, st>>>(peers, lay, world, rank, epoch, 1, nullptr);
    return cudaGetLastError();
}

cudaError_t launch_ep_wait_returns(const shrike_moe* home, cudaStream_t st, const uint8_t* mine, const EpLayout& lay,
                                   uint32_t world, uint32_t cap, uint32_t epoch, uint32_t max_polls) {
    ep_wait_kernel<<<1, SHRIKE_EP_MAX_WORLD, 0, st>>>(mine, lay, world, epoch, 1, cap, nullptr, nullptr, home->ws.status,
                                                      max_polls);
    return cudaGetLastError();
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
