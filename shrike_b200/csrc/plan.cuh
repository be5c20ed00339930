// Decode work-list builder shared by the stand-alone plan kernel and the fused
// route kernel: orders the (row, rank) pairs by pool cell and cuts the runs
// into instances of at most 8 rows. Any block size that is a multiple of 32.
#pragma once

#include "internal.h"

namespace shrike {

constexpr uint32_t kPlanMaxPairs = SHRIKE_MAX_DECODE_TOKENS * SHRIKE_MAX_TOP_K;  // 512

struct PlanSmem {
    uint32_t key[kPlanMaxPairs];    // pool cell of pair p, or SHRIKE_SLOT_MISS
    uint32_t order[kPlanMaxPairs];  // pair ids sorted by (cell, pair id)
    uint32_t start[kPlanMaxPairs];  // 1 where an instance starts in the sorted order
    uint32_t index[kPlanMaxPairs];  // instance index of each start
    uint32_t n_valid;
    uint32_t n_routed;
};

// sm.key[0 .. n_pairs) must hold the (validated) cells; entries past n_pairs
// are ignored. Writes inst, n_inst, sorted. `inst` holds max_inst entries (sized for at most
// num_experts distinct cells): instances beyond it -- possible only when the caller's slots name more
// distinct cells than the layer has experts -- are dropped and reported through the status word.
__device__ __forceinline__ void plan_body(PlanSmem& sm, uint32_t n_pairs, uint32_t T, uint32_t with_shared,
                                          Instance* __restrict__ inst, uint32_t* __restrict__ n_inst,
                                          uint32_t* __restrict__ sorted, uint32_t max_inst, uint32_t* status) {
    const uint32_t tid = threadIdx.x, bd = blockDim.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) sm.n_valid = 0;
    __syncthreads();
    uint32_t mine = 0;
    for (uint32_t p = tid; p < n_pairs; p += bd) {
        const uint32_t s = sm.key[p];
        if (s == SHRIKE_SLOT_MISS) continue;
        uint32_t rank = 0;
        for (uint32_t j = 0; j < n_pairs; ++j) {
            const uint32_t o = sm.key[j];
            rank += (o < s || (o == s && j < p)) ? 1u : 0u;  // a miss is 0xffffffff: never smaller
        }
        sm.order[rank] = p;
        ++mine;
    }
    if (mine) atomicAdd(&sm.n_valid, mine);
    __syncthreads();
    const uint32_t n_valid = sm.n_valid;
    // an instance starts at every 8th row of a run of equal cells
    for (uint32_t p = tid; p < n_valid; p += bd) {
        const uint32_t my = sm.key[sm.order[p]];
        uint32_t q = 0;
        while (q < p && sm.key[sm.order[p - q - 1]] == my) ++q;
        sm.start[p] = (q & 7u) == 0 ? 1u : 0u;
        sorted[p] = sm.order[p];
    }
    __syncthreads();
    if (warp == 0) {
        uint32_t running = 0;
        for (uint32_t base = 0; base < n_valid; base += 32) {
            const uint32_t p = base + lane;
            const uint32_t v = p < n_valid ? sm.start[p] : 0u;
            uint32_t inc = v;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t n = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= (uint32_t)o) inc += n;
            }
            if (p < n_valid) sm.index[p] = running + inc - v;
            running += __shfl_sync(0xffffffffu, inc, 31);
        }
        if (lane == 0) sm.n_routed = running;
    }
    __syncthreads();
    const uint32_t n_routed = sm.n_routed;
    for (uint32_t p = tid; p < n_valid; p += bd) {
        if (!sm.start[p]) continue;
        const uint32_t my = sm.key[sm.order[p]];
        uint32_t count = 1;
        while (count < 8 && p + count < n_valid && sm.key[sm.order[p + count]] == my) ++count;
        Instance in;
        in.kind = 0; in.slot = my; in.first = p; in.count = count;
        for (uint32_t j = 0; j < 8; ++j) in.pair[j] = sm.order[p + (j < count ? j : 0)];
        if (sm.index[p] < max_inst) inst[sm.index[p]] = in;
    }
    const uint32_t n_shared = with_shared ? (T + 7) / 8 : 0;
    for (uint32_t j = tid; j < n_shared; j += bd) {
        Instance in;
        in.kind = 1; in.slot = 0; in.first = j * 8; in.count = min(8u, T - j * 8);
        for (uint32_t q = 0; q < 8; ++q) in.pair[q] = j * 8 + (q < in.count ? q : 0);
        if (n_routed + j < max_inst) inst[n_routed + j] = in;
    }
    if (tid == 0) {
        if (n_routed + n_shared > max_inst) report_status(status, kStatusBadIndex);
        *n_inst = min(n_routed + n_shared, max_inst);
    }
}

}  // namespace shrike
