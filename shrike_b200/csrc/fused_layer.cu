// One decode row through one MoE layer in ONE launch: router logits, top-k, residency lookup, shared
// and routed gate/up + GLU, down projections, weighted combine, hidden += y.
//
//   router_gemv_r4 + router_topk_select_k8          moe.metal:324-582
//   moe_classify_expert_residency_spec              moe.metal:121-231
//   moe_phase1_gate_up_act_spec_u16load             moe.metal:950-998
//   moe_phase2_down_reduce_spec_k8 / phase2_finish  moe.metal:889-893, 1008-1057
//   shared expert (SharedExpertRuntime)             SharedExpertInt4.swift:251-342
//
// One persistent block per SM: a producer warp and sixteen consumer warps. A layer's bytes (nine 1.7 MB
// expert blocks at the Qwen shape) are about as large as the chip's shared memory, so as soon as the
// instance list is known every block asks for ALL of its share: the lanes of the producer warp each
// issue one unit's tiled TMA copies (cp.async.bulk.tensor, no multicast; the lanes run copy by copy,
// so the copy engine's queue holds the small scale/bias boxes first and the weight boxes in unit
// order) into a ring of shared-memory slots, each slot completing on an mbarrier. The consumers walk
// the slots with the dequant-fused skinny tiles (packed words -> exact fp16 integers with one logic
// op per register, mma.sync m16n8k16, fp32 accumulate, one fused multiply-add per group with the
// scale and one with the zero-point bias): gate/up units by groups of eight warps, a unit per group
// at a time; the down tile of a block by all sixteen warps, one meeting per tile. What a block does
// is a closed form of its index (BlockPlan), so no warp walks a list to find its work.
//
// The tensor maps describe a weight matrix as (bytes of one group of a row, rows, groups along the
// row [, gate/up], cells): a box of 8 or 16 rows lands in shared memory as [group][row][group
// bytes], so the rows a shared-memory wavefront reads (4 rows x 32 bytes for int4 g64) are
// contiguous -- conflict-free without swizzle or padding -- and a 16 KB tile is ONE copy. (Measured
// on B200, one block per SM pulling 112 KB: 1 KB bulk copies issue at 58 ns each and reach 2.3
// TB/s; 16 KB tensor boxes issue in 0.07 us each and reach 6.7 TB/s. 16-byte cp.async from two
// warps: 3.5 TB/s, and per-unit mbarrier arrivals serialise the units.)
//
// What used to be launch boundaries are data hand-overs through L2, with no barrier object:
//   logits   every block computes its expert rows (fp32 rows were bulk-copied to shared memory
//            before the dependency wait) and publishes {epoch, value} as one 64-bit word per expert;
//   route    the last two blocks (they have the fewest router rows) gather all words, rank them
//            (comparison counting, no serial rounds), look the picks up in the residency table and
//            publish the instance list as 16-byte entries that each carry the epoch; every other
//            block's producer warp reads one of the two copies;
//   acts     a gate/up unit (8 gate rows + 8 up rows of one expert) publishes its 8 fp16
//            activations as 16 bytes whose halves are never the sentinel 0xFFFF, into each of a few
//            copies of the buffer (block b reads copy b mod kActCopies: polls of many blocks on the
//            same lines slow the writes to them); in a block that owns a tile of output rows every
//            warp polls just the words its own items multiply until no half is the sentinel. The
//            buffer of the previous call (other parity of the epoch) is reset by this call.
// Every wait -- mbarrier or global poll -- is bounded: it gives up, reports through the status
// word and the block runs on to its end.
//
// What bounds the kernel (measured with per-warp cycle stamps): not HBM. A warp of this code issues
// an instruction every 5 to 10 cycles (dependent shared-memory loads, logic ops and tiles; four warps
// share an issue port), so the serial chain router row -> gather -> rank -> publish -> read ->
// request -> first bytes -> gate/up -> exchange -> down costs about 14 us at the Qwen shape, of which
// the bytes need 2.4. Code that runs once per launch also pays for its instruction fetches (a body
// beyond about 32 KB streams at 6 bytes a cycle), which is why the waits, the walkers and the tile
// bodies are out of line and shared.
//
// MMA row slot s of a unit is row s of its box: rows 0..7 gate and 8..15 up in phase 1 (GLU partners
// in one thread), 16 consecutive down rows in phase 2.
#include <cuda.h>

#include <algorithm>

#include "router_math.cuh"
#include "select.cuh"

namespace shrike {

namespace {

constexpr uint32_t kGroups = 2;                      // consumer groups: each takes every second gate/up unit of the block
constexpr uint32_t kGroupWarps = 8;                  // warps of a group: they split a unit's columns (measured: 4 groups
                                                     // of 4 warps +0.16 us, one group of 16 +1.2 us)
constexpr uint32_t kCW = kGroups * kGroupWarps;      // consumer warps
constexpr uint32_t kSelWarps = 8;                    // consumer warps that take part in the selection (32 experts each)
constexpr uint32_t kFusedThreads = (1 + kCW) * 32;   // + the producer warp (its lanes issue the copies)
constexpr uint32_t kMaxUnits = 64;                   // units of one block
constexpr uint32_t kSelectors = 2;                   // blocks that select and publish the instance list (measured: 1-3 best, 8 +0.3 us, all +1.5 us;
                                                     // all of them with the logits in 32 copies still +0.2 us)
constexpr uint32_t kRouteCopies = 1;                 // copies of the list each of them writes (measured: 4 and 8 change nothing)
constexpr uint32_t kActCopies = 8;                   // copies of the published activations, block b polls copy b % 8
                                                     // (measured: 1 copy +0.5 us, 4 to 16 alike, one per block +2.2 us)
constexpr uint32_t kMaxInst = SHRIKE_MAX_TOP_K + 1;  // picks + shared expert
constexpr uint32_t kMaxSlots = 16;
constexpr uint32_t kMaxRouterRowsPerBlock = 2;

}  // namespace

// Sizes and offsets the host works out once per handle.
struct FusedGeom {
    uint32_t p1_meta_off, p1_ab_off, p1_bytes;
    // phase-2 pack entries: [0] routed experts, [1] the shared expert
    uint32_t p2_meta_off[2], p2_ab_off[2], p2_expert_bytes[2];
    uint32_t experts_per_pack;           // routed experts per phase-2 unit
    uint32_t slot_bytes, n_slots;
    uint32_t off_x, off_xraw, off_rw, off_xs, off_acts, off_asum, off_ring, smem_bytes;   // dynamic shared memory
    uint32_t acts_stride;                // halves per instance in the activation buffers
    uint32_t cg_p1, cg_p2[2];            // groups per chunk (1, 2 or 4)
    uint32_t router_rows_per_block;
    // ceil(2^24 / c) for the divisors the block plan uses (numerators below 4096): a multiply and a shift
    uint32_t rcp_blocks, rcp_upe, rcp_slots, rcp_epp, rcp_bps, rcp_gmax2, rcp_cpe_r;
};

// Tensor maps of one expert block layout: entries 0..7 the pool's chunks, entry 8 the shared expert's block.
struct FusedMaps {
    CUtensorMap w1[SHRIKE_MAX_POOL_CHUNKS + 1];   // gate + up rows: (group bytes, rows, groups, 2, cells)
    CUtensorMap m1[SHRIKE_MAX_POOL_CHUNKS + 1];   // their scales and biases: (8 rows' worth, rows / 8, scale|bias, 2, cells)
    CUtensorMap w2[SHRIKE_MAX_POOL_CHUNKS + 1];   // down rows: (group bytes, rows, groups, cells)
    CUtensorMap m2[SHRIKE_MAX_POOL_CHUNKS + 1];   // their scales and biases: (8 rows' worth, rows / 8, scale|bias, cells)
};

struct FusedArgs {
    PoolView pool;
    Offsets3 routed, shared;
    const uint8_t* shared_block;
    uint32_t d, f, f_shared, top_k, activation, expert_bias, act_dtype, y_dtype;
    // router (field names as the selection helpers expect them)
    const void* rw;
    const uint16_t* rscales;
    const uint16_t* rbiases;
    uint32_t rbits;
    const float* gate_row;
    const uint16_t* eff_scale;
    const uint16_t* logit_bias;
    const uint16_t* per_expert_scale;
    uint32_t ne, sigmoid_scores, round_f16;
    float scaling;
    const uint64_t* table;
    uint32_t pool_cells;
    const uint32_t* io_status;
    const void* x;
    void* y;
    void* hidden;
    uint32_t* out_ids;
    float* out_w;
    uint32_t* out_slots;
    float* out_gate;
    unsigned long long* logits64;   // [ne + 1]: {epoch, logit bits}
    uint16_t* acts_pub;             // [2][kActCopies][kMaxInst][acts_stride] halves, 0xFFFF = not yet written
    uint32_t* epoch;
    uint32_t* status;
#ifdef SHRIKE_TRACE
    uint64_t* trace;   // debug builds: 16 timestamps per block
#endif
    uint32_t rcp_cpc;               // ceil(2^32 / cells_per_chunk): cell / cells_per_chunk = mulhi(cell, rcp_cpc)
    FusedGeom g;
    FusedMaps maps;
};

namespace {

template <int BITS, int GROUP>
struct FQ {
    static constexpr int kWords = GROUP * BITS / 128;   // u32 per thread, row and group
    static constexpr int kMmas = GROUP / 16;
    static constexpr int kBRegs = GROUP / 8;
    static constexpr uint32_t kGroupBytes = GROUP * BITS / 8;
    // what the tiles multiply is offset + q: 1024 + q for nibbles in bits 0..3 (and for bytes), 64 + q for
    // nibbles in bits 4..7 (the fp16 value 64 has its unit in the last place at bit 4): no shift to unpack
    static constexpr float kOffEven = 1024.0f;
    static constexpr float kOffOdd = BITS == 4 ? 64.0f : 1024.0f;
};

// One unit of work of a block, as every warp reads it from the block's table (8 bytes).
//   bits 0     kind: 0 phase 1 (8 gate + 8 up rows of one instance), 1 phase 2 (16 output rows x a pack)
//   bit  1     the shared expert's geometry
//   bits 4-7   first instance          bits 8-11  instances in the pack (0: the layer has no expert work at all)
//   bits 20-24 ring slot               bit 25     parity of the slot's round
struct alignas(8) UnitRec {
    uint32_t bits, r0;
    __device__ uint32_t kind() const { return bits & 1u; }
    __device__ uint32_t sh() const { return (bits >> 1) & 1u; }
    __device__ uint32_t inst() const { return (bits >> 4) & 15u; }
    __device__ uint32_t count() const { return (bits >> 8) & 15u; }
    __device__ uint32_t slot() const { return (bits >> 20) & 31u; }
    __device__ uint32_t parity() const { return (bits >> 25) & 1u; }
};

struct RouteSmem {
    uint32_t cell[kMaxInst];    // per instance (shared expert first when there is one)
    float w[kMaxInst];          // route weight, or the shared expert's gate
    uint32_t n_inst, n_routed;
};

struct FusedStatic {
    alignas(16) uint64_t table[SHRIKE_MAX_EXPERTS];
    float logits[SHRIKE_MAX_EXPERTS + 1];
    // selection: {key, ~expert id} of every expert, every selecting warp's best eight, the picks in rank order
    alignas(16) unsigned long long ckeys[SHRIKE_MAX_EXPERTS], cand[kSelWarps * 8], sel[SHRIKE_MAX_TOP_K];
    RouteSmem route;
    UnitRec units[kMaxUnits];                      // UnitRec, in the order the block takes them
    float red[kGroups][2][kGroupWarps][16];        // a group's partial sums, two units deep
    float red2[2][kCW][16];                        // every consumer warp's sums of a down tile, two tiles deep
    alignas(16) uint16_t act_stage[kGroups][8];
    uint64_t full[kMaxSlots], empty[kMaxSlots], rw_bar, tab_bar;
    uint32_t epoch, failed;
};

__device__ __forceinline__ bool try_wait_bar(uint32_t addr, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
    return ok != 0;
}
// The bounded part of a wait, out of line: the kernel's instruction stream holds one copy of it.
__device__ __noinline__ bool wait_bar_slow(uint32_t addr, uint32_t parity) {
#pragma unroll 1
    for (uint32_t it = 0; it < (1u << 17); ++it) {
        if (try_wait_bar(addr, parity)) return true;
        if (it > 128) __nanosleep(32);
    }
    return false;
}
__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    return try_wait_bar(addr, parity) || wait_bar_slow(addr, parity);
}
__device__ __forceinline__ void bar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void bar_arrive_n(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_relaxed_v4(const void* p) {
    uint4 v;
    asm volatile("ld.relaxed.gpu.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_v4(void* p, uint4 v) {
    asm volatile("st.relaxed.gpu.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}
// Named barriers: 1 the selecting warps, 2 all consumer warps, 3.. one per consumer group.
__device__ __forceinline__ void select_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kSelWarps * 32) : "memory"); }
__device__ __forceinline__ void consumers_sync() { asm volatile("bar.sync 2, %0;" ::"n"(kCW * 32) : "memory"); }
__device__ __forceinline__ void group_sync(uint32_t group) {
    asm volatile("bar.sync %0, %1;" ::"r"(3u + group), "n"(kGroupWarps * 32) : "memory");
}

__device__ __forceinline__ bool has_sentinel(uint4 v) {
    auto bad = [](uint32_t w) { return (w & 0xffffu) == 0xffffu || (w >> 16) == 0xffffu; };
    return bad(v.x) || bad(v.y) || bad(v.z) || bad(v.w);
}

// What a block does, in closed form (every lane can work out any unit on its own): phase-1 units blk, blk +
// n_blk, ... of the sequence [shared expert's units | first pick's | second pick's ...], then the packs of the
// output tiles n_blk - 1 - blk, + n_blk, ... (blocks that are light in one phase are heavy in the other).
// n / c for n < 4096 and c < 4096, with rcp = ceil(2^24 / c)
__device__ __forceinline__ uint32_t div_rcp(uint32_t n, uint32_t rcp) { return (uint32_t)(((unsigned long long)n * rcp) >> 24); }

struct BlockPlan {
    uint32_t n_blk, blk, su, upe, has_shared, tiles, epp, n_slots;
    uint32_t rcp_blocks, rcp_upe, rcp_slots, rcp_epp;
    uint32_t n_routed, n1, n_tiles, packs, packs_eff, n_units;

    __device__ void init(const FusedArgs& a) {
        n_blk = gridDim.x; blk = blockIdx.x;
        has_shared = a.shared_block ? 1u : 0u;
        su = has_shared ? a.f_shared / 8 : 0u;
        upe = a.f / 8;
        tiles = a.d / 16;
        epp = a.g.experts_per_pack;
        n_slots = a.g.n_slots;
        rcp_blocks = a.g.rcp_blocks; rcp_upe = a.g.rcp_upe; rcp_slots = a.g.rcp_slots; rcp_epp = a.g.rcp_epp;
        const uint32_t t0 = n_blk - 1u - blk;
        n_tiles = t0 < tiles ? div_rcp(tiles - t0 + n_blk - 1u, rcp_blocks) : 0u;
    }
    // phase-1 units of the shared expert: they do not depend on the routing
    __device__ uint32_t shared_units() const { return blk < su ? div_rcp(su - blk + n_blk - 1u, rcp_blocks) : 0u; }
    __device__ void route(uint32_t routed) {
        n_routed = routed;
        const uint32_t total1 = su + n_routed * upe;
        n1 = blk < total1 ? div_rcp(total1 - blk + n_blk - 1u, rcp_blocks) : 0u;
        packs = has_shared + div_rcp(n_routed + epp - 1u, rcp_epp);
        packs_eff = packs ? packs : 1u;
        n_units = n1 + n_tiles * packs_eff;
    }
    __device__ UnitRec phase1(uint32_t i) const {
        const uint32_t idx = blk + i * n_blk;
        UnitRec u;
        if (idx < su) {
            u.bits = 0u | 2u | (1u << 8);
            u.r0 = idx * 8u;
        } else {
            const uint32_t k = idx - su, e = div_rcp(k, rcp_upe);
            u.bits = ((has_shared + e) << 4) | (1u << 8);
            u.r0 = (k - e * upe) * 8u;
        }
        const uint32_t round = div_rcp(i, rcp_slots);
        u.bits |= ((i - round * n_slots) << 20) | ((round & 1u) << 25);
        return u;
    }
    __device__ UnitRec unit(uint32_t i) const {
        if (i < n1) return phase1(i);
        const uint32_t j = i - n1, m = j / packs_eff, p = j - m * packs_eff;
        UnitRec u;
        u.r0 = (n_blk - 1u - blk + m * n_blk) * 16u;
        const uint32_t round = div_rcp(i, rcp_slots);
        u.bits = 1u | ((i - round * n_slots) << 20) | ((round & 1u) << 25);
        if (packs == 0u) return u;   // count 0
        if (has_shared && p == 0u) {
            u.bits |= 2u | (1u << 8);
        } else {
            const uint32_t q = p - has_shared;
            u.bits |= ((has_shared + q * epp) << 4) | (min(epp, n_routed - q * epp) << 8);
        }
        return u;
    }
};

template <int BITS>
__device__ __forceinline__ void unpack2(const uint32_t* w, int m, uint32_t& lo, uint32_t& hi) {
    if constexpr (BITS == 4) {
        const uint32_t v = w[m >> 1] >> ((m & 1) * 8);
        lo = lop3_and_or(v, 0x000F000Fu, 0x64006400u);   // (1024 + n0, 1024 + n4)
        hi = lop3_and_or(v, 0x00F000F0u, 0x54005400u);   // (64 + n1, 64 + n5)
    } else {
        const uint32_t v = w[m];
        lo = prmt(v, 0x64646464u, 0x5140u);
        hi = prmt(v, 0x64646464u, 0x5342u);
    }
}

template <int W>
__device__ __forceinline__ void lds_words(const uint8_t* p, uint32_t (&w)[W]) {
    if constexpr (W == 1) {
        w[0] = *(const uint32_t*)p;
    } else if constexpr (W == 2) {
        const uint2 v = *(const uint2*)p;
        w[0] = v.x; w[1] = v.y;
    } else {
        const uint4 v = *(const uint4*)p;
        w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
    }
}

// CG consecutive 16-bit values starting at an address that is a multiple of min(2 * CG, 4) bytes.
template <int CG, int META>
__device__ __forceinline__ void lds_meta(const uint8_t* p, float (&out)[CG]) {
    if constexpr (CG == 1) {
        out[0] = meta_to_f32<META>(*(const uint16_t*)p);
    } else if constexpr (CG == 2) {
        const uint32_t v = *(const uint32_t*)p;
        out[0] = meta_to_f32<META>((uint16_t)(v & 0xffffu));
        out[1] = meta_to_f32<META>((uint16_t)(v >> 16));
    } else {
        // two 32-bit loads where a row of scales is only 4-byte aligned (group count even, not a multiple of 4)
        const uint2 v = make_uint2(*(const uint32_t*)p, *(const uint32_t*)(p + 4));
        out[0] = meta_to_f32<META>((uint16_t)(v.x & 0xffffu));
        out[1] = meta_to_f32<META>((uint16_t)(v.x >> 16));
        out[2] = meta_to_f32<META>((uint16_t)(v.y & 0xffffu));
        out[3] = meta_to_f32<META>((uint16_t)(v.y >> 16));
    }
}

// CG consecutive groups of two MMA rows against one activation row (the same in every column).
// rowA/rowB: this thread's address in group 0 of the two rows; slab: bytes from one group to the next;
// s*/b*: addresses of the rows' scale and bias arrays at group 0; bsm: fp16 operand copy of the activation
// row; xs: {sum x, sum offset*x} per group.
// Returns scale*sum(q x) + bias*sum(x) summed over the groups, for both rows.
// Not inlined: phase 1 and phase 2 share the code, and the kernel's instruction footprint is what a block
// pays for on every launch (each code region is run once, so every instruction line is a cache miss).
template <int BITS, int GROUP, int META, int CG>
__device__ __noinline__ float2 chunk_rows(const uint8_t* rowA, const uint8_t* rowB, uint32_t slab, const uint8_t* s0p,
                                          const uint8_t* b0p, const uint8_t* s1p, const uint8_t* b1p,
                                          const uint16_t* bsm, const float2* xs, uint32_t grp0, uint32_t t) {
    using Q = FQ<BITS, GROUP>;
    uint32_t raw[CG][2][Q::kWords];
    uint32_t bf[CG][Q::kBRegs];
    float2 xv[CG];
#pragma unroll
    for (int i = 0; i < CG; ++i) {
        lds_words<Q::kWords>(rowA + (size_t)(grp0 + i) * slab, raw[i][0]);
        lds_words<Q::kWords>(rowB + (size_t)(grp0 + i) * slab, raw[i][1]);
        const uint4* bp = (const uint4*)(bsm + (size_t)(grp0 + i) * GROUP + t * (GROUP / 4));
        const uint4 v0 = bp[0];
        bf[i][0] = v0.x; bf[i][1] = v0.y; bf[i][2] = v0.z; bf[i][3] = v0.w;
        if constexpr (GROUP == 64) {
            const uint4 v1 = bp[1];
            bf[i][4] = v1.x; bf[i][5] = v1.y; bf[i][6] = v1.z; bf[i][7] = v1.w;
        }
        xv[i] = xs[grp0 + i];
    }
    float sc0[CG], bi0[CG], sc1[CG], bi1[CG];
    lds_meta<CG, META>(s0p + (size_t)grp0 * 2, sc0);
    lds_meta<CG, META>(b0p + (size_t)grp0 * 2, bi0);
    lds_meta<CG, META>(s1p + (size_t)grp0 * 2, sc1);
    lds_meta<CG, META>(b1p + (size_t)grp0 * 2, bi1);
    float q0 = 0.f, q1 = 0.f, z0 = 0.f, z1 = 0.f;
#pragma unroll
    for (int i = 0; i < CG; ++i) {
        float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int m = 0; m < Q::kMmas; ++m) {
            uint32_t lo0, hi0, lo1, hi1;
            unpack2<BITS>(raw[i][0], m, lo0, hi0);
            unpack2<BITS>(raw[i][1], m, lo1, hi1);
            mma_16816(c, lo0, lo1, hi0, hi1, bf[i][2 * m], bf[i][2 * m + 1]);
        }
        // c = sum((offset + q) x): take the offsets out, then one multiply-add with the scale and one with the bias
        q0 = fmaf(sc0[i], c[0] - xv[i].y, q0);
        q1 = fmaf(sc1[i], c[2] - xv[i].y, q1);
        z0 = fmaf(bi0[i], xv[i].x, z0);
        z1 = fmaf(bi1[i], xv[i].x, z1);
    }
    return make_float2(q0 + z0, q1 + z1);
}

// Chunk c of a row of `groups` groups. Width 4: chunks of four groups and, when two groups are left over, a last
// chunk of two (90 groups of 32 at d = 2880: 22 + 1 chunks, not 45 of two). One call site per width.
template <int BITS, int GROUP, int META>
__device__ __forceinline__ float2 chunk_rows_cg(uint32_t cg, uint32_t groups, const uint8_t* rowA, const uint8_t* rowB,
                                                uint32_t slab, const uint8_t* s0p, const uint8_t* b0p, const uint8_t* s1p,
                                                const uint8_t* b1p, const uint16_t* bsm, const float2* xs, uint32_t c,
                                                uint32_t t) {
    if (cg == 4) {
        if (c * 4 + 4 <= groups) return chunk_rows<BITS, GROUP, META, 4>(rowA, rowB, slab, s0p, b0p, s1p, b1p, bsm, xs, c * 4, t);
        return chunk_rows<BITS, GROUP, META, 2>(rowA, rowB, slab, s0p, b0p, s1p, b1p, bsm, xs, c * 4, t);
    }
    if (cg == 2) return chunk_rows<BITS, GROUP, META, 2>(rowA, rowB, slab, s0p, b0p, s1p, b1p, bsm, xs, c * 2, t);
    return chunk_rows<BITS, GROUP, META, 1>(rowA, rowB, slab, s0p, b0p, s1p, b1p, bsm, xs, c, t);
}
// chunks of a row of `groups` groups at width cg
__device__ __forceinline__ uint32_t chunks_of(uint32_t groups, uint32_t cg) {
    return cg == 4 ? (groups + 3) >> 2 : cg == 2 ? groups >> 1 : groups;
}

// {sum x, sum offset * x} of group `grp` of an fp16 operand row in shared memory.
template <int BITS, int GROUP>
__device__ __noinline__ float2 group_sums(const uint16_t* row, uint32_t grp) {
    using Q = FQ<BITS, GROUP>;
    float even = 0.f, odd = 0.f;
    const uint4* p = (const uint4*)(row + (size_t)grp * GROUP);
#pragma unroll
    for (int b = 0; b < GROUP / 8; ++b) {
        const uint4 v = p[b];
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        float h[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            h[2 * j] = f16_bits_to_f32((uint16_t)(w[j] & 0xffffu));
            h[2 * j + 1] = f16_bits_to_f32((uint16_t)(w[j] >> 16));
        }
        if constexpr (BITS == 4) {   // positions {0,1,4,5} hold the even elements, {2,3,6,7} the odd ones
            even += (h[0] + h[1]) + (h[4] + h[5]);
            odd += (h[2] + h[3]) + (h[6] + h[7]);
        } else {
            even += ((h[0] + h[1]) + (h[2] + h[3])) + ((h[4] + h[5]) + (h[6] + h[7]));
        }
    }
    return make_float2(even + odd, Q::kOffEven * even + Q::kOffOdd * odd);
}

#ifdef SHRIKE_TRACE
// the SM's cycle counter: cheap to read (the global timer was measured to hold a warp for about 2 us per read).
// Every warp keeps 32 stamps.
#define FUSED_TS(slot) do { if (a.trace && lane == 0) a.trace[((size_t)blockIdx.x * (kFusedThreads / 32) + warp) * 32 + (slot)] = (uint64_t)clock64(); } while (0)
#else
#define FUSED_TS(slot) do { } while (0)
#endif

// Tiled TMA loads (no multicast): the box lands densely, innermost dimension first.
__device__ __forceinline__ void tma_4d(uint32_t dst, const CUtensorMap* map, int32_t c0, int32_t c1, int32_t c2, int32_t c3,
                                       uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_5d(uint32_t dst, const CUtensorMap* map, int32_t c0, int32_t c1, int32_t c2, int32_t c3,
                                       int32_t c4, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(smem_u32(bar)) : "memory");
}

// Top-k of the logits in shared memory by the first kSelWarps consumer warps, without serial rounds: (score
// descending, expert id ascending) is a total order, so the number of experts that beat one is its rank.
// An expert's key and the complement of its id make one 64-bit word whose unsigned order is that order.
// Warp w ranks experts 32w..32w+31 among themselves and keeps the best eight; two warps rank the 64
// survivors. The picks and their order are those of router_topk_select_body's insertion scan
// (moe.metal:436-456). Lane r of warp 0 returns the r-th pick. All kSelWarps warps call it.
template <class A, class S>
__device__ __forceinline__ void select_ranked(const float* lg, const A& a, S& st, uint32_t cw, uint32_t lane,
                                              uint32_t& out_id, float& out_w) {
    const uint32_t e = cw * 32 + lane;
    uint32_t key = 0;
    if (e < a.ne) key = selection_key_of(lg[e], a.logit_bias ? bf16_bits_to_f32(a.logit_bias[e]) : 0.0f, a);
    const unsigned long long mine = ((unsigned long long)key << 32) | (unsigned long long)(0xffffffffu - e);
    st.ckeys[e] = mine;
    __syncwarp();
    {
        const ulonglong2* kv = (const ulonglong2*)(st.ckeys + cw * 32);
        uint32_t rank = 0;
#pragma unroll
        for (uint32_t j = 0; j < 16; ++j) {
            const ulonglong2 v = kv[j];
            rank += (v.x > mine ? 1u : 0u) + (v.y > mine ? 1u : 0u);
        }
        if (rank < 8) st.cand[cw * 8 + rank] = mine;   // the words are distinct: one lane per rank
    }
    select_sync();
    if (cw < 2) {
        const unsigned long long c = st.cand[cw * 32 + lane];
        const ulonglong2* cv = (const ulonglong2*)st.cand;
        uint32_t rank = 0;
#pragma unroll
        for (uint32_t j = 0; j < kSelWarps * 4; ++j) {
            const ulonglong2 v = cv[j];
            rank += (v.x > c ? 1u : 0u) + (v.y > c ? 1u : 0u);
        }
        if (rank < SHRIKE_MAX_TOP_K) st.sel[rank] = c;
    }
    select_sync();
    out_id = 0;
    out_w = 0.f;
    if (cw == 0) {
        float my_score = -INFINITY;
        uint32_t my_id = 0;
        if (lane < a.top_k) {
            const unsigned long long c = st.sel[lane];
            const uint32_t k = (uint32_t)(c >> 32);
            my_score = score_of_key(k);   // key 0: no candidate, the scan's initial -inf and id 0
            my_id = k ? min(0xffffffffu - (uint32_t)c, a.ne - 1u) : 0u;
        }
        out_w = selection_weight<false>(lg, a, lane, my_score, my_id);
        out_id = my_id;
    }
}

__device__ __noinline__ float affine_row_dot(const uint8_t* row, const uint16_t* s_row, const uint16_t* b_row, uint32_t bits,
                                             uint32_t groups, uint32_t lane, const void* xrow, uint32_t dt,
                                             const uint16_t* eff_scale) {
    return lane_dot_affine(row, s_row, b_row, bits, groups, lane, xrow, dt, eff_scale);
}
__device__ __noinline__ float glu_call(float gate, float up, uint32_t activation) { return glu(gate, up, activation); }

// What the selection helpers read of the router, with the plain router's choices (softmax scores, no selection
// bias, no per-expert scale) as constants.
struct PlainRouterView {
    uint32_t ne, top_k, round_f16;
    static constexpr uint32_t sigmoid_scores = 0;
    static constexpr const uint16_t* logit_bias = nullptr;
    static constexpr const uint16_t* per_expert_scale = nullptr;
    static constexpr float scaling = 1.0f;
};

// PLAIN: the layer is bf16 rows in, fp32 router rows with softmax scores and no bias or scale operands, SiLU, no
// additive expert biases (the flagship shapes): those
// choices are then constants of the instruction stream instead of branches in it. A kernel of this kind runs
// every code region once per launch, so what it does not fetch it does not wait for.
template <int BITS, int GROUP, int META, bool PLAIN>
__global__ void __launch_bounds__(kFusedThreads, 1) decode_layer_kernel(const __grid_constant__ FusedArgs a) {
    const uint32_t cfg_act_dtype = PLAIN ? (uint32_t)SHRIKE_DTYPE_BF16 : a.act_dtype;
    const uint32_t cfg_activation = PLAIN ? (uint32_t)SHRIKE_ACT_SILU : a.activation;
    const uint32_t cfg_expert_bias = PLAIN ? 0u : a.expert_bias;
    const uint32_t cfg_rbits = PLAIN ? 0u : a.rbits;
    using Q = FQ<BITS, GROUP>;
    extern __shared__ __align__(128) uint8_t dsm[];
    __shared__ FusedStatic st;
    const FusedGeom& G = a.g;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t D = a.d, GD = D / GROUP;
    const uint32_t rb1 = D * BITS / 8;
    uint16_t* x_sm = (uint16_t*)(dsm + G.off_x);
    float2* xs_sm = (float2*)(dsm + G.off_xs);
    uint16_t* acts_sm = (uint16_t*)(dsm + G.off_acts);
    float2* asum_sm = (float2*)(dsm + G.off_asum);
    uint8_t* ring = dsm + G.off_ring;
    const uint32_t ring_smem = smem_u32(ring);
    const uint32_t has_shared = a.shared_block ? 1u : 0u;
    const uint32_t gmax2 = G.acts_stride / GROUP;
    const bool is_producer = warp == 0;
    const uint32_t cw = warp - 1u;     // consumer index of the consumer warps

    FUSED_TS(0);
    BlockPlan plan;
    plan.init(a);

    // ---- before the previous kernel in the stream is known to be complete: nothing that it produces ----
    // (Measured: the dependency wait and the row's load moved up here, ahead of this set-up, +0.5 us -- the wait
    // returns only some time after the previous kernel's last block has left, and the set-up fills that time.)
    if (tid < G.n_slots) {
        mbar_init(&st.full[tid], 1);
        mbar_init(&st.empty[tid], kGroupWarps);
    }
    if (tid == 32) { mbar_init(&st.rw_bar, 1); mbar_init(&st.tab_bar, 1); }
    if (tid <= 32) fence_mbar_init();
    if (tid == 0) st.failed = 0;
    // (No prefetch.tensormap of the descriptors here: measured, it holds the prologue back by 0.6 us -- the
    // first copy through a descriptor fetches it just as well.)
    const uint32_t router_rows = a.ne + (a.gate_row ? 1u : 0u);
    const uint32_t my_row = blockIdx.x + cw * gridDim.x;
    const bool routes = !is_producer && cw < G.router_rows_per_block && my_row < router_rows;
    const bool row_is_gate = routes && a.gate_row && my_row == a.ne;
    const bool row_f32 = cfg_rbits == 0 || row_is_gate;
    __syncthreads();   // barriers initialised
    if (tid == 32) {
        // fp32 router rows (and the gate row) of this block -> shared memory, one bulk copy each
        uint32_t bytes = 0;
        for (uint32_t k = 0; k < G.router_rows_per_block; ++k) {
            const uint32_t e = blockIdx.x + k * gridDim.x;
            const bool gate = a.gate_row && e == a.ne;
            if (e < router_rows && (cfg_rbits == 0 || gate)) bytes += D * 4;
        }
        mbar_expect_tx(&st.rw_bar, bytes);
        for (uint32_t k = 0; k < G.router_rows_per_block; ++k) {
            const uint32_t e = blockIdx.x + k * gridDim.x;
            const bool gate = a.gate_row && e == a.ne;
            if (e < router_rows && (cfg_rbits == 0 || gate))
                bulk_g2s(dsm + G.off_rw + (size_t)k * D * 4, gate ? (const void*)a.gate_row : (const void*)((const float*)a.rw + (size_t)e * D),
                         D * 4, &st.rw_bar);
        }
    }

    // One lane asks for one unit: one to four tiled copies that complete on the slot's barrier.
    auto issue = [&](const UnitRec u) {
        const uint32_t slot = u.slot();
        const uint32_t stage = ring_smem + slot * G.slot_bytes;
        uint64_t* bar = &st.full[slot];
        const uint32_t sh = u.sh();
        if (u.kind() == 0) {
            const uint32_t cell = sh ? 0u : st.route.cell[u.inst()];
            const uint32_t ch = __umulhi(cell, a.rcp_cpc);   // cell / cells_per_chunk
            const uint32_t mi = sh ? SHRIKE_MAX_POOL_CHUNKS : ch;
            const int32_t cc = sh ? 0 : (int32_t)(cell - ch * a.pool.cells_per_chunk);
            mbar_expect_tx(bar, 16 * rb1 + 64 * GD + (cfg_expert_bias ? 32u : 0u));
            tma_5d(stage + G.p1_meta_off, &a.maps.m1[mi], 0, (int32_t)(u.r0 / 8), 0, 0, cc, bar);   // the small one first
            tma_5d(stage, &a.maps.w1[mi], 0, (int32_t)u.r0, 0, 0, cc, bar);
            if (cfg_expert_bias) {
                const uint8_t* base = sh ? a.shared_block : pool_cell_base(a.pool, cell);
                const Offsets3& off = sh ? a.shared : a.routed;
                bulk_g2s(ring + (size_t)slot * G.slot_bytes + G.p1_ab_off, base + off.ab[0] + (size_t)u.r0 * 2, 16, bar);
                bulk_g2s(ring + (size_t)slot * G.slot_bytes + G.p1_ab_off + 16, base + off.ab[1] + (size_t)u.r0 * 2, 16, bar);
            }
        } else {
            const uint32_t F = sh ? a.f_shared : a.f, G2 = F / GROUP, rb2 = F * BITS / 8;
            const uint32_t count = u.count();
            mbar_expect_tx(bar, count * (16 * rb2 + 64 * G2 + (cfg_expert_bias ? 32u : 0u)));   // count 0: the arrival alone
            for (uint32_t q = 0; q < count; ++q) {
                const uint32_t cell = sh ? 0u : st.route.cell[u.inst() + q];
                const uint32_t ch = __umulhi(cell, a.rcp_cpc);   // cell / cells_per_chunk
                const uint32_t mi = sh ? SHRIKE_MAX_POOL_CHUNKS : ch;
                const int32_t cc = sh ? 0 : (int32_t)(cell - ch * a.pool.cells_per_chunk);
                const uint32_t eb = stage + q * G.p2_expert_bytes[sh];
                tma_4d(eb + G.p2_meta_off[sh], &a.maps.m2[mi], 0, (int32_t)(u.r0 / 8), 0, cc, bar);
                tma_4d(eb, &a.maps.w2[mi], 0, (int32_t)u.r0, 0, cc, bar);
                if (cfg_expert_bias) {
                    const uint8_t* base = sh ? a.shared_block : pool_cell_base(a.pool, cell);
                    const Offsets3& off = sh ? a.shared : a.routed;
                    bulk_g2s(ring + (size_t)slot * G.slot_bytes + q * G.p2_expert_bytes[sh] + G.p2_ab_off[sh],
                             base + off.ab[2] + (size_t)u.r0 * 2, 32, bar);
                }
            }
        }
    };

    // the shared expert's gate/up units do not depend on the routing (nor on the previous kernel): the lanes
    // of the producer warp ask for one each, now
    const uint32_t n_pre = min(plan.shared_units(), G.n_slots);
    if (is_producer && lane < n_pre) issue(plan.phase1(lane));

    FUSED_TS(1);
    pdl_wait();
    FUSED_TS(2);

    // ---- the activation row: every thread takes 8 elements in one round trip and leaves the fp16 operand
    // copy (permuted for the tiles, clamped to the fp16 range), the fp32 copy the router multiplies, and --
    // with the lanes that share a group -- the group's {sum x, sum offset*x} ----
    {
        if (tid == kFusedThreads - 1) st.epoch = *(volatile const uint32_t*)a.epoch;
        float* xf_sm = (float*)(dsm + G.off_xraw);
        constexpr uint32_t kLanes = GROUP / 8;   // lanes of a group
        for (uint32_t base = warp * 32; base < D / 8; base += kFusedThreads) {
            const uint32_t blk = base + lane;
            const bool valid = blk < D / 8;
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = 0.f;
            if (valid) {
                if (cfg_act_dtype == SHRIKE_DTYPE_FP32) {
                    const float4 lo = __ldg((const float4*)a.x + 2 * blk), hi = __ldg((const float4*)a.x + 2 * blk + 1);
                    v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w; v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
                } else {
                    const uint4 raw = __ldg((const uint4*)a.x + blk);
                    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (cfg_act_dtype == SHRIKE_DTYPE_FP16) {
                            v[2 * j] = f16_bits_to_f32((uint16_t)(w[j] & 0xffffu));
                            v[2 * j + 1] = f16_bits_to_f32((uint16_t)(w[j] >> 16));
                        } else {
                            v[2 * j] = __uint_as_float(w[j] << 16);
                            v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
                        }
                    }
                }
                ((float4*)xf_sm)[2 * blk] = make_float4(v[0], v[1], v[2], v[3]);
                ((float4*)xf_sm)[2 * blk + 1] = make_float4(v[4], v[5], v[6], v[7]);
            }
            if (cfg_act_dtype != SHRIKE_DTYPE_FP16) {
                bool over = false;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if (fabsf(v[j]) > kHalfMax) {   // false for NaN, which passes through
                        over = true;
                        v[j] = copysignf(kHalfMax, v[j]);
                    }
                }
                if (over) report_status(a.status, kStatusOperandRange);
            }
            uint16_t o[8];
            float even = 0.f, odd = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const __half h = __float2half_rn(v[j]);
                o[perm_index(j, BITS == 4)] = __half_as_ushort(h);
                if (BITS == 4 && (j & 1)) odd += __half2float(h);
                else even += __half2float(h);
            }
            if (valid)
                *(uint4*)(x_sm + (size_t)blk * 8) = make_uint4(o[0] | ((uint32_t)o[1] << 16), o[2] | ((uint32_t)o[3] << 16),
                                                                 o[4] | ((uint32_t)o[5] << 16), o[6] | ((uint32_t)o[7] << 16));
#pragma unroll
            for (uint32_t m = 1; m < kLanes; m <<= 1) {
                even += __shfl_xor_sync(0xffffffffu, even, m);
                odd += __shfl_xor_sync(0xffffffffu, odd, m);
            }
            if (valid && (blk & (kLanes - 1)) == 0) xs_sm[blk / kLanes] = make_float2(even + odd, Q::kOffEven * even + Q::kOffOdd * odd);
        }
    }
    // the selecting blocks need the layer's residency table (a kernel before this one may have written it)
    const uint32_t n_sel = min(kSelectors, gridDim.x);
    const bool selector = blockIdx.x >= gridDim.x - n_sel;
    const uint32_t tab_bytes = a.ne * 8u;
    const bool tab_bulk = (tab_bytes & 15u) == 0 && ((uintptr_t)a.table & 15u) == 0;
    if (selector) {
        if (tid == 32) {
            mbar_expect_tx(&st.tab_bar, tab_bulk ? tab_bytes : 0u);
            if (tab_bulk) bulk_g2s(st.table, a.table, tab_bytes, &st.tab_bar);
        }
        if (!tab_bulk)
            for (uint32_t e = tid; e < a.ne; e += kFusedThreads) st.table[e] = a.table[e];
    }
    FUSED_TS(16);
    __syncthreads();
    const uint32_t epoch = st.epoch;
    const uint32_t parity = epoch & 1u;
    // the published activations exist in a few copies, so that the polls of all the blocks do not meet on the
    // same lines; whoever finishes a gate/up unit writes the unit's 16 bytes into every copy
    const size_t acts_copy = (size_t)kMaxInst * G.acts_stride;
    uint16_t* acts_call = a.acts_pub + (size_t)parity * kActCopies * acts_copy;
    uint16_t* acts_mine = acts_call + (size_t)(blockIdx.x % kActCopies) * acts_copy;
    uint4* route_pub = (uint4*)(a.logits64 + ((a.ne + 2u) & ~1u));   // [n_sel][1 + kMaxInst] 16-byte entries

    // ---- this block's router rows ----
    if (routes) {
        float acc;
        if (row_f32) {
            const uint32_t chunks = D / 4;
            const uint16_t* es = (PLAIN || row_is_gate) ? nullptr : a.eff_scale;
            if (!wait_bar(&st.rw_bar, 0)) report_status(a.status, kStatusWaitTimeout);
            const float4* wrow = (const float4*)(dsm + G.off_rw + (size_t)cw * D * 4);
            const float4* xf = (const float4*)(dsm + G.off_xraw);
            acc = 0.f;
            // lane l takes the float4 chunks l, l + 32, ... in order: the sequence of fused multiply-adds of
            // lane_dot_f32, both operands from shared memory
#pragma unroll 4
            for (uint32_t c = lane; c < chunks; c += 32) {
                const float4 wv = wrow[c];
                float4 xv = xf[c];
                if (es) {
                    const uint2 q = __ldg((const uint2*)es + c);
                    xv.x = __fmul_rn(xv.x, __uint_as_float(q.x << 16));
                    xv.y = __fmul_rn(xv.y, __uint_as_float(q.x & 0xffff0000u));
                    xv.z = __fmul_rn(xv.z, __uint_as_float(q.y << 16));
                    xv.w = __fmul_rn(xv.w, __uint_as_float(q.y & 0xffff0000u));
                }
                acc = __fmaf_rn(wv.x, xv.x, acc);
                acc = __fmaf_rn(wv.y, xv.y, acc);
                acc = __fmaf_rn(wv.z, xv.z, acc);
                acc = __fmaf_rn(wv.w, xv.w, acc);
            }
        } else {
            const uint32_t groups = D / 64;
            acc = affine_row_dot((const uint8_t*)a.rw + (size_t)my_row * (D * cfg_rbits / 8), a.rscales + (size_t)my_row * groups,
                                 a.rbiases + (size_t)my_row * groups, cfg_rbits, groups, lane, a.x, cfg_act_dtype, a.eff_scale);
        }
        acc = butterfly_sum(acc);
        if (lane == 0)
            st_relaxed_u64(a.logits64 + my_row, ((unsigned long long)epoch << 32) | (unsigned long long)__float_as_uint(acc));
        FUSED_TS(3);   // this block's logits are published
    }
    {   // the buffer the next call will use still holds the previous call's activations
        uint4* other = (uint4*)(a.acts_pub + (size_t)(parity ^ 1u) * kActCopies * acts_copy);
        const uint32_t n16 = kActCopies * kMaxInst * G.acts_stride / 8;
        const uint4 fill = make_uint4(0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu);
        for (uint32_t i = blockIdx.x * kFusedThreads + tid; i < n16; i += gridDim.x * kFusedThreads) other[i] = fill;
    }

    // ---- the selecting blocks (the last few: they have the fewest router rows) gather every block's logits,
    // pick, look the picks up and publish the instance list; every other block reads one copy of it ----
    if (selector) {
        for (uint32_t e = tid; e < router_rows; e += kFusedThreads) {
            bool ok = false;
            for (uint32_t it = 0; it < (1u << 17); ++it) {
                const unsigned long long v = ld_relaxed_u64(a.logits64 + e);
                if ((uint32_t)(v >> 32) == epoch) {
                    st.logits[e] = __uint_as_float((uint32_t)v);
                    ok = true;
                    break;
                }
                if (it > 64) __nanosleep(64);
            }
            if (!ok) {
                report_status(a.status, kStatusWaitTimeout);
                st.logits[e] = 0.f;
            }
        }
        FUSED_TS(18);
        __syncthreads();
        FUSED_TS(4);   // logits gathered
        if (!is_producer && cw < kSelWarps) {
            uint32_t id;
            float w;
            FUSED_TS(12);
            if constexpr (PLAIN) {
                const PlainRouterView view{a.ne, a.top_k, a.round_f16};
                select_ranked(st.logits, view, st, cw, lane, id, w);
            } else {
                select_ranked(st.logits, a, st, cw, lane, id, w);
            }
            FUSED_TS(13);
            if (cw == 0) {
                uint32_t io = 1u;
                if (a.io_status) io = *(volatile const uint32_t*)a.io_status;
                const bool ready = io == 1u || io == 3u;
                const bool first = blockIdx.x == gridDim.x - n_sel;   // the one that answers the caller
                uint32_t slot = SHRIKE_SLOT_MISS;
                if (!wait_bar(&st.tab_bar, 0)) report_status(a.status, kStatusWaitTimeout);
                if (lane < a.top_k) {
                    const uint64_t word = st.table[min(id, a.ne - 1u)];
                    slot = (uint32_t)(word & 0xffffffffu);
                    const bool hit = (uint32_t)(word >> 32) == 2u && slot != SHRIKE_SLOT_MISS;
                    if (!hit) slot = SHRIKE_SLOT_MISS;
                    if (first) {
                        // what the host reads back is the table's answer; what the kernel follows is range-checked
                        a.out_ids[lane] = id;
                        a.out_w[lane] = w;
                        if (a.out_slots) a.out_slots[lane] = slot;
                    }
                    if (slot != SHRIKE_SLOT_MISS && slot >= a.pool_cells) {
                        report_status(a.status, kStatusBadIndex);
                        slot = SHRIKE_SLOT_MISS;
                    }
                    if (!ready) slot = SHRIKE_SLOT_MISS;
                }
                const uint32_t hits = __ballot_sync(0xffffffffu, slot != SHRIKE_SLOT_MISS);
                if (slot != SHRIKE_SLOT_MISS) {
                    const uint32_t pos = has_shared + __popc(hits & ((1u << lane) - 1u));
                    st.route.cell[pos] = slot;
                    st.route.w[pos] = w;
                }
                if (lane == 0) {
                    st.route.n_routed = __popc(hits);
                    st.route.n_inst = has_shared + __popc(hits);
                    if (has_shared) {
                        st.route.cell[0] = 0;
                        st.route.w[0] = a.gate_row ? sigmoid_det(st.logits[a.ne]) : 1.0f;
                        if (a.gate_row && a.out_gate && first) a.out_gate[0] = st.route.w[0];
                    }
                }
                __syncwarp();
                // entry 0: the counts; entry 1 + i: instance i. Every 16-byte entry carries the epoch.
                uint4* mine = route_pub + (size_t)(blockIdx.x - (gridDim.x - n_sel)) * kRouteCopies * (1u + kMaxInst);
                if (lane <= kMaxInst) {
                    const uint4 e = lane == 0 ? make_uint4(epoch, st.route.n_routed, st.route.n_inst, 0u)
                                              : make_uint4(epoch, st.route.cell[lane - 1], __float_as_uint(st.route.w[lane - 1]), 0u);
#pragma unroll
                    for (uint32_t c = 0; c < kRouteCopies; ++c) st_relaxed_v4(mine + c * (1u + kMaxInst) + lane, e);
                }
            }
        }
    } else if (is_producer) {
        if (lane <= kMaxInst) {
            const uint4* src = route_pub + (size_t)(blockIdx.x % (n_sel * kRouteCopies)) * (1u + kMaxInst) + lane;
            uint4 v = make_uint4(0, 0, 0, 0);
            bool ok = false;
            for (uint32_t it = 0; it < (1u << 17); ++it) {
                v = ld_relaxed_v4(src);
                if (v.x == epoch) { ok = true; break; }
                __nanosleep(it > 64 ? 256 : 100);
            }
            if (!ok) {
                report_status(a.status, kStatusWaitTimeout);
                v = make_uint4(epoch, 0u, has_shared, 0u);   // lane 0: no routed expert; the others are not read
            }
            if (lane == 0) {
                st.route.n_routed = min(v.y, (uint32_t)SHRIKE_MAX_TOP_K);
                st.route.n_inst = has_shared + min(v.y, (uint32_t)SHRIKE_MAX_TOP_K);
            } else {
                st.route.cell[lane - 1] = v.y < a.pool_cells ? v.y : 0u;
                st.route.w[lane - 1] = __uint_as_float(v.z);
            }
        }
    }
    FUSED_TS(19);
    __syncthreads();
    FUSED_TS(5);   // the instance list is known
    plan.route(st.route.n_routed);
    const uint32_t n_units = plan.n_units, packs_eff = plan.packs_eff;

    if (is_producer) {
        // ================= producer: one lane per unit =================
        // first the units whose slot is fresh; then, a ring's worth at a time, those that wait for a slot
        // (a lane never waits for a unit that a later lane of the same pass asks for)
        // (the lanes run an issue together, copy by copy: the gate/up units first, then the down units, so
        // that the copy engine's queue holds them in the order the consumers want them)
        const uint32_t ring_a = min(n_units, G.n_slots);
        if (lane >= n_pre && lane < min(plan.n1, ring_a)) issue(plan.unit(lane));
        __syncwarp();
        if (lane >= max(n_pre, plan.n1) && lane < ring_a) issue(plan.unit(lane));
        __syncwarp();
        FUSED_TS(7);   // the first ring's worth asked for
        for (uint32_t base = G.n_slots; base < n_units; base += G.n_slots) {
            const uint32_t i = base + lane;
            if (lane < G.n_slots && i < n_units) {
                const UnitRec u = plan.unit(i);
                if (!wait_bar(&st.empty[u.slot()], u.parity() ^ 1u)) {
                    report_status(a.status, kStatusWaitTimeout);
                    st.failed = 1;
                }
                issue(u);
            }
            __syncwarp();
        }
        FUSED_TS(6);   // everything asked for
        if (lane == 0) {
            // The next kernel in the stream may begin its prologue from here on.
            pdl_launch_dependents();
            // every block read the epoch before it published its logits, and this block has gathered them all
            if (blockIdx.x == 0) *(volatile uint32_t*)a.epoch = epoch + 1u;
        }
        if (st.failed && lane == 0) {
            // a copy of this block may still be in flight: give it a bounded time to land before the block's
            // shared memory goes away
            for (int k = 0; k < 200; ++k) __nanosleep(1000);
        }
    } else {
        // ================= consumers =================
        // Gate/up units: groups of eight warps, a unit per group at a time, its columns split among the warps.
        // Down tiles: all consumer warps share a tile's (expert, column chunk) items and meet once per tile.
        const uint32_t g = lane >> 2, t = lane & 3;
        const uint32_t gi = cw / kGroupWarps, wi = cw % kGroupWarps;
        // this thread's byte offset inside its row's share of a group: rows are Q::kGroupBytes apart inside a
        // group's slab of a box ([group][row][group bytes])
        const uint32_t toff = t * (Q::kWords * 4);
        const uint32_t ctid = tid - 32u;
        // the block's unit table, a unit per consumer thread (the producer works its units out itself)
        if (ctid < n_units) st.units[ctid] = plan.unit(ctid);
        consumers_sync();
        uint32_t r = 0;   // units this group has taken
        for (uint32_t n = gi; n < plan.n1; n += kGroups, ++r) {
            const UnitRec u = st.units[n];
            if (r == 0) FUSED_TS(14);
            const uint32_t slot = u.slot();
            if (!wait_bar(&st.full[slot], u.parity())) report_status(a.status, kStatusWaitTimeout);
            if (r == 0) FUSED_TS(7);   // this group's first unit landed
            const uint8_t* stage = ring + (size_t)slot * G.slot_bytes;
            float tot0 = 0.f, tot1 = 0.f;
            {
                // rows g (gate) and g + 8 (up) of the unit: [gate|up][group][row 0..7][group bytes]
                const uint8_t* rowA = stage + (size_t)g * Q::kGroupBytes + toff;
                const uint8_t* rowB = rowA + 8 * (size_t)rb1;
                const uint32_t slab = 8 * Q::kGroupBytes;
                // scales and biases: [gate|up][scale|bias][row 0..7][group]
                const uint8_t* s0p = stage + G.p1_meta_off + (size_t)g * GD * 2;
                const uint8_t* b0p = s0p + 16 * GD;
                const uint8_t* s1p = s0p + 32 * GD;
                const uint8_t* b1p = s0p + 48 * GD;
                const uint32_t cg = G.cg_p1, chunks = chunks_of(GD, cg);
                for (uint32_t c = wi; c < chunks; c += kGroupWarps) {
                    const float2 o = chunk_rows_cg<BITS, GROUP, META>(cg, GD, rowA, rowB, slab, s0p, b0p, s1p, b1p, x_sm, xs_sm, c, t);
                    tot0 += o.x;
                    tot1 += o.y;
                }
                if (cfg_expert_bias && wi == 0) {
                    const uint16_t* ab = (const uint16_t*)(stage + G.p1_ab_off);
                    tot0 += bf16_bits_to_f32(ab[g]);
                    tot1 += bf16_bits_to_f32(ab[8 + g]);
                }
            }
            // the slot's bytes are consumed: hand it back; the group's partial sums meet in shared memory
            __syncwarp();
            if (r == 0) FUSED_TS(15);
            if (lane == 0) bar_arrive(&st.empty[slot]);
            float* red = &st.red[gi][r & 1u][0][0];
            if (t == 0) {
                red[wi * 16 + g] = tot0;
                red[wi * 16 + g + 8] = tot1;
            }
            group_sync(gi);
            if (wi != r % kGroupWarps) continue;
            // ---- this warp finishes the unit (the group's warps take turns) while the others go on ----
            float v = 0.f;
            if (lane < 16) {
#pragma unroll
                for (uint32_t w = 0; w < kGroupWarps; ++w) v += red[w * 16 + lane];
            }
            // rows 0..7 are gate rows; the up row of the same output sits 8 rows further
            const float up = __shfl_down_sync(0xffffffffu, v, 8);
            uint16_t* stg = st.act_stage[gi];
            if (lane < 8) {
                const float act = PLAIN ? glu(v, up, SHRIKE_ACT_SILU) : glu_call(v, up, cfg_activation);
                stg[perm_index(lane, BITS == 4)] = act_to_half_bits(act, a.status);
            }
            __syncwarp();
            {
                const uint4 pk = *(const uint4*)stg;
                uint16_t* dst = acts_call + (size_t)u.inst() * G.acts_stride + u.r0;
                if (lane < kActCopies) st_relaxed_v4(dst + (size_t)lane * acts_copy, pk);
            }
        }
        FUSED_TS(8);   // this warp's gate/up units done
        if (plan.n_tiles > 0) {
            // (worked out before the wait for the activations, not after it)
            const uint32_t cpe_s = has_shared ? chunks_of(a.f_shared / GROUP, G.cg_p2[1]) : 0u;   // chunks of the shared expert
            const uint32_t cpe_r = chunks_of(a.f / GROUP, G.cg_p2[0]);                            // chunks of a routed expert
            const uint32_t items = cpe_s + plan.n_routed * cpe_r;
            // (each warp stages what its own items multiply -- see below -- so no warp waits for an instance it
            // does not use, and nothing in this phase needs the whole block)
            for (uint32_t m = 0; m < plan.n_tiles; ++m) {
                const uint32_t u0 = plan.n1 + m * packs_eff;   // the tile's first unit
                const uint32_t row0 = (plan.n_blk - 1u - plan.blk + m * plan.n_blk) * 16u;
                float tot0 = 0.f, tot1 = 0.f;
                for (uint32_t it = cw; it < items; it += kCW) {
                    uint32_t sh, in, c, p, q;
                    if (it < cpe_s) {
                        sh = 1u; in = 0u; c = it; p = 0u; q = 0u;
                    } else {
                        const uint32_t k = it - cpe_s, j = div_rcp(k, G.rcp_cpe_r), pj = div_rcp(j, plan.rcp_epp);
                        sh = 0u; in = has_shared + j; c = k - j * cpe_r; p = has_shared + pj; q = j - pj * plan.epp;
                    }
                    const uint32_t F = sh ? a.f_shared : a.f, G2 = F / GROUP;
                    if (m == 0) {
                        // ---- the activations this item multiplies: its chunk of its instance's row, at most 32
                        // 16-byte blocks, a lane each. Poll until published, stage, and -- with the lanes that
                        // share a group -- the group's sums. (Later tiles of the block find them staged.) ----
                        constexpr uint32_t kLanes = GROUP / 8;
                        const uint32_t cgw = G.cg_p2[sh];
                        const uint32_t grp0 = c * cgw, ngrp = min(cgw, G2 - grp0);
                        const uint32_t blk0 = (in * G.acts_stride + grp0 * GROUP) / 8, nblk = ngrp * kLanes;
                        uint4 v = make_uint4(0, 0, 0, 0);
                        if (lane < nblk) {
                            const uint16_t* src = acts_mine + (size_t)(blk0 + lane) * 8;
                            v = ld_relaxed_v4(src);
                            bool got = !has_sentinel(v);
#pragma unroll 1
                            for (uint32_t tries = 0; !got && tries < (1u << 17); ++tries) {
                                __nanosleep(tries > 32 ? 512 : 80);   // (measured with 8 copies: 300 ns +0.1 us, 150 ns +0.03 us)
                                v = ld_relaxed_v4(src);
                                got = !has_sentinel(v);
                            }
                            if (!got) {
                                report_status(a.status, kStatusWaitTimeout);
                                v = make_uint4(0, 0, 0, 0);
                            }
                            *(uint4*)(acts_sm + (size_t)(blk0 + lane) * 8) = v;
                        }
                        __syncwarp();
                        // the block's halves in operand order: positions {0,1,4,5} hold the even elements (int4)
                        const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
                        float even = 0.f, odd = 0.f;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float lo = f16_bits_to_f32((uint16_t)(w4[j] & 0xffffu)), hi = f16_bits_to_f32((uint16_t)(w4[j] >> 16));
                            if (BITS == 4 && (j & 1)) odd += lo + hi;
                            else even += lo + hi;
                        }
#pragma unroll
                        for (uint32_t o = 1; o < kLanes; o <<= 1) {
                            even += __shfl_xor_sync(0xffffffffu, even, o);
                            odd += __shfl_xor_sync(0xffffffffu, odd, o);
                        }
                        if (lane < nblk && (lane & (kLanes - 1)) == 0)
                            asum_sm[in * gmax2 + grp0 + lane / kLanes] = make_float2(even + odd, Q::kOffEven * even + Q::kOffOdd * odd);
                        __syncwarp();
                        if (it == cw) FUSED_TS(9);   // this warp's first item's activations staged
                    }
                    const UnitRec u = st.units[u0 + p];
                    if (!wait_bar(&st.full[u.slot()], u.parity())) report_status(a.status, kStatusWaitTimeout);
                    if (it == cw && m == 0) FUSED_TS(22);
                    const uint8_t* eb = ring + (size_t)u.slot() * G.slot_bytes + (size_t)q * G.p2_expert_bytes[sh];
                    // [group][row 0..15][group bytes]; scales and biases [scale|bias][row 0..15][group]
                    const uint8_t* rowA = eb + (size_t)g * Q::kGroupBytes + toff;
                    const uint8_t* rowB = rowA + 8 * Q::kGroupBytes;
                    const uint32_t slab = 16 * Q::kGroupBytes;
                    const uint8_t* s0p = eb + G.p2_meta_off[sh] + (size_t)g * G2 * 2;
                    const uint8_t* s1p = s0p + 16 * G2;
                    const uint8_t* b0p = s0p + 32 * G2;
                    const uint8_t* b1p = s1p + 32 * G2;
                    const uint16_t* bsm = acts_sm + (size_t)in * G.acts_stride;
                    const float2* xs = asum_sm + (size_t)in * gmax2;
                    const float2 o = chunk_rows_cg<BITS, GROUP, META>(G.cg_p2[sh], G2, rowA, rowB, slab, s0p, b0p, s1p, b1p, bsm, xs, c, t);
                    float o0 = o.x, o1 = o.y;
                    if (cfg_expert_bias && c == 0) {
                        const uint16_t* ab = (const uint16_t*)(eb + G.p2_ab_off[sh]);
                        o0 += bf16_bits_to_f32(ab[g]);
                        o1 += bf16_bits_to_f32(ab[g + 8]);
                    }
                    const float w = st.route.w[in];
                    tot0 = fmaf(w, o0, tot0);
                    tot1 = fmaf(w, o1, tot1);
                    if (it == cw && m == 0) FUSED_TS(17);
                }
                if (m == 0) FUSED_TS(20);
                float* red = &st.red2[m & 1u][cw][0];
                if (t == 0) {
                    red[g] = tot0;
                    red[g + 8] = tot1;
                }
                // one warp per tile adds the warps' sums up (in warp order) and writes the rows; it asks for the
                // residual's values before the warps meet
                const bool fin = cw == m % kCW;
                float hid = 0.f;
                if (fin && lane < 16 && a.hidden) hid = load_act(a.hidden, (size_t)row0 + lane, cfg_act_dtype);
                consumers_sync();
                if (m == 0) FUSED_TS(21);
                if (fin) {
                    if (lane < 16) {
                        float ysum = 0.f;
#pragma unroll
                        for (uint32_t w = 0; w < kCW; ++w) ysum += st.red2[m & 1u][w][lane];
                        const size_t o = (size_t)row0 + lane;
                        store_act(a.y, o, a.y_dtype, ysum);
                        if (a.hidden) store_act(a.hidden, o, cfg_act_dtype, hid + round_act(a.y_dtype, ysum));
                    }
                    // every warp is past its reads of the tile's slots: they go back to the producer
                    if (lane < packs_eff) bar_arrive_n(&st.empty[st.units[u0 + lane].slot()], kGroupWarps);
                }
            }
        }
        FUSED_TS(10);   // this warp done
    }
}

inline uint32_t align_up(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_tiled() {
    static EncodeFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return (EncodeFn)p;
    }();
    return fn;
}

}  // namespace

// ---- host ----------------------------------------------------------------------------------

// Sizes the ring and the unit layouts for a handle; false when the shape does not fit (the layer call then
// keeps its three launches).
bool fused_geometry(const shrike_moe_config& c, int sm_count, int max_smem_optin, FusedGeom& g) {
    memset(&g, 0, sizeof g);
    if (c.d % 64 || c.f % 64 || (c.has_shared && c.shared_f % 64)) return false;
    if (!encode_tiled()) return false;
    const uint32_t rb1 = c.d * c.weight_bits / 8, G1 = c.d / c.group_size;
    g.p1_meta_off = align_up(16 * rb1, 128);
    g.p1_ab_off = align_up(g.p1_meta_off + 64 * G1, 128);
    g.p1_bytes = g.p1_ab_off + 128;
    auto pick_cg = [](uint32_t groups) { return groups % 2 == 0 && groups >= 4 ? 4u : groups % 2 == 0 ? 2u : 1u; };
    g.cg_p1 = pick_cg(G1);
    while (g.cg_p1 > 1 && G1 / g.cg_p1 < kGroupWarps) g.cg_p1 /= 2;   // a chunk for every warp of the group
    for (int sh = 0; sh < 2; ++sh) {
        const uint32_t F = sh ? (c.has_shared ? c.shared_f : c.f) : c.f;
        const uint32_t rb2 = F * c.weight_bits / 8, G2 = F / c.group_size;
        g.p2_meta_off[sh] = align_up(16 * rb2, 128);
        g.p2_ab_off[sh] = align_up(g.p2_meta_off[sh] + 64 * G2, 128);
        g.p2_expert_bytes[sh] = g.p2_ab_off[sh] + 128;
        g.cg_p2[sh] = pick_cg(G2);
    }
    {   // the sixteen consumer warps share a down tile's (expert, chunk) items: narrower chunks when they split
        // more evenly (18 items of 4 groups are two rounds of 4; as 36 items of 2 they are three rounds of 2)
        auto rounds = [&](uint32_t cap) {
            uint32_t items = 0;
            for (int sh = 0; sh < 2; ++sh) {
                if (sh && !c.has_shared) continue;
                const uint32_t G2 = (sh ? c.shared_f : c.f) / c.group_size, cg = std::min(g.cg_p2[sh], cap);
                items += (sh ? 1u : c.top_k) * ((G2 + cg - 1) / cg);
            }
            return (items + kCW - 1) / kCW * cap;
        };
        if (g.cg_p2[0] == 4 && (!c.has_shared || g.cg_p2[1] == 4) && rounds(2) < rounds(4)) g.cg_p2[0] = g.cg_p2[1] = 2;
    }
    // a routed pack holds as many experts as fit beside the larger of the other unit kinds
    uint32_t slot = std::max(g.p1_bytes, g.p2_expert_bytes[0]);
    if (c.has_shared) slot = std::max(slot, g.p2_expert_bytes[1]);
    g.experts_per_pack = std::max(1u, std::min<uint32_t>(SHRIKE_MAX_TOP_K, slot / g.p2_expert_bytes[0]));
    g.slot_bytes = slot;
    const uint32_t n_inst = c.top_k + (c.has_shared ? 1u : 0u);
    g.acts_stride = std::max(c.f, c.has_shared ? c.shared_f : 0u);
    g.off_x = 0;
    g.off_xraw = align_up(c.d * 2, 16);
    g.off_rw = g.off_xraw + c.d * 4;   // the row in fp32
    g.off_xs = g.off_rw + kMaxRouterRowsPerBlock * c.d * 4;   // this block's fp32 router rows
    g.off_acts = g.off_xs + align_up(G1 * 8, 16);
    g.off_asum = g.off_acts + n_inst * g.acts_stride * 2;
    g.off_ring = align_up(g.off_asum + n_inst * (g.acts_stride / c.group_size) * 8, 128);
    const uint32_t budget = (uint32_t)max_smem_optin - (uint32_t)sizeof(FusedStatic) - 1024;
    if (g.off_ring + 2 * g.slot_bytes > budget) return false;
    g.n_slots = std::min<uint32_t>(kMaxSlots, (budget - g.off_ring) / g.slot_bytes);
    g.smem_bytes = g.off_ring + g.n_slots * g.slot_bytes;
    const uint32_t rows = c.num_experts + (c.shared_gated ? 1u : 0u);
    g.router_rows_per_block = (rows + (uint32_t)sm_count - 1) / (uint32_t)sm_count;
    if (g.router_rows_per_block > kMaxRouterRowsPerBlock) return false;
    auto rcp = [](uint32_t c) { return (uint32_t)(((1ull << 24) + c - 1) / c); };
    if (c.f / 8 >= 4096 || (c.has_shared ? c.shared_f / 8 : 0u) + c.top_k * (c.f / 8) + (uint32_t)sm_count >= 4096 ||
        c.d / 16 + (uint32_t)sm_count >= 4096)
        return false;   // the plan's divisions are a multiply by these reciprocals: numerators and divisors below 4096
    g.rcp_blocks = rcp((uint32_t)sm_count); g.rcp_upe = rcp(c.f / 8); g.rcp_slots = rcp(g.n_slots);
    g.rcp_epp = rcp(g.experts_per_pack);
    g.rcp_cpe_r = rcp(g.cg_p2[0] == 4 ? (c.f / c.group_size + 3) / 4 : c.f / c.group_size / g.cg_p2[0]);
    g.rcp_bps = rcp(g.acts_stride / 8); g.rcp_gmax2 = rcp(g.acts_stride / c.group_size);
    if (n_inst * (g.acts_stride / 8) >= 4096) return false;
    // the block's unit table and its per-tile sums, at the most work a block can get
    const uint32_t n_blk = (uint32_t)sm_count;
    const uint32_t units1 = ((c.has_shared ? c.shared_f / 8 : 0u) + c.top_k * (c.f / 8) + n_blk - 1) / n_blk;
    const uint32_t tiles = (c.d / 16 + n_blk - 1) / n_blk;
    const uint32_t packs = (c.has_shared ? 1u : 0u) + (c.top_k + g.experts_per_pack - 1) / g.experts_per_pack;
    // (a tile's packs are held until the tile is done: they must fit the ring together)
    return std::max(packs, 1u) <= g.n_slots && units1 + tiles * std::max(packs, 1u) <= kMaxUnits;
}

// ---- tensor maps of an expert-block layout -------------------------------------------------------------

// The four maps of one chunk of `cells` blocks at `base` (cells 1: the shared expert's block). False when the
// layout is not the regular one (gate and up sub-tensors the same distance apart for weights, scales and
// biases) or the driver refuses a map: the layer call then keeps its three launches.
static bool make_block_maps(const shrike_moe_config& c, const uint8_t* base, const Offsets3& off, uint32_t F,
                            uint64_t cells, uint64_t cell_stride, CUtensorMap* w1, CUtensorMap* m1, CUtensorMap* w2,
                            CUtensorMap* m2) {
    EncodeFn enc = encode_tiled();
    if (!enc) return false;
    const uint64_t gb = c.group_size * c.weight_bits / 8;
    const uint64_t rb1 = (uint64_t)c.d * c.weight_bits / 8, G1 = c.d / c.group_size;
    const uint64_t rb2 = (uint64_t)F * c.weight_bits / 8, G2 = F / c.group_size;
    const uint64_t mat = (uint64_t)off.w[1] - off.w[0], kind1 = (uint64_t)off.b[0] - off.s[0];
    if (off.w[1] <= off.w[0] || off.s[1] - off.s[0] != mat || off.b[1] - off.s[1] != kind1 || off.b[0] <= off.s[0] ||
        off.b[2] <= off.s[2])
        return false;
    if (mat % 16 || kind1 % 16 || (off.b[2] - off.s[2]) % 16 || cell_stride % 16 || ((uintptr_t)base & 15)) return false;
    const uint64_t cs = cells > 1 ? cell_stride : std::max<uint64_t>(cell_stride, 16);
    const cuuint32_t ones[5] = {1, 1, 1, 1, 1};
    auto ok = [](CUresult r) { return r == CUDA_SUCCESS; };
    {   // gate + up weights: (group bytes, F rows, G1 groups, 2, cells); a box = 8 rows of both
        const cuuint64_t dims[5] = {gb, F, G1, 2, cells};
        const cuuint64_t strides[4] = {rb1, gb, mat, cs};
        const cuuint32_t box[5] = {(cuuint32_t)gb, 8, (cuuint32_t)G1, 2, 1};
        if (!ok(enc(w1, CU_TENSOR_MAP_DATA_TYPE_UINT8, 5, (void*)(base + off.w[0]), dims, strides, box, ones,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)))
            return false;
    }
    {   // their scales and biases, 8 rows (16*G1 bytes) at a time in 8-byte units: (2*G1, F/8, scale|bias, 2, cells)
        const cuuint64_t dims[5] = {2 * G1, F / 8, 2, 2, cells};
        const cuuint64_t strides[4] = {16 * G1, kind1, mat, cs};
        const cuuint32_t box[5] = {(cuuint32_t)(2 * G1), 1, 2, 2, 1};
        if (!ok(enc(m1, CU_TENSOR_MAP_DATA_TYPE_UINT64, 5, (void*)(base + off.s[0]), dims, strides, box, ones,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)))
            return false;
    }
    {   // down weights: (group bytes, D rows, G2 groups, cells); a box = 16 rows
        const cuuint64_t dims[4] = {gb, c.d, G2, cells};
        const cuuint64_t strides[3] = {rb2, gb, cs};
        const cuuint32_t box[4] = {(cuuint32_t)gb, 16, (cuuint32_t)G2, 1};
        if (!ok(enc(w2, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, (void*)(base + off.w[2]), dims, strides, box, ones,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)))
            return false;
    }
    {   // their scales and biases, 8 rows at a time: (2*G2, D/8, scale|bias, cells); a box = 16 rows of both
        const cuuint64_t dims[4] = {2 * G2, c.d / 8, 2, cells};
        const cuuint64_t strides[3] = {16 * G2, (uint64_t)off.b[2] - off.s[2], cs};
        const cuuint32_t box[4] = {(cuuint32_t)(2 * G2), 2, 2, 1};
        if (!ok(enc(m2, CU_TENSOR_MAP_DATA_TYPE_UINT64, 4, (void*)(base + off.s[2]), dims, strides, box, ones,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)))
            return false;
    }
    return true;
}

// The maps of a call's pool and shared block, cached on the handle: they change only when the host changes
// the pool, the offsets or the shared block.
struct FusedMapCache {
    PoolView pool;
    Offsets3 routed, shared;
    const uint8_t* shared_block;
    bool valid, usable;
    FusedMaps maps;
};

static const FusedMaps* fused_maps_for(const shrike_moe* m, const ExpertArgs& ea) {
    FusedMapCache* cache = (FusedMapCache*)m->ws.fused_maps;
    if (!cache) return nullptr;
    const bool same = cache->valid && memcmp(&cache->pool, &ea.pool, sizeof(PoolView)) == 0 &&
                      memcmp(&cache->routed, &ea.routed, sizeof(Offsets3)) == 0 &&
                      memcmp(&cache->shared, &ea.shared, sizeof(Offsets3)) == 0 && cache->shared_block == ea.shared_block;
    if (same) return cache->usable ? &cache->maps : nullptr;
    const shrike_moe_config& c = m->cfg;
    memset(cache, 0, sizeof *cache);   // padding bytes included: the comparison above is bytewise
    cache->pool = ea.pool; cache->routed = ea.routed; cache->shared = ea.shared; cache->shared_block = ea.shared_block;
    cache->valid = true;
    bool ok = true;
    uint32_t left = ea.pool.cells;
    for (uint32_t ch = 0; ch < SHRIKE_MAX_POOL_CHUNKS && ok && left; ++ch) {
        if (!ea.pool.base[ch]) break;
        const uint32_t cells = left < ea.pool.cells_per_chunk ? left : ea.pool.cells_per_chunk;
        ok = make_block_maps(c, ea.pool.base[ch], ea.routed, c.f, cells, ea.pool.stride, &cache->maps.w1[ch],
                             &cache->maps.m1[ch], &cache->maps.w2[ch], &cache->maps.m2[ch]);
        left -= cells;
    }
    if (ok && c.has_shared)
        ok = make_block_maps(c, ea.shared_block, ea.shared, c.shared_f, 1, 16, &cache->maps.w1[SHRIKE_MAX_POOL_CHUNKS],
                             &cache->maps.m1[SHRIKE_MAX_POOL_CHUNKS], &cache->maps.w2[SHRIKE_MAX_POOL_CHUNKS],
                             &cache->maps.m2[SHRIKE_MAX_POOL_CHUNKS]);
    cache->usable = ok;
    return ok ? &cache->maps : nullptr;
}

size_t fused_map_cache_bytes() { return sizeof(FusedMapCache); }

size_t fused_geom_bytes() { return sizeof(FusedGeom); }
// {epoch, logit} words of the experts and the gate row, then the selecting blocks' copies of the instance list
size_t fused_logits_bytes(const shrike_moe_config& c) {
    return (size_t)((c.num_experts + 2u) & ~1u) * 8 + (size_t)kSelectors * kRouteCopies * (1 + kMaxInst) * 16;
}
size_t fused_acts_bytes(const shrike_moe_config& c) {
    return (size_t)2 * kActCopies * kMaxInst * std::max(c.f, c.has_shared ? c.shared_f : 0u) * 2;
}

template <int BITS, int GROUP, int META, bool PLAIN>
static cudaError_t launch_fused_tp(const shrike_moe* m, cudaStream_t st, const FusedArgs& a) {
    auto k = decode_layer_kernel<BITS, GROUP, META, PLAIN>;
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)a.g.smem_bytes);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)m->sm_count);
    cfg.blockDim = dim3(kFusedThreads);
    cfg.dynamicSmemBytes = a.g.smem_bytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    unsigned n = 0;
    // The blocks wait on each other's results, so all of them must be resident together. A cooperative launch
    // guarantees it, whatever else runs on the GPU: it is the default. It also keeps every block from starting
    // until the previous kernel has left, prologue and launch latency exposed (0.5 us per layer). A host that
    // runs one stream on the GPU does not need the guarantee -- the grid is one block per SM and a block needs
    // most of an SM, so the blocks are together as soon as the stream's previous kernel has ended -- and says so
    // with SHRIKE_SINGLE_STREAM at handle creation. (Two such layers on two streams without the guarantee could
    // each hold half of the SMs and wait for the other half: the bounded waits would end that with a timeout
    // status, not a hang, but the call would have failed.)
    if (!m->single_stream || m->no_pdl) {
        attr[n].id = cudaLaunchAttributeCooperative;
        attr[n].val.cooperative = 1;
        ++n;
    }
    if (!m->no_pdl) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, k, a);
}

template <int BITS, int GROUP, int META>
static cudaError_t launch_fused_t(const shrike_moe* m, cudaStream_t st, const FusedArgs& a) {
    const bool plain = a.act_dtype == SHRIKE_DTYPE_BF16 && a.activation == SHRIKE_ACT_SILU && !a.expert_bias && a.rbits == 0 &&
                       !a.sigmoid_scores && !a.logit_bias && !a.per_expert_scale && !a.eff_scale;
    return plain ? launch_fused_tp<BITS, GROUP, META, true>(m, st, a) : launch_fused_tp<BITS, GROUP, META, false>(m, st, a);
}

cudaError_t launch_fused_layer(const shrike_moe* m, cudaStream_t st, const ExpertArgs& ea,
                               const shrike_router_operands& ops, const uint64_t* table, uint32_t pool_cells,
                               const uint32_t* io_status, const void* x, uint32_t* ids, float* weights,
                               uint32_t* slots, float* gate, void* y, void* hidden) {
    const shrike_moe_config& c = m->cfg;
    const FusedMaps* maps = fused_maps_for(m, ea);
    if (!maps) return cudaErrorNotSupported;   // the caller falls back to the three launches
    FusedArgs a;
    memset(&a, 0, sizeof a);
    a.maps = *maps;
    a.pool = ea.pool; a.routed = ea.routed; a.shared = ea.shared; a.shared_block = ea.shared_block;
    {   // cell -> (chunk, cell in chunk) by a multiply: exact while cells * cells_per_chunk < 2^32
        const uint64_t cpc = ea.pool.cells_per_chunk ? ea.pool.cells_per_chunk : 1;
        if (cpc < 2 || (uint64_t)ea.pool.cells * cpc >= (1ull << 32)) return cudaErrorNotSupported;   // (the three launches)
        a.rcp_cpc = (uint32_t)(((1ull << 32) + cpc - 1) / cpc);
    }
    a.d = c.d; a.f = c.f; a.f_shared = c.has_shared ? c.shared_f : 0; a.top_k = c.top_k;
    a.activation = c.activation; a.expert_bias = c.expert_bias; a.act_dtype = c.act_dtype; a.y_dtype = c.y_dtype;
    a.rw = ops.weights; a.rscales = ops.scales; a.rbiases = ops.biases; a.rbits = c.router_weight_bits;
    a.gate_row = c.shared_gated ? ops.shared_gate : nullptr;
    a.eff_scale = ops.effective_scale; a.logit_bias = ops.logit_bias; a.per_expert_scale = ops.per_expert_scale;
    a.ne = c.num_experts; a.sigmoid_scores = c.router_kind == SHRIKE_ROUTER_SIGMOID; a.round_f16 = c.round_route_weights_f16;
    a.scaling = c.routed_scaling;
    a.table = table; a.pool_cells = pool_cells; a.io_status = io_status;
    a.x = x; a.y = y; a.hidden = hidden;
    a.out_ids = ids; a.out_w = weights; a.out_slots = slots; a.out_gate = gate;
    a.logits64 = (unsigned long long*)m->ws.fused_logits; a.acts_pub = m->ws.fused_acts; a.epoch = m->ws.fused_epoch;
    a.status = m->ws.status;
#ifdef SHRIKE_TRACE
    a.trace = m->trace;
#endif
    a.g = *(const FusedGeom*)m->ws.fused_geom;
    const uint32_t bits = c.weight_bits, grp = c.group_size;
    const bool f16 = c.meta_dtype == SHRIKE_DTYPE_FP16;
    if (bits == 4 && grp == 64 && !f16) return launch_fused_t<4, 64, SHRIKE_DTYPE_BF16>(m, st, a);
    if (bits == 4 && grp == 64 && f16) return launch_fused_t<4, 64, SHRIKE_DTYPE_FP16>(m, st, a);
    if (bits == 4 && grp == 32 && !f16) return launch_fused_t<4, 32, SHRIKE_DTYPE_BF16>(m, st, a);
    if (bits == 4 && grp == 32 && f16) return launch_fused_t<4, 32, SHRIKE_DTYPE_FP16>(m, st, a);
    if (bits == 8 && grp == 64 && !f16) return launch_fused_t<8, 64, SHRIKE_DTYPE_BF16>(m, st, a);
    if (bits == 8 && grp == 64 && f16) return launch_fused_t<8, 64, SHRIKE_DTYPE_FP16>(m, st, a);
    if (bits == 8 && grp == 32 && !f16) return launch_fused_t<8, 32, SHRIKE_DTYPE_BF16>(m, st, a);
    if (bits == 8 && grp == 32 && f16) return launch_fused_t<8, 32, SHRIKE_DTYPE_FP16>(m, st, a);
    return cudaErrorInvalidValue;
}

}  // namespace shrike
