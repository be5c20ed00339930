// One decode row through one MoE layer in ONE launch: router logits, top-k, residency lookup, shared
// and routed gate/up + GLU, down projections, weighted combine, hidden += y.
//
//   router_gemv_r4 + router_topk_select_k8          moe.metal:324-582
//   moe_classify_expert_residency_spec              moe.metal:121-231
//   moe_phase1_gate_up_act_spec_u16load             moe.metal:950-998
//   moe_phase2_down_reduce_spec_k8 / phase2_finish  moe.metal:889-893, 1008-1057
//   shared expert (SharedExpertRuntime)             SharedExpertInt4.swift:251-342
//
// One persistent block per SM. A layer's bytes (nine 1.7 MB expert blocks at the Qwen shape) are
// about as large as the chip's shared memory, so after the selection every block asks for ALL of
// its share at once: one producer lane issues a few large tiled TMA copies (cp.async.bulk.tensor,
// no multicast) into a ring of shared-memory slots, each slot completing on an mbarrier, and eight
// consumer warps walk the slots with the dequant-fused skinny tiles (packed words -> exact fp16
// integers with one logic op per register, mma.sync m16n8k16, fp32 accumulate, one fused
// multiply-add per group with the scale and one with the zero-point bias). HBM streams the whole
// layer in one burst instead of one load-then-compute pass per block and per launch.
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
//   logits   every block computes its expert rows and publishes {epoch, value} as one 64-bit word
//            per expert; every block gathers all words and repeats the (cheap) selection itself;
//   acts     a phase-1 unit (8 gate rows + 8 up rows of one expert) publishes its 8 fp16
//            activations as 16 bytes whose halves are never the sentinel 0xFFFF; the blocks that
//            own a tile of output rows poll until no half is the sentinel. The buffer of the
//            previous call (other parity of the epoch) is reset by this call.
// Every wait -- mbarrier or global poll -- is bounded: it gives up, reports through the status
// word and the block runs on to its end. The launch is cooperative (all blocks resident).
//
// MMA row slot s of a unit is row s of its box: rows 0..7 gate and 8..15 up in phase 1 (GLU partners
// in one thread), 16 consecutive down rows in phase 2.
#include <cuda.h>

#include <algorithm>

#include "router_math.cuh"
#include "select.cuh"

namespace shrike {

namespace {

constexpr uint32_t kPW = 1;                          // producer warps (one lane issues the copies)
constexpr uint32_t kCW = 8;                          // consumer warps
constexpr uint32_t kFusedThreads = (kPW + kCW + 1) * 32;   // + epilogue warp
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
    uint16_t* acts_pub;             // [2][kMaxInst][acts_stride] halves, 0xFFFF = not yet written
    uint32_t* epoch;
    uint32_t* status;
#ifdef SHRIKE_TRACE
    uint64_t* trace;   // debug builds: 16 timestamps per block
#endif
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

struct RouteSmem {
    uint32_t cell[kMaxInst];    // per instance (shared expert first when there is one)
    float w[kMaxInst];          // route weight, or the shared expert's gate
    uint32_t n_inst, n_routed;
};

struct FusedStatic {
    uint64_t table[SHRIKE_MAX_EXPERTS];
    float logits[SHRIKE_MAX_EXPERTS + 1];
    uint32_t cand_key[kCW * 8], cand_id[kCW * 8];   // every consumer warp's best picks
    RouteSmem route;
    float red[2][kCW][16];
    alignas(16) uint16_t act_stage[8];
    uint64_t full[kMaxSlots], empty[kMaxSlots], red_full[2], red_empty[2], rw_bar;
    uint32_t epoch, failed;
};

__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t it = 0; it < (1u << 21); ++it) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
        if (ok) return true;
        if (it > 128) __nanosleep(32);
    }
    return false;
}
__device__ __forceinline__ void bar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
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
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kCW * 32) : "memory"); }

__device__ __forceinline__ bool has_sentinel(uint4 v) {
    auto bad = [](uint32_t w) { return (w & 0xffffu) == 0xffffu || (w >> 16) == 0xffffu; };
    return bad(v.x) || bad(v.y) || bad(v.z) || bad(v.w);
}

// One unit of work of a block. The producer, the consumers and the epilogue warp walk the same sequence.
struct Unit {
    uint32_t kind;    // 0: phase 1 (8 gate + 8 up rows of one instance); 1: phase 2 (16 output rows x a pack)
    uint32_t inst;    // first instance
    uint32_t count;   // phase 2: instances in the pack (0: the layer has no expert work at all)
    uint32_t r0;      // first weight row
    uint32_t sh;      // the shared expert's geometry
    uint32_t last;    // phase 2: last pack of its tile
};

struct Walker {
    uint32_t n_blk, blk, su, upe, n_routed, has_shared, tiles, epp;
    uint32_t phase, idx, pack;

    __device__ void init(const FusedArgs& a) {
        n_blk = gridDim.x; blk = blockIdx.x;
        has_shared = a.shared_block ? 1u : 0u;
        su = has_shared ? a.f_shared / 8 : 0u;
        upe = a.f / 8;
        tiles = a.d / 16;
        epp = a.g.experts_per_pack;
        n_routed = 0;
        phase = 0; idx = blk; pack = 0;
    }
    // Next unit; false when exhausted, or when the next one needs the routing result and `routed` is false.
    __device__ __noinline__ bool next(Unit& u, bool routed) {
        if (phase == 0) {
            if (idx < su) {
                u = Unit{0u, 0u, 1u, idx * 8u, 1u, 0u};
                idx += n_blk;
                return true;
            }
            if (!routed) return false;
            const uint32_t k = idx - su;
            if (k < n_routed * upe) {
                u = Unit{0u, has_shared + k / upe, 1u, (k % upe) * 8u, 0u, 0u};
                idx += n_blk;
                return true;
            }
            phase = 1; idx = n_blk - 1u - blk; pack = 0;
        }
        if (!routed) return false;
        if (idx >= tiles) return false;
        const uint32_t routed_packs = (n_routed + epp - 1u) / epp;
        const uint32_t packs = has_shared + routed_packs;
        if (packs == 0) {
            u = Unit{1u, 0u, 0u, idx * 16u, 0u, 1u};
            idx += n_blk;
            return true;
        }
        if (has_shared && pack == 0) {
            u = Unit{1u, 0u, 1u, idx * 16u, 1u, packs == 1u ? 1u : 0u};
        } else {
            const uint32_t p = pack - has_shared;
            u = Unit{1u, has_shared + p * epp, min(epp, n_routed - p * epp), idx * 16u, 0u, pack + 1u == packs ? 1u : 0u};
        }
        if (++pack == packs) { pack = 0; idx += n_blk; }
        return true;
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

// CG consecutive 16-bit values starting at an address that is a multiple of 2 * CG bytes.
template <int CG, int META>
__device__ __forceinline__ void lds_meta(const uint8_t* p, float (&out)[CG]) {
    if constexpr (CG == 1) {
        out[0] = meta_to_f32<META>(*(const uint16_t*)p);
    } else if constexpr (CG == 2) {
        const uint32_t v = *(const uint32_t*)p;
        out[0] = meta_to_f32<META>((uint16_t)(v & 0xffffu));
        out[1] = meta_to_f32<META>((uint16_t)(v >> 16));
    } else {
        const uint2 v = *(const uint2*)p;
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

// The chunk width is uniform for a unit; one call site per width.
template <int BITS, int GROUP, int META>
__device__ __forceinline__ float2 chunk_rows_cg(uint32_t cg, const uint8_t* rowA, const uint8_t* rowB, uint32_t slab,
                                                const uint8_t* s0p, const uint8_t* b0p, const uint8_t* s1p,
                                                const uint8_t* b1p, const uint16_t* bsm, const float2* xs, uint32_t c,
                                                uint32_t t) {
    if (cg == 4) return chunk_rows<BITS, GROUP, META, 4>(rowA, rowB, slab, s0p, b0p, s1p, b1p, bsm, xs, c * 4, t);
    if (cg == 2) return chunk_rows<BITS, GROUP, META, 2>(rowA, rowB, slab, s0p, b0p, s1p, b1p, bsm, xs, c * 2, t);
    return chunk_rows<BITS, GROUP, META, 1>(rowA, rowB, slab, s0p, b0p, s1p, b1p, bsm, xs, c, t);
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
#define FUSED_TS(slot) do { if (a.trace && lane == 0) a.trace[(size_t)blockIdx.x * 16 + (slot)] = globaltimer_ns(); } while (0)
#else
#define FUSED_TS(slot) do { } while (0)
#endif

// Asks the TMA unit to fetch a descriptor ahead of its first use (a first use otherwise waits for the fetch:
// a block whose experts sit in eight pool chunks met a different descriptor with almost every copy).
__device__ __forceinline__ void prefetch_map(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// Tiled TMA loads (no multicast): the box lands densely, innermost dimension first.
__device__ __forceinline__ void tma_3d(uint32_t dst, const CUtensorMap* map, int32_t c0, int32_t c1, int32_t c2, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar)) : "memory");
}
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

// Top-k of the logits in shared memory by the eight consumer warps, then a merge by the first of them: warp w
// holds experts 32w..32w+31 one per lane and takes its best top_k by rounds of a warp-wide maximum (equal keys:
// the lowest lane, i.e. the lowest expert id); the candidates are merged the same way. The picks and their
// order are those of router_topk_select_body's insertion scan (moe.metal:436-456). Lane r of the merging warp
// returns the r-th pick. `cw`: consumer warp index; all consumer warps call it.
template <class A>
__device__ __forceinline__ void select_warps(const float* lg, const A& a, uint32_t* cand_key, uint32_t* cand_id,
                                             uint32_t cw, uint32_t lane, uint32_t& out_id, float& out_w) {
    const uint32_t e = cw * 32 + lane;
    uint32_t key = 0;
    if (e < a.ne) key = selection_key_of(lg[e], a.logit_bias ? bf16_bits_to_f32(a.logit_bias[e]) : 0.0f, a);
    for (uint32_t r = 0; r < a.top_k; ++r) {
        const uint32_t best = __reduce_max_sync(0xffffffffu, key);
        const uint32_t who = __ffs(__ballot_sync(0xffffffffu, key == best && best != 0u));   // 0: nobody left
        if (lane == 0) {
            cand_key[cw * 8 + r] = who ? best : 0u;
            cand_id[cw * 8 + r] = who ? cw * 32 + who - 1 : 0u;
        }
        if (who && lane == who - 1) key = 0u;
    }
    consumer_sync();
    out_id = 0;
    out_w = 0.f;
    if (cw == 0) {
        // 64 candidates (8 warps x 8, unused entries 0), two per lane: lane l holds warp l/4's entries 2(l%4), +1
        uint32_t k0 = 0, k1 = 0, i0 = 0, i1 = 0;
        {
            const uint32_t w = lane >> 2, q = (lane & 3) * 2;
            if (q < a.top_k) { k0 = cand_key[w * 8 + q]; i0 = cand_id[w * 8 + q]; }
            if (q + 1 < a.top_k) { k1 = cand_key[w * 8 + q + 1]; i1 = cand_id[w * 8 + q + 1]; }
        }
        float my_score = -INFINITY;
        uint32_t my_id = 0;
        for (uint32_t r = 0; r < a.top_k; ++r) {
            const uint32_t best = __reduce_max_sync(0xffffffffu, max(k0, k1));
            uint32_t cand = 0xffffffffu;
            if (best != 0u) {
                if (k1 == best) cand = i1;
                if (k0 == best) cand = min(cand, i0);
            }
            const uint32_t win = __reduce_min_sync(0xffffffffu, cand);   // equal keys: the lower expert id
            if (win != 0xffffffffu) {
                if (k0 == best && i0 == win) k0 = 0u;
                else if (k1 == best && i1 == win) k1 = 0u;
            }
            if (lane == r) {
                my_score = score_of_key(win == 0xffffffffu ? 0u : best);
                my_id = win == 0xffffffffu ? 0u : min(win, a.ne - 1u);
            }
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

template <int BITS, int GROUP, int META>
__global__ void __launch_bounds__(kFusedThreads, 1) decode_layer_kernel(const __grid_constant__ FusedArgs a) {
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
    const bool is_producer = warp < kPW, is_consumer = warp >= kPW && warp < kPW + kCW;
    const uint32_t cw = warp - kPW;    // consumer index of the consumer warps

    if (warp == 0) FUSED_TS(0);
    Walker prod;   // the producers' position survives the routing
    prod.init(a);
    uint32_t prod_n = 0;

    // ---- before the previous kernel in the stream is known to be complete: nothing that it produces ----
    if (tid == 0) {
        for (uint32_t s = 0; s < G.n_slots; ++s) { mbar_init(&st.full[s], 1); mbar_init(&st.empty[s], kCW); }
        for (uint32_t s = 0; s < 2; ++s) { mbar_init(&st.red_full[s], kCW); mbar_init(&st.red_empty[s], 1); }
        mbar_init(&st.rw_bar, 1);
        fence_mbar_init();
        st.failed = 0;
    }
    for (uint32_t e = tid; e < a.ne; e += kFusedThreads) st.table[e] = a.table[e];
    {   // the descriptors this block may use: the shared expert's, and every pool chunk's
        const uint32_t n_chunks = (a.pool.cells + a.pool.cells_per_chunk - 1) / a.pool.cells_per_chunk;
        const uint32_t which = tid >> 2, kind = tid & 3;
        const bool wanted = which < n_chunks || (which == SHRIKE_MAX_POOL_CHUNKS && a.shared_block);
        if (tid < 4 * (SHRIKE_MAX_POOL_CHUNKS + 1) && wanted)
            prefetch_map(kind == 0 ? &a.maps.w1[which] : kind == 1 ? &a.maps.m1[which] : kind == 2 ? &a.maps.w2[which] : &a.maps.m2[which]);
    }
    // this block's router rows (fp32 rows are fetched into registers now, used after the wait)
    const uint32_t router_rows = a.ne + (a.gate_row ? 1u : 0u);
    const uint32_t my_row = blockIdx.x + cw * gridDim.x;
    const bool routes = is_consumer && cw < G.router_rows_per_block && my_row < router_rows;
    const bool row_is_gate = routes && a.gate_row && my_row == a.ne;
    const bool row_f32 = a.rbits == 0 || row_is_gate;
    __syncthreads();   // barriers initialised
    if (tid == 0) {
        // fp32 router rows (and the gate row) of this block -> shared memory, one bulk copy each
        uint32_t bytes = 0;
        for (uint32_t k = 0; k < G.router_rows_per_block; ++k) {
            const uint32_t e = blockIdx.x + k * gridDim.x;
            const bool gate = a.gate_row && e == a.ne;
            if (e < router_rows && (a.rbits == 0 || gate)) bytes += D * 4;
        }
        mbar_expect_tx(&st.rw_bar, bytes);
        for (uint32_t k = 0; k < G.router_rows_per_block; ++k) {
            const uint32_t e = blockIdx.x + k * gridDim.x;
            const bool gate = a.gate_row && e == a.ne;
            if (e < router_rows && (a.rbits == 0 || gate))
                bulk_g2s(dsm + G.off_rw + (size_t)k * D * 4, gate ? (const void*)a.gate_row : (const void*)((const float*)a.rw + (size_t)e * D),
                         D * 4, &st.rw_bar);
        }
    }

    auto issue = [&](const Unit& u, uint32_t n) {
        // lane 0 of the producer warp: a unit is one to four tiled copies that complete on the slot's barrier
        const uint32_t slot = n % G.n_slots, round = n / G.n_slots;
        if (round > 0 && !wait_bar(&st.empty[slot], (round - 1) & 1)) {
            report_status(a.status, kStatusWaitTimeout);
            st.failed = 1;
        }
        const uint32_t stage = ring_smem + slot * G.slot_bytes;
        uint64_t* bar = &st.full[slot];
        if (u.kind == 0) {
            const uint32_t cell = u.sh ? 0u : st.route.cell[u.inst];
            const uint32_t mi = u.sh ? SHRIKE_MAX_POOL_CHUNKS : cell / a.pool.cells_per_chunk;
            const int32_t cc = u.sh ? 0 : (int32_t)(cell % a.pool.cells_per_chunk);
            mbar_expect_tx(bar, 16 * rb1 + 64 * GD + (a.expert_bias ? 32u : 0u));
            tma_5d(stage, &a.maps.w1[mi], 0, (int32_t)u.r0, 0, 0, cc, bar);
            tma_5d(stage + G.p1_meta_off, &a.maps.m1[mi], 0, (int32_t)(u.r0 / 8), 0, 0, cc, bar);
            if (a.expert_bias) {
                const uint8_t* base = u.sh ? a.shared_block : pool_cell_base(a.pool, cell);
                const Offsets3& off = u.sh ? a.shared : a.routed;
                bulk_g2s(ring + (size_t)slot * G.slot_bytes + G.p1_ab_off, base + off.ab[0] + (size_t)u.r0 * 2, 16, bar);
                bulk_g2s(ring + (size_t)slot * G.slot_bytes + G.p1_ab_off + 16, base + off.ab[1] + (size_t)u.r0 * 2, 16, bar);
            }
        } else {
            const uint32_t F = u.sh ? a.f_shared : a.f, G2 = F / GROUP, rb2 = F * BITS / 8;
            mbar_expect_tx(bar, u.count * (16 * rb2 + 64 * G2 + (a.expert_bias ? 32u : 0u)));   // count 0: the arrival alone
            for (uint32_t q = 0; q < u.count; ++q) {
                const uint32_t cell = u.sh ? 0u : st.route.cell[u.inst + q];
                const uint32_t mi = u.sh ? SHRIKE_MAX_POOL_CHUNKS : cell / a.pool.cells_per_chunk;
                const int32_t cc = u.sh ? 0 : (int32_t)(cell % a.pool.cells_per_chunk);
                const uint32_t eb = stage + q * G.p2_expert_bytes[u.sh];
                tma_4d(eb, &a.maps.w2[mi], 0, (int32_t)u.r0, 0, cc, bar);
                tma_4d(eb + G.p2_meta_off[u.sh], &a.maps.m2[mi], 0, (int32_t)(u.r0 / 8), 0, cc, bar);
                if (a.expert_bias) {
                    const uint8_t* base = u.sh ? a.shared_block : pool_cell_base(a.pool, cell);
                    const Offsets3& off = u.sh ? a.shared : a.routed;
                    bulk_g2s(ring + (size_t)slot * G.slot_bytes + q * G.p2_expert_bytes[u.sh] + G.p2_ab_off[u.sh],
                             base + off.ab[2] + (size_t)u.r0 * 2, 32, bar);
                }
            }
        }
    };

    // the shared expert's gate/up units do not depend on the routing (nor on the previous kernel): ask now
    if (tid == 0) {
        Unit u;
        while (prod_n < G.n_slots && prod.next(u, false)) issue(u, prod_n++);
    }

    if (warp == 0) FUSED_TS(1);
    pdl_wait();
    if (warp == 0) FUSED_TS(2);

    // ---- the activation row, as it is, into shared memory (one round trip, every thread a piece; the epoch
    // word travels in the same round trip); then this block's router rows from there ----
    {
        const uint32_t n16 = D * (a.act_dtype == SHRIKE_DTYPE_FP32 ? 4u : 2u) / 16;
        uint4* xr = (uint4*)(dsm + G.off_xraw);
        if (tid == 0) st.epoch = *(volatile const uint32_t*)a.epoch;
        for (uint32_t c = tid; c < n16; c += kFusedThreads) xr[c] = __ldg((const uint4*)a.x + c);
    }
    __syncthreads();
    const uint8_t* xraw = dsm + G.off_xraw;
    if (routes) {
        float acc;
        if (row_f32) {
            const uint32_t chunks = D / 4;
            const uint16_t* es = row_is_gate ? nullptr : a.eff_scale;
            if (!wait_bar(&st.rw_bar, 0)) report_status(a.status, kStatusWaitTimeout);
            const float4* wrow = (const float4*)(dsm + G.off_rw + (size_t)cw * D * 4);
            acc = 0.f;
            // lane l takes the float4 chunks l, l + 32, ... in order: the sequence of fused multiply-adds of
            // lane_dot_f32, both operands from shared memory
#pragma unroll 2
            for (uint32_t c = lane; c < chunks; c += 32) {
                const float4 wv = wrow[c];
                float xv[4];
                if (a.act_dtype == SHRIKE_DTYPE_FP32) {
                    const float4 v = ((const float4*)xraw)[c];
                    xv[0] = v.x; xv[1] = v.y; xv[2] = v.z; xv[3] = v.w;
                } else {
                    const uint2 v = ((const uint2*)xraw)[c];
                    if (a.act_dtype == SHRIKE_DTYPE_FP16) {
                        xv[0] = f16_bits_to_f32(v.x & 0xffff); xv[1] = f16_bits_to_f32(v.x >> 16);
                        xv[2] = f16_bits_to_f32(v.y & 0xffff); xv[3] = f16_bits_to_f32(v.y >> 16);
                    } else {
                        xv[0] = __uint_as_float(v.x << 16); xv[1] = __uint_as_float(v.x & 0xffff0000u);
                        xv[2] = __uint_as_float(v.y << 16); xv[3] = __uint_as_float(v.y & 0xffff0000u);
                    }
                }
                if (es) {
                    const uint2 q = __ldg((const uint2*)es + c);
                    xv[0] = __fmul_rn(xv[0], __uint_as_float(q.x << 16));
                    xv[1] = __fmul_rn(xv[1], __uint_as_float(q.x & 0xffff0000u));
                    xv[2] = __fmul_rn(xv[2], __uint_as_float(q.y << 16));
                    xv[3] = __fmul_rn(xv[3], __uint_as_float(q.y & 0xffff0000u));
                }
                acc = __fmaf_rn(wv.x, xv[0], acc);
                acc = __fmaf_rn(wv.y, xv[1], acc);
                acc = __fmaf_rn(wv.z, xv[2], acc);
                acc = __fmaf_rn(wv.w, xv[3], acc);
            }
        } else {
            const uint32_t groups = D / 64;
            acc = affine_row_dot((const uint8_t*)a.rw + (size_t)my_row * (D * a.rbits / 8), a.rscales + (size_t)my_row * groups,
                                 a.rbiases + (size_t)my_row * groups, a.rbits, groups, lane, xraw, a.act_dtype, a.eff_scale);
        }
        acc = butterfly_sum(acc);
        if (lane == 0)
            st_relaxed_u64(a.logits64 + my_row, ((unsigned long long)st.epoch << 32) | (unsigned long long)__float_as_uint(acc));
        if (cw == 0) FUSED_TS(3);   // this block's logits are published
    }
    for (uint32_t blk = tid; blk < D / 8; blk += kFusedThreads)
        xprep_block8(xraw, blk, a.act_dtype, BITS == 4, x_sm, a.status);
    __syncthreads();
    const uint32_t epoch = st.epoch;
    const uint32_t parity = epoch & 1u;
    uint16_t* acts_mine = a.acts_pub + (size_t)parity * kMaxInst * G.acts_stride;
    for (uint32_t grp = tid; grp < GD; grp += kFusedThreads) xs_sm[grp] = group_sums<BITS, GROUP>(x_sm, grp);

    // ---- gather every block's logits ----
    if (tid < router_rows) {
        bool ok = false;
        for (uint32_t it = 0; it < (1u << 17); ++it) {
            const unsigned long long v = ld_relaxed_u64(a.logits64 + tid);
            if ((uint32_t)(v >> 32) == epoch) {
                st.logits[tid] = __uint_as_float((uint32_t)v);
                ok = true;
                break;
            }
            if (it > 64) __nanosleep(64);
        }
        if (!ok) {
            report_status(a.status, kStatusWaitTimeout);
            st.logits[tid] = 0.f;
        }
    }
    uint32_t io = 1u;
    if (warp == kPW && a.io_status) io = *(volatile const uint32_t*)a.io_status;
    {   // the buffer the next call will use still holds the previous call's activations
        uint4* other = (uint4*)(a.acts_pub + (size_t)(parity ^ 1u) * kMaxInst * G.acts_stride);
        const uint32_t n16 = kMaxInst * G.acts_stride / 8;
        const uint4 fill = make_uint4(0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu);
        for (uint32_t i = blockIdx.x * kFusedThreads + tid; i < n16; i += gridDim.x * kFusedThreads) other[i] = fill;
    }
    __syncthreads();
    if (warp == 0) FUSED_TS(4);   // logits gathered

    // ---- selection (every block repeats it), residency lookup, instance list ----
    if (is_consumer) {
        uint32_t id;
        float w;
        select_warps(st.logits, a, st.cand_key, st.cand_id, cw, lane, id, w);
        if (cw == 0) {
            const bool ready = io == 1u || io == 3u;
            uint32_t slot = SHRIKE_SLOT_MISS;
            if (lane < a.top_k) {
                const uint64_t word = st.table[min(id, a.ne - 1u)];
                slot = (uint32_t)(word & 0xffffffffu);
                const bool hit = (uint32_t)(word >> 32) == 2u && slot != SHRIKE_SLOT_MISS;
                if (!hit) slot = SHRIKE_SLOT_MISS;
                if (blockIdx.x == 0) {
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
                    if (a.gate_row && a.out_gate && blockIdx.x == 0) a.out_gate[0] = st.route.w[0];
                }
            }
        }
    }
    __syncthreads();
    if (warp == 0) FUSED_TS(5);   // selection done
    const uint32_t n_routed = st.route.n_routed, n_inst = st.route.n_inst;

    if (is_producer) {
        // ================= producer =================
        if (lane == 0) {
            prod.n_routed = n_routed;
            Unit u;
#ifdef SHRIKE_TRACE
            uint32_t k = 12;
            if (a.trace) a.trace[(size_t)blockIdx.x * 16 + k++] = globaltimer_ns();
            while (prod.next(u, true)) {
                issue(u, prod_n++);
                if (a.trace && k < 16) a.trace[(size_t)blockIdx.x * 16 + k++] = globaltimer_ns();
            }
#else
            while (prod.next(u, true)) issue(u, prod_n++);
#endif
        }
        FUSED_TS(6);   // everything asked for
    } else if (is_consumer) {
        // ================= consumers =================
        const uint32_t g = lane >> 2, t = lane & 3;
        // this thread's byte offset inside its row's share of a group: rows are Q::kGroupBytes apart inside a
        // group's slab of a box ([group][row][group bytes])
        const uint32_t toff = t * (Q::kWords * 4);
        const uint32_t ctid = tid - kPW * 32;
        Walker wk;
        wk.init(a);
        wk.n_routed = n_routed;
        Unit u;
        uint32_t n = 0;
        bool staged = false;
        while (wk.next(u, true)) {
            if (u.kind == 1 && !staged) {
                if (cw == 0) FUSED_TS(8);   // this block's phase-1 units done
                // ---- all instances' activations: poll until published, stage, group sums. A thread's blocks
                // are all requested before the first is examined. ----
                constexpr uint32_t kMaxPer = 4;
                const uint32_t bps = G.acts_stride / 8;          // 16-byte blocks per instance (padded)
                const uint32_t total = n_inst * bps;
                for (uint32_t i0 = ctid; i0 < total; i0 += kCW * 32 * kMaxPer) {
                    uint4 v[kMaxPer];
                    bool need[kMaxPer];
#pragma unroll
                    for (uint32_t k = 0; k < kMaxPer; ++k) {
                        const uint32_t i = i0 + k * kCW * 32;
                        const uint32_t in = i / bps, b = i - in * bps;
                        const uint32_t F = (has_shared && in == 0) ? a.f_shared : a.f;
                        need[k] = i < total && b < F / 8;
                        v[k] = make_uint4(0xffffffffu, 0, 0, 0);
                        if (need[k]) v[k] = ld_relaxed_v4(acts_mine + (size_t)i * 8);
                    }
#pragma unroll
                    for (uint32_t k = 0; k < kMaxPer; ++k) {
                        if (!need[k]) continue;
                        const uint32_t i = i0 + k * kCW * 32;
                        bool ok = !has_sentinel(v[k]);
#pragma unroll 1
                        for (uint32_t it = 0; !ok && it < (1u << 17); ++it) {
                            if (it > 32) __nanosleep(64);
                            v[k] = ld_relaxed_v4(acts_mine + (size_t)i * 8);
                            ok = !has_sentinel(v[k]);
                        }
                        if (!ok) {
                            report_status(a.status, kStatusWaitTimeout);
                            v[k] = make_uint4(0, 0, 0, 0);
                        }
                        *(uint4*)(acts_sm + (size_t)i * 8) = v[k];
                    }
                }
                consumer_sync();
                for (uint32_t i = ctid; i < n_inst * gmax2; i += kCW * 32) {
                    const uint32_t in = i / gmax2, grp = i - in * gmax2;
                    const uint32_t F = (has_shared && in == 0) ? a.f_shared : a.f;
                    if (grp < F / GROUP) asum_sm[i] = group_sums<BITS, GROUP>(acts_sm + (size_t)in * G.acts_stride, grp);
                }
                consumer_sync();
                if (cw == 0) FUSED_TS(9);   // activations of every instance staged
                staged = true;
            }
            const uint32_t slot = n % G.n_slots, round = n / G.n_slots;
            if (!wait_bar(&st.full[slot], round & 1)) report_status(a.status, kStatusWaitTimeout);
            if (cw == 0 && n == 0) FUSED_TS(7);   // first unit landed
            const uint8_t* stage = ring + (size_t)slot * G.slot_bytes;
            float tot0 = 0.f, tot1 = 0.f;
            if (u.kind == 0) {
                // rows g (gate) and g + 8 (up) of the unit: [gate|up][group][row 0..7][group bytes]
                const uint8_t* rowA = stage + (size_t)g * Q::kGroupBytes + toff;
                const uint8_t* rowB = rowA + 8 * (size_t)rb1;
                const uint32_t slab = 8 * Q::kGroupBytes;
                // scales and biases: [gate|up][scale|bias][row 0..7][group]
                const uint8_t* s0p = stage + G.p1_meta_off + (size_t)g * GD * 2;
                const uint8_t* b0p = s0p + 16 * GD;
                const uint8_t* s1p = s0p + 32 * GD;
                const uint8_t* b1p = s0p + 48 * GD;
                const uint32_t cg = G.cg_p1, chunks = GD / cg;
                for (uint32_t c = cw; c < chunks; c += kCW) {
                    const float2 o = chunk_rows_cg<BITS, GROUP, META>(cg, rowA, rowB, slab, s0p, b0p, s1p, b1p, x_sm, xs_sm, c, t);
                    tot0 += o.x;
                    tot1 += o.y;
                }
                if (a.expert_bias && cw == 0) {
                    const uint16_t* ab = (const uint16_t*)(stage + G.p1_ab_off);
                    tot0 += bf16_bits_to_f32(ab[g]);
                    tot1 += bf16_bits_to_f32(ab[8 + g]);
                }
            } else {
                const uint32_t sh = u.sh;
                const uint32_t F = sh ? a.f_shared : a.f, G2 = F / GROUP;
                const uint32_t cg = G.cg_p2[sh], cpe = G2 / cg;
                for (uint32_t cc = cw; cc < u.count * cpe; cc += kCW) {
                    const uint32_t q = cc / cpe, c = cc - q * cpe;
                    const uint32_t in = u.inst + q;
                    const uint8_t* eb = stage + (size_t)q * G.p2_expert_bytes[sh];
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
                    const float2 o = chunk_rows_cg<BITS, GROUP, META>(cg, rowA, rowB, slab, s0p, b0p, s1p, b1p, bsm, xs, c, t);
                    float o0 = o.x, o1 = o.y;
                    if (a.expert_bias && c == 0) {
                        const uint16_t* ab = (const uint16_t*)(eb + G.p2_ab_off[sh]);
                        o0 += bf16_bits_to_f32(ab[g]);
                        o1 += bf16_bits_to_f32(ab[g + 8]);
                    }
                    const float w = st.route.w[in];
                    tot0 = fmaf(w, o0, tot0);
                    tot1 = fmaf(w, o1, tot1);
                }
            }
            // the slot's bytes are consumed; hand it back, then leave the partial sums for the epilogue warp
            __syncwarp();
            if (lane == 0) bar_arrive(&st.empty[slot]);
            const uint32_t rbuf = n & 1u, rround = n >> 1;
            if (rround > 0 && !wait_bar(&st.red_empty[rbuf], (rround - 1) & 1)) report_status(a.status, kStatusWaitTimeout);
            if (t == 0) {
                st.red[rbuf][cw][g] = tot0;
                st.red[rbuf][cw][g + 8] = tot1;
            }
            __syncwarp();
            if (lane == 0) bar_arrive(&st.red_full[rbuf]);
            ++n;
        }
        if (cw == 0) FUSED_TS(10);   // consumers done
    } else {
        // ================= epilogue warp =================
        // The next kernel in the stream may begin its prologue (its own weight prefetch) from here on. One lane
        // says so for the block: the instruction was measured to hold a warp for about 3 us, and this warp has
        // nothing to do until the first unit has been reduced.
        if (lane == 0) pdl_launch_dependents();
        Walker wk;
        wk.init(a);
        wk.n_routed = n_routed;
        Unit u;
        uint32_t n = 0;
        float ysum = 0.f;
        while (wk.next(u, true)) {
            const uint32_t rbuf = n & 1u, rround = n >> 1;
            if (!wait_bar(&st.red_full[rbuf], rround & 1)) report_status(a.status, kStatusWaitTimeout);
            float v = 0.f;
            if (lane < 16) {
#pragma unroll
                for (uint32_t w = 0; w < kCW; ++w) v += st.red[rbuf][w][lane];
            }
            __syncwarp();
            if (lane == 0) bar_arrive(&st.red_empty[rbuf]);
            if (u.kind == 0) {
                // rows 0..7 are gate rows; the up row of the same output sits 8 rows further
                const float up = __shfl_down_sync(0xffffffffu, v, 8);
                if (lane < 8) {
                    const float act = glu_call(v, up, a.activation);
                    st.act_stage[perm_index(lane, BITS == 4)] = act_to_half_bits(act, a.status);
                }
                __syncwarp();
                if (lane == 0) {
                    const uint4 pk = *(const uint4*)st.act_stage;
                    st_relaxed_v4(acts_mine + (size_t)u.inst * G.acts_stride + u.r0, pk);
                }
                __syncwarp();
            } else {
                ysum += v;
                if (u.last) {
                    if (lane < 16) {
                        const size_t o = (size_t)u.r0 + lane;
                        store_act(a.y, o, a.y_dtype, ysum);
                        if (a.hidden) {
                            const float h = load_act(a.hidden, o, a.act_dtype) + round_act(a.y_dtype, ysum);
                            store_act(a.hidden, o, a.act_dtype, h);
                        }
                    }
                    ysum = 0.f;
                }
            }
            ++n;
        }
        // every block read the epoch before it published its logits, and this block has gathered them all
        if (blockIdx.x == 0 && lane == 0) *(volatile uint32_t*)a.epoch = epoch + 1u;
        FUSED_TS(11);   // block done
    }
    if (st.failed && warp == 0 && lane == 0) {
        // a copy of this block may still be in flight: give it a bounded time to land before the block's
        // shared memory goes away
        for (int k = 0; k < 200; ++k) __nanosleep(1000);
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
    auto pick_cg = [](uint32_t groups) { return groups % 4 == 0 ? 4u : groups % 2 == 0 ? 2u : 1u; };
    g.cg_p1 = pick_cg(G1);
    for (int sh = 0; sh < 2; ++sh) {
        const uint32_t F = sh ? (c.has_shared ? c.shared_f : c.f) : c.f;
        const uint32_t rb2 = F * c.weight_bits / 8, G2 = F / c.group_size;
        g.p2_meta_off[sh] = align_up(16 * rb2, 128);
        g.p2_ab_off[sh] = align_up(g.p2_meta_off[sh] + 64 * G2, 128);
        g.p2_expert_bytes[sh] = g.p2_ab_off[sh] + 128;
        g.cg_p2[sh] = pick_cg(G2);
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
    g.off_rw = g.off_xraw + align_up(c.d * (c.act_dtype == SHRIKE_DTYPE_FP32 ? 4u : 2u), 16);
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
    return g.router_rows_per_block <= kMaxRouterRowsPerBlock && rows <= kFusedThreads;
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
size_t fused_logits_bytes(const shrike_moe_config& c) { return (size_t)(c.num_experts + 1) * 8; }
size_t fused_acts_bytes(const shrike_moe_config& c) {
    return (size_t)2 * kMaxInst * std::max(c.f, c.has_shared ? c.shared_f : 0u) * 2;
}

template <int BITS, int GROUP, int META>
static cudaError_t launch_fused_t(const shrike_moe* m, cudaStream_t st, const FusedArgs& a) {
    auto k = decode_layer_kernel<BITS, GROUP, META>;
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)a.g.smem_bytes);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)m->sm_count);
    cfg.blockDim = dim3(kFusedThreads);
    cfg.dynamicSmemBytes = a.g.smem_bytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    unsigned n = 0;
    if (!getenv("SHRIKE_NO_COOP")) {
        attr[n].id = cudaLaunchAttributeCooperative;   // every block resident: the blocks wait on each other's results
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
