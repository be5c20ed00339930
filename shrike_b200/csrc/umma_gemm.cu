// Ragged prefill on the 5th-generation tensor cores: an expert-grouped GEMM with
// the dequantisation in the producer warps (the B200 counterpart of
// mpp_prefill_affine_grouped_f16, tensorops.metal:145-248, and of
// encodeGroupedExpertGEMMs, PrefillGroupedRoutedMoE.swift:925-1035).
//
// One block = 256 weight rows of one expert against up to 256 of the rows routed
// to it ("swap-AB": the weights are the M operand -- two 128-row tiles, each
// with its own TMEM accumulator -- and the activation rows the N operand, so an
// expert with few rows still fills the MMA's M dimension). A 256 x 256 block
// reads each activation byte once per 256 weight rows and dequantises each
// weight once per 256 activation rows.
//
//   warp 18    one thread streams the packed weights (64 bytes of every row
//              per copy: a 3-D TMA box of 128 rows of one matrix of one pool
//              cell, 64-byte swizzle) and the group scales / biases (16 bytes
//              of every row per copy) into shared-memory rings. Whole-line TMA
//              requests keep the packed experts streaming at HBM speed where
//              per-thread 32-byte loads ran out of outstanding requests.
//   warp 17    one thread copies the activation tiles: a 64 x 256 box of the
//              expert-sorted fp16 rows per K block, 128-byte swizzle.
//   warps 0-15 converters: two threads per weight row; per 64-wide K block
//              they turn the packed nibbles/bytes into fp16 (q - Z) * scale +
//              (bias + Z*scale) -- the reference's half(fma(q, scale, bias)),
//              tensorops.metal:106 -- and writes them, 16 bytes at a time, into
//              the K-major 128-byte-swizzled tile the MMA reads. After the K
//              loop the same warps run the epilogue.
//   warp 16    one thread issues tcgen05.mma (M 128, N = rows, K 16, fp16 in,
//              fp32 accumulate in TMEM) for both tiles and commits to the
//              mbarriers that free the converted tile and the activation tile.
//
// PHASE 0: tile 0 = 128 gate rows, tile 1 = the matching 128 up rows; epilogue
//          GLU -> fp16 activations in operand layout, one row per sorted pair.
// PHASE 1: tiles = 256 consecutive down rows; epilogue (+ additive bias) x route
//          weight -> red.global.add into the token's fp32 accumulator row (the
//          weighted reduce, with no per-(row, rank) partial rows in between).
//
// Every wait is bounded; a wait that gives up sets the status word and the
// block falls through to the TMEM release.
#include <cuda.h>
// -DSHRIKE_TRACE: every block records entry / set-up / accumulators-ready / exit timestamps
// in the handle's trace buffer (shrike_debug_set_trace, debug builds only); compiled out of the shipped library.

#include "internal.h"

namespace shrike {

constexpr uint32_t kUmmaMaxN = 256;
constexpr int kActBoxes = 5;
constexpr uint32_t kConverters = 512;                  // two threads per weight row
constexpr uint32_t kConvWarps = kConverters / 32;
constexpr uint32_t kUmmaThreads = kConverters + 96;    // + MMA warp, activation-copy warp, weight-copy warp
constexpr uint32_t kAStages = 2, kMaxAStages = 4, kBStages = 3, kPkSlots = 3;   // kAStages: at the widest activation tile
constexpr uint32_t kTileBytes = 128 * 128;             // 128 rows x 64 fp16, one swizzle-128B K block
constexpr uint32_t kAStageBytes = 2 * kTileBytes;      // both weight tiles
constexpr uint32_t kBTileBytes = kUmmaMaxN * 128;      // 256 rows x 64 fp16
constexpr uint32_t kPkSlotBytes = 256 * 64;            // 64 packed bytes of 256 rows
constexpr uint32_t kScHalfBytes = 256 * 16;            // 8 scales (or biases) of 256 rows
constexpr uint32_t kOffA = kBStages * kBTileBytes;
constexpr uint32_t kOffPk = kOffA + kAStages * kAStageBytes;
constexpr uint32_t kOffSc = kOffPk + kPkSlots * kPkSlotBytes;
constexpr uint32_t kOffBar = kOffSc + 2 * kScHalfBytes;
constexpr uint32_t kNumBars = 2 * kMaxAStages + 2 * kBStages + 2 * kPkSlots + 3;
constexpr uint32_t kUmmaSmemBytes = kOffBar + kNumBars * 8 + 2 * kUmmaMaxN * 4 + 16 + 1024 /*alignment slack*/;

struct WeightMaps {       // TMA descriptors of the two 128-row tiles of a block
    CUtensorMap w[2];     // packed weights   [cells][rows][row bytes]
    CUtensorMap s[2];     // group scales     [cells][rows][groups]
    CUtensorMap b[2];     // group biases
};
struct UmmaMaps {
    WeightMaps routed[SHRIKE_MAX_POOL_CHUNKS];
    WeightMaps shared;
    CUtensorMap act_routed[kActBoxes], act_shared[kActBoxes];   // boxes of 16, 32, 64, 128 and 256 activation rows
};

// ---- tcgen05 wrappers -------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// K-major, 128-byte swizzle, rows packed at 128 bytes: 8-row atoms 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);   // start address
    d |= (uint64_t)1 << 16;                          // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;                // stride byte offset
    d |= (uint64_t)1 << 46;                          // descriptor version
    d |= (uint64_t)2 << 61;                          // 128-byte swizzle
    return d;
}
// D fp32, A/B fp16, both K-major, M 128, N n.
__device__ __forceinline__ uint32_t umma_idesc(uint32_t n) {
    return (1u << 4) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}

// 8 packed nibbles -> 8 fp16 weights in operand order {0,4,1,5,2,6,3,7}; 4 bytes -> 4 fp16 in order.
template <int BITS>
__device__ __forceinline__ void dequant_word(uint32_t w, uint32_t s2, uint32_t z2, uint32_t* out) {
    if constexpr (BITS == 4) {
        // nibbles j and j + 4 of the word make pair j. A nibble in bits 0..3 of a half is read as the fp16
        // value 1024 + q, one in bits 4..7 as 64 + q (64's unit in the last place sits at bit 4): one shift
        // per word instead of three.
        const uint32_t v = w >> 8;
        const uint32_t h0 = hsub2_u32(lop3_and_or(w, 0x000F000Fu, 0x64006400u), 0x64086408u);   // (1024 + q) - 1032
        const uint32_t h1 = hsub2_u32(lop3_and_or(w, 0x00F000F0u, 0x54005400u), 0x54805480u);   // (64 + q) - 72
        const uint32_t h2 = hsub2_u32(lop3_and_or(v, 0x000F000Fu, 0x64006400u), 0x64086408u);
        const uint32_t h3 = hsub2_u32(lop3_and_or(v, 0x00F000F0u, 0x54005400u), 0x54805480u);
        asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(out[0]) : "r"(h0), "r"(s2), "r"(z2));
        asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(out[1]) : "r"(h1), "r"(s2), "r"(z2));
        asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(out[2]) : "r"(h2), "r"(s2), "r"(z2));
        asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(out[3]) : "r"(h3), "r"(s2), "r"(z2));
    } else {
        const uint32_t lo = hsub2_u32(prmt(w, 0x64646464u, 0x5140u), 0x64806480u);
        const uint32_t hi = hsub2_u32(prmt(w, 0x64646464u, 0x5342u), 0x64806480u);
        asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(out[0]) : "r"(lo), "r"(s2), "r"(z2));
        asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(out[1]) : "r"(hi), "r"(s2), "r"(z2));
    }
}

__device__ __forceinline__ uint32_t half2_dup(float v) {
    const uint32_t h = __half_as_ushort(__float2half_rn(v));
    return h | (h << 16);
}

__device__ __forceinline__ void tmem_ld16_issue(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Tiled TMA loads (no multicast). x is the element column, then row, then cell.
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* map, int32_t x, int32_t y,
                                            uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_dst), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t smem_dst, const CUtensorMap* map, int32_t x, int32_t y, int32_t z,
                                            uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(smem_dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar)) : "memory");
}

// SiLU / clamped-SwiGLU gates with the fast exponential and reciprocal: the
// epilogue runs one per output element, and the result is rounded to fp16.
__device__ __forceinline__ float glu_epilogue(float gate, float up, uint32_t activation) {
    if (activation == SHRIKE_ACT_CLAMPED_SWIGLU) {
        const float gc = fminf(gate, 7.0f);
        const float uc = fmaxf(-7.0f, fminf(up, 7.0f));
        return __fdividef(gc, 1.0f + __expf(-1.702f * gc)) * (uc + 1.0f);
    }
    if (activation == SHRIKE_ACT_GELU_TANH) return glu(gate, up, activation);
    return __fdividef(gate, 1.0f + __expf(-gate)) * up;
}

// Bounded wait for the pipeline barriers: these are on the critical path of every K block, so the
// first polls do not sleep.
__device__ __forceinline__ bool pipe_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t it = 0; it < (1u << 21); ++it) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
        if (ok) return true;
        if (it > 256) __nanosleep(32);
    }
    return false;
}

// 16-bit field `idx` (0..7) of four registers.
__device__ __forceinline__ uint16_t pick16(const uint32_t (&v)[4], uint32_t idx) {
    const uint32_t lo = (idx & 2u) ? v[1] : v[0], hi = (idx & 2u) ? v[3] : v[2];
    const uint32_t w = (idx & 4u) ? hi : lo;
    return (uint16_t)((idx & 1u) ? (w >> 16) : (w & 0xffffu));
}

struct ChunkInstance {  // up to 256 rows that share one expert block
    uint32_t kind, slot, first, count;
};

// grid (row tiles, max chunk instances); block 608.
template <int BITS, int GROUP, int META, int PHASE>
__global__ void __launch_bounds__(kUmmaThreads, 1)
umma_expert_kernel(const ExpertArgs a, const ChunkInstance* __restrict__ inst, const uint32_t* __restrict__ n_inst,
                   const __grid_constant__ UmmaMaps maps) {
    constexpr uint32_t kRowBlockBytes = 64 * BITS / 8;  // packed bytes of one row per K block (32 or 64)
    constexpr uint32_t kWordsPerBlock = kRowBlockBytes / 4;
    constexpr uint32_t kGroupsPerBlock = 64 / GROUP;    // 1 (g64) or 2 (g32)
    constexpr uint32_t kKbPerPk = 64 / kRowBlockBytes;  // K blocks per packed copy (2 or 1)
    constexpr uint32_t kKbPerSc = 8 / kGroupsPerBlock;  // K blocks per scale copy (8 or 4)
    constexpr float kZero = BITS == 4 ? 8.0f : 128.0f;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
#ifdef SHRIKE_TRACE
    const uint64_t t_entry = globaltimer_ns();
#endif
    const uint32_t ii = blockIdx.y;
    if (ii >= *n_inst) return;
    const ChunkInstance in = inst[ii];
    const bool shared = in.kind == 1;
    const uint32_t F = shared ? a.f_shared : a.f;
    const uint32_t kdim = PHASE == 0 ? a.d : F;
    const uint32_t out_rows = PHASE == 0 ? F : a.d;       // rows of the weight matrix
    const uint32_t r0 = blockIdx.x * (PHASE == 0 ? 128u : 256u);
    if (r0 >= out_rows) return;
    const Offsets3& off = shared ? a.shared : a.routed;
    const uint8_t* base = shared ? a.shared_block : pool_cell_base(a.pool, in.slot);
    const uint32_t KB = kdim / 64;
    const uint32_t G = kdim / GROUP;
    // scale rows that are whole 16-byte units come by TMA; others (G % 8 != 0) are read by the converters
    const bool sc_tma = (G & 7u) == 0;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t N = (in.count + 15u) & ~15u;           // MMA N: rows padded to 16
    uint32_t ncols = 32;                                   // TMEM columns of one accumulator
    while (ncols < N) ncols <<= 1;
    // The activation tiles and the converted weight tiles share one region of shared memory: an instance with
    // few rows needs narrow activation tiles and gets more weight stages instead. What paces such a block is the
    // round trip converters -> tensor core -> converters (barrier, issue, commit, barrier: about half a
    // microsecond against a few hundred nanoseconds of arithmetic), so it wants more tiles in flight.
    // the instance's rows as one or two boxes of 16 << i rows: the largest that fits, then the smallest that
    // holds the rest
    uint32_t n1 = 16, b1 = 0;
    while ((n1 << 1) <= N && b1 + 1 < (uint32_t)kActBoxes) { n1 <<= 1; ++b1; }
    uint32_t n2 = 0, b2 = 0;
    if (N > n1) {
        n2 = 16;
        while (n2 < N - n1) { n2 <<= 1; ++b2; }
    }
    const uint32_t b_stage = (((n1 + n2) * 128u + 2047u) / 2048u) * 2048u;   // bytes of one activation stage
    const uint32_t off_a = kBStages * b_stage;
    const uint32_t a_stages = min(kMaxAStages, (kOffPk - off_a) / kAStageBytes);

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
    uint64_t* bars = (uint64_t*)(smem + kOffBar);
    uint64_t* a_full = bars;                       // converters -> MMA
    uint64_t* a_empty = a_full + kMaxAStages;      // MMA -> converters
    uint64_t* b_full = a_empty + kMaxAStages;      // activation copy -> MMA
    uint64_t* b_empty = b_full + kBStages;         // MMA -> activation copy
    uint64_t* pk_full = b_empty + kBStages;        // weight copy -> converters
    uint64_t* pk_empty = pk_full + kPkSlots;       // converters -> weight copy
    uint64_t* sc_full = pk_empty + kPkSlots;
    uint64_t* sc_empty = sc_full + 1;
    uint64_t* accum = sc_empty + 1;
    uint32_t* rowid = (uint32_t*)(bars + kNumBars);   // token of column n
    float* roww = (float*)(rowid + kUmmaMaxN);        // route weight (routed) or gate (shared) of column n
    uint32_t* tmem_slot = (uint32_t*)(roww + kUmmaMaxN);
    __shared__ uint32_t s_failed;

    if (tid == 0) {
        for (uint32_t s = 0; s < kMaxAStages; ++s) { mbar_init(&a_full[s], kConvWarps); mbar_init(&a_empty[s], 1); }
        for (uint32_t s = 0; s < kBStages; ++s) { mbar_init(&b_full[s], 1); mbar_init(&b_empty[s], 1); }
        for (uint32_t s = 0; s < kPkSlots; ++s) { mbar_init(&pk_full[s], 1); mbar_init(&pk_empty[s], kConvWarps); }
        mbar_init(sc_full, 1);
        mbar_init(sc_empty, kConvWarps);
        mbar_init(accum, 1);
        fence_mbar_init();
        s_failed = 0;
    }
    // the descriptors this block's copy threads will use: fetched while the barriers are set up
    if (warp == kConvWarps + 1 && lane < 2) {
        const CUtensorMap* mb = shared ? maps.act_shared : maps.act_routed;
        asm volatile("prefetch.tensormap [%0];" ::"l"(&mb[lane == 0 ? b1 : b2]) : "memory");
    }
    if (warp == kConvWarps + 2 && lane < 6) {
        const WeightMaps* wm = shared ? &maps.shared : &maps.routed[in.slot / a.pool.cells_per_chunk];
        const CUtensorMap* mp = lane < 2 ? &wm->w[lane] : lane < 4 ? &wm->s[lane - 2] : &wm->b[lane - 4];
        asm volatile("prefetch.tensormap [%0];" ::"l"(mp) : "memory");
    }
    if (warp == kConvWarps) tmem_alloc(smem_u32(tmem_slot), 2 * ncols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
#ifdef SHRIKE_TRACE
    uint64_t* const tr = a.trace ? a.trace + 8 * ((size_t)(PHASE * 4096 + blockIdx.y) * 8 + blockIdx.x) : nullptr;
    if (tr && tid == 0) { tr[0] = t_entry; tr[1] = globaltimer_ns(); tr[7] = ((uint64_t)N << 32) | KB; }
#endif
    auto give_up = [&]() {
        report_status(a.status, kStatusWaitTimeout);
        s_failed = 1;
    };

    if (warp < kConvWarps) {
        // ---------------- converters ----------------
        // the tokens and route weights of the columns: the epilogue reads them, long after these loads
        if (PHASE == 1) {
            for (uint32_t n = tid; n < kUmmaMaxN; n += kConverters) {
                const uint32_t src = n < in.count ? n : 0;
                if (shared) {
                    rowid[n] = in.first + src;
                    roww[n] = a.shared_gate ? a.shared_gate[in.first + src] : 1.0f;
                } else {
                    const uint32_t pair = a.sorted[in.first + src];
                    rowid[n] = pair / a.top_k;
                    roww[n] = a.route_w[pair];
                }
            }
        }
        // Two threads per weight row: thread `half` converts 32 of the K block's 64 weights.
        const uint32_t tile = tid >> 8, r = (tid >> 1) & 127, half = tid & 1;
        constexpr uint32_t kWordsPerThread = kWordsPerBlock / 2;   // 4 (int4) or 8 (int8)
        const uint32_t pk_row = kOffPk + tile * (kPkSlotBytes / 2) + r * 64, pk_xor = (r >> 1) & 3;
        uint32_t sreg[4] = {0, 0, 0, 0}, breg[4] = {0, 0, 0, 0};
        uint32_t snext[4] = {0, 0, 0, 0}, bnext[4] = {0, 0, 0, 0};
        const uint32_t mrow = r0 + (PHASE == 0 ? r : tile * 128 + r);
        const int mat = PHASE == 0 ? (int)tile : 2;
        const uint16_t* srow = (const uint16_t*)(base + off.s[mat]) + (size_t)mrow * G;
        const uint16_t* brow = (const uint16_t*)(base + off.b[mat]) + (size_t)mrow * G;
        // groups 8*blk .. 8*blk+7 of this thread's row, straight from global memory (rows past the matrix
        // and groups past the row read as zero: the converted weights are then zero)
        auto fetch_scales = [&](uint32_t blk) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t gi = blk * 8 + 2 * i;
                uint32_t sv = 0, bv = 0;
                if (mrow < out_rows && gi < G) {
                    sv = __ldg(srow + gi);
                    bv = __ldg(brow + gi);
                    if (gi + 1 < G) {
                        sv |= (uint32_t)__ldg(srow + gi + 1) << 16;
                        bv |= (uint32_t)__ldg(brow + gi + 1) << 16;
                    }
                }
                snext[i] = sv;
                bnext[i] = bv;
            }
        };
        if (!sc_tma) fetch_scales(0);
        // What does not change along K: this thread's chunk positions in a packed slot and in the converted
        // tile (both swizzled by the row), and the tile rows of the two stages.
        uint32_t pk_off[kKbPerPk * (kWordsPerThread / 4)];
#pragma unroll
        for (uint32_t sub = 0; sub < kKbPerPk; ++sub)
#pragma unroll
            for (uint32_t q = 0; q < kWordsPerThread / 4; ++q) {
                // 16-byte chunk of the 64-byte row: the K block's share, then this thread's half of it
                const uint32_t c = sub * (kRowBlockBytes / 16) + half * (kWordsPerThread / 4) + q;
                pk_off[sub * (kWordsPerThread / 4) + q] = pk_row + ((c ^ pk_xor) << 4);
            }
        constexpr uint32_t kStores = BITS == 4 ? kWordsPerThread : kWordsPerThread / 2;   // 16-byte chunks written
        uint32_t a_off[kStores];
#pragma unroll
        for (uint32_t i = 0; i < kStores; ++i)   // A row r: 8 chunks of 8 fp16; chunk c lives at position c ^ (r & 7)
            a_off[i] = off_a + tile * kTileBytes + r * 128 + (((half * kStores + i) ^ (r & 7)) << 4);
        // A scale block (8 groups of the row) at a time, its K blocks unrolled: the position in the packed slot
        // and the group of a K block are then constants of the instruction stream.
        uint32_t st = 0, a_round = 0;   // the stage of the next K block and how often the stages have gone round
        for (uint32_t kb0 = 0; kb0 < KB; kb0 += kKbPerSc) {
            if (*(volatile uint32_t*)&s_failed) break;
            if (sc_tma) {
                if (!pipe_wait(sc_full, (kb0 / kKbPerSc) & 1)) { give_up(); break; }
                const uint4 sv = *(const uint4*)(smem + kOffSc + tile * (kScHalfBytes / 2) + r * 16);
                const uint4 bv = *(const uint4*)(smem + kOffSc + kScHalfBytes + tile * (kScHalfBytes / 2) + r * 16);
                sreg[0] = sv.x; sreg[1] = sv.y; sreg[2] = sv.z; sreg[3] = sv.w;
                breg[0] = bv.x; breg[1] = bv.y; breg[2] = bv.z; breg[3] = bv.w;
                // the values are in registers: the copy thread may fetch the next block's
                __syncwarp();
                if (lane == 0) mbar_arrive(sc_empty);
            } else {
                // this block's 8 groups were fetched one block ago; fetch the next block's now
#pragma unroll
                for (int i = 0; i < 4; ++i) { sreg[i] = snext[i]; breg[i] = bnext[i]; }
                fetch_scales(kb0 / kKbPerSc + 1);
            }
            uint32_t slot_base = 0, slot = 0;
#pragma unroll
            for (uint32_t j = 0; j < kKbPerSc; ++j) {
                const uint32_t kb = kb0 + j;
                if (kb >= KB) break;
                constexpr uint32_t kSubMask = kKbPerPk - 1;
                const uint32_t sub = j & kSubMask;         // K block within its packed slot
                if (sub == 0) {
                    const uint32_t u = kb / kKbPerPk;
                    slot = u % kPkSlots;
                    slot_base = slot * kPkSlotBytes;
                    if (!pipe_wait(&pk_full[slot], (u / kPkSlots) & 1)) { give_up(); break; }
                }
                uint32_t pk[kWordsPerThread];
#pragma unroll
                for (uint32_t q = 0; q < kWordsPerThread / 4; ++q) {
                    const uint4 v = *(const uint4*)(smem + slot_base + pk_off[sub * (kWordsPerThread / 4) + q]);
                    pk[4 * q] = v.x; pk[4 * q + 1] = v.y; pk[4 * q + 2] = v.z; pk[4 * q + 3] = v.w;
                }
                // a thread's half of a 64-wide block lies inside one group of 32 or 64
                const uint32_t gsel = j * kGroupsPerBlock + (GROUP == 64 ? 0u : half);
                const float sc = meta_to_f32<META>(pick16(sreg, gsel));
                const float zf = fmaf(kZero, sc, meta_to_f32<META>(pick16(breg, gsel)));
                const uint32_t s2 = half2_dup(sc), z2 = half2_dup(zf);
                if (a_round && !pipe_wait(&a_empty[st], (a_round - 1) & 1)) { give_up(); break; }
                uint8_t* a_stage = smem + st * kAStageBytes;
#pragma unroll
                for (uint32_t i = 0; i < kWordsPerThread; ++i) {
                    uint32_t o[4];
                    dequant_word<BITS>(pk[i], s2, z2, o);
                    if constexpr (BITS == 4) {
                        *(uint4*)(a_stage + a_off[i]) = make_uint4(o[0], o[1], o[2], o[3]);
                    } else {
                        // two words make one 16-byte chunk
                        *((uint2*)(a_stage + a_off[i >> 1]) + (i & 1)) = make_uint2(o[0], o[1]);
                    }
                }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) {
                    // one arrival per warp: 512 arrivals on one barrier word would serialise every K block
                    mbar_arrive(&a_full[st]);
                    // The ring slots are handed back only here: by now the values read from them have been
                    // consumed, so the reads are complete before the copy thread may overwrite the slot.
                    if (sub == kSubMask || kb + 1 == KB) mbar_arrive(&pk_empty[slot]);
                }
                if (++st == a_stages) { st = 0; ++a_round; }
            }
        }
    } else if (warp == kConvWarps && lane == 0) {
        // ---------------- MMA issue ----------------
        const uint32_t idesc = umma_idesc(N);
        uint32_t sa = 0, a_round = 0;
        for (uint32_t kb = 0; kb < KB; ++kb) {
            const uint32_t sb = kb % kBStages;
            if (!pipe_wait(&a_full[sa], a_round & 1) || !pipe_wait(&b_full[sb], (kb / kBStages) & 1)) {
                give_up();
                break;
            }
            tc_fence_after();
            const uint32_t a_addr = smem_base + off_a + sa * kAStageBytes;
            const uint64_t da0 = umma_smem_desc(a_addr), da1 = umma_smem_desc(a_addr + kTileBytes);
            const uint64_t db = umma_smem_desc(smem_base + sb * b_stage);
            // 4 x K16 per 64-wide block: 32 bytes further along the row. The two tiles alternate: consecutive
            // instructions then add into different accumulators.
#pragma unroll
            for (uint32_t k = 0; k < 4; ++k) {
                umma_f16(tmem_base, da0 + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
                umma_f16(tmem_base + ncols, da1 + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
            }
            umma_commit(&a_empty[sa]);
            umma_commit(&b_empty[sb]);
            if (++sa == a_stages) { sa = 0; ++a_round; }
        }
        umma_commit(accum);
    } else if (warp == kConvWarps + 1 && lane == 0) {
        // ---------------- activation tiles ----------------
        // One or two boxes per K block: these tiles are most of what a block pulls out of L2, and a short instance
        // does not pay for 256 rows, nor one of 80 rows for 128.
        const CUtensorMap* maps_b = shared ? maps.act_shared : maps.act_routed;
        const uint32_t b_bytes = (n1 + n2) * 128u;
        for (uint32_t kb = 0; kb < KB; ++kb) {
            if (*(volatile uint32_t*)&s_failed) break;
            const uint32_t sb = kb % kBStages;
            if (kb >= kBStages && !pipe_wait(&b_empty[sb], ((kb / kBStages) - 1) & 1)) { give_up(); break; }
            mbar_expect_tx(&b_full[sb], b_bytes);
            tma_load_2d(smem_base + sb * b_stage, &maps_b[b1], (int32_t)(kb * 64), (int32_t)in.first, &b_full[sb]);
            if (n2)
                tma_load_2d(smem_base + sb * b_stage + n1 * 128u, &maps_b[b2], (int32_t)(kb * 64),
                            (int32_t)(in.first + n1), &b_full[sb]);
        }
    } else if (warp == kConvWarps + 2 && lane == 0) {
        // ---------------- packed weights, scales, biases ----------------
        const WeightMaps* wm = shared ? &maps.shared : &maps.routed[in.slot / a.pool.cells_per_chunk];
        const int32_t cell = shared ? 0 : (int32_t)(in.slot % a.pool.cells_per_chunk);
        const int32_t y0 = (int32_t)r0, y1 = (int32_t)(PHASE == 0 ? r0 : r0 + 128);
        for (uint32_t kb = 0; kb < KB; ++kb) {
            if (*(volatile uint32_t*)&s_failed) break;
            if (sc_tma && kb % kKbPerSc == 0) {
                const uint32_t blk = kb / kKbPerSc;
                if (blk > 0 && !pipe_wait(sc_empty, (blk - 1) & 1)) { give_up(); break; }
                mbar_expect_tx(sc_full, 2 * kScHalfBytes);
                const uint32_t dst = smem_base + kOffSc;
                tma_load_3d(dst, &wm->s[0], (int32_t)(blk * 8), y0, cell, sc_full);
                tma_load_3d(dst + kScHalfBytes / 2, &wm->s[1], (int32_t)(blk * 8), y1, cell, sc_full);
                tma_load_3d(dst + kScHalfBytes, &wm->b[0], (int32_t)(blk * 8), y0, cell, sc_full);
                tma_load_3d(dst + kScHalfBytes + kScHalfBytes / 2, &wm->b[1], (int32_t)(blk * 8), y1, cell, sc_full);
            }
            if (kb % kKbPerPk == 0) {
                const uint32_t u = kb / kKbPerPk, slot = u % kPkSlots;
                if (u >= kPkSlots && !pipe_wait(&pk_empty[slot], ((u / kPkSlots) - 1) & 1)) { give_up(); break; }
                mbar_expect_tx(&pk_full[slot], kPkSlotBytes);
                const uint32_t dst = smem_base + kOffPk + slot * kPkSlotBytes;
                tma_load_3d(dst, &wm->w[0], (int32_t)(u * 64), y0, cell, &pk_full[slot]);
                tma_load_3d(dst + kPkSlotBytes / 2, &wm->w[1], (int32_t)(u * 64), y1, cell, &pk_full[slot]);
            }
        }
    }

    // ---------------- epilogue (warp w: TMEM lanes 32*(w & 3) .. +31, every fourth 16-column group) ----------------
    if (warp < kConvWarps) {
        bool ok = pipe_wait(accum, 0);
        if (!ok) report_status(a.status, kStatusWaitTimeout);
        if (*(volatile uint32_t*)&s_failed) ok = false;
        tc_fence_after();
        // the columns' tokens and weights were written by other converter threads at the start of the block
        if (PHASE == 1) asm volatile("bar.sync 1, %0;" ::"n"(kConverters) : "memory");
#ifdef SHRIKE_TRACE
        if (tr && tid == 0) tr[5] = globaltimer_ns();
#endif
        const uint32_t q = warp & 3, h = warp >> 2;
        const uint32_t trow = q * 32 + lane;                       // row inside each 128-row tile
        const uint32_t taddr = tmem_base + ((q * 32) << 16);
        constexpr uint32_t kColStep = 16 * (kConvWarps / 4);
        if (PHASE == 0) {
            const uint32_t f = r0 + trow;
            const bool f_ok = f < F && ok;
            float gab = 0.f, uab = 0.f;
            if (a.expert_bias && f < F) {
                gab = bf16_bits_to_f32(((const uint16_t*)(base + off.ab[0]))[f]);
                uab = bf16_bits_to_f32(((const uint16_t*)(base + off.ab[1]))[f]);
            }
            uint16_t* dst = (shared ? a.acts_shared : a.acts) + (size_t)in.first * F + perm_index(f, BITS == 4);
            for (uint32_t c0 = h * 16; c0 < N; c0 += kColStep) {
                uint32_t g[16], u[16];
                tmem_ld16_issue(taddr + c0, g);
                tmem_ld16_issue(taddr + ncols + c0, u);
                tmem_ld_wait();
                uint16_t* p = dst + (size_t)c0 * F;
                const uint32_t live = f_ok ? min(16u, in.count > c0 ? in.count - c0 : 0u) : 0u;   // rows of this group
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float v = glu_epilogue(__uint_as_float(g[j]) + gab, __uint_as_float(u[j]) + uab, a.activation);
                    if ((uint32_t)j < live) *p = act_to_half_bits(v, a.status);
                    p += F;
                }
            }
        } else {
            const uint32_t d0 = r0 + trow, d1 = d0 + 128;
            float ab0 = 0.f, ab1 = 0.f;
            if (a.expert_bias) {
                const uint16_t* dab = (const uint16_t*)(base + off.ab[2]);
                if (d0 < a.d) ab0 = bf16_bits_to_f32(dab[d0]);
                if (d1 < a.d) ab1 = bf16_bits_to_f32(dab[d1]);
            }
            const bool ok0 = ok && d0 < a.d, ok1 = ok && d1 < a.d;
            for (uint32_t c0 = h * 16; c0 < N; c0 += kColStep) {
                uint32_t v0[16], v1[16];
                tmem_ld16_issue(taddr + c0, v0);
                tmem_ld16_issue(taddr + ncols + c0, v1);
                tmem_ld_wait();
                const uint32_t live = min(16u, in.count > c0 ? in.count - c0 : 0u);
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    if ((uint32_t)j < live) {
                        // lanes hold consecutive output rows: one 128-byte reduction per warp and column
                        float* o = a.yacc + (size_t)rowid[c0 + j] * a.d + d0;
                        const float w = roww[c0 + j];
                        if (ok0) atomicAdd(o, w * (__uint_as_float(v0[j]) + ab0));
                        if (ok1) atomicAdd(o + 128, w * (__uint_as_float(v1[j]) + ab1));
                    }
                }
            }
        }
    }
#ifdef SHRIKE_TRACE
    if (tr && tid == 0) tr[6] = globaltimer_ns();
#endif
    if (*(volatile uint32_t*)&s_failed && lane == 0 && warp > kConvWarps) {
        // a copy of this block may still be in flight: give it a bounded time to land
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kConvWarps) {
        __syncwarp();
        tmem_dealloc(tmem_base, 2 * ncols);
    }
}

// One thread per expert: ceil(count/256) chunk instances each, then the shared expert's.
// n_inst[0] = instances, n_inst[1] = sorted rows in total.
__global__ void __launch_bounds__(256)
chunk_instances_kernel(const uint32_t* __restrict__ offsets, const uint32_t* __restrict__ counts,
                       const uint32_t* __restrict__ slot_of_expert, uint32_t ne, uint32_t T, uint32_t with_shared,
                       uint32_t pool_cells, ChunkInstance* __restrict__ inst, uint32_t* __restrict__ n_inst,
                       uint32_t* status) {
    __shared__ uint32_t warp_sums[8], warp_rows[8];
    const uint32_t e = threadIdx.x;
    uint32_t n = 0, slot = SHRIKE_SLOT_MISS, c = 0;
    if (e < ne && counts[e] > 0) {
        c = counts[e];
        slot = slot_of_expert[e];
        if (slot != SHRIKE_SLOT_MISS && slot >= pool_cells) {
            report_status(status, kStatusBadIndex);
            slot = SHRIKE_SLOT_MISS;
        }
        if (slot != SHRIKE_SLOT_MISS) n = (c + kUmmaMaxN - 1) / kUmmaMaxN;
    }
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t inc = n, rows = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t v = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= (uint32_t)o) inc += v;
        rows += __shfl_xor_sync(0xffffffffu, rows, o);
    }
    if (lane == 31) warp_sums[warp] = inc;
    if (lane == 0) warp_rows[warp] = rows;
    __syncthreads();
    uint32_t base = 0, total = 0, total_rows = 0;
    for (uint32_t w = 0; w < 8; ++w) {
        if (w < warp) base += warp_sums[w];
        total += warp_sums[w];
        total_rows += warp_rows[w];
    }
    // The shared expert's instances come first in the list: they are full (256 rows), and the blocks of the
    // list's end are the last to start -- a launch that ends on its longest blocks ends late.
    const uint32_t n_shared = with_shared ? (T + kUmmaMaxN - 1) / kUmmaMaxN : 0;
    base += inc - n + n_shared;
    for (uint32_t j = 0; j < n; ++j) {
        ChunkInstance in;
        in.kind = 0; in.slot = slot; in.first = offsets[e] + kUmmaMaxN * j; in.count = min(kUmmaMaxN, c - kUmmaMaxN * j);
        inst[base + j] = in;
    }
    for (uint32_t j = threadIdx.x; j < n_shared; j += blockDim.x) {
        ChunkInstance in;
        in.kind = 1; in.slot = 0; in.first = kUmmaMaxN * j; in.count = min(kUmmaMaxN, T - kUmmaMaxN * j);
        inst[j] = in;
    }
    if (threadIdx.x == 0) {
        n_inst[0] = total + n_shared;
        n_inst[1] = total_rows;
    }
}

// The activation rows in expert-sorted order: xs[pos] = xh[token of sorted pair pos].
// grid (pairs); one block copies one row.
__global__ void __launch_bounds__(128)
gather_sorted_rows_kernel(const uint16_t* __restrict__ xh, const uint32_t* __restrict__ sorted,
                          const uint32_t* __restrict__ n_inst, uint32_t top_k, uint32_t d, uint16_t* __restrict__ xs) {
    const uint32_t pos = blockIdx.x;
    if (pos >= n_inst[1]) return;
    const uint4* src = (const uint4*)(xh + (size_t)(sorted[pos] / top_k) * d);
    uint4* dst = (uint4*)(xs + (size_t)pos * d);
    for (uint32_t i = threadIdx.x; i < d / 8; i += blockDim.x) dst[i] = __ldg(src + i);
}

// ---- tensor maps -------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            p = nullptr;
        return (EncodeTiledFn)p;
    }();
    return fn;
}

// fp16 activation rows [rows][cols]: box = 64 columns (one 128-byte swizzle row) x box_rows rows.
static bool make_rows_map(CUtensorMap* map, const uint16_t* base, uint64_t cols, uint64_t rows, uint32_t box_rows) {
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2};
    const cuuint32_t box[2] = {64, box_rows};
    const cuuint32_t elem[2] = {1, 1};
    return encode_tiled_fn()(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, (void*)base, dims, strides, box, elem,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// One matrix of every cell of a pool chunk: [cells][rows][row_bytes] bytes (packed weights, 64-byte
// boxes of 128 rows, 64-byte swizzle) or [cells][rows][groups] 16-bit (scales / biases, 8 per row).
static bool make_matrix_map(CUtensorMap* map, const uint8_t* base, bool meta, uint64_t row_elems, uint64_t rows,
                            uint64_t cells, uint64_t cell_stride) {
    const uint64_t esz = meta ? 2 : 1;
    const cuuint64_t dims[3] = {row_elems, rows, cells};
    // a single cell (the shared expert's block) still needs a valid outer pitch
    const cuuint64_t strides[2] = {row_elems * esz, cells > 1 ? cell_stride : row_elems * esz * rows};
    const cuuint32_t box[3] = {meta ? 8u : 64u, 128, 1};
    const cuuint32_t elem[3] = {1, 1, 1};
    return encode_tiled_fn()(map, meta ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, (void*)base,
                             dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             meta ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_64B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The two tiles of one phase: gate + up (phase 0) or down twice (phase 1).
static bool make_weight_maps(WeightMaps* wm, const uint8_t* base, const Offsets3& off, int phase, uint32_t kdim,
                             uint32_t rows, uint32_t bits, uint32_t group, uint64_t cells, uint64_t cell_stride) {
    for (int t = 0; t < 2; ++t) {
        const int mat = phase == 0 ? t : 2;
        if (!make_matrix_map(&wm->w[t], base + off.w[mat], false, (uint64_t)kdim * bits / 8, rows, cells, cell_stride))
            return false;
        if ((kdim / group) % 8 != 0) continue;   // such scale rows are read by the converter threads
        if (!make_matrix_map(&wm->s[t], base + off.s[mat], true, kdim / group, rows, cells, cell_stride) ||
            !make_matrix_map(&wm->b[t], base + off.b[mat], true, kdim / group, rows, cells, cell_stride))
            return false;
    }
    return true;
}

// K in whole 64-wide blocks (packed rows are then whole 16-byte units, which the TMA copies need).
bool umma_supported(const shrike_moe_config& c) {
    if (c.d % 64 || c.f % 64) return false;
    if (c.has_shared && c.shared_f % 64) return false;
    return encode_tiled_fn() != nullptr;
}

// Called once per handle, after the workspace exists: the activation operands' maps.
cudaError_t umma_prepare(shrike_moe* m) {
    const shrike_moe_config& c = m->cfg;
    Workspace& ws = m->ws;
    if (!ws.xs || !umma_supported(c)) return cudaSuccess;
    // maps[operand][box]: operands xs, acts, xh, acts_shared; boxes of 32, 64, 128, 256 rows
    CUtensorMap* am = (CUtensorMap*)ws.tensor_maps;
    const uint64_t pairs = (uint64_t)c.max_tokens * c.top_k;
    bool ok = true;
    for (int bi = 0; bi < kActBoxes && ok; ++bi) {
        const uint32_t box_rows = 16u << bi;
        ok = make_rows_map(&am[0 * kActBoxes + bi], ws.xs, c.d, pairs, box_rows) &&
             make_rows_map(&am[1 * kActBoxes + bi], ws.acts, c.f, pairs, box_rows);
        if (ok && c.has_shared)
            ok = make_rows_map(&am[2 * kActBoxes + bi], ws.xh, c.d, c.max_tokens, box_rows) &&
                 make_rows_map(&am[3 * kActBoxes + bi], ws.acts_shared, c.shared_f, c.max_tokens, box_rows);
    }
    return ok ? cudaSuccess : cudaErrorInvalidValue;
}

template <int BITS, int GROUP, int META>
static cudaError_t launch_umma_t(cudaStream_t st, const ExpertArgs& a, const ChunkInstance* inst,
                                 const uint32_t* n_inst, uint32_t max_inst, const UmmaMaps& m0, const UmmaMaps& m1) {
    auto k0 = umma_expert_kernel<BITS, GROUP, META, 0>;
    auto k1 = umma_expert_kernel<BITS, GROUP, META, 1>;
    cudaError_t e = cudaFuncSetAttribute(k0, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kUmmaSmemBytes);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kUmmaSmemBytes);
    if (e != cudaSuccess) return e;
    const uint32_t fmax = a.f_shared > a.f ? a.f_shared : a.f;
    k0<<<dim3((fmax + 127) / 128, max_inst), kUmmaThreads, kUmmaSmemBytes, st>>>(a, inst, n_inst, m0);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    k1<<<dim3((a.d + 255) / 256, max_inst), kUmmaThreads, kUmmaSmemBytes, st>>>(a, inst, n_inst, m1);
    return cudaGetLastError();
}

uint32_t umma_max_chunk_instances(const shrike_moe_config& c, uint32_t T) {
    const uint32_t pairs = T * c.top_k;
    uint32_t routed = c.num_experts + pairs / kUmmaMaxN;
    if (routed > pairs) routed = pairs;
    return routed + (c.has_shared ? (T + kUmmaMaxN - 1) / kUmmaMaxN : 0);
}

size_t umma_chunk_instance_bytes() { return sizeof(ChunkInstance); }
size_t umma_tensor_map_bytes() { return 4 * kActBoxes * sizeof(CUtensorMap); }

// Gate/up + GLU, then down, for the instances built from the grouping the
// prefill plan left in the workspace.
cudaError_t launch_umma_prefill(const shrike_moe* m, cudaStream_t st, const ExpertArgs& a, uint32_t T,
                                uint32_t pool_cells) {
    const shrike_moe_config& c = m->cfg;
    const Workspace& ws = m->ws;
    const CUtensorMap* am = (const CUtensorMap*)ws.tensor_maps;
    if (!am || !umma_supported(c)) return cudaErrorNotSupported;
    // descriptors of this call's pool and shared block (host work only)
    UmmaMaps maps[2];
    for (int phase = 0; phase < 2; ++phase) {
        UmmaMaps& mp = maps[phase];
        memset(&mp, 0, sizeof mp);
        const uint32_t kdim = phase == 0 ? c.d : c.f, rows = phase == 0 ? c.f : c.d;
        uint32_t left = a.pool.cells;
        for (uint32_t ch = 0; ch < SHRIKE_MAX_POOL_CHUNKS && a.pool.base[ch] && left; ++ch) {
            const uint32_t cells = left < a.pool.cells_per_chunk ? left : a.pool.cells_per_chunk;
            if (!make_weight_maps(&mp.routed[ch], a.pool.base[ch], a.routed, phase, kdim, rows, c.weight_bits,
                                  c.group_size, cells, a.pool.stride))
                return cudaErrorInvalidValue;
            left -= cells;
        }
        for (int bi = 0; bi < kActBoxes; ++bi) mp.act_routed[bi] = am[phase * kActBoxes + bi];
        if (c.has_shared) {
            const uint32_t kds = phase == 0 ? c.d : c.shared_f, rws = phase == 0 ? c.shared_f : c.d;
            if (!make_weight_maps(&mp.shared, a.shared_block, a.shared, phase, kds, rws, c.weight_bits, c.group_size, 1,
                                  16))
                return cudaErrorInvalidValue;
            for (int bi = 0; bi < kActBoxes; ++bi) mp.act_shared[bi] = am[(2 + phase) * kActBoxes + bi];
        } else {
            mp.shared = mp.routed[0];
            for (int bi = 0; bi < kActBoxes; ++bi) mp.act_shared[bi] = mp.act_routed[bi];
        }
    }
    ChunkInstance* inst = (ChunkInstance*)ws.chunk_inst;
    const uint32_t max_inst = umma_max_chunk_instances(c, T);
    chunk_instances_kernel<<<1, 256, 0, st>>>(ws.expert_offsets, ws.expert_counts, ws.slot_of_expert, c.num_experts, T,
                                              c.has_shared, pool_cells, inst, ws.n_chunk_inst, ws.status);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    gather_sorted_rows_kernel<<<T * c.top_k, 128, 0, st>>>(ws.xh, ws.sorted, ws.n_chunk_inst, c.top_k, c.d, ws.xs);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    const uint32_t bits = c.weight_bits, grp = c.group_size;
    const bool f16 = c.meta_dtype == SHRIKE_DTYPE_FP16;
#define SHRIKE_UMMA(B, G, M) \
    return launch_umma_t<B, G, M>(st, a, inst, ws.n_chunk_inst, max_inst, maps[0], maps[1])
    if (bits == 4 && grp == 64 && !f16) SHRIKE_UMMA(4, 64, SHRIKE_DTYPE_BF16);
    if (bits == 4 && grp == 64 && f16) SHRIKE_UMMA(4, 64, SHRIKE_DTYPE_FP16);
    if (bits == 4 && grp == 32 && !f16) SHRIKE_UMMA(4, 32, SHRIKE_DTYPE_BF16);
    if (bits == 4 && grp == 32 && f16) SHRIKE_UMMA(4, 32, SHRIKE_DTYPE_FP16);
    if (bits == 8 && grp == 64 && !f16) SHRIKE_UMMA(8, 64, SHRIKE_DTYPE_BF16);
    if (bits == 8 && grp == 64 && f16) SHRIKE_UMMA(8, 64, SHRIKE_DTYPE_FP16);
    if (bits == 8 && grp == 32 && !f16) SHRIKE_UMMA(8, 32, SHRIKE_DTYPE_BF16);
    if (bits == 8 && grp == 32 && f16) SHRIKE_UMMA(8, 32, SHRIKE_DTYPE_FP16);
#undef SHRIKE_UMMA
    return cudaErrorInvalidValue;
}

}  // namespace shrike
