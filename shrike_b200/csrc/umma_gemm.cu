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
//   warps 0-7  producers: each thread owns one weight row; per 64-wide K block
//              it turns the packed nibbles/bytes into fp16 (q - Z) * scale +
//              (bias + Z*scale) -- the reference's half(fma(q, scale, bias)),
//              tensorops.metal:106 -- and writes them, 16 bytes at a time, into
//              the K-major 128-byte-swizzled shared-memory tile the MMA reads.
//              Thread 0 also starts the TMA copy of the K block's activation
//              tile (a 64 x 256 box of the expert-sorted fp16 rows, landing in
//              the same swizzled layout). After the K loop the same warps run
//              the epilogue.
//   warp 8     one thread issues tcgen05.mma (M 128, N = rows, K 16, fp16 in,
//              fp32 accumulate in TMEM) for both tiles and commits to the
//              stage's mbarrier.
//
// PHASE 0: tile 0 = 128 gate rows, tile 1 = the matching 128 up rows; epilogue
//          GLU -> fp16 activations in operand layout, one row per sorted pair.
// PHASE 1: tiles = 256 consecutive down rows; epilogue (+ additive bias) -> one
//          fp32 partial row per (row, rank) pair for the weighted combine.
//
// Every wait is bounded; a wait that gives up sets the status word and the
// block falls through to the TMEM release.
#include <cuda.h>

#include <type_traits>

#include "internal.h"

namespace shrike {

constexpr uint32_t kUmmaStages = 3;
constexpr uint32_t kUmmaMaxN = 256;
constexpr uint32_t kUmmaProducers = 256;
constexpr uint32_t kUmmaThreads = kUmmaProducers + 32;
constexpr uint32_t kTileBytes = 128 * 128;              // 128 rows x 64 fp16, one swizzle-128B K block
constexpr uint32_t kBTileBytes = kUmmaMaxN * 128;       // 256 rows x 64 fp16
constexpr uint32_t kStageBytes = 2 * kTileBytes + kBTileBytes;
static_assert(kUmmaStages == 3, "the producers' register buffers double as the stage index");

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
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t h = hsub2_u32(lop3_and_or(w >> (4 * j), 0x000F000Fu, 0x64006400u), 0x64086408u);
            asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(out[j]) : "r"(h), "r"(s2), "r"(z2));
        }
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

// 2-D tiled TMA load (no multicast): box origin (x = element column, y = row).
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* map, int32_t x, int32_t y,
                                            uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_dst), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}

struct ChunkInstance {  // up to 256 rows that share one expert block
    uint32_t kind, slot, first, count;
};

// grid (row tiles, max chunk instances); block 288.
template <int BITS, int GROUP, int META, int PHASE>
__global__ void __launch_bounds__(kUmmaThreads, 1)
umma_expert_kernel(const ExpertArgs a, const ChunkInstance* __restrict__ inst, const uint32_t* __restrict__ n_inst,
                   float* __restrict__ partials, float* __restrict__ partial_shared,
                   const __grid_constant__ CUtensorMap tm_routed, const __grid_constant__ CUtensorMap tm_shared) {
    constexpr uint32_t kRowBlockBytes = 64 * BITS / 8;  // packed bytes of one row per K block (32 or 64)
    constexpr uint32_t kWordsPerBlock = kRowBlockBytes / 4;
    constexpr uint32_t kGroupsPerBlock = 64 / GROUP;    // 1 (g64) or 2 (g32)
    constexpr float kZero = BITS == 4 ? 8.0f : 128.0f;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
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
    const CUtensorMap* tmap = shared ? &tm_shared : &tm_routed;
    const uint32_t G = kdim / GROUP;
    const uint32_t KB = kdim / 64;
    const uint32_t row_bytes = kdim * BITS / 8;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t N = (in.count + 15u) & ~15u;           // MMA N: rows padded to 16
    uint32_t ncols = 32;                                   // TMEM columns of one accumulator
    while (ncols < N) ncols <<= 1;

    // shared memory (1024-byte aligned): stages x [A0 16 KB][A1 16 KB][B 32 KB] | barriers | row ids | tmem slot
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
    uint64_t* full = (uint64_t*)(smem + kUmmaStages * kStageBytes);
    uint64_t* empty = full + kUmmaStages;
    uint64_t* accum = empty + kUmmaStages;
    uint32_t* rowid = (uint32_t*)(accum + 1);   // output row of column n: pair id (routed) or row (shared)
    uint32_t* tmem_slot = rowid + kUmmaMaxN;
    __shared__ uint32_t s_failed;

    if (tid == 0) {
        for (uint32_t s = 0; s < kUmmaStages; ++s) {
            mbar_init(&full[s], kUmmaProducers + 1);   // every producer + the expect_tx arrival of the TMA copy
            mbar_init(&empty[s], 1);
        }
        mbar_init(accum, 1);
        fence_mbar_init();
        s_failed = 0;
    }
    if (PHASE == 1) {
        for (uint32_t n = tid; n < kUmmaMaxN; n += kUmmaThreads) {
            const uint32_t src = n < in.count ? n : 0;
            rowid[n] = shared ? in.first + src : a.sorted[in.first + src];
        }
    }
    if (warp == 8) tmem_alloc(smem_u32(tmem_slot), 2 * ncols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < 8) {
        // ---------------- producers ----------------
        const uint32_t tile = tid >> 7, r = tid & 127;   // A tile and row inside it
        uint32_t mrow;                                    // row of the weight matrix, which matrix
        int mat;
        if (PHASE == 0) { mat = (int)tile; mrow = r0 + r; } else { mat = 2; mrow = r0 + tid; }
        const bool row_ok = mrow < out_rows;
        const uint8_t* wrow = base + off.w[mat] + (size_t)(row_ok ? mrow : 0) * row_bytes;
        const uint16_t* srow = (const uint16_t*)(base + off.s[mat]) + (size_t)(row_ok ? mrow : 0) * G;
        const uint16_t* brow_meta = (const uint16_t*)(base + off.b[mat]) + (size_t)(row_ok ? mrow : 0) * G;

        uint32_t pk[3][kWordsPerBlock];
        uint16_t sraw[3][kGroupsPerBlock], braw[3][kGroupsPerBlock];
        // three register buffers, indexed at compile time so that they stay in registers
        auto fetch = [&](uint32_t kb, auto bufc) {
            constexpr int buf = decltype(bufc)::value;
            const uint4* p = (const uint4*)(wrow + (size_t)kb * kRowBlockBytes);
#pragma unroll
            for (uint32_t q = 0; q < kWordsPerBlock / 4; ++q) {
                const uint4 v = ldg_stream_u128(p + q);
                pk[buf][4 * q] = v.x; pk[buf][4 * q + 1] = v.y; pk[buf][4 * q + 2] = v.z; pk[buf][4 * q + 3] = v.w;
            }
#pragma unroll
            for (uint32_t gq = 0; gq < kGroupsPerBlock; ++gq) {
                sraw[buf][gq] = __ldg(srow + kb * kGroupsPerBlock + gq);
                braw[buf][gq] = __ldg(brow_meta + kb * kGroupsPerBlock + gq);
            }
        };
        auto step = [&](uint32_t kb, auto bufc) {
            constexpr int buf = decltype(bufc)::value;     // also the pipeline stage: kb % 3
            if (kb + 2 < KB) fetch(kb + 2, std::integral_constant<int, (buf + 2) % 3>{});
            if (kb >= kUmmaStages && !mbar_wait_bounded(&empty[buf], ((kb / kUmmaStages) - 1) & 1)) {
                report_status(a.status, kStatusWaitTimeout);
                s_failed = 1;
            }
            uint8_t* a_tile = smem + buf * kStageBytes + tile * kTileBytes;
            if (tid == 0) {
                mbar_expect_tx(&full[buf], kBTileBytes);
                tma_load_2d(smem_base + buf * kStageBytes + 2 * kTileBytes, tmap, (int32_t)(kb * 64), (int32_t)in.first,
                            &full[buf]);
            }
            uint32_t sz[kGroupsPerBlock][2];
#pragma unroll
            for (uint32_t gq = 0; gq < kGroupsPerBlock; ++gq) {
                const float s = meta_to_f32<META>(sraw[buf][gq]);
                const float z = fmaf(kZero, s, meta_to_f32<META>(braw[buf][gq]));
                sz[gq][0] = row_ok ? half2_dup(s) : 0u;
                sz[gq][1] = row_ok ? half2_dup(z) : 0u;
            }
            // A row r: 8 chunks of 8 fp16; chunk c lives at chunk position c ^ (r & 7)
#pragma unroll
            for (uint32_t w = 0; w < kWordsPerBlock; ++w) {
                constexpr uint32_t kPerWord = BITS == 4 ? 8 : 4;           // weights per packed word
                const uint32_t gq = (w * kPerWord) / GROUP;                // group of this word inside the K block
                uint32_t o[4];
                dequant_word<BITS>(pk[buf][w], sz[gq][0], sz[gq][1], o);
                if constexpr (BITS == 4) {
                    *(uint4*)(a_tile + r * 128 + ((w ^ (r & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                } else {
                    // two words make one 16-byte chunk
                    uint2* dst = (uint2*)(a_tile + r * 128 + (((w >> 1) ^ (r & 7)) << 4)) + (w & 1);
                    *dst = make_uint2(o[0], o[1]);
                }
            }
            fence_async_smem();
            mbar_arrive(&full[buf]);
        };
        fetch(0, std::integral_constant<int, 0>{});
        if (KB > 1) fetch(1, std::integral_constant<int, 1>{});
        for (uint32_t kb = 0; kb < KB; kb += 3) {
            if (*(volatile uint32_t*)&s_failed) break;
            step(kb, std::integral_constant<int, 0>{});
            if (kb + 1 < KB) step(kb + 1, std::integral_constant<int, 1>{});
            if (kb + 2 < KB) step(kb + 2, std::integral_constant<int, 2>{});
        }
    } else if (lane == 0) {
        // ---------------- MMA issue ----------------
        const uint32_t idesc = umma_idesc(N);
        for (uint32_t kb = 0; kb < KB; ++kb) {
            const uint32_t s = kb % kUmmaStages;
            if (!mbar_wait_bounded(&full[s], (kb / kUmmaStages) & 1)) {
                report_status(a.status, kStatusWaitTimeout);
                s_failed = 1;
                break;
            }
            tc_fence_after();
            const uint32_t a_addr = smem_base + s * kStageBytes;
            const uint64_t da0 = umma_smem_desc(a_addr), da1 = umma_smem_desc(a_addr + kTileBytes);
            const uint64_t db = umma_smem_desc(a_addr + 2 * kTileBytes);
#pragma unroll
            for (uint32_t k = 0; k < 4; ++k)  // 4 x K16 per 64-wide block: 32 bytes further along the row
                umma_f16(tmem_base, da0 + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
#pragma unroll
            for (uint32_t k = 0; k < 4; ++k)
                umma_f16(tmem_base + ncols, da1 + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
            umma_commit(&empty[s]);
        }
        umma_commit(accum);
    }

    // ---------------- epilogue (warp w: TMEM lanes 32*(w & 3) .. +31, every other 16-column group) ----------------
    if (warp < 8) {
        bool ok = mbar_wait_bounded(accum, 0);
        if (!ok) report_status(a.status, kStatusWaitTimeout);
        if (*(volatile uint32_t*)&s_failed) ok = false;
        tc_fence_after();
        const uint32_t q = warp & 3, h = warp >> 2;
        const uint32_t trow = q * 32 + lane;                       // row inside each 128-row tile
        const uint32_t taddr = tmem_base + ((q * 32) << 16);
        if (PHASE == 0) {
            const uint32_t f = r0 + trow;
            const bool f_ok = f < F;
            float gab = 0.f, uab = 0.f;
            if (a.expert_bias && f_ok) {
                gab = bf16_bits_to_f32(((const uint16_t*)(base + off.ab[0]))[f]);
                uab = bf16_bits_to_f32(((const uint16_t*)(base + off.ab[1]))[f]);
            }
            uint16_t* dst = (shared ? a.acts_shared : a.acts) + (size_t)in.first * F + perm_index(f, BITS == 4);
            for (uint32_t c0 = h * 16; c0 < N; c0 += 32) {
                uint32_t g[16], u[16];
                tmem_ld16_issue(taddr + c0, g);
                tmem_ld16_issue(taddr + ncols + c0, u);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float v = glu(__uint_as_float(g[j]) + gab, __uint_as_float(u[j]) + uab, a.activation);
                    if (ok && f_ok && c0 + j < in.count) dst[(size_t)(c0 + j) * F] = __half_as_ushort(__float2half_rn(v));
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
            float* out = shared ? partial_shared : partials;
            for (uint32_t c0 = h * 16; c0 < N; c0 += 32) {
                uint32_t v0[16], v1[16];
                tmem_ld16_issue(taddr + c0, v0);
                tmem_ld16_issue(taddr + ncols + c0, v1);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    if (ok && c0 + j < in.count) {
                        float* o = out + (size_t)rowid[c0 + j] * a.d;
                        if (d0 < a.d) o[d0] = __uint_as_float(v0[j]) + ab0;
                        if (d1 < a.d) o[d1] = __uint_as_float(v1[j]) + ab1;
                    }
                }
            }
        }
    }
    if (*(volatile uint32_t*)&s_failed && tid == 0) {
        // a copy of this block may still be in flight: give it a bounded time to land
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
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
    base += inc - n;
    for (uint32_t j = 0; j < n; ++j) {
        ChunkInstance in;
        in.kind = 0; in.slot = slot; in.first = offsets[e] + kUmmaMaxN * j; in.count = min(kUmmaMaxN, c - kUmmaMaxN * j);
        inst[base + j] = in;
    }
    const uint32_t n_shared = with_shared ? (T + kUmmaMaxN - 1) / kUmmaMaxN : 0;
    for (uint32_t j = threadIdx.x; j < n_shared; j += blockDim.x) {
        ChunkInstance in;
        in.kind = 1; in.slot = 0; in.first = kUmmaMaxN * j; in.count = min(kUmmaMaxN, T - kUmmaMaxN * j);
        inst[total + j] = in;
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

// ---- tensor maps of the activation operands ---------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static cudaError_t make_rows_map(EncodeTiledFn encode, CUtensorMap* map, const uint16_t* base, uint64_t cols,
                                 uint64_t rows) {
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2};             // bytes between rows
    const cuuint32_t box[2] = {64, kUmmaMaxN};            // 64 fp16 = one 128-byte swizzle row, 256 rows
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, (void*)base, dims, strides, box, elem,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// Called once per handle, after the workspace exists. Handles that only decode
// (max_tokens <= 64) have no prefill buffers and no maps.
cudaError_t umma_prepare(shrike_moe* m) {
    const shrike_moe_config& c = m->cfg;
    Workspace& ws = m->ws;
    if (!ws.xs) return cudaSuccess;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess) return e;
    if (!fn || qres != cudaDriverEntryPointSuccess) return cudaErrorNotSupported;
    EncodeTiledFn encode = (EncodeTiledFn)fn;
    CUtensorMap* maps = (CUtensorMap*)ws.tensor_maps;
    const uint64_t pairs = (uint64_t)c.max_tokens * c.top_k;
    if ((e = make_rows_map(encode, &maps[0], ws.xs, c.d, pairs)) != cudaSuccess) return e;
    if ((e = make_rows_map(encode, &maps[1], ws.acts, c.f, pairs)) != cudaSuccess) return e;
    if (c.has_shared) {
        if ((e = make_rows_map(encode, &maps[2], ws.xh, c.d, c.max_tokens)) != cudaSuccess) return e;
        if ((e = make_rows_map(encode, &maps[3], ws.acts_shared, c.shared_f, c.max_tokens)) != cudaSuccess) return e;
    } else {
        maps[2] = maps[0];
        maps[3] = maps[1];
    }
    return cudaSuccess;
}

template <int BITS, int GROUP, int META>
static cudaError_t launch_umma_t(cudaStream_t st, const ExpertArgs& a, const ChunkInstance* inst,
                                 const uint32_t* n_inst, uint32_t max_inst, float* partials, float* partial_shared,
                                 const CUtensorMap* maps) {
    const uint32_t smem = kUmmaStages * kStageBytes + 1024 /*alignment slack*/ + (2 * kUmmaStages + 1) * 8 +
                          kUmmaMaxN * 4 + 16;
    auto k0 = umma_expert_kernel<BITS, GROUP, META, 0>;
    auto k1 = umma_expert_kernel<BITS, GROUP, META, 1>;
    cudaError_t e = cudaFuncSetAttribute(k0, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    const uint32_t fmax = a.f_shared > a.f ? a.f_shared : a.f;
    k0<<<dim3((fmax + 127) / 128, max_inst), kUmmaThreads, smem, st>>>(a, inst, n_inst, partials, partial_shared,
                                                                     maps[0], maps[2]);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    k1<<<dim3((a.d + 255) / 256, max_inst), kUmmaThreads, smem, st>>>(a, inst, n_inst, partials, partial_shared,
                                                                    maps[1], maps[3]);
    return cudaGetLastError();
}

uint32_t umma_max_chunk_instances(const shrike_moe_config& c, uint32_t T) {
    const uint32_t pairs = T * c.top_k;
    uint32_t routed = c.num_experts + pairs / kUmmaMaxN;
    if (routed > pairs) routed = pairs;
    return routed + (c.has_shared ? (T + kUmmaMaxN - 1) / kUmmaMaxN : 0);
}

size_t umma_chunk_instance_bytes() { return sizeof(ChunkInstance); }
size_t umma_tensor_map_bytes() { return 4 * sizeof(CUtensorMap); }

// Gate/up + GLU, then down, for the instances built from the grouping the
// prefill plan left in the workspace.
cudaError_t launch_umma_prefill(const shrike_moe* m, cudaStream_t st, const ExpertArgs& a, uint32_t T,
                                uint32_t pool_cells, float* partials, float* partial_shared) {
    const shrike_moe_config& c = m->cfg;
    const Workspace& ws = m->ws;
    ChunkInstance* inst = (ChunkInstance*)ws.chunk_inst;
    const uint32_t max_inst = umma_max_chunk_instances(c, T);
    chunk_instances_kernel<<<1, 256, 0, st>>>(ws.expert_offsets, ws.expert_counts, ws.slot_of_expert, c.num_experts, T,
                                              c.has_shared, pool_cells, inst, ws.n_chunk_inst, ws.status);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    gather_sorted_rows_kernel<<<T * c.top_k, 128, 0, st>>>(ws.xh, ws.sorted, ws.n_chunk_inst, c.top_k, c.d, ws.xs);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    const CUtensorMap* maps = (const CUtensorMap*)ws.tensor_maps;
    if (!maps) return cudaErrorInvalidValue;
    const uint32_t bits = c.weight_bits, grp = c.group_size;
    const bool f16 = c.meta_dtype == SHRIKE_DTYPE_FP16;
#define SHRIKE_UMMA(B, G, M) return launch_umma_t<B, G, M>(st, a, inst, ws.n_chunk_inst, max_inst, partials, partial_shared, maps)
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
