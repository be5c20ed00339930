// A small C++ host that plays the reference runner's role for one routed layer
// (RealForwardRunner.encodeDecodeTailStage + encodeSpeculativeRouted): it keeps
// the slot table, fills the pool, and encodes router -> classification -> plan ->
// phase 1 -> phase 2, then the same layer through the one-call form, and writes
// both outputs so that a test can compare them with the CPU oracle.
//
//   harness <seed> <rows> <out.bin>
//
// Layer: d 512, f 256, 32 experts top-8, int4 g64, gated shared expert, fp32
// activations. Router rows and activations are read from stdin as raw fp32
// (32*512 + 512 gate + rows*512 values) so that the test controls them.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <vector>

#include "shrike_moe.hpp"

#define CUDA_OK(call)                                                                  \
    do {                                                                               \
        cudaError_t e_ = (call);                                                       \
        if (e_ != cudaSuccess) { std::fprintf(stderr, "%s: %s\n", #call, cudaGetErrorString(e_)); return 2; } \
    } while (0)

int main(int argc, char** argv) {
    if (argc != 4) { std::fprintf(stderr, "usage: harness <seed> <rows> <out.bin>\n"); return 64; }
    const uint64_t seed = std::strtoull(argv[1], nullptr, 10);
    const uint32_t rows = (uint32_t)std::atoi(argv[2]);
    shrike_moe_config cfg{};
    cfg.d = 512; cfg.f = 256; cfg.num_experts = 32; cfg.top_k = 8; cfg.weight_bits = 4; cfg.group_size = 64;
    cfg.meta_dtype = SHRIKE_DTYPE_BF16; cfg.act_dtype = SHRIKE_DTYPE_FP32; cfg.y_dtype = SHRIKE_DTYPE_FP32; cfg.activation = SHRIKE_ACT_SILU;
    cfg.router_kind = SHRIKE_ROUTER_SOFTMAX; cfg.routed_scaling = 1.0f; cfg.round_route_weights_f16 = 1;
    cfg.has_shared = 1; cfg.shared_gated = 1; cfg.shared_f = 256; cfg.max_tokens = 16;
    try {
        const size_t nr = (size_t)cfg.num_experts * cfg.d, nx = (size_t)rows * cfg.d;
        std::vector<float> in(nr + cfg.d + nx);
        if (std::fread(in.data(), sizeof(float), in.size(), stdin) != in.size()) {
            std::fprintf(stderr, "short read on stdin\n");
            return 65;
        }
        shrike_host::MoE moe(cfg, 0);
        uint64_t blockBytes = 0, sharedBytes = 0;
        const shrike_expert_offsets off = shrike_host::makeExpertOffsets(cfg, false, &blockBytes);
        const shrike_expert_offsets soff = shrike_host::makeExpertOffsets(cfg, true, &sharedBytes);
        const uint64_t stride = (blockBytes + 255) / 256 * 256;
        shrike_host::ExpertCellArena pool(moe, cfg.num_experts + 1, stride, 2);
        pool.fillSynthetic(0, cfg.num_experts, seed, 0);
        pool.fillSynthetic(cfg.num_experts, 1, seed, 0, 100000, true);
        moe.createResidency(1);
        moe.residencySetLayerIdentity(0, 0);

        float *dRouter, *dGate, *dX, *dY, *dY2, *dW, *dSg;
        uint32_t *dIds, *dSlots;
        CUDA_OK(cudaMalloc(&dRouter, nr * 4)); CUDA_OK(cudaMalloc(&dGate, cfg.d * 4));
        CUDA_OK(cudaMalloc(&dX, nx * 4)); CUDA_OK(cudaMalloc(&dY, nx * 4)); CUDA_OK(cudaMalloc(&dY2, nx * 4));
        CUDA_OK(cudaMalloc(&dW, rows * cfg.top_k * 4)); CUDA_OK(cudaMalloc(&dSg, rows * 4));
        CUDA_OK(cudaMalloc(&dIds, rows * cfg.top_k * 4)); CUDA_OK(cudaMalloc(&dSlots, rows * cfg.top_k * 4));
        CUDA_OK(cudaMemcpy(dRouter, in.data(), nr * 4, cudaMemcpyHostToDevice));
        CUDA_OK(cudaMemcpy(dGate, in.data() + nr, cfg.d * 4, cudaMemcpyHostToDevice));
        CUDA_OK(cudaMemcpy(dX, in.data() + nr + cfg.d, nx * 4, cudaMemcpyHostToDevice));

        shrike_router_operands router{};
        router.weights = dRouter;
        router.shared_gate = dGate;
        shrike_shared_expert shared{pool.cellAddress(cfg.num_experts), soff};

        // the runner's call order, one encode per stage
        moe.encodeRouter(nullptr, router, dX, rows, cfg.d, dIds, dW, dSg);
        moe.encodeResidencyClassification(nullptr, dIds, 0, rows, dSlots);
        moe.encodeDecodePlan(nullptr, pool, dSlots, dX, rows);
        moe.encodeSpecPhase1(nullptr, pool, off, &shared, rows);
        moe.encodeSpecPhase2Reduce(nullptr, pool, off, dW, &shared, dSg, rows, dY, nullptr);
        // and the one-call form
        moe.encodeDecodeLayer(nullptr, pool, off, 0, router, &shared, dX, rows, dY2, nullptr);
        moe.status();

        std::vector<float> y(nx), y2(nx);
        std::vector<uint32_t> ids(rows * cfg.top_k);
        CUDA_OK(cudaMemcpy(y.data(), dY, nx * 4, cudaMemcpyDeviceToHost));
        CUDA_OK(cudaMemcpy(y2.data(), dY2, nx * 4, cudaMemcpyDeviceToHost));
        CUDA_OK(cudaMemcpy(ids.data(), dIds, ids.size() * 4, cudaMemcpyDeviceToHost));
        FILE* f = std::fopen(argv[3], "wb");
        if (!f) return 66;
        std::fwrite(ids.data(), 4, ids.size(), f);
        std::fwrite(y.data(), 4, y.size(), f);
        std::fwrite(y2.data(), 4, y2.size(), f);
        std::fclose(f);

        // a shape the handle was not built for must throw, not abort
        bool threw = false;
        try {
            moe.encodeRouter(nullptr, router, dX, cfg.max_tokens + 1, cfg.d, dIds, dW, dSg);
        } catch (const shrike_host::Error& e) {
            threw = e.code == SHRIKE_ERANGE;
        }
        if (!threw) { std::fprintf(stderr, "expected SHRIKE_ERANGE\n"); return 3; }
        std::printf("ok rows=%u block=%llu\n", rows, (unsigned long long)blockBytes);
    } catch (const shrike_host::Error& e) {
        std::fprintf(stderr, "shrike error %d: %s\n", e.code, e.what());
        return 1;
    }
    return 0;
}
