// C++ host-side mirror of the reference's MoE dispatch surface over the C ABI.
//
// The reference's host is Swift (sources/Shrike/Kernels/MoE/MoE.swift,
// sources/Shrike/Kernels/Prefill/MoE, sources/Shrike/Infrastructure/Streaming).
// These classes keep its names, argument meaning and error behaviour (shape and
// resource errors throw, like the Swift wrappers' `throw`) so that a runner
// written against `MoE.encodeRouter`, `encodeResidencyClassification`,
// `encodeSpecPhase1U16Load`, `encodeSpecPhase2Reduce` reads the same here.
// Header only; link with libshrike_b200.so.
#pragma once

#include <cstdint>
#include <stdexcept>
#include <string>

#include "../../include/shrike_b200.h"

namespace shrike_host {

struct Error : std::runtime_error {
    int code;
    Error(int c, const std::string& what) : std::runtime_error(what), code(c) {}
};

inline void check(int rc, const shrike_moe* handle) {
    if (rc != SHRIKE_OK) throw Error(rc, shrike_last_error(handle));
}

/// `MoEExpertOffsets` (MoE.swift:4-39) from the shapes alone, as
/// `CPUExpertFFN.Offsets(d:f:)` does (CPUExpertFFN.swift:34-61).
inline shrike_expert_offsets makeExpertOffsets(const shrike_moe_config& config, bool shared, uint64_t* blockBytes) {
    shrike_expert_offsets o{};
    check(shrike_expert_offsets_make(&config, shared ? 1 : 0, &o, blockBytes), nullptr);
    return o;
}

class MoE;

/// `ExpertCellArena` (ExpertCellArena.swift:16-132): whole experts in HBM cells.
class ExpertCellArena {
public:
    ExpertCellArena(MoE& moe, uint32_t cells, uint64_t cellStride, uint32_t chunks = 1);
    ~ExpertCellArena() { shrike_pool_destroy(pool_); }
    ExpertCellArena(const ExpertCellArena&) = delete;
    ExpertCellArena& operator=(const ExpertCellArena&) = delete;

    void upload(uint32_t cell, const void* blockHost, uint64_t bytes, void* stream = nullptr);
    void fillSynthetic(uint32_t firstCell, uint32_t count, uint64_t seed, uint32_t layer, uint32_t firstExpert = 0,
                       bool shared = false, void* stream = nullptr);
    void* cellAddress(uint32_t cell) const;
    shrike_pool* raw() const { return pool_; }

private:
    MoE& moe_;
    shrike_pool* pool_ = nullptr;
};

/// `final class MoE` (MoE.swift:41-1071) plus the prefill wrappers.
class MoE {
public:
    explicit MoE(const shrike_moe_config& config, int device = 0) : config_(config) {
        check(shrike_moe_create(&config, device, &handle_), nullptr);
    }
    ~MoE() { shrike_moe_destroy(handle_); }
    MoE(const MoE&) = delete;
    MoE& operator=(const MoE&) = delete;

    const shrike_moe_config& config() const { return config_; }
    shrike_moe* raw() const { return handle_; }

    /// ExpertResidencyTable: one {slot, state} word per (layer, expert).
    uint64_t* createResidency(uint32_t layers) {
        uint64_t* table = nullptr;
        check(shrike_residency_create(handle_, layers, &table), handle_);
        table_ = table;
        return table;
    }
    const uint64_t* residencyRow(uint32_t layer) const { return table_ + (size_t)layer * config_.num_experts; }
    void residencySet(uint32_t layer, uint32_t expert, uint32_t slot, uint32_t state, void* stream = nullptr) {
        check(shrike_residency_set(handle_, layer, expert, slot, state, stream), handle_);
    }
    void residencySetLayerIdentity(uint32_t layer, uint32_t firstCell, void* stream = nullptr) {
        check(shrike_residency_set_layer_identity(handle_, layer, firstCell, stream), handle_);
    }

    /// MoE.encodeRouter (MoE.swift:249-316) / PrefillRouter.encodeBlock (PrefillRouter.swift:75-152).
    void encodeRouter(void* stream, const shrike_router_operands& operands, const void* hidden, uint32_t queryCount,
                      uint32_t hiddenStrideElements, uint32_t* outIndices, float* outWeights, float* outSharedGate) {
        check(shrike_encode_router(handle_, stream, &operands, hidden, queryCount, hiddenStrideElements, outIndices,
                                   outWeights, outSharedGate), handle_);
    }

    /// MoE.encodeResidencyClassification (MoE.swift:552-613).
    void encodeResidencyClassification(void* stream, const uint32_t* topKIndices, uint32_t layer, uint32_t queryCount,
                                       uint32_t* resolvedSlots, uint32_t* counts = nullptr,
                                       uint32_t* missPositions = nullptr, uint32_t* missExperts = nullptr) {
        check(shrike_encode_residency_classification(handle_, stream, topKIndices, residencyRow(layer), queryCount,
                                                     resolvedSlots, counts, missPositions, missExperts), handle_);
    }

    /// The slot lookup at the head of the spec kernels, for the rows of one call.
    void encodeDecodePlan(void* stream, const ExpertCellArena& pool, const uint32_t* resolvedSlots, const void* x,
                          uint32_t queryCount, const uint32_t* ioStatus = nullptr) {
        check(shrike_encode_decode_plan(handle_, stream, pool.raw(), resolvedSlots, x, queryCount, ioStatus), handle_);
    }

    /// MoE.encodeSpecPhase1U16Load (MoE.swift:906-948) + the shared expert's gate/up.
    void encodeSpecPhase1(void* stream, const ExpertCellArena& pool, const shrike_expert_offsets& routedOffsets,
                          const shrike_shared_expert* shared, uint32_t queryCount) {
        check(shrike_encode_phase1(handle_, stream, pool.raw(), &routedOffsets, shared, queryCount), handle_);
    }

    /// MoE.encodeSpecPhase2Reduce (MoE.swift:992-1049) + the shared expert's down projection.
    void encodeSpecPhase2Reduce(void* stream, const ExpertCellArena& pool, const shrike_expert_offsets& routedOffsets,
                                const float* routingWeights, const shrike_shared_expert* shared,
                                const float* sharedGate, uint32_t queryCount, void* y, void* hidden) {
        check(shrike_encode_phase2_reduce(handle_, stream, pool.raw(), &routedOffsets, routingWeights, shared,
                                          sharedGate, queryCount, y, hidden), handle_);
    }

    /// encodeSpeculativeRouted (RealForwardRunner.swift:5520-5572) with the router of the tail stage in front.
    void encodeDecodeLayer(void* stream, const ExpertCellArena& pool, const shrike_expert_offsets& routedOffsets,
                           uint32_t layer, const shrike_router_operands& router, const shrike_shared_expert* shared,
                           const void* x, uint32_t queryCount, void* y, void* hidden, uint32_t* outIndices = nullptr,
                           float* outWeights = nullptr, const uint32_t* ioStatus = nullptr) {
        check(shrike_encode_decode_layer(handle_, stream, pool.raw(), &routedOffsets, residencyRow(layer), &router,
                                         shared, x, queryCount, ioStatus, outIndices, outWeights, y, hidden), handle_);
    }

    /// encodeRoutedMoEPrefill's expert work (RealForwardRunner.swift:4552-4665).
    void encodePrefill(void* stream, const ExpertCellArena& pool, const shrike_expert_offsets& routedOffsets,
                       const uint32_t* topKIndices, const uint32_t* resolvedSlots, const float* routingWeights,
                       const void* x, uint32_t queryCount, const shrike_shared_expert* shared, const float* sharedGate,
                       void* y, void* hidden) {
        check(shrike_encode_moe_prefill(handle_, stream, pool.raw(), &routedOffsets, topKIndices, resolvedSlots,
                                        routingWeights, x, queryCount, shared, sharedGate, y, hidden), handle_);
    }

    /// Synchronises and throws if the device reported a failure (commandBuffer.error in the reference).
    void status(void* stream = nullptr) { check(shrike_moe_status(handle_, stream), handle_); }

private:
    shrike_moe_config config_;
    shrike_moe* handle_ = nullptr;
    uint64_t* table_ = nullptr;
};

inline ExpertCellArena::ExpertCellArena(MoE& moe, uint32_t cells, uint64_t cellStride, uint32_t chunks) : moe_(moe) {
    check(shrike_pool_create(moe.raw(), cells, cellStride, chunks, &pool_), moe.raw());
}
inline void ExpertCellArena::upload(uint32_t cell, const void* blockHost, uint64_t bytes, void* stream) {
    check(shrike_pool_upload(pool_, cell, blockHost, bytes, stream), moe_.raw());
}
inline void ExpertCellArena::fillSynthetic(uint32_t firstCell, uint32_t count, uint64_t seed, uint32_t layer,
                                           uint32_t firstExpert, bool shared, void* stream) {
    check(shrike_pool_fill_synthetic(moe_.raw(), pool_, firstCell, count, seed, layer, firstExpert, shared ? 1 : 0,
                                     stream), moe_.raw());
}
inline void* ExpertCellArena::cellAddress(uint32_t cell) const {
    void* p = nullptr;
    check(shrike_pool_cell_address(pool_, cell, &p), moe_.raw());
    return p;
}

}  // namespace shrike_host
