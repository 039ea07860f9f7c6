// Shared between the two aligned-writer kernels (warp-MMA and tcgen05).
#pragma once

#include "tq_common.cuh"

namespace tq {

constexpr long long kIngestWaitBudget = 2000000000LL;   // clock cycles, about a second

struct IngestParams {
    const void* key;
    const void* value;
    uint8_t* key_cache;
    uint8_t* value_cache;
    float* scale_cache;
    const int32_t* slots;
    const void* signs;
    uint32_t sign_source;
    uint32_t num_strips, H, S, P;
    uint32_t chunks;                 // num_strips * 2 * H, below 2^31
    uint32_t div_mul, div_shift;     // exact division by 2H: see fast_div
    uint32_t page_mul, page_shift;   // exact division by S (the tcgen05 writer's slot -> page)
    float inv_sqrt_len;
    uint32_t* status;
    // ragged requests (the varlen entry only): request b owns tokens cu_seqlens[b] ..
    // cu_seqlens[b+1] and strips strip_begin[b] .. strip_begin[b+1]
    const int32_t* cu_seqlens = nullptr;
    const int32_t* strip_begin = nullptr;
    uint32_t num_requests = 0;
    // tcgen05 writer: clock cycles one wait on a tile fetch or on a product may take before the
    // kernel reports TQ_STATUS_WAIT_EXPIRED and stops storing; zero gives up without looking
    long long wait_budget = kIngestWaitBudget;
};

// The tcgen05 writer for head size 128 (tq_ingest_umma.cu). `bf16` selects the element type.
cudaError_t launch_ingest_umma(cudaStream_t stream, const IngestParams& p, bool bf16);

}  // namespace tq
