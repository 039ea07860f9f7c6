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

// (shared by both aligned writers)
// Eight packed codes from eight rounded values r_e = 1.5 * 2^23 + u_e (u_e = code + 8 in
// 0..16: a value that rounds up to code 8 has yet to be clamped to 7), lowest nibble first.
// The low byte of r_e is u_e. The even and the odd elements are gathered into four bytes
// each; min(u, 15) = (15 u + 15) >> 4 for u <= 16 and no byte of 15 u + 15 exceeds 255, so
// one multiply-add clamps four elements at once and leaves them in the high nibbles; the two
// words interleave into eight nibbles and u -> two's complement flips each nibble's top bit.
__device__ __forceinline__ uint32_t pack8(const float (&r)[8])
{
    const uint32_t e02 = __byte_perm(__float_as_uint(r[0]), __float_as_uint(r[2]), 0x0040);
    const uint32_t e46 = __byte_perm(__float_as_uint(r[4]), __float_as_uint(r[6]), 0x0040);
    const uint32_t o13 = __byte_perm(__float_as_uint(r[1]), __float_as_uint(r[3]), 0x0040);
    const uint32_t o57 = __byte_perm(__float_as_uint(r[5]), __float_as_uint(r[7]), 0x0040);
    const uint32_t even = __byte_perm(e02, e46, 0x5410), odd = __byte_perm(o13, o57, 0x5410);
    const uint32_t ye = even * 15u + 0x0F0F0F0Fu, yo = odd * 15u + 0x0F0F0F0Fu;
    return (((ye >> 4) & 0x0F0F0F0Fu) | (yo & 0xF0F0F0F0u)) ^ 0x88888888u;
}

// The tcgen05 writer for head size 128 (tq_ingest_umma.cu). `bf16` selects the element type.
cudaError_t launch_ingest_umma(cudaStream_t stream, const IngestParams& p, bool bf16);
// The tcgen05 writer for head size 256 (tq_ingest_umma256.cu).
cudaError_t launch_ingest_umma256(cudaStream_t stream, const IngestParams& p, bool bf16);

}  // namespace tq
