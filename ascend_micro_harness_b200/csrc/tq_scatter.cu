// reshape_and_cache, scatter writer: 1..16 bf16 tokens per request at arbitrary
// slots -- the decode-step and prefill-tail writer.
//
// Reference: kernels/ops/turboquant/turboquant_reshape_scatter_aiv.cpp:16-81,:660-730
// and its oracle tests/common/turboquant_scatter_oracle.hpp:185-217,:291-342.
//   * unit of work = (request, kv_head), one warp; the request's tokens are taken
//     in order, so two tokens that share a value byte are written by the same
//     lane in program order;
//   * y = Pi x as the FP32 radix-2 cascade in the oracle's stage order (strides
//     1..16, sign diagonal, strides 32..d/2), so even non-integer rows agree bit
//     for bit with the host model;
//   * absmax == 0 selects scale 1.0 and codes 0; otherwise the power-of-two scale
//     comes from the exponent field of absmax, with no floor at 1;
//   * key: the token's d/2 bytes are written whole. value: nibble-granular
//     read-modify-write inside the 16-token strip, every unowned nibble preserved.
#include "tq_common.cuh"

namespace tq {

struct ScatterParams {
    const uint16_t* key;
    const uint16_t* value;
    uint8_t* key_cache;
    uint8_t* value_cache;
    float* scale_cache;
    const int32_t* slots;
    const float* signs;
    const int32_t* cu_seqlens;
    uint32_t num_requests, H, S, P, item_begin, item_count;
    float inv_sqrt_len;
    uint32_t* status;
};

constexpr int kScatterWarps = 4;

template <int D>
__global__ void __launch_bounds__(kScatterWarps * 32) tq_scatter_kernel(const ScatterParams p)
{
    // a decode launched as this kernel's programmatic dependent may be scheduled from here on
    // (it waits for this grid's completion before it reads the cache)
    asm volatile("griddepcontrol.launch_dependents;\n");
    constexpr int K = D / 32;  // consecutive channels per lane
    const int lane = threadIdx.x & 31;
    const uint32_t warp_global = blockIdx.x * kScatterWarps + (threadIdx.x >> 5);
    const uint32_t warps_total = gridDim.x * kScatterWarps;

    float sgn[K];
#pragma unroll
    for (int i = 0; i < K; ++i) sgn[i] = p.signs[lane * K + i];

    for (uint32_t it = warp_global; it < p.item_count; it += warps_total) {
        const uint32_t item = p.item_begin + it;
        const uint32_t request = item / p.H, head = item % p.H;
        if (request >= p.num_requests) continue;
        const int tok_begin = p.cu_seqlens ? p.cu_seqlens[request] : static_cast<int>(request);
        const int tok_end = p.cu_seqlens ? p.cu_seqlens[request + 1] : static_cast<int>(request) + 1;
        for (int tok = tok_begin; tok < tok_end; ++tok) {
            const int32_t slot = p.slots[tok];
            if (slot < 0) continue;  // a padded token owns nothing
            const uint32_t page = static_cast<uint32_t>(slot) / p.S, tib = static_cast<uint32_t>(slot) % p.S;
            if (page >= p.P) {
                if (lane == 0) report(p.status, TQ_STATUS_BAD_PAGE);
                continue;
            }
            const size_t row = (static_cast<size_t>(tok) * p.H + head) * D + lane * K;
            const size_t head_base = (static_cast<size_t>(page) * p.H + head) * p.S * (D / 2);
            // Everything the token needs from memory is requested up front: both activation
            // rows and the value-strip bytes whose other nibble has to survive.
            uint32_t raw[2][K / 2];
#pragma unroll
            for (int plane = 0; plane < 2; ++plane) {
                const uint16_t* src = (plane == 0 ? p.key : p.value) + row;
                if constexpr (K == 4) {
                    const uint2 w = *reinterpret_cast<const uint2*>(src);
                    raw[plane][0] = w.x;
                    raw[plane][1] = w.y;
                } else {
                    const uint4 w = *reinterpret_cast<const uint4*>(src);
                    raw[plane][0] = w.x;
                    raw[plane][1] = w.y;
                    raw[plane][2] = w.z;
                    raw[plane][3] = w.w;
                }
            }
            uint8_t* strip = p.value_cache + head_base + static_cast<size_t>(tib / kStrip) * (kStrip * D / 2);
            const uint32_t t = tib % kStrip;
            uint32_t old_bytes[K];
#pragma unroll
            for (int i = 0; i < K; ++i) old_bytes[i] = strip[(lane * K + i) * 8 + t / 2];
#pragma unroll
            for (int plane = 0; plane < 2; ++plane) {
                float v[K];
#pragma unroll
                for (int i = 0; i < K / 2; ++i) {
                    v[2 * i] = __uint_as_float(raw[plane][i] << 16);
                    v[2 * i + 1] = __uint_as_float(raw[plane][i] & 0xFFFF0000u);
                }
                cascade_ingress<K>(v, sgn, lane);

                float amax = 0.0f;
#pragma unroll
                for (int i = 0; i < K; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));

                float scale = 1.0f, inv = 0.0f;  // the absmax == 0 branch: codes 0, scale 1
                if (amax != 0.0f) {
                    const int pow_bits = (__float_as_int(amax) & 0x7F800000) - (2 << 23);
                    scale = __int_as_float(pow_bits) * p.inv_sqrt_len;
                    inv = __int_as_float((254 << 23) - pow_bits);
                }
                uint32_t codes = 0;  // K nibbles, channel lane*K + i at bits 4i
#pragma unroll
                for (int i = 0; i < K; ++i) {
                    const int q = __float2int_rn(fminf(v[i] * inv, 7.0f));
                    codes |= (static_cast<uint32_t>(q) & 0xFu) << (4 * i);
                }
                if (plane == 0) {
                    uint8_t* dst = p.key_cache + head_base + static_cast<size_t>(tib) * (D / 2) + lane * (K / 2);
                    if constexpr (K == 4) *reinterpret_cast<uint16_t*>(dst) = static_cast<uint16_t>(codes);
                    else *reinterpret_cast<uint32_t*>(dst) = codes;
                } else {
#pragma unroll
                    for (int i = 0; i < K; ++i) {
                        const uint32_t nib = (codes >> (4 * i)) & 0xFu;
                        const uint32_t old = old_bytes[i];
                        strip[(lane * K + i) * 8 + t / 2] =
                            static_cast<uint8_t>((t & 1u) ? ((old & 0x0Fu) | (nib << 4)) : ((old & 0xF0u) | nib));
                    }
                }
                if (lane == 0)
                    p.scale_cache[((static_cast<size_t>(plane) * p.P + page) * p.H + head) * p.S + tib] = scale;
            }
        }
    }
}

}  // namespace tq

extern "C" int tq_reshape_scatter(void* stream, const uint16_t* key, const uint16_t* value,
                                  int8_t* key_cache, int8_t* value_cache, float* scale_cache,
                                  const int32_t* slot_mapping, const float* pi_signs,
                                  const int32_t* cu_seqlens, uint32_t num_requests,
                                  uint32_t num_kv_heads, uint32_t head_size, uint32_t block_size,
                                  uint32_t num_blocks, uint32_t item_begin, uint32_t item_count,
                                  float inv_sqrt_len, uint32_t* status)
{
    using namespace tq;
    if (!num_kv_heads || !num_blocks || !block_size || block_size % kStrip != 0 ||
        (head_size != 128 && head_size != 256))
        return TQ_ERR_INVALID_ARGUMENT;
    if (num_requests == 0 || item_count == 0) return TQ_OK;
    if (!key || !value || !key_cache || !value_cache || !scale_cache || !slot_mapping || !pi_signs)
        return TQ_ERR_INVALID_ARGUMENT;
    ScatterParams p{key, value, reinterpret_cast<uint8_t*>(key_cache),
                    reinterpret_cast<uint8_t*>(value_cache), scale_cache, slot_mapping, pi_signs,
                    cu_seqlens, num_requests, num_kv_heads, block_size, num_blocks, item_begin,
                    item_count, inv_sqrt_len, status};
    const unsigned blocks = (item_count + kScatterWarps - 1) / kScatterWarps;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (head_size == 128) tq_scatter_kernel<128><<<blocks, kScatterWarps * 32, 0, s>>>(p);
    else tq_scatter_kernel<256><<<blocks, kScatterWarps * 32, 0, s>>>(p);
    return cudaGetLastError() == cudaSuccess ? TQ_OK : TQ_ERR_LAUNCH;
}

// kernels/ops/turboquant/turboquant_reshape_scatter_aiv.cpp:760-773. block_dim
// was the AI-core count to spread items over; the grid is sized from item_count
// here. launch_probe published Ascend block indices for a probe and is unused.
#include <stdexcept>
extern "C" void launch_turboquant_reshape_scatter_aiv(
    void* stream, uint32_t /*block_dim*/, uint16_t* key, uint16_t* value, int8_t* key_cache,
    int8_t* value_cache, float* scale_cache, int32_t* slot_mapping, float* pi_signs,
    int32_t* cu_seqlens, int32_t* /*launch_probe*/, uint32_t num_requests, uint32_t num_kv_heads,
    uint32_t head_size, uint32_t block_size, uint32_t num_blocks, uint32_t item_begin,
    uint32_t item_count, float inv_sqrt_len)
{
    const int st = tq_reshape_scatter(stream, key, value, key_cache, value_cache, scale_cache,
                                      slot_mapping, pi_signs, cu_seqlens, num_requests,
                                      num_kv_heads, head_size, block_size, num_blocks, item_begin,
                                      item_count, inv_sqrt_len, nullptr);
    if (st == TQ_ERR_INVALID_ARGUMENT)
        throw std::invalid_argument("reshape_scatter_aiv: unsupported geometry");
    if (st != TQ_OK) throw std::runtime_error("reshape_scatter_aiv: launch failed");
}
