// reshape_and_cache, aligned writer: one warp turns one (strip, plane, head)
// panel of 16 tokens x d channels into a packed 4-bit page plus 16 FP32 scales.
//
// What the reference computes per panel (tests/common/turboquant_oracle.hpp:357-449;
// device: kernels/ops/turboquant/turboquant_reshape_and_cache_a8.cpp:714-744,:1083-1226):
//   y = M x,  M = (H_G (x) I32) diag(s) (I_G (x) H32),  G = d/32
//   absmax = max(1, max|y|), 2^e <= absmax < 2^(e+1), scale = 2^(e-2) * inv_sqrt_len
//   q = rint_even(min(y * 2^(2-e), 7)),  two codes per byte, low nibble first
//   key page token-major, value page channel-major inside the strip.
//
// How this kernel computes it:
//   * the 16 x d panel is read straight into MMA A-fragments with 64/128-bit
//     loads; the contraction index of the MMA is permuted so that each thread's
//     contiguous bytes ARE its fragment -- no shared-memory staging on the way in;
//   * the inner factor I_G (x) H32 is the only dense contraction: per 32-channel
//     group, 4 (int8, m16n8k32) or 8 (bf16, m16n8k16) warp MMAs against +-1
//     operands generated from popcount parity. Products of +-1 with int8 / small
//     bf16 integers accumulate exactly in INT32 / FP32;
//   * the MMA's output columns are permuted so each thread ends up with 8
//     consecutive channels of every group: the sign diagonal and the outer
//     H_G factor are then register-local (a log2(G)-stage butterfly), and one
//     thread's 8 codes are one 32-bit word of the key page;
//   * fragment rows r and r+8 carry tokens 2r and 2r+1, so one thread owns both
//     nibbles of every value-page byte it produces;
//   * the scale comes from the exponent field of absmax by integer arithmetic,
//     no division enters; the page is staged in shared memory and leaves as
//     128-bit stores of the whole contiguous (page, head) block.
#include <type_traits>

#include "tq_common.cuh"

namespace tq {

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
    float inv_sqrt_len;
    uint32_t* status;
};

constexpr int kIngestWarps = 4;
constexpr int kIngestCtasPerSm = 3;

template <int D, bool BF16>
struct Panel {
    static constexpr int G = D / kGroup;
    using Vec = typename std::conditional<BF16, uint4, uint2>::type;
    Vec lo[G], hi[G];   // token 2r and token 2r+1, 8 channels per group
    int32_t slot;       // slot of token (lane & 15) of the strip
};

// Issue the loads of one (strip, plane, head) panel: straight into what will be
// the MMA A-fragments.
template <int D, bool BF16>
__device__ __forceinline__ void load_panel(Panel<D, BF16>& f, const IngestParams& p, uint64_t chunk,
                                           int lane)
{
    constexpr int G = D / kGroup;
    using Vec = typename Panel<D, BF16>::Vec;
    using Elem = typename std::conditional<BF16, uint16_t, int8_t>::type;
    const int r = lane >> 2, qd = lane & 3;
    const uint32_t head = static_cast<uint32_t>(chunk % p.H);
    const uint32_t plane = static_cast<uint32_t>((chunk / p.H) & 1u);
    const uint32_t strip = static_cast<uint32_t>(chunk / (2u * p.H));
    const size_t row_pitch = static_cast<size_t>(p.H) * D;  // elements
    const Elem* base = static_cast<const Elem*>(plane == 0 ? p.key : p.value) +
                       (static_cast<size_t>(strip) * kStrip + 2 * r) * row_pitch +
                       static_cast<size_t>(head) * D + qd * 8;
#pragma unroll
    for (int g = 0; g < G; ++g) {
        f.lo[g] = __ldg(reinterpret_cast<const Vec*>(base + g * kGroup));
        f.hi[g] = __ldg(reinterpret_cast<const Vec*>(base + row_pitch + g * kGroup));
    }
    f.slot = __ldg(p.slots + static_cast<size_t>(strip) * kStrip + (lane & 15));
}

// Rotate, quantise, pack and store one panel.
template <int D, bool BF16>
__device__ __forceinline__ void process_panel(const Panel<D, BF16>& f, const IngestParams& p,
                                              uint64_t chunk, int lane,
                                              const uint32_t (&bfrag)[BF16 ? 16 : 8],
                                              const float* sgn_s, uint32_t* stage)
{
    constexpr int G = D / kGroup;
    constexpr int kPageWords = kStrip * D / 8;
    const int r = lane >> 2, qd = lane & 3;
    const uint32_t head = static_cast<uint32_t>(chunk % p.H);
    const uint32_t plane = static_cast<uint32_t>((chunk / p.H) & 1u);

    // ---- the strip's page, from its slots; the contract is checked, not assumed
    // (tests/common/turboquant_oracle.hpp:278-287).
    const int32_t slot0 = __shfl_sync(0xffffffffu, f.slot, 0);
    const bool run_ok = (f.slot == slot0 + (lane & 15));
    const bool strip_ok = __all_sync(0xffffffffu, run_ok) && slot0 >= 0 && (slot0 % kStrip) == 0 &&
                          static_cast<uint32_t>(slot0) / p.S < p.P;
    if (!strip_ok) {
        if (lane == 0) report(p.status, TQ_STATUS_BAD_SLOT);
        return;
    }
    const uint32_t page = static_cast<uint32_t>(slot0) / p.S;
    const uint32_t tok_in_page = static_cast<uint32_t>(slot0) % p.S;

    // y[tt][g][e]: token 2r+tt, channel g*32 + qd*8 + e, as float (exact integers
    // for int8 and integer-valued bf16 inputs).
    float y[2][G][8];
    if constexpr (!BF16) {
        // The INT32 accumulator starts at the bit pattern of 1.5 * 2^23, so what comes
        // out, read as a float, is 12582912 + sum exactly; one FP32 subtract recovers
        // the sum without an integer-to-float conversion.
        constexpr int kBias = 0x4B400000;
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const uint32_t a[4] = {f.lo[g].x, f.hi[g].x, f.lo[g].y, f.hi[g].y};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                int c[4] = {kBias, kBias, kBias, kBias};
                mma_s8_16832(c, a, bfrag[j * 2 + 0], bfrag[j * 2 + 1]);
                y[0][g][j * 2 + 0] = __int_as_float(c[0]) - 12582912.0f;
                y[0][g][j * 2 + 1] = __int_as_float(c[1]) - 12582912.0f;
                y[1][g][j * 2 + 0] = __int_as_float(c[2]) - 12582912.0f;
                y[1][g][j * 2 + 1] = __int_as_float(c[3]) - 12582912.0f;
            }
        }
    } else {
#pragma unroll
        for (int g = 0; g < G; ++g) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float c[4] = {0.f, 0.f, 0.f, 0.f};
                mma_bf16_16816(c, f.lo[g].x, f.hi[g].x, f.lo[g].y, f.hi[g].y, bfrag[j * 2 + 0],
                               bfrag[j * 2 + 1]);
                mma_bf16_16816(c, f.lo[g].z, f.hi[g].z, f.lo[g].w, f.hi[g].w, bfrag[8 + j * 2 + 0],
                               bfrag[8 + j * 2 + 1]);
                y[0][g][j * 2 + 0] = c[0];
                y[0][g][j * 2 + 1] = c[1];
                y[1][g][j * 2 + 0] = c[2];
                y[1][g][j * 2 + 1] = c[3];
            }
        }
    }

    // ---- sign diagonal folded into the first stage of the outer factor H_G, then
    // the remaining stages, per (token, e). All multiplies are by +-1: exact.
    float amax[2] = {1.0f, 1.0f};  // the writer floors absmax at 1
    {
        float sgn[G][8];
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const float4 s0 = *reinterpret_cast<const float4*>(sgn_s + qd * (G * 8) + g * 8);
            const float4 s1 = *reinterpret_cast<const float4*>(sgn_s + qd * (G * 8) + g * 8 + 4);
            sgn[g][0] = s0.x; sgn[g][1] = s0.y; sgn[g][2] = s0.z; sgn[g][3] = s0.w;
            sgn[g][4] = s1.x; sgn[g][5] = s1.y; sgn[g][6] = s1.z; sgn[g][7] = s1.w;
        }
#pragma unroll
        for (int tt = 0; tt < 2; ++tt)
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                float x[G];
#pragma unroll
                for (int g = 0; g < G; g += 2) {
                    const float a = sgn[g][e] * y[tt][g][e];
                    x[g] = fmaf(sgn[g + 1][e], y[tt][g + 1][e], a);
                    x[g + 1] = fmaf(-sgn[g + 1][e], y[tt][g + 1][e], a);
                }
#pragma unroll
                for (int s = 2; s < G; s <<= 1)
#pragma unroll
                    for (int i = 0; i < G; ++i)
                        if ((i & s) == 0) {
                            const float a = x[i], bb = x[i + s];
                            x[i] = a + bb;
                            x[i + s] = a - bb;
                        }
#pragma unroll
                for (int g = 0; g < G; g += 2) {
                    y[tt][g][e] = x[g];
                    y[tt][g + 1][e] = x[g + 1];
                    amax[tt] = fmaxf(amax[tt], fmaxf(fabsf(x[g]), fabsf(x[g + 1])));
                }
            }
    }
#pragma unroll
    for (int tt = 0; tt < 2; ++tt) {
        amax[tt] = fmaxf(amax[tt], __shfl_xor_sync(0xffffffffu, amax[tt], 1));
        amax[tt] = fmaxf(amax[tt], __shfl_xor_sync(0xffffffffu, amax[tt], 2));
    }

    // ---- power-of-two scale from the exponent field
    // (kernels/ops/turboquant/turboquant_reshape_and_cache_a8.cpp:1136-1158).
    float inv[2], pow2[2];
#pragma unroll
    for (int tt = 0; tt < 2; ++tt) {
        const int exp_bits = __float_as_int(amax[tt]) & 0x7F800000;
        const int pow_bits = exp_bits - (2 << 23);
        pow2[tt] = __int_as_float(pow_bits);
        inv[tt] = __int_as_float((254 << 23) - pow_bits);
    }

    // ---- quantise. y * inv is exact (power of two), so one fused multiply-add onto
    // 1.5 * 2^23 + 8 rounds it to nearest-even at integer granularity: the result is
    // 12582912 + u with u = code + 8 in 0..16, and its bit pattern is 0x4B400000 + u;
    // the upper clamp (code 7, u = 15) is a float min. Biased codes pack by integer
    // multiply-add with no masks and no borrows; a final xor with 0x88.. turns u back
    // into the two's-complement nibble.
    constexpr float kMagic = 12582920.0f;           // 1.5 * 2^23 + 8
    constexpr float kMagicTop = 12582927.0f;        // 1.5 * 2^23 + 15
    constexpr uint32_t kMagicBits = 0x4B400000u;    // bits of 1.5 * 2^23
    __syncwarp();  // the previous panel's copy-out has finished reading the stage
    if (plane == 0) {
        // key page: token-major, row of D/8 words; this thread's word is g*4 + qd.
        // Horner over e = 7..0: w = sum (K + u_e) 16^e = K * 0x11111111 + packed.
        constexpr uint32_t kHorner = kMagicBits * 0x11111111u;
#pragma unroll
        for (int tt = 0; tt < 2; ++tt)
#pragma unroll
            for (int g = 0; g < G; ++g) {
                uint32_t w = 0;
#pragma unroll
                for (int e = 7; e >= 0; --e) {
                    const float rr = fminf(fmaf(y[tt][g][e], inv[tt], kMagic), kMagicTop);
                    w = w * 16u + __float_as_uint(rr);
                }
                stage[(2 * r + tt) * (D / 8) + ((g * 4 + qd) ^ (r & 3) * 4)] = (w - kHorner) ^ 0x88888888u;
            }
    } else {
        // value page: byte (channel*8 + r) = u(token 2r) + 16 u(token 2r+1); the store
        // keeps the low byte, to which 17 * 0x4B400000 contributes nothing.
        uint8_t* sb = reinterpret_cast<uint8_t*>(stage);
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float r0 = fminf(fmaf(y[0][g][e], inv[0], kMagic), kMagicTop);
                const float r1 = fminf(fmaf(y[1][g][e], inv[1], kMagic), kMagicTop);
                const uint32_t byte = __float_as_uint(r1) * 16u + __float_as_uint(r0);
                sb[(g * kGroup + qd * 8 + e) * 8 + r] = static_cast<uint8_t>(byte);
            }
    }
    __syncwarp();

    // ---- whole contiguous block out with 128-bit stores.
    uint8_t* cache = plane == 0 ? p.key_cache : p.value_cache;
    const size_t block_bytes = static_cast<size_t>(kStrip) * D / 2;
    uint8_t* dst = cache + (static_cast<size_t>(page) * p.H + head) * (static_cast<size_t>(p.S) * D / 2) +
                   static_cast<size_t>(tok_in_page / kStrip) * block_bytes;
    const uint4* s4 = reinterpret_cast<const uint4*>(stage);
#pragma unroll
    for (int i = 0; i < kPageWords / 4 / 32; ++i) {
        const int unit = i * 32 + lane;  // 16-byte unit of the page
        uint4 v;
        if (plane == 0) {
            // undo the store swizzle: unit = row * (D/32) + chunk, chunk ^= (row/2) & 3
            const int row = unit / (D / 32), chunk16 = unit % (D / 32);
            v = s4[row * (D / 32) + (chunk16 ^ ((row >> 1) & 3))];
        } else {
            v = s4[unit];
            v.x ^= 0x88888888u;  // u -> two's-complement nibble
            v.y ^= 0x88888888u;
            v.z ^= 0x88888888u;
            v.w ^= 0x88888888u;
        }
        __stcs(reinterpret_cast<uint4*>(dst) + unit, v);
    }

    if (qd == 0) {
        const size_t at = ((static_cast<size_t>(plane) * p.P + page) * p.H + head) * p.S +
                          tok_in_page + 2 * r;
        *reinterpret_cast<float2*>(p.scale_cache + at) =
            make_float2(pow2[0] * p.inv_sqrt_len, pow2[1] * p.inv_sqrt_len);
    }
}

// Persistent: every warp walks panels warp_global, warp_global + warps_total, ...
// with the next panel's loads in flight while the current one is processed.
template <int D, bool BF16>
__global__ void __launch_bounds__(kIngestWarps * 32, kIngestCtasPerSm)
tq_ingest_kernel(const IngestParams p)
{
    constexpr int G = D / kGroup;
    constexpr int kPageWords = kStrip * D / 8;
    __shared__ __align__(16) uint32_t stage_all[kIngestWarps][kPageWords];
    __shared__ __align__(16) float sgn_s[4 * G * 8];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = lane >> 2, qd = lane & 3;

    // sign diagonal per quad position: sgn_s[qd][g*8 + e] for channel g*32 + qd*8 + e
    for (int i = threadIdx.x; i < 4 * G * 8; i += blockDim.x) {
        const int q = i / (G * 8), k = i % (G * 8);
        sgn_s[i] = sign_is_negative(p.signs, p.sign_source, (k / 8) * kGroup + q * 8 + (k % 8)) ? -1.0f : 1.0f;
    }

    // +-1 B fragments of H32, once per thread. Column n of tile j is output channel
    // c0 = (n/2)*8 + j*2 + n%2, so a thread ends up with 8 consecutive channels.
    uint32_t bfrag[BF16 ? 16 : 8];
    if constexpr (!BF16) {
        // contraction slot k of the low half is input channel (k/4)*8 + k%4, of the
        // high half (k/4)*8 + 4 + k%4 -- the order the 8-byte loads deliver.
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const unsigned c0 = (r >> 1) * 8 + j * 2 + (r & 1);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t w = 0;
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    w |= (hneg(c0, qd * 8 + h * 4 + e) ? 0xFFu : 0x01u) << (8 * e);
                bfrag[j * 2 + h] = w;
            }
        }
    } else {
        // Two k16 steps per group; step s slot qd'*2+e <-> channel qd'*8 + 4s + e,
        // slot 8+qd'*2+e <-> channel qd'*8 + 4s + 2 + e.
#pragma unroll
        for (int s = 0; s < 2; ++s)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const unsigned c0 = (r >> 1) * 8 + j * 2 + (r & 1);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const unsigned ch = qd * 8 + 4 * s + 2 * h;
                    bfrag[s * 8 + j * 2 + h] = (hneg(c0, ch) ? 0xBF80u : 0x3F80u) |
                                               ((hneg(c0, ch + 1) ? 0xBF80u : 0x3F80u) << 16);
                }
            }
    }
    __syncthreads();

    const uint64_t total = static_cast<uint64_t>(p.num_strips) * 2u * p.H;
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kIngestWarps;
    uint64_t c0 = static_cast<uint64_t>(blockIdx.x) * kIngestWarps + warp;
    uint32_t* stage = stage_all[warp];

    Panel<D, BF16> pa, pb;
    if (c0 < total) load_panel<D, BF16>(pa, p, c0, lane);
    while (c0 < total) {
        const uint64_t c1 = c0 + stride;
        if (c1 < total) load_panel<D, BF16>(pb, p, c1, lane);
        process_panel<D, BF16>(pa, p, c0, lane, bfrag, sgn_s, stage);
        if (c1 >= total) break;
        c0 = c1 + stride;
        if (c0 < total) load_panel<D, BF16>(pa, p, c0, lane);
        process_panel<D, BF16>(pb, p, c1, lane, bfrag, sgn_s, stage);
    }
}

template <int D, bool BF16>
static cudaError_t launch_ingest(cudaStream_t stream, const IngestParams& p)
{
    const uint64_t chunks = static_cast<uint64_t>(p.num_strips) * 2u * p.H;
    uint64_t blocks = (chunks + kIngestWarps - 1) / kIngestWarps;
    if (blocks == 0) return cudaSuccess;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess)
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const uint64_t resident = static_cast<uint64_t>(sms) * kIngestCtasPerSm;
    if (blocks > resident) blocks = resident;  // persistent: one resident wave
    tq_ingest_kernel<D, BF16><<<static_cast<unsigned>(blocks), kIngestWarps * 32, 0, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace tq

extern "C" int tq_reshape_and_cache(void* stream, const void* key, const void* value,
                                    int8_t* key_cache, int8_t* value_cache, float* scale_cache,
                                    const int32_t* slot_mapping, const void* signs,
                                    uint32_t sign_source, uint32_t in_dtype, uint32_t num_tokens,
                                    uint32_t num_kv_heads, uint32_t head_size, uint32_t block_size,
                                    uint32_t num_blocks, float inv_sqrt_len, uint32_t* status)
{
    using namespace tq;
    if (num_kv_heads == 0 || num_blocks == 0 || block_size == 0 || block_size % kStrip != 0 ||
        (head_size != 128 && head_size != 256) || in_dtype > TQ_IN_BF16 ||
        sign_source > TQ_SIGNS_TABLES_BF16)
        return TQ_ERR_INVALID_ARGUMENT;
    // A partial trailing strip would be silently dropped; refuse it like the
    // reference launcher (turboquant_reshape_and_cache_a8.cpp:1606-1609).
    if (num_tokens % kStrip != 0) return TQ_ERR_PARTIAL_STRIP;
    if (num_tokens == 0) return TQ_OK;
    if (!key || !value || !key_cache || !value_cache || !scale_cache || !slot_mapping || !signs)
        return TQ_ERR_INVALID_ARGUMENT;

    IngestParams p;
    p.key = key;
    p.value = value;
    p.key_cache = reinterpret_cast<uint8_t*>(key_cache);
    p.value_cache = reinterpret_cast<uint8_t*>(value_cache);
    p.scale_cache = scale_cache;
    p.slots = slot_mapping;
    p.signs = signs;
    p.sign_source = sign_source;
    p.num_strips = num_tokens / kStrip;
    p.H = num_kv_heads;
    p.S = block_size;
    p.P = num_blocks;
    p.inv_sqrt_len = inv_sqrt_len;
    p.status = status;

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t err;
    if (head_size == 128)
        err = in_dtype == TQ_IN_BF16 ? launch_ingest<128, true>(s, p) : launch_ingest<128, false>(s, p);
    else
        err = in_dtype == TQ_IN_BF16 ? launch_ingest<256, true>(s, p) : launch_ingest<256, false>(s, p);
    return err == cudaSuccess ? TQ_OK : TQ_ERR_LAUNCH;
}
