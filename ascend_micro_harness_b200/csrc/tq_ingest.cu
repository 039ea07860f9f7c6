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
//   * persistent warps walk the panels; each thread copies exactly the bytes that
//     are its MMA A-fragments into a private two-stage shared-memory ring with
//     cp.async (the MMA's contraction order is permuted so a thread's contiguous
//     8/16 bytes ARE its fragment), one panel ahead of the arithmetic, and reads them
//     back itself -- no cross-thread synchronisation on the way in;
//   * the inner factor I_G (x) H32 is the only dense contraction: per 32-channel
//     group, 4 (int8, m16n8k32) or 8 (bf16, m16n8k16) warp MMAs against +-1
//     operands generated from popcount parity. Products of +-1 with int8 / small
//     bf16 integers accumulate exactly in INT32 / FP32;
//   * the MMA's output columns are permuted so each thread ends up with 8
//     consecutive channels of every group: the sign diagonal and the outer H_G
//     factor are register-local butterflies on packed f32x2 operations, and one
//     thread's 8 codes are one 32-bit word of the key page;
//   * fragment rows r and r+8 carry tokens 2r and 2r+1, so one thread owns both
//     nibbles of every value-page byte it produces;
//   * the scale comes from the exponent field of absmax by integer arithmetic, the
//     rounding is one fused multiply-add onto 1.5 * 2^23 (no float-to-int
//     conversion), codes pack by integer multiply-add; the page is staged in shared
//     memory and leaves as 128-bit stores of the whole contiguous (page, head) block.
#include <atomic>
#include <type_traits>

#include "tq_ingest.cuh"

namespace tq {

constexpr int kIngestWarps = 4;
#ifndef TQ_D256_INGEST_CTAS
#define TQ_D256_INGEST_CTAS 3
#endif
// Resident CTAs per SM: a thread holds a 16 x d / 32 slice of the rotated panel in
// registers (64 floats at d = 128, 128 at d = 256), which fixes the register budget.
template <int D>
constexpr int kIngestCtasPerSm = D == 128 ? 4 : TQ_D256_INGEST_CTAS;
// Floats per quad position in the shared sign table: d/4 signs plus two of padding, so
// that the four positions a warp reads at once sit in different banks.
template <int D>
constexpr int kSignPitchOf = D / 4 + 2;
// Bytes of the per-CTA table behind the warps' stages. bf16: the sign diagonal as floats per quad
// position. int8: the +-1 MMA operands of H32 with the group's signs folded into their columns,
// [group][half][lane] x 16 bytes.
template <int D, bool BF16>
constexpr int kTableBytes = BF16 ? 4 * kSignPitchOf<D> * 4 : (D / kGroup) * 2 * 32 * 16;

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src));
}
// 16 bytes of which the first `bytes` come from memory and the rest are zeros.
__device__ __forceinline__ void cp_async_16_zfill(uint32_t dst, const void* src, uint32_t bytes)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_8(uint32_t dst, const void* src)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(dst), "l"(src));
}

struct PanelId {
    uint32_t strip, plane, head;
};
__device__ __forceinline__ PanelId panel_of(const IngestParams& p, uint32_t chunk)
{
    PanelId id;
    id.strip = fast_div(chunk, p.div_mul, p.div_shift);
    const uint32_t rem = chunk - id.strip * 2u * p.H;
    id.plane = rem >= p.H ? 1u : 0u;
    id.head = rem - id.plane * p.H;
    return id;
}

// First token and token count of a strip. Dense launches: strip s holds tokens 16 s .. 16 s + 15.
// Ragged launches: the request is found by bisection over the strips' prefix sum; the last
// strip of a request may hold fewer than 16 tokens.
struct StripRun {
    uint32_t token0, count;
};
template <bool VARLEN>
__device__ __forceinline__ StripRun strip_run(const IngestParams& p, uint32_t strip)
{
    if constexpr (!VARLEN) {
        return {strip * kStrip, static_cast<uint32_t>(kStrip)};
    } else {
        uint32_t lo = 0, hi = p.num_requests;   // strip_begin[lo] <= strip < strip_begin[hi]
        while (hi - lo > 1u) {
            const uint32_t mid = (lo + hi) >> 1;
            if (static_cast<uint32_t>(__ldg(p.strip_begin + mid)) <= strip) lo = mid;
            else hi = mid;
        }
        const uint32_t begin = static_cast<uint32_t>(__ldg(p.cu_seqlens + lo));
        const uint32_t len = static_cast<uint32_t>(__ldg(p.cu_seqlens + lo + 1)) - begin;
        const uint32_t r = strip - static_cast<uint32_t>(__ldg(p.strip_begin + lo));
        return {begin + r * kStrip, min(static_cast<uint32_t>(kStrip), len - r * kStrip)};
    }
}

// Queue the copies of one panel: per 32-channel group the 8 channels of token 2r and
// of token 2r+1 that this thread will feed to the MMA. Returns the slot of token
// (lane & 15) of the strip, fetched alongside.
template <int D, bool BF16, bool VARLEN>
__device__ __forceinline__ int32_t stage_panel(const IngestParams& p, uint32_t chunk, int lane,
                                               uint32_t stage_s)
{
    constexpr int G = D / kGroup;
    constexpr int kElem = BF16 ? 2 : 1;
    constexpr int kPiece = 8 * kElem;   // bytes of 8 channels
    const int r = lane >> 2, qd = lane & 3;
    const PanelId id = panel_of(p, chunk);
    const StripRun run = strip_run<VARLEN>(p, id.strip);
    const size_t row_pitch = static_cast<size_t>(p.H) * D * kElem;  // bytes
    const uint8_t* strip_base = static_cast<const uint8_t*>(id.plane == 0 ? p.key : p.value) +
                                static_cast<size_t>(run.token0) * row_pitch +
                                (static_cast<size_t>(id.head) * D + qd * 8) * kElem;
    const uint8_t* base = strip_base + static_cast<size_t>(2 * r) * row_pitch;
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t dst = stage_s + ((g * 2 + h) * 32 + lane) * kPiece;
            const uint8_t* src = base + h * row_pitch + g * kGroup * kElem;
            if constexpr (VARLEN) {
                // tokens past a short last strip read as zeros (from the strip's first row)
                const bool live = static_cast<uint32_t>(2 * r + h) < run.count;
                cp_async_16_zfill(dst, live ? src : strip_base, live ? 16u : 0u);
            } else if constexpr (BF16) {
                cp_async_16(dst, src);
            } else {
                cp_async_8(dst, src);
            }
        }
    const uint32_t t = lane & 15;
    if constexpr (VARLEN) {
        // slots of absent tokens are synthesised so that the run check sees a whole strip
        const int32_t first = __ldg(p.slots + run.token0);
        return t < run.count ? __ldg(p.slots + run.token0 + t) : first + static_cast<int32_t>(t);
    } else {
        return __ldg(p.slots + static_cast<size_t>(run.token0) + t);
    }
}

__device__ __forceinline__ float2 f2(float a, float b) { return make_float2(a, b); }

// max(a, |b|, |c|) in one three-input instruction.
__device__ __forceinline__ float max3_abs(float a, float b, float c)
{
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(fabsf(b)), "f"(fabsf(c)));
    return r;
}

// Rotate, quantise, pack and store one panel whose fragments sit in `in` (this
// thread's own bytes) and whose slot run is `slot`.
template <int D, bool BF16, bool VARLEN>
__device__ __forceinline__ void process_panel(const IngestParams& p, uint32_t chunk, int lane,
                                              const uint8_t* in, int32_t slot,
                                              const uint32_t (&bfrag)[16],
                                              const float* sgn_s, uint32_t* stage)
{
    constexpr int G = D / kGroup;
    constexpr int kPageWords = kStrip * D / 8;
    constexpr int kPiece = BF16 ? 16 : 8;
    constexpr int kSignPitch = kSignPitchOf<D>;
    const int r = lane >> 2, qd = lane & 3;
    const PanelId id = panel_of(p, chunk);
    // tokens the strip really holds (16 except for the last strip of a ragged request)
    const uint32_t live_tokens = VARLEN ? strip_run<VARLEN>(p, id.strip).count : static_cast<uint32_t>(kStrip);

    // ---- the strip's page, from its slots; the contract is checked, not assumed
    // (tests/common/turboquant_oracle.hpp:278-287).
    const int32_t slot0 = __shfl_sync(0xffffffffu, slot, 0);
    const bool run_ok = (slot == slot0 + (lane & 15));
    // slot0 / S by the precomputed multiplier (a division in software is dozens of dependent instructions)
    const uint32_t page = fast_div(static_cast<uint32_t>(slot0), p.page_mul, p.page_shift);
    const bool strip_ok = __all_sync(0xffffffffu, run_ok) && slot0 >= 0 && (slot0 % kStrip) == 0 && page < p.P;
    if (!strip_ok) {
        if (lane == 0) report(p.status, TQ_STATUS_BAD_SLOT);
        return;
    }
    const uint32_t tok_in_page = static_cast<uint32_t>(slot0) - page * p.S;

    // y[tt][g][ep]: token 2r+tt, channels g*32 + qd*8 + 2ep, +1 as one float pair
    // (exact integers for int8 and integer-valued bf16 inputs).
    float2 y[2][G][4];
    if constexpr (!BF16) {
        // The INT32 accumulator starts at the bit pattern of 1.5 * 2^23, so what comes
        // out, read as a float, is 12582912 + sum exactly; the first butterfly below takes
        // the offset out again. The operands carry the sign diagonal already (a column of
        // the +-1 operand is an output channel), so y is s . (H32 x) up to that offset.
        constexpr int kBias = 0x4B400000;
        const uint4* bsg = reinterpret_cast<const uint4*>(sgn_s);
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const uint2 lo = *reinterpret_cast<const uint2*>(in + ((g * 2 + 0) * 32 + lane) * kPiece);
            const uint2 hi = *reinterpret_cast<const uint2*>(in + ((g * 2 + 1) * 32 + lane) * kPiece);
            const uint32_t a[4] = {lo.x, hi.x, lo.y, hi.y};
            const uint4 b01 = bsg[(g * 2 + 0) * 32 + lane], b23 = bsg[(g * 2 + 1) * 32 + lane];
            const uint32_t bw[8] = {b01.x, b01.y, b01.z, b01.w, b23.x, b23.y, b23.z, b23.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                int c[4] = {kBias, kBias, kBias, kBias};
                mma_s8_16832(c, a, bw[j * 2 + 0], bw[j * 2 + 1]);
                y[0][g][j] = f2(__int_as_float(c[0]), __int_as_float(c[1]));
                y[1][g][j] = f2(__int_as_float(c[2]), __int_as_float(c[3]));
            }
        }
    } else {
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const uint4 lo = *reinterpret_cast<const uint4*>(in + ((g * 2 + 0) * 32 + lane) * kPiece);
            const uint4 hi = *reinterpret_cast<const uint4*>(in + ((g * 2 + 1) * 32 + lane) * kPiece);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float c[4] = {0.f, 0.f, 0.f, 0.f};
                mma_bf16_16816(c, lo.x, hi.x, lo.y, hi.y, bfrag[j * 2 + 0], bfrag[j * 2 + 1]);
                mma_bf16_16816(c, lo.z, hi.z, lo.w, hi.w, bfrag[8 + j * 2 + 0], bfrag[8 + j * 2 + 1]);
                y[0][g][j] = f2(c[0], c[1]);
                y[1][g][j] = f2(c[2], c[3]);
            }
        }
    }

    // ---- the outer factor H_G on packed pairs. bf16: the sign diagonal is folded into its first
    // stage (multiplies by +-1: exact). int8: the inputs are B + a and B + b with B = 1.5 * 2^23;
    // b - 2B = b' - B, a + (b' - B) = a' + b' and a - b = a' - b' are all exact in FP32.
    const float2 minus1 = f2(-1.0f, -1.0f);
    const float2 minus2bias = f2(-25165824.0f, -25165824.0f);
    float amax[2] = {1.0f, 1.0f};  // the writer floors absmax at 1
#pragma unroll
    for (int ep = 0; ep < 4; ++ep) {
        float2 sg[G];
        if constexpr (BF16) {
#pragma unroll
            for (int g = 0; g < G; ++g)
                sg[g] = *reinterpret_cast<const float2*>(sgn_s + qd * kSignPitch + g * 8 + ep * 2);
        }
#pragma unroll
        for (int tt = 0; tt < 2; ++tt) {
            float2 x[G];
#pragma unroll
            for (int g = 0; g < G; g += 2) {
                if constexpr (BF16) {
                    const float2 a = __fmul2_rn(sg[g], y[tt][g][ep]);
                    const float2 b = __fmul2_rn(sg[g + 1], y[tt][g + 1][ep]);
                    x[g] = __fadd2_rn(a, b);
                    x[g + 1] = __ffma2_rn(b, minus1, a);
                } else {
                    const float2 a = y[tt][g][ep], b = y[tt][g + 1][ep];
                    x[g] = __fadd2_rn(a, __fadd2_rn(b, minus2bias));
                    x[g + 1] = __ffma2_rn(b, minus1, a);
                }
            }
#pragma unroll
            for (int s = 2; s < G; s <<= 1)
#pragma unroll
                for (int i = 0; i < G; ++i)
                    if ((i & s) == 0) {
                        const float2 a = x[i], b = x[i + s];
                        x[i] = __fadd2_rn(a, b);
                        x[i + s] = __ffma2_rn(b, minus1, a);
                    }
#pragma unroll
            for (int g = 0; g < G; ++g) {
                y[tt][g][ep] = x[g];
                amax[tt] = max3_abs(amax[tt], x[g].x, x[g].y);
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
    // the upper clamp (code 7, u = 15) is part of the packing of the key page (pack8) and a
    // float min in the value page, whose bytes pair two tokens; a final xor with 0x88.. turns
    // u back into the two's-complement nibble.
    constexpr float kMagic = 12582920.0f;           // 1.5 * 2^23 + 8
    constexpr float kMagicTop = 12582927.0f;        // 1.5 * 2^23 + 15
    const float2 magic2 = f2(kMagic, kMagic);
    __syncwarp();  // the previous panel's copy-out has finished reading the stage
    if (id.plane == 0) {
        // key page: token-major, row of D/8 words; this thread's word is g*4 + qd: eight codes
        // clamped and packed four at a time (pack8)
#pragma unroll
        for (int tt = 0; tt < 2; ++tt) {
            const float2 inv2 = f2(inv[tt], inv[tt]);
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float rounded[8];
#pragma unroll
                for (int ep = 0; ep < 4; ++ep) {
                    const float2 rr = __ffma2_rn(y[tt][g][ep], inv2, magic2);
                    rounded[2 * ep] = rr.x;
                    rounded[2 * ep + 1] = rr.y;
                }
                stage[(2 * r + tt) * (D / 8) + ((g * 4 + qd) ^ (r & 3) * 4)] = pack8(rounded);
            }
        }
    } else {
        // value page: byte (channel*8 + r) = u(token 2r) + 16 u(token 2r+1); the store
        // keeps the low byte, to which 17 * 0x4B400000 contributes nothing.
        uint8_t* sb = reinterpret_cast<uint8_t*>(stage);
        const float2 inv0 = f2(inv[0], inv[0]), inv1 = f2(inv[1], inv[1]);
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int ep = 0; ep < 4; ++ep) {
                const float2 r0 = __ffma2_rn(y[0][g][ep], inv0, magic2);
                const float2 r1 = __ffma2_rn(y[1][g][ep], inv1, magic2);
                const uint32_t b0 = __float_as_uint(fminf(r1.x, kMagicTop)) * 16u +
                                    __float_as_uint(fminf(r0.x, kMagicTop));
                const uint32_t b1 = __float_as_uint(fminf(r1.y, kMagicTop)) * 16u +
                                    __float_as_uint(fminf(r0.y, kMagicTop));
                // channels c, c+1 fill one 16-byte unit (index c/2); units of quad positions
                // qd and qd^2 would share banks, so bit 0 of the unit index takes qd's bit 1
                const int unit = ((g * kGroup + qd * 8 + ep * 2) >> 1) ^ (qd >> 1);
                sb[unit * 16 + r] = static_cast<uint8_t>(b0);
                sb[unit * 16 + 8 + r] = static_cast<uint8_t>(b1);
            }
    }
    __syncwarp();

    // ---- whole contiguous block out with 128-bit stores.
    uint8_t* cache = id.plane == 0 ? p.key_cache : p.value_cache;
    const size_t block_bytes = static_cast<size_t>(kStrip) * D / 2;
    uint8_t* dst = cache + (static_cast<size_t>(page) * p.H + id.head) * (static_cast<size_t>(p.S) * D / 2) +
                   static_cast<size_t>(tok_in_page / kStrip) * block_bytes;
    const uint4* s4 = reinterpret_cast<const uint4*>(stage);
#pragma unroll
    for (int i = 0; i < kPageWords / 4 / 32; ++i) {
        const int unit = i * 32 + lane;  // 16-byte unit of the page
        uint4 v;
        if (id.plane == 0) {
            // undo the store swizzle: unit = row * (D/32) + chunk, chunk ^= (row/2) & 3
            const int row = unit / (D / 32), chunk16 = unit % (D / 32);
            if (VARLEN && static_cast<uint32_t>(row) >= live_tokens) continue;   // key rows past a short strip stay
            v = s4[row * (D / 32) + (chunk16 ^ ((row >> 1) & 3))];
        } else {
            v = s4[unit ^ ((unit >> 3) & 1)];   // undo the store swizzle
            v.x ^= 0x88888888u;  // u -> two's-complement nibble
            v.y ^= 0x88888888u;
            v.z ^= 0x88888888u;
            v.w ^= 0x88888888u;
        }
        __stcs(reinterpret_cast<uint4*>(dst) + unit, v);
    }

    if (qd == 0) {
        const size_t at = ((static_cast<size_t>(id.plane) * p.P + page) * p.H + id.head) * p.S +
                          tok_in_page + 2 * r;
        if (!VARLEN || static_cast<uint32_t>(2 * r + 1) < live_tokens) {
            *reinterpret_cast<float2*>(p.scale_cache + at) =
                make_float2(pow2[0] * p.inv_sqrt_len, pow2[1] * p.inv_sqrt_len);
        } else if (static_cast<uint32_t>(2 * r) < live_tokens) {
            p.scale_cache[at] = pow2[0] * p.inv_sqrt_len;
        }
    }
}

// Persistent: every warp walks panels warp_global, warp_global + warps_total, ...
// with the next panel's bytes in flight while the current one is processed.
template <int D, bool BF16, bool VARLEN = false>
__global__ void __launch_bounds__(kIngestWarps * 32, kIngestCtasPerSm<D>)
tq_ingest_kernel(const IngestParams p)
{
    constexpr int G = D / kGroup;
    constexpr int kPageWords = kStrip * D / 8;
    constexpr int kInBytes = kStrip * D * (BF16 ? 2 : 1);   // one panel of activations
    extern __shared__ __align__(16) uint8_t smem_raw[];
    // per warp: two input stages, one output stage; then the CTA's table (kTableBytes)
    uint8_t* warp_base = smem_raw + (threadIdx.x >> 5) * (2 * kInBytes + kPageWords * 4);
    float* sgn_s = reinterpret_cast<float*>(smem_raw + kIngestWarps * (2 * kInBytes + kPageWords * 4));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = lane >> 2, qd = lane & 3;

    // +-1 B fragments of H32. Column n of tile j is output channel c0 = (n/2)*8 + j*2 + n%2 of
    // its group, so a thread ends up with 8 consecutive channels.
    uint32_t bfrag[16] = {};
    if constexpr (!BF16) {
        // contraction slot k of the low half is input channel (k/4)*8 + k%4, of the
        // high half (k/4)*8 + 4 + k%4 -- the order the 8-byte pieces deliver. A fragment word is
        // one column of the operand: negating it (0x01 <-> 0xFF, xor 0xFE per byte) applies the
        // sign of that output channel, so the table holds every group's operands ready signed.
        uint4* bsg = reinterpret_cast<uint4*>(sgn_s);
        for (int g = warp; g < G; g += kIngestWarps) {
            uint32_t w8[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const unsigned c0 = (r >> 1) * 8 + j * 2 + (r & 1);
                const uint32_t flip = sign_is_negative(p.signs, p.sign_source, g * kGroup + c0) ? 0xFEFEFEFEu : 0u;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t w = 0;
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        w |= (hneg(c0, qd * 8 + h * 4 + e) ? 0xFFu : 0x01u) << (8 * e);
                    w8[j * 2 + h] = w ^ flip;
                }
            }
            bsg[(g * 2 + 0) * 32 + lane] = make_uint4(w8[0], w8[1], w8[2], w8[3]);
            bsg[(g * 2 + 1) * 32 + lane] = make_uint4(w8[4], w8[5], w8[6], w8[7]);
        }
    } else {
        // sign diagonal per quad position: sgn_s[qd][g*8 + e] for channel g*32 + qd*8 + e
        for (int i = threadIdx.x; i < 4 * G * 8; i += blockDim.x) {
            const int q = i / (G * 8), k = i % (G * 8);
            sgn_s[q * kSignPitchOf<D> + k] =
                sign_is_negative(p.signs, p.sign_source, (k / 8) * kGroup + q * 8 + (k % 8)) ? -1.0f : 1.0f;
        }
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

    const uint32_t stride = gridDim.x * kIngestWarps;
    uint32_t c = blockIdx.x * kIngestWarps + warp;
    const uint32_t in_s = static_cast<uint32_t>(__cvta_generic_to_shared(warp_base));
    uint32_t* stage = reinterpret_cast<uint32_t*>(warp_base + 2 * kInBytes);

    int32_t slot_cur = 0, slot_nxt = 0;
    if (c < p.chunks) slot_cur = stage_panel<D, BF16, VARLEN>(p, c, lane, in_s);
    asm volatile("cp.async.commit_group;\n" ::);
    uint32_t buf = 0;
#pragma unroll 1
    for (; c < p.chunks; c += stride, buf ^= 1u) {
        const uint32_t cn = c + stride;
        if (cn < p.chunks) slot_nxt = stage_panel<D, BF16, VARLEN>(p, cn, lane, in_s + (buf ^ 1u) * kInBytes);
        asm volatile("cp.async.commit_group;\n" ::);
        asm volatile("cp.async.wait_group 1;\n" ::: "memory");   // this thread's own bytes of panel c
        process_panel<D, BF16, VARLEN>(p, c, lane, warp_base + buf * kInBytes, slot_cur, bfrag, sgn_s, stage);
        slot_cur = slot_nxt;
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
}

template <int D, bool BF16, bool VARLEN = false>
static cudaError_t launch_ingest(cudaStream_t stream, const IngestParams& p)
{
    constexpr int kInBytes = kStrip * D * (BF16 ? 2 : 1);
    constexpr int kSmem = kIngestWarps * (2 * kInBytes + kStrip * D / 2) + kTableBytes<D, BF16>;
    uint32_t blocks = (p.chunks + kIngestWarps - 1) / kIngestWarps;
    if (blocks == 0) return cudaSuccess;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) != cudaSuccess) return cudaErrorNoDevice;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    static bool configured[64] = {};   // benign race: the attribute is idempotent
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(tq_ingest_kernel<D, BF16, VARLEN>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    const uint32_t resident = static_cast<uint32_t>(sms) * kIngestCtasPerSm<D>;
    if (blocks > resident) blocks = resident;  // persistent: one resident wave
    tq_ingest_kernel<D, BF16, VARLEN><<<blocks, kIngestWarps * 32, kSmem, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace tq

// Clock cycles the tcgen05 writer lets one of its waits take; every launch reads it.
static std::atomic<long long> g_wait_budget{tq::kIngestWaitBudget};

extern "C" void tq_ingest_set_wait_budget(long long cycles)
{
    g_wait_budget.store(cycles < 0 ? tq::kIngestWaitBudget : cycles, std::memory_order_relaxed);
}

// Which kernel serves a call. kAuto: the tcgen05 kernels, which measure faster on B200 for either
// head size and element type (int8 at head size 256 by a hair: 3.43 against 3.40 TB/s), and the
// warp-MMA kernel wherever the driver cannot encode a tensor map.
enum class Writer { kAuto, kWarpMma, kTcgen05 };

static int reshape_and_cache(void* stream, const void* key, const void* value,
                             int8_t* key_cache, int8_t* value_cache, float* scale_cache,
                             const int32_t* slot_mapping, const void* signs,
                             uint32_t sign_source, uint32_t in_dtype, uint32_t num_tokens,
                             uint32_t num_kv_heads, uint32_t head_size, uint32_t block_size,
                             uint32_t num_blocks, float inv_sqrt_len, uint32_t* status,
                             Writer writer)
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
    // 16-byte accesses on every operand; panels are indexed in 32 bits
    const uintptr_t align = reinterpret_cast<uintptr_t>(key) | reinterpret_cast<uintptr_t>(value) |
                            reinterpret_cast<uintptr_t>(key_cache) |
                            reinterpret_cast<uintptr_t>(value_cache) |
                            reinterpret_cast<uintptr_t>(scale_cache);
    const uint64_t chunks = static_cast<uint64_t>(num_tokens / kStrip) * 2u * num_kv_heads;
    if ((align & 15u) != 0u || chunks >= 0x7FFFFFFFull || num_kv_heads > 0x10000u)
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
    p.chunks = static_cast<uint32_t>(chunks);
    fast_div_constants(2u * num_kv_heads, &p.div_mul, &p.div_shift);
    fast_div_constants(block_size, &p.page_mul, &p.page_shift);   // block_size >= 16
    p.inv_sqrt_len = inv_sqrt_len;
    p.status = status;
    p.wait_budget = g_wait_budget.load(std::memory_order_relaxed);

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t err = cudaErrorNotSupported;
    const bool bf16 = in_dtype == TQ_IN_BF16;
    const bool tensor_memory = writer != Writer::kWarpMma;
    if (tensor_memory) err = head_size == 128 ? launch_ingest_umma(s, p, bf16) : launch_ingest_umma256(s, p, bf16);
    if (err == cudaErrorNotSupported && writer != Writer::kTcgen05) {
        // the explicit warp-MMA entry, or a driver without tensor maps
        if (head_size == 128)
            err = in_dtype == TQ_IN_BF16 ? launch_ingest<128, true>(s, p) : launch_ingest<128, false>(s, p);
        else
            err = in_dtype == TQ_IN_BF16 ? launch_ingest<256, true>(s, p) : launch_ingest<256, false>(s, p);
    }
    return err == cudaSuccess ? TQ_OK : TQ_ERR_LAUNCH;
}

extern "C" int tq_reshape_and_cache(void* stream, const void* key, const void* value,
                                    int8_t* key_cache, int8_t* value_cache, float* scale_cache,
                                    const int32_t* slot_mapping, const void* signs,
                                    uint32_t sign_source, uint32_t in_dtype, uint32_t num_tokens,
                                    uint32_t num_kv_heads, uint32_t head_size, uint32_t block_size,
                                    uint32_t num_blocks, float inv_sqrt_len, uint32_t* status)
{
    return reshape_and_cache(stream, key, value, key_cache, value_cache, scale_cache, slot_mapping,
                             signs, sign_source, in_dtype, num_tokens, num_kv_heads, head_size,
                             block_size, num_blocks, inv_sqrt_len, status, Writer::kAuto);
}

extern "C" int tq_reshape_and_cache_warp_mma(void* stream, const void* key, const void* value,
                                             int8_t* key_cache, int8_t* value_cache,
                                             float* scale_cache, const int32_t* slot_mapping,
                                             const void* signs, uint32_t sign_source,
                                             uint32_t in_dtype, uint32_t num_tokens,
                                             uint32_t num_kv_heads, uint32_t head_size,
                                             uint32_t block_size, uint32_t num_blocks,
                                             float inv_sqrt_len, uint32_t* status)
{
    return reshape_and_cache(stream, key, value, key_cache, value_cache, scale_cache, slot_mapping,
                             signs, sign_source, in_dtype, num_tokens, num_kv_heads, head_size,
                             block_size, num_blocks, inv_sqrt_len, status, Writer::kWarpMma);
}

extern "C" int tq_reshape_and_cache_tcgen05(void* stream, const void* key, const void* value,
                                            int8_t* key_cache, int8_t* value_cache,
                                            float* scale_cache, const int32_t* slot_mapping,
                                            const void* signs, uint32_t sign_source,
                                            uint32_t in_dtype, uint32_t num_tokens,
                                            uint32_t num_kv_heads, uint32_t head_size,
                                            uint32_t block_size, uint32_t num_blocks,
                                            float inv_sqrt_len, uint32_t* status)
{
    return reshape_and_cache(stream, key, value, key_cache, value_cache, scale_cache, slot_mapping,
                             signs, sign_source, in_dtype, num_tokens, num_kv_heads, head_size,
                             block_size, num_blocks, inv_sqrt_len, status, Writer::kTcgen05);
}

// The aligned writer over ragged requests: strips are cut per request, the last strip of a
// request may hold fewer than 16 tokens (key plane: its rows only; value plane: the whole
// channel-major strip with the missing tokens as zeros; scales: its tokens only).
extern "C" int tq_reshape_and_cache_varlen(void* stream, const uint16_t* key, const uint16_t* value,
                                           int8_t* key_cache, int8_t* value_cache,
                                           float* scale_cache, const int32_t* slot_mapping,
                                           const float* pi_signs, const int32_t* cu_seqlens,
                                           const int32_t* strip_begin, uint32_t num_requests,
                                           uint32_t total_strips, uint32_t num_kv_heads,
                                           uint32_t head_size, uint32_t block_size,
                                           uint32_t num_blocks, float inv_sqrt_len, uint32_t* status)
{
    using namespace tq;
    if (num_kv_heads == 0 || num_blocks == 0 || block_size == 0 || block_size % kStrip != 0 ||
        (head_size != 128 && head_size != 256))
        return TQ_ERR_INVALID_ARGUMENT;
    if (num_requests == 0 || total_strips == 0) return TQ_OK;
    if (!key || !value || !key_cache || !value_cache || !scale_cache || !slot_mapping || !pi_signs ||
        !cu_seqlens || !strip_begin)
        return TQ_ERR_INVALID_ARGUMENT;
    const uintptr_t align = reinterpret_cast<uintptr_t>(key) | reinterpret_cast<uintptr_t>(value) |
                            reinterpret_cast<uintptr_t>(key_cache) |
                            reinterpret_cast<uintptr_t>(value_cache) |
                            reinterpret_cast<uintptr_t>(scale_cache);
    const uint64_t chunks = static_cast<uint64_t>(total_strips) * 2u * num_kv_heads;
    if ((align & 15u) != 0u || chunks >= 0x7FFFFFFFull || num_kv_heads > 0x10000u)
        return TQ_ERR_INVALID_ARGUMENT;
    IngestParams p;
    p.key = key;
    p.value = value;
    p.key_cache = reinterpret_cast<uint8_t*>(key_cache);
    p.value_cache = reinterpret_cast<uint8_t*>(value_cache);
    p.scale_cache = scale_cache;
    p.slots = slot_mapping;
    p.signs = pi_signs;
    p.sign_source = TQ_SIGNS_F32;
    p.num_strips = total_strips;
    p.H = num_kv_heads;
    p.S = block_size;
    p.P = num_blocks;
    p.chunks = static_cast<uint32_t>(chunks);
    fast_div_constants(2u * num_kv_heads, &p.div_mul, &p.div_shift);
    fast_div_constants(block_size, &p.page_mul, &p.page_shift);
    p.inv_sqrt_len = inv_sqrt_len;
    p.status = status;
    p.cu_seqlens = cu_seqlens;
    p.strip_begin = strip_begin;
    p.num_requests = num_requests;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const cudaError_t err = head_size == 128 ? launch_ingest<128, true, true>(s, p)
                                             : launch_ingest<256, true, true>(s, p);
    return err == cudaSuccess ? TQ_OK : TQ_ERR_LAUNCH;
}
