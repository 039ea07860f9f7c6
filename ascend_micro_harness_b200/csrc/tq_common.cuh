// Shared device helpers for the TurboQuant kernels (sm_100a).
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "../../include/tq_b200.h"

namespace tq {

constexpr int kStrip = 16;   // tokens per strip: the unit both operators walk
constexpr int kGroup = 32;   // width of the inner Hadamard factor
constexpr float kMaskedScore = -3.0e38f;  // neutral softmax maximum of an empty range

// (-1)^popcount(a & b): the Sylvester Hadamard sign, true when negative.
__device__ __forceinline__ bool hneg(unsigned a, unsigned b) { return __popc(a & b) & 1u; }

// Sign of channel `ch` from whichever operand the caller supplied:
//   F32 vector, or column 0 of row c0 of resident block g (sign half 0).
__device__ __forceinline__ bool sign_is_negative(const void* signs, uint32_t source, int ch)
{
    if (source == TQ_SIGNS_F32) return static_cast<const float*>(signs)[ch] < 0.0f;
    const size_t at = static_cast<size_t>(ch) * kGroup;  // (g*32 + c0) * 32 + 0
    if (source == TQ_SIGNS_TABLES_I8) return static_cast<const int8_t*>(signs)[at] < 0;
    return (static_cast<const uint16_t*>(signs)[at] & 0x8000u) != 0u;
}

__device__ __forceinline__ void mma_s8_16832(int (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                             uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1,
                                               uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// In-register Sylvester transform over N values: x[c1] = sum_g H_N[c1][g] x[g].
template <int N, class T>
__device__ __forceinline__ void fwht_inplace(T (&x)[N])
{
#pragma unroll
    for (int s = 1; s < N; s <<= 1)
#pragma unroll
        for (int i = 0; i < N; ++i)
            if ((i & s) == 0) {
                const T a = x[i], b = x[i + s];
                x[i] = a + b;
                x[i + s] = a - b;
            }
}

// y = Pi x * sqrt(d) for one row spread over a warp: lane l holds the K = d/32
// consecutive channels l*K .. l*K+K-1. FP32 radix-2 cascade in the stage order of the
// reference's host model (tests/common/rotate_butterfly_oracle.hpp:44-48,:130-142):
// strides 1..16, the sign diagonal, strides 32..d/2, each stage
// out[i] = in[i ^ s] + ((i & s) ? -in[i] : in[i]) -- so the result is reproducible
// bit for bit, integer-valued rows or not.
template <int K>
__device__ __forceinline__ void cascade_ingress(float (&v)[K], const float (&sgn)[K], int lane)
{
    auto stage = [&](int s) {
        if (s < K) {
#pragma unroll
            for (int i = 0; i < K; ++i)
                if ((i & s) == 0) {
                    const float a = v[i], b = v[i + s];
                    v[i] = b + a;
                    v[i + s] = a - b;
                }
        } else {
            const int lm = s / K;
            const bool upper = (lane & lm) != 0;
#pragma unroll
            for (int i = 0; i < K; ++i) {
                const float other = __shfl_xor_sync(0xffffffffu, v[i], lm);
                v[i] = other + (upper ? -v[i] : v[i]);
            }
        }
    };
#pragma unroll
    for (int s = 1; s < kGroup; s <<= 1) stage(s);
#pragma unroll
    for (int i = 0; i < K; ++i) v[i] *= sgn[i];
#pragma unroll
    for (int s = kGroup; s < 32 * K; s <<= 1) stage(s);
}

__device__ __forceinline__ float bf16_bits_to_f32(uint16_t raw)
{
    return __uint_as_float(static_cast<uint32_t>(raw) << 16);
}

__device__ __forceinline__ uint16_t f32_to_bf16_bits(float v)
{
    return __bfloat16_as_ushort(__float2bfloat16_rn(v));
}

// n / d for any 32-bit n with the precomputed (mul, shift) of divisor d >= 2
// (round-up method: mul = floor(2^32 (2^l - d) / d) + 1, l = ceil(log2 d)).
__device__ __forceinline__ uint32_t fast_div(uint32_t n, uint32_t mul, uint32_t shift)
{
    const uint32_t t = __umulhi(mul, n);
    return (t + ((n - t) >> 1)) >> shift;
}

// The (mul, shift) pair of fast_div for divisor d >= 2.
inline void fast_div_constants(uint32_t d, uint32_t* mul, uint32_t* shift)
{
    uint32_t l = 0;
    while ((1ull << l) < d) ++l;
    *mul = static_cast<uint32_t>(((1ull << 32) * ((1ull << l) - d)) / d + 1ull);
    *shift = l - 1u;
}

// A divisor fixed at launch, any value >= 1: the host prepares it, the kernel divides by it
// with a multiply and two shifts instead of the dozens of dependent instructions of a division
// in software.
struct Divider {
    uint32_t d = 1, mul = 0, shift = 0;
    Divider() = default;
    explicit Divider(uint32_t divisor) : d(divisor)
    {
        if (d >= 2u) fast_div_constants(d, &mul, &shift);
    }
    __device__ __forceinline__ uint32_t quotient(uint32_t n) const { return d == 1u ? n : fast_div(n, mul, shift); }
};

__device__ __forceinline__ void report(uint32_t* status, uint32_t bits)
{
    if (status != nullptr) atomicOr(status, bits);
}

}  // namespace tq
