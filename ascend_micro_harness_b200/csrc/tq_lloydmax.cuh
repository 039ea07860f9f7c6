// The 16-level Lloyd-Max codebook for N(0,1) and the in-register block Hadamard shared by
// the routine kernels and the Lloyd-Max cache variant.
#pragma once

#include "tq_common.cuh"

namespace tq {

// Gaussian conditional-mean fixed point with midpoint thresholds
// (include/routines/routine_vector_lloydmax_quantize.hpp:18-30). Both tables are odd:
// centroid[15 - q] = -centroid[q], thresholds -t7 .. -t1, 0, t1 .. t7.
__device__ __forceinline__ float lloydmax4_positive_threshold(int j)   // j = 1..7
{
    constexpr float t[8] = {0.f,          0.258221665f, 0.522403709f, 0.799549788f,
                            1.099285827f, 1.437138792f, 1.843531806f, 2.400803399f};
    return t[j];
}

__device__ __forceinline__ float lloydmax4_centroid(unsigned q)
{
    constexpr float c[8] = {0.128395030f, 0.388048299f, 0.656759119f, 0.942340456f,
                            1.256231197f, 1.618046386f, 2.069017227f, 2.732589571f};
    float m = c[0];
    const unsigned k = q >= 8u ? q - 8u : 7u - q;   // magnitude index
#pragma unroll
    for (int i = 1; i < 8; ++i) m = k == static_cast<unsigned>(i) ? c[i] : m;
    return q >= 8u ? m : -m;
}

// code = #{thresholds <= x}, equality to the upper bin (same header :32-38). With a = |x|
// and n = #{j : a >= t_j} over the seven positive thresholds: for x >= 0 (including -0) the
// code is 8 + n; for x < 0 it is #{j : a <= t_j} = 7 - #{j : a > t_j}, and a > t is
// nextdown(a) >= t, so one three-step binary search serves both signs. A NaN compares false
// everywhere and gets code 0, as in the reference.
__device__ __forceinline__ unsigned lloydmax4_code(float x)
{
    const bool nonneg = x >= 0.0f;
    // |x|, stepped down by one ulp for negative x (x < 0 implies |x| > 0: no wrap)
    const float a = __uint_as_float((__float_as_uint(x) & 0x7FFFFFFFu) - (x < 0.0f ? 1u : 0u));
    const bool c4 = a >= lloydmax4_positive_threshold(4);
    const float ta = c4 ? lloydmax4_positive_threshold(6) : lloydmax4_positive_threshold(2);
    const bool c2 = a >= ta;
    const float tb = c4 ? (c2 ? lloydmax4_positive_threshold(7) : lloydmax4_positive_threshold(5))
                        : (c2 ? lloydmax4_positive_threshold(3) : lloydmax4_positive_threshold(1));
    const bool c1 = a >= tb;
    const unsigned n = (c4 ? 4u : 0u) + (c2 ? 2u : 0u) + (c1 ? 1u : 0u);
    const unsigned code = nonneg ? 8u + n : 7u - n;
    return x != x ? 0u : code;
}

// x <- x H16 for 16 values held by one thread (H16[k][c] = (-1)^popcount(k & c); symmetric),
// as the radix-2 cascade out[i] = in[i ^ s] + ((i & s) ? -in[i] : in[i]), s = 1, 2, 4, 8.
__device__ __forceinline__ void hadamard16_inplace(float (&v)[16])
{
#pragma unroll
    for (int s = 1; s < 16; s <<= 1)
#pragma unroll
        for (int i = 0; i < 16; ++i)
            if ((i & s) == 0) {
                const float a = v[i], b = v[i + s];
                v[i] = b + a;
                v[i + s] = a - b;
            }
}

}  // namespace tq
