// The reference's single-purpose routines that its cache writers and decoders do not call,
// as standalone kernels behind the C ABI:
//   * Y = X x H16 on 16x16 FP16 tiles (routines/routine_cube_hadamard16.hpp:32-84; golden
//     model include/sim_micro_testbed.hpp:181-198) -- one warp per tile, two tensor-core MMAs
//     against +-1 operands generated from popcount parity, FP32 accumulation (exact for the
//     dyadic inputs the reference pins it with);
//   * the 16-level Lloyd-Max codec for N(0,1) inputs
//     (include/routines/routine_vector_lloydmax_quantize.hpp:18-38; packing
//     tests/common/lloydmax_oracle.hpp:65-69): code = number of thresholds <= x, equality to
//     the upper bin, unsigned codes packed low nibble first, reconstruction = centroid;
//   * the inverse-CDF int4 quantiser (routines/routine_vector_icdf_quantize.hpp:95-132;
//     oracle tests/cpu/icdf_fixture.hpp:124-142): y = 14 sigmoid(x) - 7, round to nearest
//     even, saturate to [-8, 7], two's-complement nibbles packed low first;
//   * the stand-alone query rotation Q_rot = Q Pi^T, rounded to bf16
//     (routines/routine_cube_decode_score.hpp:202-223), which the decoders otherwise do in
//     their own prologue.
#include <cuda_fp16.h>

#include "tq_lloydmax.cuh"

namespace tq {

__global__ void __launch_bounds__(128) tq_hadamard16_kernel(const uint16_t* __restrict__ x,
                                                            void* __restrict__ y, uint32_t out_dtype,
                                                            uint32_t tiles)
{
    const int lane = threadIdx.x & 31, r = lane >> 2, qd = lane & 3;
    const uint32_t tile = blockIdx.x * 4u + (threadIdx.x >> 5);
    if (tile >= tiles) return;
    const uint32_t* xt = reinterpret_cast<const uint32_t*>(x + static_cast<size_t>(tile) * 256);
    // A fragment: rows r and r+8, contraction slots 2qd, 2qd+1 and 8+2qd, 8+2qd+1
    const uint32_t a0 = xt[r * 8 + qd], a1 = xt[(r + 8) * 8 + qd];
    const uint32_t a2 = xt[r * 8 + 4 + qd], a3 = xt[(r + 8) * 8 + 4 + qd];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const unsigned col = j * 8 + r;   // B fragment column
        auto pm1 = [&](unsigned k) { return hneg(k, col) ? 0xBC00u : 0x3C00u; };   // f16 -1 / +1
        const uint32_t b0 = pm1(2 * qd) | (pm1(2 * qd + 1) << 16);
        const uint32_t b1 = pm1(8 + 2 * qd) | (pm1(8 + 2 * qd + 1) << 16);
        float c[4] = {0.f, 0.f, 0.f, 0.f};
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
            "{%8,%9}, {%0,%1,%2,%3};\n"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const size_t at = static_cast<size_t>(tile) * 256 + (r + 8 * h) * 16 + j * 8 + 2 * qd;
            const float lo = c[2 * h], hi = c[2 * h + 1];
            if (out_dtype == TQ_DTYPE_F32)
                *reinterpret_cast<float2*>(static_cast<float*>(y) + at) = make_float2(lo, hi);
            else if (out_dtype == TQ_DTYPE_F16)
                *reinterpret_cast<__half2*>(static_cast<__half*>(y) + at) = __floats2half2_rn(lo, hi);
            else
                *reinterpret_cast<uint32_t*>(static_cast<uint16_t*>(y) + at) =
                    f32_to_bf16_bits(lo) | (static_cast<uint32_t>(f32_to_bf16_bits(hi)) << 16);
        }
    }
}

// Eight elements per thread: two float4 in, one packed word out.
__global__ void __launch_bounds__(256) tq_lloydmax4_kernel(const float* __restrict__ x,
                                                           uint32_t* __restrict__ packed,
                                                           float* __restrict__ recon, size_t groups)
{
    const size_t g = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (g >= groups) return;
    const float4 lo = reinterpret_cast<const float4*>(x)[2 * g], hi = reinterpret_cast<const float4*>(x)[2 * g + 1];
    const float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
    uint32_t w = 0;
    float rc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const unsigned q = lloydmax4_code(v[e]);
        w |= q << (4 * e);
        rc[e] = lloydmax4_centroid(q);
    }
    packed[g] = w;
    if (recon != nullptr) {
        reinterpret_cast<float4*>(recon)[2 * g] = make_float4(rc[0], rc[1], rc[2], rc[3]);
        reinterpret_cast<float4*>(recon)[2 * g + 1] = make_float4(rc[4], rc[5], rc[6], rc[7]);
    }
}

__global__ void __launch_bounds__(256) tq_icdf_kernel(const uint16_t* __restrict__ x, uint32_t is_bf16,
                                                      uint32_t* __restrict__ packed, size_t groups)
{
    const size_t g = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (g >= groups) return;
    const uint4 raw = reinterpret_cast<const uint4*>(x)[g];
    const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t w = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const uint16_t bits = static_cast<uint16_t>(words[e >> 1] >> (16 * (e & 1)));
        const float v = is_bf16 ? bf16_bits_to_f32(bits) : __half2float(__ushort_as_half(bits));
        const float yv = 14.0f / (1.0f + expf(-v)) - 7.0f;
        const int q = max(-8, min(7, __float2int_rn(yv)));
        w |= (static_cast<uint32_t>(q) & 0xFu) << (4 * e);
    }
    packed[g] = w;
}

// q_rot = bf16(Pi q): one warp per row, the FP32 ingress cascade of the decoders.
template <int D>
__global__ void __launch_bounds__(128) tq_rotate_query_kernel(const uint16_t* __restrict__ q,
                                                              const float* __restrict__ signs,
                                                              uint16_t* __restrict__ q_rot, uint32_t rows,
                                                              float inv_sqrt_len)
{
    constexpr int K = D / 32;
    const int lane = threadIdx.x & 31;
    const uint32_t row = blockIdx.x * 4u + (threadIdx.x >> 5);
    if (row >= rows) return;
    float sgn[K], v[K];
#pragma unroll
    for (int i = 0; i < K; ++i) {
        sgn[i] = signs[lane * K + i] < 0.0f ? -1.0f : 1.0f;
        v[i] = bf16_bits_to_f32(q[static_cast<size_t>(row) * D + lane * K + i]);
    }
    cascade_ingress<K>(v, sgn, lane);
#pragma unroll
    for (int i = 0; i < K; ++i)
        q_rot[static_cast<size_t>(row) * D + lane * K + i] = f32_to_bf16_bits(v[i] * inv_sqrt_len);
}

// q_rot = Pi q with Pi = diag(s) H diag(s) / sqrt(D), FP32 out: the query prologue of the fused
// decoder's raw-query entry (tests/common/fused_decode_opt_fixture.hpp:104-117,:166-182). One
// warp per row, lane l holds channels l*K .. l*K+K-1: strides below K are register
// butterflies, the others exchange whole registers between lanes.
template <int D>
__global__ void __launch_bounds__(128) tq_rotate_query_pi_kernel(const uint16_t* __restrict__ q,
                                                                 uint32_t is_bf16,
                                                                 const float* __restrict__ signs,
                                                                 float* __restrict__ q_rot, uint32_t rows,
                                                                 float inv_sqrt_len)
{
    constexpr int K = D / 32;
    const int lane = threadIdx.x & 31;
    const uint32_t row = blockIdx.x * 4u + (threadIdx.x >> 5);
    if (row >= rows) return;
    float sgn[K], v[K];
#pragma unroll
    for (int i = 0; i < K; ++i) {
        sgn[i] = signs[lane * K + i] < 0.0f ? -1.0f : 1.0f;
        const uint16_t bits = q[static_cast<size_t>(row) * D + lane * K + i];
        v[i] = (is_bf16 ? bf16_bits_to_f32(bits) : __half2float(__ushort_as_half(bits))) * sgn[i];
    }
#pragma unroll
    for (int s = 1; s < K; s <<= 1)
#pragma unroll
        for (int i = 0; i < K; ++i)
            if ((i & s) == 0) {
                const float a = v[i], b = v[i + s];
                v[i] = a + b;
                v[i + s] = a - b;
            }
#pragma unroll
    for (int o = 1; o < 32; o <<= 1)
#pragma unroll
        for (int i = 0; i < K; ++i) {
            const float other = __shfl_xor_sync(0xffffffffu, v[i], o);
            v[i] = (lane & o) ? other - v[i] : v[i] + other;
        }
#pragma unroll
    for (int i = 0; i < K; ++i) q_rot[static_cast<size_t>(row) * D + lane * K + i] = v[i] * sgn[i] * inv_sqrt_len;
}

}  // namespace tq

// Q_rot = Q Pi^T for `rows` bf16 query vectors, rounded to bf16: the operand the decoders pin
// (routines/routine_cube_decode_score.hpp:202-223; tests/common/paged_decode_oracle.hpp:486-515).
// The decode entry points rotate in the kernel; this is the stand-alone form.
extern "C" int tq_rotate_query(void* stream, const uint16_t* query, const float* pi_signs,
                               uint16_t* query_rot, uint32_t rows, uint32_t head_size,
                               float inv_sqrt_len)
{
    if (head_size != 128 && head_size != 256) return TQ_ERR_INVALID_ARGUMENT;
    if (rows == 0) return TQ_OK;
    if (!query || !pi_signs || !query_rot) return TQ_ERR_INVALID_ARGUMENT;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const unsigned blocks = (rows + 3u) / 4u;
    if (head_size == 128) tq::tq_rotate_query_kernel<128><<<blocks, 128, 0, s>>>(query, pi_signs, query_rot, rows, inv_sqrt_len);
    else tq::tq_rotate_query_kernel<256><<<blocks, 128, 0, s>>>(query, pi_signs, query_rot, rows, inv_sqrt_len);
    return cudaGetLastError() == cudaSuccess ? TQ_OK : TQ_ERR_LAUNCH;
}

extern "C" int tq_hadamard16(void* stream, const uint16_t* x_f16, void* y, uint32_t out_dtype,
                             uint32_t tiles)
{
    if (out_dtype > TQ_DTYPE_F32) return TQ_ERR_INVALID_ARGUMENT;
    if (tiles == 0) return TQ_OK;
    if (!x_f16 || !y || (reinterpret_cast<uintptr_t>(x_f16) & 3u) || (reinterpret_cast<uintptr_t>(y) & 7u))
        return TQ_ERR_INVALID_ARGUMENT;
    tq::tq_hadamard16_kernel<<<(tiles + 3u) / 4u, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        x_f16, y, out_dtype, tiles);
    return cudaGetLastError() == cudaSuccess ? TQ_OK : TQ_ERR_LAUNCH;
}

extern "C" int tq_lloydmax4_quantize(void* stream, const float* x, uint8_t* packed, float* recon,
                                     size_t count)
{
    if (count % 8u != 0u) return TQ_ERR_INVALID_ARGUMENT;
    if (count == 0) return TQ_OK;
    if (!x || !packed || (reinterpret_cast<uintptr_t>(x) & 15u) || (reinterpret_cast<uintptr_t>(packed) & 3u) ||
        (reinterpret_cast<uintptr_t>(recon) & 15u))
        return TQ_ERR_INVALID_ARGUMENT;
    const size_t groups = count / 8u, blocks = (groups + 255u) / 256u;
    if (blocks > 0x7FFFFFFFull) return TQ_ERR_INVALID_ARGUMENT;
    tq::tq_lloydmax4_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        x, reinterpret_cast<uint32_t*>(packed), recon, groups);
    return cudaGetLastError() == cudaSuccess ? TQ_OK : TQ_ERR_LAUNCH;
}

extern "C" int tq_icdf_quantize(void* stream, const uint16_t* x, uint32_t in_dtype, uint8_t* packed,
                                size_t count)
{
    if (count % 8u != 0u || (in_dtype != TQ_DTYPE_BF16 && in_dtype != TQ_DTYPE_F16))
        return TQ_ERR_INVALID_ARGUMENT;
    if (count == 0) return TQ_OK;
    if (!x || !packed || (reinterpret_cast<uintptr_t>(x) & 15u) || (reinterpret_cast<uintptr_t>(packed) & 3u))
        return TQ_ERR_INVALID_ARGUMENT;
    const size_t groups = count / 8u, blocks = (groups + 255u) / 256u;
    if (blocks > 0x7FFFFFFFull) return TQ_ERR_INVALID_ARGUMENT;
    tq::tq_icdf_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        x, in_dtype == TQ_DTYPE_BF16 ? 1u : 0u, reinterpret_cast<uint32_t*>(packed), groups);
    return cudaGetLastError() == cudaSuccess ? TQ_OK : TQ_ERR_LAUNCH;
}

// Pi q for `rows` FP16 or BF16 query vectors, FP32 out: the rotated image
// tq_decode_splitk_prerotated takes, with Pi = diag(pi_signs) H diag(pi_signs) / sqrt(head_size)
// (the fused decoder's raw-query prologue, include/turboquant_fused_decode_opt.hpp:160-169).
extern "C" int tq_rotate_query_pi(void* stream, const uint16_t* query, uint32_t elem_dtype,
                                  const float* pi_signs, float* query_rot, uint32_t rows,
                                  uint32_t head_size)
{
    if ((head_size != 128 && head_size != 256) || (elem_dtype != TQ_DTYPE_BF16 && elem_dtype != TQ_DTYPE_F16))
        return TQ_ERR_INVALID_ARGUMENT;
    if (rows == 0) return TQ_OK;
    if (!query || !pi_signs || !query_rot) return TQ_ERR_INVALID_ARGUMENT;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const unsigned blocks = (rows + 3u) / 4u;
    const uint32_t bf = elem_dtype == TQ_DTYPE_BF16 ? 1u : 0u;
    if (head_size == 128)
        tq::tq_rotate_query_pi_kernel<128><<<blocks, 128, 0, s>>>(query, bf, pi_signs, query_rot, rows, 0.08838834764831845f);
    else
        tq::tq_rotate_query_pi_kernel<256><<<blocks, 128, 0, s>>>(query, bf, pi_signs, query_rot, rows, 0.0625f);
    return cudaGetLastError() == cudaSuccess ? TQ_OK : TQ_ERR_LAUNCH;
}
