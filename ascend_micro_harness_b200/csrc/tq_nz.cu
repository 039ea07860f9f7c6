// Import of a KV4/FP8 cache in the NZ-tiled layout of the reference's fused decoder into this
// library's native page layout, so that such a cache can be decoded here
// (tq_decode_splitk_prerotated with the mid-rise code grid).
//
// Source format (head size 256 only, include/turboquant_fused_decode_opt.hpp:10,:85-88):
//   * packed planes, one pool for keys and one for values: inside a page of S slots (S = 64 or
//     128) the byte of packed column `column` (0..127) of (slot, kv head) sits at
//     NzTiledPackedByte(slot, head, column, H, 128)
//       = (slot - slot % 64) * H * 128 + head * 64 * 128 + ((column / 32) * 64 + slot % 64) * 32
//         + column % 32
//     (kernels/ops/turboquant/fused_decode/common/turboquant_layout.h:80-92): every
//     (64-row tile, kv head) is one contiguous 8 KiB image [column group][row][32 bytes];
//   * bits 3:0 of that byte are channel `column`, bits 7:4 channel `column + 128`
//     (tests/common/fused_decode_opt_fixture.hpp:286-293); a nibble is a two's-complement
//     code c that stands for (c + 0.5) * scale / gain (the uniform mid-rise grid b - 7.5 with
//     b = c + 8; fused_decode/common/turboquant_mode.h:100-124);
//   * scales: ceil(2H / 8) * 8 floats per slot, the H key scales first, then the H value
//     scales (fused_decode/common/turboquant_common.h:62-65; fixture :283-284).
//
// Destination: the native planes -- key token-major with channels 2j | 2j+1 in byte j, value
// channel-major inside each 16-token strip with tokens 2j | 2j+1 in byte j -- and the planar
// scale cache holding scale / gain (IEEE FP32 division). Codes are copied, never re-quantised,
// so the import loses nothing. Pages keep their numbers.
//
// One CTA of 128 threads per (page, 64-row tile, kv head): the two 8 KiB images are staged in
// shared memory; the key plane is a nibble re-pairing inside each row, the value plane a
// 16 x 8 nibble transpose done on 32-bit words with byte permutes.
#include "tq_common.cuh"

namespace tq {

constexpr int kNzTileRows = 64;
constexpr int kNzPacked = 128;                       // packed bytes per (slot, head) at head size 256
constexpr int kNzTileBytes = kNzTileRows * kNzPacked;  // 8192

struct NzImportParams {
    const uint8_t* nz_key;
    const uint8_t* nz_value;
    const float* nz_scales;
    uint8_t* key_cache;
    uint8_t* value_cache;
    float* scale_cache;
    uint32_t H, S, P, slot_floats;
    float gain;
};

__global__ void __launch_bounds__(128) tq_nz_kv4_import_kernel(const NzImportParams p)
{
    __shared__ __align__(16) uint8_t img[2][kNzTileBytes];
    const uint32_t tid = threadIdx.x;
    const uint32_t tiles_per_page = p.S / kNzTileRows;
    uint32_t lin = blockIdx.x;
    const uint32_t head = lin % p.H;
    lin /= p.H;
    const uint32_t tile = lin % tiles_per_page, page = lin / tiles_per_page;

    const size_t page_bytes = static_cast<size_t>(p.S) * p.H * kNzPacked;
    const size_t src_off = static_cast<size_t>(page) * page_bytes +
                           static_cast<size_t>(tile) * kNzTileRows * p.H * kNzPacked +
                           static_cast<size_t>(head) * kNzTileBytes;
    const uint4* ksrc = reinterpret_cast<const uint4*>(p.nz_key + src_off);
    const uint4* vsrc = reinterpret_cast<const uint4*>(p.nz_value + src_off);
#pragma unroll
    for (int i = 0; i < kNzTileBytes / 16 / 128; ++i) {
        reinterpret_cast<uint4*>(img[0])[i * 128 + tid] = __ldg(ksrc + i * 128 + tid);
        reinterpret_cast<uint4*>(img[1])[i * 128 + tid] = __ldg(vsrc + i * 128 + tid);
    }

    // scales: thread t < 64 the key scale of row t, thread 64 + t its value scale
    {
        const uint32_t plane = tid >> 6, row = tile * kNzTileRows + (tid & 63u);
        const float sc = __ldg(p.nz_scales + (static_cast<size_t>(page) * p.S + row) * p.slot_floats +
                               plane * p.H + head);
        p.scale_cache[((static_cast<size_t>(plane) * p.P + page) * p.H + head) * p.S + row] =
            __fdiv_rn(sc, p.gain);
    }
    __syncthreads();

    // native (page, head) block of either plane, and this tile's place in it
    const size_t block = (static_cast<size_t>(page) * p.H + head) * (static_cast<size_t>(p.S) * 128u) +
                         static_cast<size_t>(tile) * kNzTileBytes;

    // ---- key plane. Output chunk q (16 bytes = channels 32q .. 32q+31) of row t comes from the
    // 32-byte segment of column group q % 4: its low nibbles for q < 4, its high nibbles above.
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t item = i * 128 + tid, row = item >> 3, q = item & 7u;
        const uint4* seg = reinterpret_cast<const uint4*>(img[0] + ((q & 3u) * kNzTileRows + row) * 32);
        const uint4 a = seg[0], b = seg[1];
        const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        uint32_t o[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            // four source bytes -> two destination bytes, (byte 2e) | (byte 2e+1) << 4
            auto pair = [&](uint32_t word) {
                const uint32_t x = (q < 4u ? word : word >> 4) & 0x0F0F0F0Fu;
                return x | (x >> 4);   // bytes 0 and 2 hold the two results
            };
            o[k] = __byte_perm(pair(w[2 * k]), pair(w[2 * k + 1]), 0x6420u);
        }
        *reinterpret_cast<uint4*>(p.key_cache + block + row * 128u + q * 16u) = make_uint4(o[0], o[1], o[2], o[3]);
    }

    // ---- value plane. Thread = (strip s of the tile, packed word-column wc): the 16 words of
    // its tokens carry channels 4wc .. 4wc+3 (low nibbles) and 128 + 4wc .. (high nibbles).
    {
        const uint32_t s = tid >> 5, wc = tid & 31u;
        const uint8_t* colbase = img[1] + ((wc >> 3) * kNzTileRows + s * 16u) * 32 + (wc & 7u) * 4;
        uint32_t lo[8], hi[8];   // per token pair j: byte i = destination byte j of channel 4wc+i (or 128+4wc+i)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t w0 = *reinterpret_cast<const uint32_t*>(colbase + (2 * j) * 32);
            const uint32_t w1 = *reinterpret_cast<const uint32_t*>(colbase + (2 * j + 1) * 32);
            lo[j] = (w0 & 0x0F0F0F0Fu) | ((w1 & 0x0F0F0F0Fu) << 4);
            hi[j] = ((w0 >> 4) & 0x0F0F0F0Fu) | (w1 & 0xF0F0F0F0u);
        }
        // 8 x 4 byte transpose: channel i's eight bytes are byte i of words 0..7
        auto gather = [](const uint32_t (&v)[8], int i, int half) {
            const uint32_t sel = static_cast<uint32_t>(i) | (static_cast<uint32_t>(4 + i) << 4);
            const uint32_t ab = __byte_perm(v[4 * half], v[4 * half + 1], sel);
            const uint32_t cd = __byte_perm(v[4 * half + 2], v[4 * half + 3], sel);
            return __byte_perm(ab, cd, 0x5410u);
        };
        uint8_t* strip = p.value_cache + block + s * 2048u;
#pragma unroll
        for (int i = 0; i < 4; i += 2) {
            *reinterpret_cast<uint4*>(strip + (4u * wc + i) * 8u) =
                make_uint4(gather(lo, i, 0), gather(lo, i, 1), gather(lo, i + 1, 0), gather(lo, i + 1, 1));
            *reinterpret_cast<uint4*>(strip + (128u + 4u * wc + i) * 8u) =
                make_uint4(gather(hi, i, 0), gather(hi, i, 1), gather(hi, i + 1, 0), gather(hi, i + 1, 1));
        }
    }
}

}  // namespace tq

// Imports `num_blocks` pages of `block_size` (64 or 128) slots, `num_kv_heads` heads of size
// 256. nz_key / nz_value: num_blocks * block_size * num_kv_heads * 128 bytes each; nz_scales:
// num_blocks * block_size * ceil(2 num_kv_heads / 8) * 8 floats; key_cache / value_cache /
// scale_cache: the native pools of the same geometry (see tq_reshape_and_cache). gain is the
// codebook gain the decode divides out of the scales (2.9832882881 for KV4/FP8).
extern "C" int tq_nz_kv4_import(void* stream, const uint8_t* nz_key, const uint8_t* nz_value,
                                const float* nz_scales, int8_t* key_cache, int8_t* value_cache,
                                float* scale_cache, uint32_t num_kv_heads, uint32_t block_size,
                                uint32_t num_blocks, float gain)
{
    if (!num_kv_heads || (block_size != 64 && block_size != 128) || !(gain > 0.0f))
        return TQ_ERR_INVALID_ARGUMENT;
    if (num_blocks == 0) return TQ_OK;
    auto misaligned = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) != 0u; };
    if (!nz_key || !nz_value || !nz_scales || !key_cache || !value_cache || !scale_cache ||
        misaligned(nz_key) || misaligned(nz_value) || misaligned(key_cache) || misaligned(value_cache))
        return TQ_ERR_INVALID_ARGUMENT;
    const uint64_t grid = static_cast<uint64_t>(num_blocks) * (block_size / tq::kNzTileRows) * num_kv_heads;
    if (grid > 0x7FFFFFFFull) return TQ_ERR_INVALID_ARGUMENT;
    tq::NzImportParams p{nz_key,
                         nz_value,
                         nz_scales,
                         reinterpret_cast<uint8_t*>(key_cache),
                         reinterpret_cast<uint8_t*>(value_cache),
                         scale_cache,
                         num_kv_heads,
                         block_size,
                         num_blocks,
                         (2u * num_kv_heads + 7u) / 8u * 8u,
                         gain};
    tq::tq_nz_kv4_import_kernel<<<static_cast<unsigned>(grid), 128, 0, static_cast<cudaStream_t>(stream)>>>(p);
    return cudaGetLastError() == cudaSuccess ? TQ_OK : TQ_ERR_LAUNCH;
}
