// The cache variant built from the reference's stand-alone routines -- block-diagonal
// 16x16 Sylvester Hadamard rotation, per-token RMS scale, 16-level Lloyd-Max codes -- in
// the same planes as the power-of-two cache (key token-major, value channel-major per
// 16-token strip, planar FP32 scales):
//   writer   y = x H16 per 16-channel block, y_rot = y / 4,
//            scale = sqrt(sum y_rot^2) * inv_sqrt_len + 1e-20
//            (kernels/ops/turboquant/baseline/common/turboquant_codec_950.h:194-207),
//            code = lloydmax(y_rot * (1 / scale))
//            (include/routines/routine_vector_lloydmax_quantize.hpp:32-38), unsigned, low
//            nibble first (tests/common/lloydmax_oracle.hpp:65-69);
//   decode   q_rot = bf16((q H16 per block) / 4), score = sum q_rot centroid[K] * kscale *
//            softmax_scale, acc += p * vscale * centroid[V], per-split {m x8, l x8, acc[d]}
//            records in the layout of include/turboquant_splitk_contract.hpp:23-27, merged by
//            the ordinary combine kernel with the block-diagonal egress.
// The reference pins the stages (Hadamard tile, codec), not this composite. Its arithmetic is
// fixed here operation by operation (butterfly order, squares summed four at a time in FP32,
// the groups in FP64 per half of the channels, IEEE sqrt / divide / multiply without fusion),
// so the CPU restatement reproduces every scale bit and every code for any finite input.
#include <cuda_fp16.h>

#include "tq_lloydmax.cuh"

namespace tq {

// ------------------------------------------------------------------- writer
struct LmWriterParams {
    const void* key;
    const void* value;
    uint8_t* key_cache;
    uint8_t* value_cache;
    float* scale_cache;
    const int32_t* slots;
    uint32_t num_strips, H, S, P, bf16;
    float inv_sqrt_len;
    uint32_t* status;
};

// One warp per (strip, plane, head) panel: lane = (channel half, token). A lane rotates
// and quantises d/2 channels of its token; the value page's byte (channel, token pair) is
// assembled after one exchange with the neighbouring token's lane.
template <int D>
__global__ void __launch_bounds__(128) tq_lm_writer_kernel(const LmWriterParams p)
{
    constexpr int kHalf = D / 2;            // channels per lane
    constexpr int kBlocks = kHalf / 16;     // Hadamard blocks per lane
    constexpr int kWords = kHalf / 8;       // packed words per lane
    __shared__ __align__(16) uint8_t stage_all[4][kStrip * D / 2];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = lane & 15, hsel = lane >> 4;
    uint8_t* stage = stage_all[warp];
    const uint64_t panels = static_cast<uint64_t>(p.num_strips) * 2u * p.H;
    for (uint64_t panel = static_cast<uint64_t>(blockIdx.x) * 4u + warp; panel < panels;
         panel += static_cast<uint64_t>(gridDim.x) * 4u) {
        const uint32_t strip = static_cast<uint32_t>(panel / (2u * p.H));
        const uint32_t rem = static_cast<uint32_t>(panel % (2u * p.H));
        const uint32_t plane = rem >= p.H ? 1u : 0u, head = rem - plane * p.H;
        // the strip's slot run, checked as in the power-of-two writer
        const int32_t slot = __ldg(p.slots + static_cast<size_t>(strip) * kStrip + t);
        const int32_t slot0 = __shfl_sync(0xffffffffu, slot, 0);
        const bool ok = __all_sync(0xffffffffu, slot == slot0 + t) && slot0 >= 0 &&
                        (slot0 % kStrip) == 0 && static_cast<uint32_t>(slot0) / p.S < p.P;
        if (!ok) {
            if (lane == 0) report(p.status, TQ_STATUS_BAD_SLOT);
            continue;
        }
        const uint32_t page = static_cast<uint32_t>(slot0) / p.S, tip = static_cast<uint32_t>(slot0) % p.S;

        // ---- this lane's d/2 channels of token t
        float y[kHalf];
        const size_t row = (static_cast<size_t>(strip) * kStrip + t) * p.H * D + static_cast<size_t>(head) * D +
                           hsel * kHalf;
        if (p.bf16 != 0u) {
            const uint4* src = reinterpret_cast<const uint4*>(
                static_cast<const uint16_t*>(plane == 0 ? p.key : p.value) + row);
#pragma unroll
            for (int i = 0; i < kHalf / 8; ++i) {
                const uint4 raw = __ldg(src + i);
                const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    y[i * 8 + 2 * j] = __uint_as_float(w[j] << 16);
                    y[i * 8 + 2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
                }
            }
        } else {
            const uint4* src = reinterpret_cast<const uint4*>(
                static_cast<const int8_t*>(plane == 0 ? p.key : p.value) + row);
#pragma unroll
            for (int i = 0; i < kHalf / 16; ++i) {
                const uint4 raw = __ldg(src + i);
                const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int j = 0; j < 4; ++j)
#pragma unroll
                    for (int b = 0; b < 4; ++b)
                        y[i * 16 + j * 4 + b] = static_cast<float>(static_cast<int8_t>(w[j] >> (8 * b)));
            }
        }
        double s2 = 0.0;
#pragma unroll
        for (int b = 0; b < kBlocks; ++b) {
            float v[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = y[b * 16 + i];
            hadamard16_inplace(v);
#pragma unroll
            for (int i = 0; i < 16; ++i) y[b * 16 + i] = v[i];
            // squares summed four at a time in FP32 (exact for int8-range integers: 4 * 2032^2
            // < 2^24), the groups in FP64, in channel order
#pragma unroll
            for (int i = 0; i < 16; i += 4) {
                float q4 = __fmul_rn(v[i], v[i]);
                q4 = __fadd_rn(q4, __fmul_rn(v[i + 1], v[i + 1]));
                q4 = __fadd_rn(q4, __fmul_rn(v[i + 2], v[i + 2]));
                q4 = __fadd_rn(q4, __fmul_rn(v[i + 3], v[i + 3]));
                s2 += static_cast<double>(q4);
            }
        }
        {   // first half of the channels + second half, in that order on both lanes
            const double other = __shfl_xor_sync(0xffffffffu, s2, 16);
            s2 = hsel == 0 ? s2 + other : other + s2;
        }
        const float root = static_cast<float>(sqrt(s2));
        const float scale = __fadd_rn(__fmul_rn(__fmul_rn(root, 0.25f), p.inv_sqrt_len), 1e-20f);
        const float inv = __fdiv_rn(1.0f, scale);
        uint32_t words[kWords];
#pragma unroll
        for (int w = 0; w < kWords; ++w) {
            uint32_t packed = 0;
#pragma unroll
            for (int e = 0; e < 8; ++e)
                packed |= lloydmax4_code(__fmul_rn(__fmul_rn(y[w * 8 + e], 0.25f), inv)) << (4 * e);
            words[w] = packed;
        }
        if (hsel == 0)
            p.scale_cache[((static_cast<size_t>(plane) * p.P + page) * p.H + head) * p.S + tip + t] = scale;

        uint8_t* dst = (plane == 0 ? p.key_cache : p.value_cache) +
                       (static_cast<size_t>(page) * p.H + head) * (static_cast<size_t>(p.S) * D / 2) +
                       static_cast<size_t>(tip / kStrip) * (kStrip * D / 2);
        __syncwarp();   // the previous panel's copy-out has finished reading the stage
        if (plane == 0) {
            // key page, token-major: the lane's d/4 bytes of row t
            uint4* srow = reinterpret_cast<uint4*>(stage + t * (D / 2) + hsel * (D / 4));
#pragma unroll
            for (int i = 0; i < kWords / 4; ++i)
                srow[i] = make_uint4(words[4 * i], words[4 * i + 1], words[4 * i + 2], words[4 * i + 3]);
        } else {
            // value page, channel-major: byte (channel, t / 2) = code(t even) | code(t odd) << 4.
            // The even-token lane assembles the first half of its channels, the odd one the rest.
#pragma unroll
            for (int w = 0; w < kWords; ++w) {
                const uint32_t other = __shfl_xor_sync(0xffffffffu, words[w], 1);
                const bool mine = ((w < kWords / 2) == ((t & 1) == 0));
                const uint32_t even = (t & 1) ? other : words[w], odd = (t & 1) ? words[w] : other;
                if (mine) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const uint32_t byte = ((even >> (4 * e)) & 0xFu) | (((odd >> (4 * e)) & 0xFu) << 4);
                        stage[(hsel * kHalf + w * 8 + e) * 8 + (t >> 1)] = static_cast<uint8_t>(byte);
                    }
                }
            }
        }
        __syncwarp();
        const uint4* s4 = reinterpret_cast<const uint4*>(stage);
#pragma unroll
        for (int i = 0; i < kStrip * D / 2 / 16 / 32; ++i)
            __stcs(reinterpret_cast<uint4*>(dst) + i * 32 + lane, s4[i * 32 + lane]);
    }
}

// ------------------------------------------------------------------- decode
struct LmDecodeParams {
    const uint16_t* q;            // [batch][Hq][D] bf16
    const uint8_t* key_cache;
    const uint8_t* value_cache;
    const float* scale_cache;
    const int32_t* table;
    const int32_t* context_lens;
    float* workspace;             // [item][split][rows]{m x8, l x8, acc[D]}
    uint32_t items, H, rows, S, P, table_stride, splits;
    float softmax_scale;
    uint32_t* status;
    // A cache on another 16-level codebook (the fused decoder's Lloyd-Max toggle): the query is
    // FP32 and already in the cache's basis (q_f32 != null: no rotation), and a stored nibble n
    // stands for levels[n ^ 8] (bin b is stored as the signed nibble b - 8).
    const float* q_f32 = nullptr;
    float levels[16] = {};
};

constexpr float kLmLog2e = 1.4426950408889634f;

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1)
{
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void cp_async16(uint32_t smem_dst, const void* gmem_src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_dst), "l"(gmem_src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait()
{
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}
__device__ __forceinline__ uint32_t lm_movmatrix_trans(uint32_t a)
{
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
    return d;
}
__device__ __forceinline__ float lm_ex2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t lm_pack_f16x2(float lo, float hi)
{
    uint32_t d;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;\n" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}

template <int D>
struct LmDecodeSmem {
    static constexpr int kStages = 2;
    static constexpr int kStripBytes = kStrip * D / 2;
    static constexpr int kBufBytes = 2 * kStripBytes + 128;          // key strip, value strip, two scale runs
    static constexpr int kLutBytes = 256 * 32 * 4;                   // one copy of the table per bank
    static constexpr int kRingBytes = 4 * kStages * kBufBytes;
    static constexpr int kQueryBytes = 8 * D * 4;
    static constexpr int kMergeBytes = 4 * 8 * (D + 2) * 4;          // reuses ring + query after the loop
    static constexpr int kTotal = kLutBytes + kRingBytes + kQueryBytes;
    static constexpr int kCtasPerSm = D == 128 ? 4 : 3;
    static_assert(kMergeBytes <= kRingBytes + kQueryBytes, "the merge area must fit the ring");
};

// One CTA per (sequence, KV head, split); up to 8 query rows (the GQA group). Four warps
// take the strips of the split's page range in turn, each through its own 2-stage cp.async
// ring (a strip's key block, value block and two scale runs). Codes become f16 centroids
// through a byte -> (centroid[low nibble], centroid[high nibble]) table that is kept 32
// times in shared memory, entry e of lane l at word 32 e + l, so a lookup never leaves the
// lane's own bank; both contractions are f16 tensor-core MMAs with tokens as the M
// dimension. P carries the value scale relative to a running power-of-two normaliser, and
// the accumulator is rescaled only by strips that raise a row maximum or that normaliser.
template <int D, bool WIDE_Q>
__global__ void __launch_bounds__(128, LmDecodeSmem<D>::kCtasPerSm) tq_lm_decode_kernel(const LmDecodeParams p)
{
    using L = LmDecodeSmem<D>;
    constexpr int kRecord = 16 + D;
    constexpr int kStripBytes = L::kStripBytes;
    constexpr int MT = D / 16;
    constexpr int kChunks = D / 2 / 16 / 4;   // 16-byte chunks of a key row per thread: 1 or 2
    extern __shared__ __align__(128) uint8_t lm_smem[];
    uint32_t* lut = reinterpret_cast<uint32_t*>(lm_smem);
    uint8_t* ring = lm_smem + L::kLutBytes;
    float (*qs)[D] = reinterpret_cast<float (*)[D]>(ring + L::kRingBytes);
    float (*merge)[8][D + 2] = reinterpret_cast<float (*)[8][D + 2]>(ring);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, r = lane >> 2, qd = lane & 3;
    const uint32_t split = blockIdx.x % p.splits, item = blockIdx.x / p.splits;
    const uint32_t seq = item / p.H, head = item % p.H;

    // page range of this split (include/turboquant_splitk_contract.hpp:129-136)
    const int32_t c0 = p.context_lens[seq];
    const uint32_t ctx = c0 > 0 ? min(static_cast<uint32_t>(c0), p.table_stride * p.S) : 0u;
    const uint32_t pages = (ctx + p.S - 1u) / p.S;
    const uint32_t width = (pages + p.splits - 1u) / p.splits;
    const uint32_t pb = min(split * width, pages), pe = min(pb + width, pages);
    const uint32_t SP = p.S / kStrip;
    const uint32_t s0 = pb * SP, s1 = min(pe * SP, (ctx + kStrip - 1u) / kStrip);
    float* rec = p.workspace + (static_cast<size_t>(item) * p.splits + split) * p.rows * kRecord;
    if (s1 <= s0) {   // nothing to read: the neutral record
        for (int i = tid; i < static_cast<int>(p.rows) * kRecord; i += blockDim.x)
            rec[i] = (i % kRecord) < 8 ? kMaskedScore : 0.0f;
        return;
    }

    // byte -> packed (centroid[low nibble], centroid[high nibble]) as f16: the 256 entries
    // first (lane 0's copy), then the other 31 copies
    for (int i = tid; i < 256; i += blockDim.x) {
        const __half2 h = p.q_f32 != nullptr
                              ? __floats2half2_rn(p.levels[(i & 15) ^ 8], p.levels[(i >> 4) ^ 8])
                              : __floats2half2_rn(lloydmax4_centroid(i & 15), lloydmax4_centroid(i >> 4));
        lut[i * 32] = *reinterpret_cast<const uint32_t*>(&h);
    }
    // q_rot: FP32 butterfly inside each 16-channel block, / 4, bf16 (or the caller's rotated FP32 rows)
    for (int i = tid; i < 8 * (D / 16); i += blockDim.x) {
        const int row = i / (D / 16), blk = i % (D / 16);
        if (p.q_f32 != nullptr) {
#pragma unroll
            for (int k = 0; k < 16; ++k)
                qs[row][blk * 16 + k] = row < static_cast<int>(p.rows)
                                            ? p.q_f32[(static_cast<size_t>(item) * p.rows + row) * D + blk * 16 + k]
                                            : 0.f;
            continue;
        }
        float v[16];
#pragma unroll
        for (int k = 0; k < 16; ++k)
            v[k] = row < static_cast<int>(p.rows)
                       ? bf16_bits_to_f32(p.q[(static_cast<size_t>(item) * p.rows + row) * D + blk * 16 + k])
                       : 0.f;
        hadamard16_inplace(v);
#pragma unroll
        for (int k = 0; k < 16; ++k) qs[row][blk * 16 + k] = bf16_bits_to_f32(f32_to_bf16_bits(v[k] * 0.25f));
    }
    __syncthreads();
    for (int i = tid; i < 256 * 32; i += blockDim.x)
        if ((i & 31) != 0) lut[i] = lut[i & ~31];

    // B fragments of q_rot^T: MMA j of a key row takes this thread's bytes 2j, 2j+1, i.e.
    // channels qd*(D/4) + 4j .. 4j+3
    // An FP32 query (q_f32) is carried as two f16 halves, hi + lo, so that its rounding to f16
    // (2^-11 relative, which a bf16 query never sees: it is exact in f16) does not reach the logits.
    constexpr bool wide_q = WIDE_Q;   // the instantiation an FP32 query gets
    uint32_t bq[D / 16][2];
    [[maybe_unused]] uint32_t bq_lo[WIDE_Q ? D / 16 : 1][2];
#pragma unroll
    for (int j = 0; j < D / 16; ++j) {
        const float* qr = &qs[r][qd * (D / 4) + 4 * j];
        bq[j][0] = lm_pack_f16x2(qr[0], qr[1]);
        bq[j][1] = lm_pack_f16x2(qr[2], qr[3]);
        if constexpr (WIDE_Q) {
            const __half2 h0 = *reinterpret_cast<const __half2*>(&bq[j][0]),
                          h1 = *reinterpret_cast<const __half2*>(&bq[j][1]);
            bq_lo[j][0] = lm_pack_f16x2(qr[0] - __low2float(h0), qr[1] - __high2float(h0));
            bq_lo[j][1] = lm_pack_f16x2(qr[2] - __low2float(h1), qr[3] - __high2float(h1));
        }
    }
    __syncthreads();   // the table is complete

    // Online-softmax state for query rows 2qd and 2qd+1, in units of raw * key_scale.
    const float fac = p.softmax_scale * kLmLog2e;
    float m_run[2] = {kMaskedScore, kMaskedScore}, l_run[2] = {0.f, 0.f};
    float m_fac[2] = {0.f, 0.f};   // m_run * fac, the exponent offset (0 while m_run is the sentinel)
    float vnorm = 0.f, inv_vnorm = 0.f;   // running power-of-two bound of the value scales
    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[mt][i] = 0.f;

    uint8_t* my_ring = ring + warp * L::kStages * L::kBufBytes;
    const uint32_t my_ring_s = smem_u32(my_ring);
    const uint32_t* my_lut = lut + lane;   // entry e of this lane: my_lut[32 e]
    const int32_t* table_row = p.table + static_cast<size_t>(seq) * p.table_stride;
    const size_t head_block = static_cast<size_t>(p.S) * D / 2;
    auto load_page = [&](uint32_t strip) { return strip < s1 ? __ldg(table_row + strip / SP) : -1; };
    auto issue = [&](uint32_t strip, uint32_t stage, int32_t pg) {
        if (pg < 0 && strip >= s1) return;   // warp-uniform: past the range
        if (pg < 0 || static_cast<uint32_t>(pg) >= p.P) {
            if (lane == 0) report(p.status, TQ_STATUS_BAD_PAGE);
            pg = 0;
        }
        const size_t block = (static_cast<size_t>(pg) * p.H + head) * head_block +
                             static_cast<size_t>(strip % SP) * kStripBytes;
        const uint8_t* ks = p.key_cache + block + lane * 16;
        const uint8_t* vs = p.value_cache + block + lane * 16;
        const uint32_t dst = my_ring_s + stage * L::kBufBytes + lane * 16;
#pragma unroll
        for (int i = 0; i < kStripBytes / 16 / 32; ++i) {
            cp_async16(dst + i * 512, ks + i * 512);
            cp_async16(dst + kStripBytes + i * 512, vs + i * 512);
        }
        if (lane < 8) {
            const size_t sc = ((static_cast<size_t>(lane >> 2) * p.P + pg) * p.H + head) * p.S +
                              (strip % SP) * kStrip + (lane & 3) * 4;
            cp_async16(my_ring_s + stage * L::kBufBytes + 2 * kStripBytes + lane * 16, p.scale_cache + sc);
        }
    };

    // byte k of a word as a table offset (in words): 32 * byte
    auto entry = [&](uint32_t word, int k) { return my_lut[__byte_perm(word, 0u, 0x4440u | k) << 5]; };

    issue(s0 + warp, 0, load_page(s0 + warp));
    cp_async_commit();
    int32_t pg_next = load_page(s0 + warp + 4u);
    uint32_t stage = 0;
#pragma unroll 1
    for (uint32_t strip = s0 + warp; strip < s1; strip += 4u) {
        issue(strip + 4u, stage ^ 1u, pg_next);
        cp_async_commit();
        pg_next = load_page(strip + 8u);
        cp_async_wait<1>();
        __syncwarp();
        const uint8_t* buf = my_ring + stage * L::kBufBytes;
        stage ^= 1u;
        const float* scales = reinterpret_cast<const float*>(buf + 2 * kStripBytes);

        // ---- scores^T: rows = tokens r and r+8, columns = query rows
        float c[4] = {0.f, 0.f, 0.f, 0.f}, c_lo[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ch = 0; ch < kChunks; ++ch) {
            const uint4 lo = *reinterpret_cast<const uint4*>(buf + r * (D / 2) + (qd * kChunks + ch) * 16);
            const uint4 hi = *reinterpret_cast<const uint4*>(buf + (r + 8) * (D / 2) + (qd * kChunks + ch) * 16);
            const uint32_t wl[4] = {lo.x, lo.y, lo.z, lo.w}, wh[4] = {hi.x, hi.y, hi.z, hi.w};
#pragma unroll
            for (int w = 0; w < 4; ++w)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int j = ch * 8 + w * 2 + h;   // bytes 2j, 2j+1 of this thread's part of the row
                    const uint32_t a0 = entry(wl[w], 2 * h), a1 = entry(wh[w], 2 * h), a2 = entry(wl[w], 2 * h + 1),
                                   a3 = entry(wh[w], 2 * h + 1);
                    mma_f16(c, a0, a1, a2, a3, bq[j][0], bq[j][1]);
                    if constexpr (WIDE_Q) mma_f16(c_lo, a0, a1, a2, a3, bq_lo[j][0], bq_lo[j][1]);
                }
        }
        if constexpr (wide_q) {
#pragma unroll
            for (int i = 0; i < 4; ++i) c[i] += c_lo[i];
        }
        const uint32_t tok_lo = strip * kStrip + r, tok_hi = tok_lo + 8;
        const bool live_lo = tok_lo < ctx, live_hi = tok_hi < ctx;
        float sc[4];
        sc[0] = live_lo ? c[0] * scales[r] : kMaskedScore;
        sc[1] = live_lo ? c[1] * scales[r] : kMaskedScore;
        sc[2] = live_hi ? c[2] * scales[r + 8] : kMaskedScore;
        sc[3] = live_hi ? c[3] * scales[r + 8] : kMaskedScore;
        const float vs_lo = live_lo ? scales[kStrip + r] : 0.f, vs_hi = live_hi ? scales[kStrip + r + 8] : 0.f;
        float mx[2] = {fmaxf(sc[0], sc[2]), fmaxf(sc[1], sc[3])};
        float vmax = fmaxf(fabsf(vs_lo), fabsf(vs_hi));
        // m_run and vnorm are uniform over the lanes that share them: only a strip that raises
        // a row maximum or the normaliser pays for the reductions and the rescale
        const bool grow = mx[0] > m_run[0] || mx[1] > m_run[1] || vmax > vnorm;
        if (__any_sync(0xffffffffu, grow)) {
#pragma unroll
            for (int o = 4; o <= 16; o <<= 1) {
                mx[0] = fmaxf(mx[0], __shfl_xor_sync(0xffffffffu, mx[0], o));
                mx[1] = fmaxf(mx[1], __shfl_xor_sync(0xffffffffu, mx[1], o));
                vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, o));
            }
            float alpha[2];
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const float m_new = fmaxf(m_run[q], mx[q]);
                alpha[q] = lm_ex2((m_run[q] - m_new) * fac);
                m_run[q] = m_new;
                m_fac[q] = m_new > -1.0e37f ? m_new * fac : 0.f;
                l_run[q] *= alpha[q];
            }
            if (vmax > vnorm) {   // warp-uniform: value scales depend on the token only
                const float nv = __int_as_float((__float_as_int(vmax) & 0x7F800000) + (1 << 23));
                inv_vnorm = __int_as_float((254 << 23) - __float_as_int(nv));
                alpha[0] *= vnorm * inv_vnorm;
                alpha[1] *= vnorm * inv_vnorm;
                vnorm = nv;
            }
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                acc[mt][0] *= alpha[0];
                acc[mt][1] *= alpha[1];
                acc[mt][2] *= alpha[0];
                acc[mt][3] *= alpha[1];
            }
        }
        float pw[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float pr = lm_ex2(fmaf(sc[i], fac, -m_fac[i & 1]));
            l_run[i & 1] += pr;
            pw[i] = pr * ((i < 2 ? vs_lo : vs_hi) * inv_vnorm);
        }
        // P^T as the B operand: tokens 2qd, 2qd+1 (from rows r) and 8+2qd, 8+2qd+1 (rows r+8)
        const uint32_t bh0 = lm_movmatrix_trans(lm_pack_f16x2(pw[0], pw[1]));
        const uint32_t bh1 = lm_movmatrix_trans(lm_pack_f16x2(pw[2], pw[3]));
        // ---- acc^T += V^T P^T: MMA rows r and r+8 = channels mt*16 + 2r and + 2r+1 (one
        // 16-byte read), contraction = tokens: byte qd of a channel's first word holds tokens
        // 2qd, 2qd+1, byte qd of its second word tokens 8+2qd, 8+2qd+1
        const uint8_t* vrow = buf + kStripBytes + (2 * r) * 8;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            const uint4 v = *reinterpret_cast<const uint4*>(vrow + mt * 128);
            mma_f16(acc[mt], entry(v.x, qd), entry(v.z, qd), entry(v.y, qd), entry(v.w, qd), bh0, bh1);
        }
        __syncwarp();   // the stage is free for the copy two iterations ahead
    }
    cp_async_wait<0>();

    // ---- merge the four warps, export the record
    __syncthreads();   // every warp is done with its ring: the merge area reuses it
#pragma unroll
    for (int q = 0; q < 2; ++q) {
        l_run[q] += __shfl_xor_sync(0xffffffffu, l_run[q], 4);
        l_run[q] += __shfl_xor_sync(0xffffffffu, l_run[q], 8);
        l_run[q] += __shfl_xor_sync(0xffffffffu, l_run[q], 16);
    }
    if (r == 0) {
        merge[warp][qd * 2 + 0][0] = m_run[0];
        merge[warp][qd * 2 + 0][1] = l_run[0];
        merge[warp][qd * 2 + 1][0] = m_run[1];
        merge[warp][qd * 2 + 1][1] = l_run[1];
    }
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        const int ch = mt * 16 + 2 * r;
        *reinterpret_cast<float2*>(&merge[warp][qd * 2 + 0][2 + ch]) =
            make_float2(acc[mt][0] * vnorm, acc[mt][2] * vnorm);
        *reinterpret_cast<float2*>(&merge[warp][qd * 2 + 1][2 + ch]) =
            make_float2(acc[mt][1] * vnorm, acc[mt][3] * vnorm);
    }
    __syncthreads();
    for (int i = tid; i < static_cast<int>(p.rows) * kRecord; i += blockDim.x) {
        const int q = i / kRecord, cc = i % kRecord;
        float mm = kMaskedScore;
#pragma unroll
        for (int w = 0; w < 4; ++w) mm = fmaxf(mm, merge[w][q][0]);
        float out;
        if (cc < 8) {
            out = mm > -1.0e37f ? mm * p.softmax_scale : kMaskedScore;   // natural-log units
        } else {
            const int src = cc < 16 ? 1 : 2 + (cc - 16);
            out = 0.f;
#pragma unroll
            for (int w = 0; w < 4; ++w) out += merge[w][q][src] * lm_ex2((merge[w][q][0] - mm) * fac);
        }
        rec[i] = out;
    }
}

template <int D, bool WIDE_Q = false>
static cudaError_t launch_lm_decode(cudaStream_t stream, const LmDecodeParams& p, unsigned grid)
{
    // Opt in to the large dynamic shared-memory carve-out once per device.
    static bool configured[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return cudaErrorNoDevice;
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        const cudaError_t e = cudaFuncSetAttribute(tq_lm_decode_kernel<D, WIDE_Q>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   LmDecodeSmem<D>::kTotal);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    tq_lm_decode_kernel<D, WIDE_Q><<<grid, 128, LmDecodeSmem<D>::kTotal, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace tq

using namespace tq;

extern "C" int tq_reshape_and_cache_lloydmax(void* stream, const void* key, const void* value,
                                             int8_t* key_cache, int8_t* value_cache,
                                             float* scale_cache, const int32_t* slot_mapping,
                                             uint32_t in_dtype, uint32_t num_tokens,
                                             uint32_t num_kv_heads, uint32_t head_size,
                                             uint32_t block_size, uint32_t num_blocks,
                                             float inv_sqrt_len, uint32_t* status)
{
    if (!num_kv_heads || !num_blocks || !block_size || block_size % kStrip != 0 ||
        (head_size != 128 && head_size != 256) || in_dtype > TQ_IN_BF16)
        return TQ_ERR_INVALID_ARGUMENT;
    if (num_tokens % kStrip != 0) return TQ_ERR_PARTIAL_STRIP;
    if (num_tokens == 0) return TQ_OK;
    if (!key || !value || !key_cache || !value_cache || !scale_cache || !slot_mapping)
        return TQ_ERR_INVALID_ARGUMENT;
    const uintptr_t align = reinterpret_cast<uintptr_t>(key) | reinterpret_cast<uintptr_t>(value) |
                            reinterpret_cast<uintptr_t>(key_cache) | reinterpret_cast<uintptr_t>(value_cache);
    if (align & 15u) return TQ_ERR_INVALID_ARGUMENT;
    LmWriterParams p{key, value, reinterpret_cast<uint8_t*>(key_cache), reinterpret_cast<uint8_t*>(value_cache),
                     scale_cache, slot_mapping, num_tokens / kStrip, num_kv_heads, block_size, num_blocks,
                     in_dtype == TQ_IN_BF16 ? 1u : 0u, inv_sqrt_len, status};
    const uint64_t panels = static_cast<uint64_t>(p.num_strips) * 2u * num_kv_heads;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) != cudaSuccess) return TQ_ERR_NO_DEVICE;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const uint64_t want = (panels + 3u) / 4u, cap = static_cast<uint64_t>(sms) * 8u;
    const unsigned blocks = static_cast<unsigned>(want < cap ? want : cap);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (head_size == 128) tq_lm_writer_kernel<128><<<blocks, 128, 0, s>>>(p);
    else tq_lm_writer_kernel<256><<<blocks, 128, 0, s>>>(p);
    return cudaGetLastError() == cudaSuccess ? TQ_OK : TQ_ERR_LAUNCH;
}

// The split-K export over native planes whose codes index a caller's 16-level table (levels by
// bin index; nibble n is bin n ^ 8), with a pre-rotated FP32 query [batch][num_heads][d]: the
// read side of the fused decoder's Lloyd-Max toggle after tq_nz_kv4_import with gain 1.
extern "C" int tq_decode_levels_export(void* stream, const float* query_rot, const float* levels16,
                                       const int8_t* key_cache, const int8_t* value_cache,
                                       const float* scale_cache, const int32_t* block_tables,
                                       const int32_t* context_lens, float* workspace, uint32_t batch,
                                       uint32_t num_heads, uint32_t num_kv_heads, uint32_t head_size,
                                       uint32_t block_size, uint32_t num_blocks, uint32_t max_blocks,
                                       uint32_t splits, float softmax_scale, uint32_t* status)
{
    if (!num_heads || !num_kv_heads || num_heads % num_kv_heads != 0 || !block_size ||
        block_size % kStrip != 0 || !num_blocks || !max_blocks || !splits || splits > 16 ||
        (head_size != 128 && head_size != 256) || num_heads / num_kv_heads > 8 || !levels16 ||
        !(softmax_scale > 0.0f) || !(softmax_scale <= 3.0e38f))
        return TQ_ERR_INVALID_ARGUMENT;
    if (batch == 0) return TQ_OK;
    if (!query_rot || !key_cache || !value_cache || !scale_cache || !block_tables || !context_lens || !workspace)
        return TQ_ERR_INVALID_ARGUMENT;
    const uintptr_t align = reinterpret_cast<uintptr_t>(key_cache) | reinterpret_cast<uintptr_t>(value_cache) |
                            reinterpret_cast<uintptr_t>(scale_cache);
    if (align & 15u) return TQ_ERR_INVALID_ARGUMENT;
    LmDecodeParams p{nullptr, reinterpret_cast<const uint8_t*>(key_cache),
                     reinterpret_cast<const uint8_t*>(value_cache), scale_cache, block_tables, context_lens,
                     workspace, batch * num_kv_heads, num_kv_heads, num_heads / num_kv_heads, block_size,
                     num_blocks, max_blocks, splits, softmax_scale, status};
    p.q_f32 = query_rot;
    for (int i = 0; i < 16; ++i) {
        if (!(levels16[i] == levels16[i]) || levels16[i] > 60000.0f || levels16[i] < -60000.0f)
            return TQ_ERR_INVALID_ARGUMENT;   // the table is carried in f16
        p.levels[i] = levels16[i];
    }
    const uint64_t grid = static_cast<uint64_t>(p.items) * splits;
    if (grid > 0x7FFFFFFFull) return TQ_ERR_INVALID_ARGUMENT;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const cudaError_t e = head_size == 128 ? launch_lm_decode<128, true>(s, p, static_cast<unsigned>(grid))
                                           : launch_lm_decode<256, true>(s, p, static_cast<unsigned>(grid));
    return e == cudaSuccess ? TQ_OK : TQ_ERR_LAUNCH;
}

extern "C" int tq_decode_lloydmax_export(void* stream, const uint16_t* query, const int8_t* key_cache,
                                         const int8_t* value_cache, const float* scale_cache,
                                         const int32_t* block_tables, const int32_t* context_lens,
                                         float* workspace, uint32_t batch, uint32_t num_heads,
                                         uint32_t num_kv_heads, uint32_t head_size,
                                         uint32_t block_size, uint32_t num_blocks,
                                         uint32_t max_blocks, uint32_t splits, float softmax_scale,
                                         uint32_t* status)
{
    if (!num_heads || !num_kv_heads || num_heads % num_kv_heads != 0 || !block_size ||
        block_size % kStrip != 0 || !num_blocks || !max_blocks || !splits || splits > 16 ||
        (head_size != 128 && head_size != 256) || num_heads / num_kv_heads > 8)
        return TQ_ERR_INVALID_ARGUMENT;
    if (batch == 0) return TQ_OK;
    if (!query || !key_cache || !value_cache || !scale_cache || !block_tables || !context_lens || !workspace)
        return TQ_ERR_INVALID_ARGUMENT;
    const uintptr_t align = reinterpret_cast<uintptr_t>(key_cache) | reinterpret_cast<uintptr_t>(value_cache) |
                            reinterpret_cast<uintptr_t>(scale_cache);
    if (align & 15u) return TQ_ERR_INVALID_ARGUMENT;
    LmDecodeParams p{query, reinterpret_cast<const uint8_t*>(key_cache),
                     reinterpret_cast<const uint8_t*>(value_cache), scale_cache, block_tables, context_lens,
                     workspace, batch * num_kv_heads, num_kv_heads, num_heads / num_kv_heads, block_size,
                     num_blocks, max_blocks, splits, softmax_scale, status};
    const uint64_t grid = static_cast<uint64_t>(p.items) * splits;
    if (grid > 0x7FFFFFFFull) return TQ_ERR_INVALID_ARGUMENT;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const cudaError_t e = head_size == 128 ? launch_lm_decode<128>(s, p, static_cast<unsigned>(grid))
                                           : launch_lm_decode<256>(s, p, static_cast<unsigned>(grid));
    return e == cudaSuccess ? TQ_OK : TQ_ERR_LAUNCH;
}
