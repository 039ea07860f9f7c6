// Paged split-K decode attention over the 4-bit strip cache, and the log-sum-exp
// combine that merges the per-split partial states.
//
// Arithmetic (reference: tests/common/paged_decode_oracle.hpp:516-596,
// tests/common/aic_splitk_decode_fixture.hpp:32-77):
//   q_rot   = bf16(Pi q),  Pi = M / sqrt(d)           rotated once per query row
//   score_t = (sum_c q_rot[c] Kq[t][c]) * kscale[t] * softmax_scale
//   tokens >= seq_len are overwritten with -3e38, fully dead strips are dropped
//   online softmax (m, l);  acc[c] += p_t * vscale[t] * Vq[c][t]
//   partial record per (item, split, row) = { m x8, l x8, acc[d] }
//   (include/turboquant_splitk_contract.hpp:23-27), empty range = (-3e38, 0, 0).
//
// Mapping onto the SM:
//   * one CTA per (sequence, KV head, split, 8-row query tile); its page range
//     is the reference Partition (include/turboquant_splitk_contract.hpp:129-136);
//     four warps each own every fourth tile (3 strips at d = 128, 2 at d = 256) of the
//     range and keep their own (m, l, acc), merged through shared memory at the end;
//   * every warp streams its tiles through a private 2-stage cp.async ring:
//     whole packed key strips, value strips and both scale runs, resolved through
//     the block table one tile ahead, so every KV byte crosses HBM once for all
//     query rows of the GQA group;
//   * tokens are the M dimension of both contractions. scores^T = K (16 tokens x d)
//     times q_rot^T (d x 8 rows) runs on the integer tensor path: a packed key word
//     becomes two s8 operand registers (16 * code) with a shift and two masks, and
//     q_rot, scaled per row by a power of two, is a fixed-point integer split into
//     8-bit limbs (one MMA chain per limb). No per-element scale is applied: the key
//     scale multiplies the 16 score columns and the value scale folds into P, as the
//     reference does;
//   * acc^T = V^T (d channels x 16 tokens) times P^T in f16 with FP32 accumulation:
//     the value strip is already channel-major, so 16 bytes of it are the A fragment
//     of two channels after in-register int4 -> f16 expansion (mask, xor-magic, one
//     packed subtract per two codes). P is kept in [0, 1] by a running power-of-two
//     normaliser of the value scales; the reference-contract entry carries it as a
//     hi + lo pair (two MMAs). P^T reaches its B-fragment layout with movmatrix.
#include <cuda_fp16.h>
#include <atomic>
#include <stdexcept>
#include <type_traits>

#include "tq_common.cuh"

namespace tq {

constexpr int kDecWarps = 4;
// kernel modes: export one record per (sequence, KV head, split); the same grid with one split,
// every CTA finishing its head and writing the output; the persistent grid with the merge folded in
constexpr int kModeRecords = 0, kModeDirect = 1, kModePersistent = 2;
constexpr int kCensusWords = 10;   // 64-bit words per CTA of the worker census
// a plan's chunk_pages with this bit set asks for pieces of equal width (the one-wave plan)
constexpr uint32_t kEqualPieces = 0x80000000u;
constexpr int kMaxSplits = TQ_MAX_SPLITS;   // record slots per head a workspace can be asked to hold
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// floor(2^32 / d) + 1 for d = 2 .. kMaxSplits: n / d == umulhi(n, table[d]) for n < 2^27
struct SmallReciprocals {
    uint32_t v[kMaxSplits + 1];
    constexpr SmallReciprocals() : v{}
    {
        for (uint32_t d = 2; d <= static_cast<uint32_t>(kMaxSplits); ++d)
            v[d] = static_cast<uint32_t>((1ull << 32) / d + 1ull);
    }
    __device__ __forceinline__ uint32_t operator[](uint32_t d) const { return v[d]; }
};
__constant__ SmallReciprocals kSmallReciprocal;

struct DecodeParams {
    const uint16_t* q;        // [items*rows][D] bf16
    const void* signs;
    uint32_t sign_source;
    const uint8_t* key_cache;
    const uint8_t* value_cache;
    const float* scale_cache;
    const int32_t* table;     // block table rows
    const int32_t* context_lens;  // null: fixed_ctx applies
    uint16_t* q_rot;          // optional export [items*splits][rows_stride][D]
    float* workspace;
    uint32_t items, H, rows, rows_stride, S, P;
    uint32_t table_stride, splits, page_begin, page_count, fixed_ctx;
    uint32_t sp_shift;        // log2(strips per page); pages hold 16 * 2^k tokens
    uint32_t chunk_pages;     // 0: every sequence uses `splits`; else at most ceil(pages/chunk)
    // launch-constant divisors of the prologue, prepared on the host
    Divider by_heads_tiles, by_row_tiles, by_heads, by_chunk_pages;
    // The library's own plan (graded != 0): piece k of every sequence covers the pages
    // [cuts[k], cuts[k + 1]) that the sequence has; the last cut is past any sequence.
    uint32_t graded;
    uint32_t cuts[TQ_MAX_SPLITS + 1];
    uint32_t q_f16;           // 1: the query is FP16 and its rotation stays FP32 (no bf16 rounding)
    uint32_t tokens_per_req;  // query tokens per request (1 + speculative): row = token * G + head-in-group
    const float* q_f32;       // non-null: the query is FP32 and already rotated (no rotation, no rounding)
    uint32_t midrise;         // 1: a code c stands for (c + 0.5) * scale (uniform mid-rise grid)
    float inv_sqrt_len, softmax_scale;
    uint32_t* status;
    // NZ-tiled source pools (the fused decoder's KV4 cache read where it lies): floats per slot
    // of the scale records and the codebook gain the stored scales are divided by
    uint32_t nz_slot_floats;
    float nz_gain;
    // persistent grid with the combine folded in: arrival counters (one word per (sequence, KV
    // head, row tile)), the tag that tells this launch's counts from stale bytes, and what the
    // egress needs (see CombineParams)
    uint32_t* counters;
    unsigned long long* ticket;   // two words behind the counters: the chunk ticket, the count of CTAs that left
    uint32_t tag;
    const float* egress_signs;
    const void* gate;
    void* output;
    uint32_t output_stage, out_dtype, gate_dtype, rotation;
    // host side only: the launch directly follows, in the same stream, the scatter writer of the
    // same step and may be scheduled under it (the kernel holds its cache reads back)
    uint32_t follows_writer;
    // optional worker census of the persistent grid: per CTA {start, end} in nanoseconds of the
    // global timer (null: off)
    unsigned long long* census;
};

// Shared-memory plan of one CTA. A key strip is stored in 16-byte chunks whose
// position is swizzled by one bit of the token row, so that the two token rows one
// quarter-warp reads (tokens t and t+4) fall into different banks.
template <int D>
struct DecodeSmem {
    // Tile (strips per pipeline stage of one warp), ring depth and resident CTAs per SM.
    // d = 128: two stages of 3 strips for each of four warps are 51 KiB, four CTAs fit and the
    // kernel stays within 128 registers (measured against 3 stages of 2 strips: +1.7 %, the
    // per-tile bookkeeping is spread over more strips; 6 stages of 1 strip: -8 %). d = 256
    // doubles both the strips and the accumulator registers: three CTAs of up to 168 registers,
    // two stages of 2 strips, and the query's B fragments (2..3 limbs x 8 words x 2 registers
    // per lane) are kept in shared memory behind the ring and re-read per key word instead of
    // occupying 32..48 registers (measured: fragments in registers with 3 stages of 1 strip
    // 3913 GB/s, the same with the fragments in shared memory 4011, 2 stages of 2 strips 4195;
    // with the fragments in registers the 2-strip tile had been 13 % slower than the 1-strip one).
    static constexpr int kTileStrips = D == 128 ? 3 : 2;
    static constexpr int kStages = 2;
    // (at d = 128 the fragments are 16 registers and stay there: in shared memory -2.8 %)
    static constexpr bool kQFragSmem = D == 256;
    static constexpr int kQFragBytes = kQFragSmem ? 3 * (D / 32) * 2 * 4 * 32 : 0;
    static constexpr int kCtasPerSm = D == 128 ? 4 : 3;
    static constexpr int kRowBytes = D / 2;
    static constexpr int kStripBytes = kStrip * D / 2;
    static constexpr int kStripStage = 2 * kStripBytes + 2 * kStrip * 4;   // K, V, both scale runs
    static constexpr int kStageBytes = kTileStrips * kStripStage;
    static constexpr int kRingBytes = kDecWarps * kStages * kStageBytes;
    // The fixed-point query of the prologue (8 rows, padded, see q_index) sits at the END of the
    // ring, inside the last warp's last stage, which no copy targets before the main loop: the
    // first tiles can be in flight while the query is rotated.
    static constexpr int kQFixInts = 8 * (D + 16);
    static constexpr int kQBytes = kQFixInts * 4;
    static constexpr int kMergePitch = D + 4;   // floats per merged row: {m, l, acc[d]} + pad, see the epilogue
    static constexpr int kMergeBytes = kDecWarps * 8 * kMergePitch * 4;
    // after the merge area (persistent grid only): the segment's combined record, then the two
    // buffers of the egress butterfly
    static constexpr int kRecPitch = D + 2;     // {m, l, acc[d]}
    static constexpr int kRecBytes = 8 * kRecPitch * 4;
    static constexpr int kEgressBytes = 2 * 8 * D * 4;
    static constexpr int kTailBytes = kMergeBytes + kRecBytes + kEgressBytes;
    static_assert(kTailBytes <= kRingBytes, "the epilogue buffers alias the ring");
    static_assert(kQBytes <= kRingBytes, "the prologue buffer aliases the ring");
    static constexpr int kBody = kRingBytes;
    static constexpr int kTotal = kBody + kQFragBytes;
    // warps whose first stage stays clear of the fixed-point query may start copying before it
    __host__ __device__ static constexpr bool early_issue(int warp)
    {
        return (warp * kStages + 1) * kStageBytes <= kRingBytes - kQBytes;
    }
    // 16-byte chunk `c` of token row `row` lands at this chunk index of the strip.
    __host__ __device__ static constexpr int key_chunk(int row, int c)
    {
        return D == 128 ? ((row * 4 + c) ^ (((row >> 2) & 1) << 2)) : ((row * 8 + c) ^ ((row >> 2) & 1));
    }
    // NZ-tiled source: a strip is staged as [32-byte column group][row slot][32 bytes]. Token t
    // = 8a + 4c + 2b + e goes to row slot (a e c b) of the key image and (e c a b) of the value
    // image, so that the rows one shared-memory instruction touches are four consecutive slots.
    __host__ __device__ static constexpr int nz_key_slot(int t)
    {
        return (t & 8) | ((t & 1) << 2) | ((t & 4) >> 1) | ((t & 2) >> 1);
    }
    __host__ __device__ static constexpr int nz_value_slot(int t)
    {
        return ((t & 1) << 3) | (t & 4) | ((t & 8) >> 2) | ((t & 2) >> 1);
    }
};

// ---- per-thread asynchronous copies. A bulk (TMA) copy per strip was measured
// here first: with the 1 KiB scattered strips of a 16-token page it costs more issue
// slots than it saves, because a copy whose operands differ per lane is serialised
// lane by lane (about 14 instructions per copy); 16-byte cp.async with per-lane
// precomputed offsets is 5 instructions per strip.
__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void cp_async16(uint32_t smem_dst, const void* gmem_src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_dst), "l"(gmem_src));
}
__device__ __forceinline__ void cp_async4(uint32_t smem_dst, const void* gmem_src)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(smem_dst), "l"(gmem_src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait()
{
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// Two packed INT4 codes -> two exact f16 integers. The low variant takes the codes
// at bits 0-3 / 16-19 of x, the high variant those at bits 4-7 / 20-23:
//   (x & 0x000F000F) ^ 0x64086408 = f16(1024 + (code ^ 8));  minus 1032 = code
//   (x & 0x00F000F0) ^ 0x64806480 = f16(1024 + 16 (code ^ 8)); /16 minus 72 = code
__device__ __forceinline__ uint32_t dq_lo(uint32_t x)
{
    uint32_t t;
    asm("lop3.b32 %0, %1, 0x000F000F, 0x64086408, 0x6A;\n" : "=r"(t) : "r"(x));
    asm("sub.rn.f16x2 %0, %1, %2;\n" : "=r"(t) : "r"(t), "r"(0x64086408u));
    return t;
}
__device__ __forceinline__ uint32_t dq_hi(uint32_t x)
{
    uint32_t t;
    asm("lop3.b32 %0, %1, 0x00F000F0, 0x64806480, 0x6A;\n" : "=r"(t) : "r"(x));
    // 0x2C00 = 1/16, 0xD480 = -72
    asm("fma.rn.f16x2 %0, %1, %2, %3;\n" : "=r"(t) : "r"(t), "r"(0x2C002C00u), "r"(0xD480D480u));
    return t;
}

__device__ __forceinline__ void mma_f16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                              uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// D = A (16 tokens x 32 channels, s8) * B (32 channels x 8 query rows) + C on the integer
// tensor path. B is one 8-bit limb of the fixed-point query: the top limb is signed, the
// lower limbs unsigned. D and C are separate so a chain can start from a constant C.
__device__ __forceinline__ void mma_s8_limb(bool b_signed, int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                            uint32_t a3, uint32_t b0, uint32_t b1, const int (&c)[4])
{
    if (b_signed)   // a constant after unrolling
        asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
            "{%8,%9}, {%10,%11,%12,%13};\n"
            : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c[0]), "r"(c[1]), "r"(c[2]),
              "r"(c[3]));
    else
        asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
            "{%8,%9}, {%10,%11,%12,%13};\n"
            : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c[0]), "r"(c[1]), "r"(c[2]),
              "r"(c[3]));
}

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a)
{
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
    return d;
}

__device__ __forceinline__ unsigned long long global_timer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ float ex2f(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float max3(float a, float b, float c)
{
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi)
{
    uint32_t d;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;\n" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}
__device__ __forceinline__ float2 unpack_f16x2(uint32_t v)
{
    return __half22float2(*reinterpret_cast<const __half2*>(&v));
}

// Which tokens of a strip ride in MMA rows i (c0,c1) and i+8 (c2,c3). Chosen so
// that after movmatrix a thread's P^T pairs cover tokens (t, t+4) of one value word,
// the pairs one mask extracts, and a byte permute replaces the shifts.
__device__ __forceinline__ int token_row_lo(int i) { return ((i >> 2) << 3) + (((i >> 1) & 1) << 1) + ((i & 1) << 2); }
__device__ __forceinline__ int token_row_hi(int i) { return token_row_lo(i) + 1; }

// Element-wise end of a decode: the normalised context of up to 8 query rows of one
// (sequence, KV head), in buf[0][row][channel], is rotated back (output stages 1 and 2),
// gated (stage 2), narrowed and stored. 128 threads; thread c serves channels c, c + 128.
// The butterfly stages and their order are those of tq_combine_kernel, so both routes give
// the same bits for the same normalised context.
template <int D>
__device__ __forceinline__ void egress_rows(const DecodeParams& p, float* buf, int rows_here, uint32_t seq,
                                            uint32_t head, uint32_t row_tile, uint32_t tokens_per_req, int tid)
{
    constexpr int CPT = D / 128;   // channels per thread
    int cur = 0;
    auto at = [&](int b, int q, int c) -> float& { return buf[(b * 8 + q) * D + c]; };
    if (p.output_stage != TQ_OUT_ROTATED) {
        if (p.rotation == 2u) {
            for (int q = 0; q < rows_here; ++q)
#pragma unroll
                for (int j = 0; j < CPT; ++j) at(0, q, tid + 128 * j) *= p.egress_signs[tid + 128 * j];
            __syncthreads();
        }
        auto stage = [&](int s) {
            for (int q = 0; q < rows_here; ++q)
#pragma unroll
                for (int j = 0; j < CPT; ++j) {
                    const int c = tid + 128 * j;
                    const float mine = at(cur, q, c), other = at(cur, q, c ^ s);
                    at(cur ^ 1, q, c) = other + ((c & s) ? -mine : mine);
                }
            __syncthreads();
            cur ^= 1;
        };
        if (p.rotation == 1u) {
            for (int s = 1; s < 16; s <<= 1) stage(s);
        } else if (p.rotation == 2u) {
            for (int s = 1; s < D; s <<= 1) stage(s);
        } else {
            for (int s = kGroup; s < D; s <<= 1) stage(s);
            for (int q = 0; q < rows_here; ++q)
#pragma unroll
                for (int j = 0; j < CPT; ++j) at(cur, q, tid + 128 * j) *= p.egress_signs[tid + 128 * j];
            __syncthreads();
            for (int s = 1; s < kGroup; s <<= 1) stage(s);
        }
    }
    const uint32_t grp = p.rows / tokens_per_req;
    for (int q = 0; q < rows_here; ++q) {
        const uint32_t row = row_tile * 8u + q, o_tok = row / grp, o_g = row - o_tok * grp;
        const size_t out_row = (static_cast<size_t>(seq) * tokens_per_req + o_tok) * (p.H * grp) +
                               static_cast<size_t>(head) * grp + o_g;
#pragma unroll
        for (int j = 0; j < CPT; ++j) {
            const int c = tid + 128 * j;
            float v = at(cur, q, c);
            if (p.output_stage != TQ_OUT_ROTATED) {
                v = p.rotation == 1u ? v * 0.25f
                    : p.rotation == 2u ? v * p.egress_signs[c] * p.inv_sqrt_len : v * p.inv_sqrt_len;
                if (p.output_stage == TQ_OUT_GATED) {
                    const size_t gi = out_row * D + c;
                    const float gt = p.gate_dtype == TQ_DTYPE_F32 ? static_cast<const float*>(p.gate)[gi]
                                     : p.gate_dtype == TQ_DTYPE_F16
                                         ? __half2float(static_cast<const __half*>(p.gate)[gi])
                                         : bf16_bits_to_f32(static_cast<const uint16_t*>(p.gate)[gi]);
                    v = v / (1.0f + __expf(-gt));
                }
            }
            const size_t o = out_row * D + c;
            if (p.out_dtype == TQ_DTYPE_F32) static_cast<float*>(p.output)[o] = v;
            else if (p.out_dtype == TQ_DTYPE_F16) static_cast<__half*>(p.output)[o] = __float2half_rn(v);
            else static_cast<uint16_t*>(p.output)[o] = f32_to_bf16_bits(v);
        }
    }
}

// The persistent grid's schedule: the flattened tiles [0, W) are cut into chunks whose sizes
// are a function of the chunk index alone -- G chunks of c0 tiles (G = CTAs of the grid, c0
// 85 % of an equal share), G chunks of c1 (an eighth of a share), then chunks of c2 (a
// sixteenth) to the end -- so
// every CTA can name the chunk that holds a tile and the tiles a chunk holds without any table.
// The first round is dealt statically (chunk c to CTA c); the rest is taken from an atomic
// ticket, so CTAs that run faster take more (their speeds differ by some +-10 % on this
// part), and the chunks are small where the work runs out.
struct ChunkSchedule {
    unsigned long long W;
    uint32_t G, c0, c1, c2;
};
__device__ __forceinline__ unsigned long long chunk_start(const ChunkSchedule& sc, uint32_t k, uint32_t* size)
{
    if (k < sc.G) {
        *size = sc.c0;
        return static_cast<unsigned long long>(k) * sc.c0;
    }
    if (k < 2u * sc.G) {
        *size = sc.c1;
        return static_cast<unsigned long long>(sc.G) * sc.c0 + static_cast<unsigned long long>(k - sc.G) * sc.c1;
    }
    *size = sc.c2;
    return static_cast<unsigned long long>(sc.G) * (sc.c0 + sc.c1) +
           static_cast<unsigned long long>(k - 2u * sc.G) * sc.c2;
}
__device__ __forceinline__ uint32_t chunk_of(const ChunkSchedule& sc, unsigned long long pos)
{
    const unsigned long long r0 = static_cast<unsigned long long>(sc.G) * sc.c0;
    if (pos < r0) return static_cast<uint32_t>(pos / sc.c0);
    const unsigned long long r1 = r0 + static_cast<unsigned long long>(sc.G) * sc.c1;
    if (pos < r1) return sc.G + static_cast<uint32_t>((pos - r0) / sc.c1);
    return 2u * sc.G + static_cast<uint32_t>((pos - r1) / sc.c2);
}

// Puts a 64-bit word under the launch's tag (count zero) unless it is there already.
__device__ __forceinline__ bool ensure_tag(unsigned long long* word, uint32_t tag)
{
    const unsigned long long mine = static_cast<unsigned long long>(tag) << 40;
    unsigned long long old = *reinterpret_cast<volatile unsigned long long*>(word);
    for (int it = 0; it < 64; ++it) {
        if ((old >> 40) == tag) return true;
        const unsigned long long prev = atomicCAS(word, old, mine);
        if (prev == old) return true;
        old = prev;
    }
    return false;
}

// A 64-bit counter that needs no clearing between launches: the top 24 bits carry the
// launch's tag, and a word under another tag (stale, or never written) reads as zero. Returns
// the count before the addition. Every retry means another CTA changed the word, so the loop
// ends after at most a few rounds; it gives up after 64 and reports through *ok.
__device__ __forceinline__ unsigned long long tagged_fetch_add(unsigned long long* word, uint32_t tag,
                                                               unsigned long long add, bool* ok)
{
    const unsigned long long mine = static_cast<unsigned long long>(tag) << 40;
    unsigned long long old = *reinterpret_cast<volatile unsigned long long*>(word);
    *ok = false;
    for (int it = 0; it < 64; ++it) {
        if ((old >> 40) == tag) {
            *ok = true;
            break;
        }
        const unsigned long long prev = atomicCAS(word, old, mine);
        if (prev == old) {
            *ok = true;
            break;
        }
        old = prev;
    }
    if (!*ok) return 0ull;
    return atomicAdd(word, add) & ((1ull << 40) - 1ull);
}

// EXT compiles in the extensions of the serving path -- f16 or pre-rotated FP32 query
// elements, several query tokens per request, mid-rise codes -- so that the plain
// instantiation carries neither their branches nor their registers. NZ reads the packed planes
// and scale records of the fused decoder's NZ-tiled KV4 cache in place (head size 256).
// STREAMK is the persistent grid: the batch's tiles, flattened sequence by sequence and head
// by head, are dealt to the CTAs in equal contiguous shares; a CTA walks the (sequence, KV
// head) segments of its share, and the CTA that completes a head's last outstanding segment
// merges the partial records and writes the output itself (one arrival count per head, no
// waiting anywhere). Without STREAMK one CTA serves one (sequence, KV head, split).
template <int D, bool PRECISE, bool EXT, bool NZ, int MODE>
__global__ void __launch_bounds__(kDecWarps * 32, DecodeSmem<D>::kCtasPerSm)
tq_decode_partial_kernel(const DecodeParams p)
{
    // What a CTA does with a head's state is a compile-time choice, so that the record-only
    // kernel carries none of the finishing code (its presence alone cost 2.4 % there).
    constexpr bool STREAMK = MODE == kModePersistent;
    constexpr bool DIRECT = MODE == kModeDirect;
    // The combine that follows a record export may be scheduled as soon as every CTA of this
    // grid has started (it waits for the grid's completion before it reads a record).
    if constexpr (MODE == kModeRecords) asm volatile("griddepcontrol.launch_dependents;\n");
    static_assert(!NZ || D == 256, "the NZ-tiled cache has head size 256");
    static_assert(!(STREAMK && PRECISE), "the persistent grid serves the native path");
    using L = DecodeSmem<D>;
    const uint32_t tokens_per_req = EXT ? p.tokens_per_req : 1u;
    const bool q_f16 = EXT && p.q_f16 != 0u;
    const bool prerot = EXT && p.q_f32 != nullptr;
    const bool midrise = EXT && p.midrise != 0u;
    constexpr int kStages = L::kStages;
    constexpr int kTileStrips = L::kTileStrips;
    constexpr int kRecord = 16 + D;
    constexpr int MT = D / 16;    // 16-channel m-tiles of the value contraction
    constexpr int WPT = D / 32;   // packed words per thread per key row
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring = smem;
    int* qfix = reinterpret_cast<int*>(smem + L::kRingBytes - L::kQBytes);   // prologue only
    __shared__ float row_unscale[8];                         // per query row: 2^-k * softmax_scale * log2e
    __shared__ int row_qsum8[8];                             // mid-rise codes: sum of the row's fixed-point query (enters a score times 8)
    __shared__ uint32_t sk_scan[2 * kDecWarps];              // persistent grid: warp totals / maxima of the tile scan
    __shared__ uint32_t sk_prefix[kDecWarps * 32 + 1];       // tiles per head before each thread's slice of sequences, and in all
    __shared__ uint32_t sk_start[2];                         // first sequence of a chunk, tiles per head before it
    __shared__ uint32_t sk_chunk;                            // the chunk the ticket handed out
    constexpr uint32_t kCtxCache = 512;                       // sequences whose live context is kept in shared memory
    __shared__ uint32_t sk_ctx[STREAMK ? kCtxCache : 1];
    __shared__ float sk_sgn[STREAMK ? D : 1];                 // the sign diagonal, read once
    __shared__ uint32_t sk_last;                             // this CTA completed the head's last segment
    __shared__ uint32_t sk_seen;                             // the head's arrival counter as read at the segment's start

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int r = lane >> 2, qd = lane & 3;

    const uint32_t row_tiles = (p.rows + 7u) / 8u;
    const uint32_t SP = p.S / kStrip;  // strips per page

    // live context of a sequence, clamped to what its block-table row can address
    auto context_of = [&](uint32_t seq) -> uint32_t {
        const int32_t c = p.context_lens[seq];
        uint32_t ctx = c > 0 ? static_cast<uint32_t>(c) : 0u;
        const uint32_t cap = p.table_stride * p.S;
        if (ctx > cap) {
            ctx = cap;
            if (tid == 0) report(p.status, TQ_STATUS_BAD_PAGE);
        }
        return ctx;
    };
    // persistent grid: the same from shared memory once the scan has cached it (small batches)
    auto context_cached = [&](uint32_t seq) -> uint32_t {
        if constexpr (STREAMK) {
            if (p.items / p.H <= kCtxCache) return sk_ctx[seq];
        }
        return context_of(seq);
    };
    auto tiles_of = [&](uint32_t ctx) -> uint32_t {
        return ((ctx + kStrip - 1u) / kStrip + kTileStrips - 1u) / kTileStrips;
    };

    // ---- everything below that does not depend on the segment
    const size_t head_block = static_cast<size_t>(p.S) * D / 2;  // bytes of one (page, head)
    const size_t scale_plane = static_cast<size_t>(p.P) * p.H * p.S;
    const uint32_t sp_shift = p.sp_shift;                        // strips per page = 1 << sp_shift
    constexpr uint32_t kTileStep = kDecWarps * kTileStrips;      // strips between a warp's tiles
    uint8_t* my_ring = ring + warp * kStages * L::kStageBytes;
    const uint32_t my_ring_s = smem_u32(my_ring);
    // Per-lane copy plan, fixed for the whole kernel: lane l moves 16-byte chunks
    // l, l+32, ... of the key strip (to their swizzled places) and of the value strip,
    // lanes 0..7 the two 64-byte scale runs. NZ-tiled source: chunk i*32 + l is half l&1 of
    // token row l>>1 of column group i, 512 contiguous source bytes per group; every lane
    // copies one scale (lanes 0..15 the key scales, 16..31 the value scales of its token).
    constexpr int kChunksPerLane = L::kStripBytes / 16 / 32;     // 2 (d=128) or 4 (d=256)
    constexpr int kChunksPerRow = L::kRowBytes / 16;
    uint32_t kdst[kChunksPerLane];
    [[maybe_unused]] uint32_t vdst_nz = 0;
#pragma unroll
    for (int i = 0; i < kChunksPerLane; ++i) {
        const int c = i * 32 + lane;
        if constexpr (NZ) kdst[i] = i * 512 + L::nz_key_slot(lane >> 1) * 32 + (lane & 1) * 16;
        else kdst[i] = L::key_chunk(c / kChunksPerRow, c % kChunksPerRow) * 16;
    }
    if constexpr (NZ) vdst_nz = L::kStripBytes + L::nz_value_slot(lane >> 1) * 32 + (lane & 1) * 16;
    // strides fit 32 bits (one page of one cache), so a page's offset is one widening
    // multiply-add on the lane's base pointer
    const uint32_t page_stride = p.H * static_cast<uint32_t>(head_block);
    const uint32_t page_stride_scale = p.H * p.S;
    const uint32_t sip_mask = (1u << sp_shift) - 1u;

    const int tok_lo = token_row_lo(r), tok_hi = token_row_hi(r);
    // this thread's chunks of its two key rows (d=128: one chunk each; d=256: two). NZ: the
    // eight bytes qd*8.. of both rows in each of the four column groups.
    int koff_lo[NZ ? 1 : WPT / 4], koff_hi[NZ ? 1 : WPT / 4];
    if constexpr (NZ) {
        koff_lo[0] = L::nz_key_slot(tok_lo) * 32 + qd * 8;
        koff_hi[0] = L::nz_key_slot(tok_hi) * 32 + qd * 8;
    } else {
#pragma unroll
        for (int w4 = 0; w4 < WPT / 4; ++w4) {
            koff_lo[w4] = L::key_chunk(tok_lo, qd * (WPT / 4) + w4) * 16;
            koff_hi[w4] = L::key_chunk(tok_hi, qd * (WPT / 4) + w4) * 16;
        }
    }
    // byte-permute selector that brings this thread's value-token pairs to bits 0-7 / 16-23
    const uint32_t vsel = qd == 0 ? 0x3210u : qd == 1 ? 0x4321u : qd == 2 ? 0x7654u : 0x0765u;

    // Two limbs are combined in INT32 and converted once. With three limbs (the
    // reference-contract entry) the sum no longer fits: at d = 128 an accumulator of one limb
    // stays below 2^22 in magnitude (128 channels x |16 code| <= 128 x limb <= 255), so a chain
    // that starts at the bit pattern of 1.5 * 2^23 ends, read as a float, at 12582912 + sum
    // exactly and one FP32 subtract recovers it; d = 256 can exceed that range and converts.
    constexpr int NL = PRECISE ? 3 : 2;
    constexpr bool kBiasedAcc = D == 128 && NL != 2;
    const int cinit[4] = {kBiasedAcc ? 0x4B400000 : 0, kBiasedAcc ? 0x4B400000 : 0,
                          kBiasedAcc ? 0x4B400000 : 0, kBiasedAcc ? 0x4B400000 : 0};
    auto limb_value = [](int v) {
        if constexpr (kBiasedAcc) return __int_as_float(v) - 12582912.0f;
        else return __int2float_rn(v);
    };

    // ---- persistent grid: the schedule, and the chunk this CTA starts with
    uint32_t seq = 0, head = 0, row_tile = 0, split = 0;
    uint32_t sk_n = 0, sk_loc = 0, sk_left = 0;   // tiles of `seq`, position inside its block of heads, tiles to go
    uint32_t sk_before = 0, cur_chunk = 0;       // tiles (per head) of the sequences before `seq`; the chunk in hand
    ChunkSchedule sched{0ull, gridDim.x, 1u, 1u, 1u};
    const uint32_t heads_per_seq = p.H * row_tiles;
    const uint32_t batch = p.items / p.H;
    const uint32_t seqs_per_thread = (batch + blockDim.x - 1u) / blockDim.x;
    // Takes chunk k: its tiles [w0, w1), the sequence that holds w0 (found by the thread whose
    // slice of sequences covers it). False when the chunk lies past the work. Uniform over the CTA.
    auto begin_chunk = [&](uint32_t k) -> bool {
        uint32_t size;
        const unsigned long long w0 = chunk_start(sched, k, &size);
        if (w0 >= sched.W) return false;
        sk_left = static_cast<uint32_t>(min(sched.W, w0 + size) - w0);
        cur_chunk = k;
        if (tid == 0) sk_start[0] = 0xFFFFFFFFu;
        __syncthreads();
        const unsigned long long lo = static_cast<unsigned long long>(sk_prefix[tid]) * heads_per_seq;
        const unsigned long long hi = static_cast<unsigned long long>(sk_prefix[tid + 1]) * heads_per_seq;
        if (w0 >= lo && w0 < hi) {
            uint32_t at = sk_prefix[tid];
            const uint32_t b0 = min(batch, tid * seqs_per_thread), b1 = min(batch, b0 + seqs_per_thread);
            for (uint32_t b = b0; b < b1; ++b) {
                const uint32_t n = tiles_of(context_cached(b));
                if (w0 < static_cast<unsigned long long>(at + n) * heads_per_seq) {
                    sk_start[0] = b;
                    sk_start[1] = at;
                    break;
                }
                at += n;
            }
        }
        __syncthreads();
        seq = sk_start[0];
        if (seq >= batch) return false;   // no slice claimed the tile: nothing to walk
        sk_before = sk_start[1];
        sk_n = tiles_of(context_cached(seq));
        sk_loc = static_cast<uint32_t>(w0 - static_cast<unsigned long long>(sk_before) * heads_per_seq);
        return true;
    };
    // The CTA is done: it counts itself out, and the last one out clears the two schedule
    // words, so that a replay of the same launch (same tag) starts from a clean ticket.
    auto leave = [&]() {
        if (tid != 0) return;
        if (p.census != nullptr) p.census[kCensusWords * blockIdx.x + 1] = global_timer_ns();
        bool ok;
        const unsigned long long gone = tagged_fetch_add(p.ticket + 1, p.tag, 1ull, &ok);
        if (!ok) report(p.status, TQ_STATUS_WAIT_EXPIRED);
        if (ok && gone + 1ull == gridDim.x) {
            *reinterpret_cast<volatile unsigned long long*>(p.ticket) = 0ull;
            *reinterpret_cast<volatile unsigned long long*>(p.ticket + 1) = 0ull;
        }
    };
    // census only: time since the previous mark, added to word `slot` of this CTA's census line
    unsigned long long mark_at = 0;
    auto mark = [&](int slot) {
        if constexpr (STREAMK) {
            if (p.census != nullptr && tid == 0) {
                const unsigned long long now = global_timer_ns();
                if (slot >= 0) p.census[kCensusWords * blockIdx.x + slot] += now - mark_at;
                mark_at = now;
            }
        }
    };
    if constexpr (STREAMK) {
        if (p.census != nullptr && tid == 0) {
            for (int i = 4; i < kCensusWords; ++i) p.census[kCensusWords * blockIdx.x + i] = 0ull;
            p.census[kCensusWords * blockIdx.x] = global_timer_ns();
            p.census[kCensusWords * blockIdx.x + 1] = 0ull;
            p.census[kCensusWords * blockIdx.x + 2] = 0ull;   // nanoseconds warp 0 spent inside its tile loops
            p.census[kCensusWords * blockIdx.x + 3] = 0ull;   // segments
        }
        mark(-1);
        if (!prerot)
            for (int c = tid; c < D; c += blockDim.x)
                sk_sgn[c] = sign_is_negative(p.signs, p.sign_source, c) ? -1.0f : 1.0f;
        // the ticket word goes under this launch's tag once, so that every later draw is a
        // single atomic add whose result can be awaited late
        if (tid == blockDim.x - 1 && !ensure_tag(p.ticket, p.tag)) report(p.status, TQ_STATUS_WAIT_EXPIRED);
        const uint32_t b0 = min(batch, tid * seqs_per_thread), b1 = min(batch, b0 + seqs_per_thread);
        uint32_t mine = 0, nmax = 0;
        for (uint32_t b = b0; b < b1; ++b) {
            const uint32_t live = context_of(b);
            if (b < kCtxCache) sk_ctx[b] = live;
            const uint32_t n = tiles_of(live);
            mine += n;
            nmax = max(nmax, n);
            if (n == 0u && blockIdx.x == 0u) {
                // a sequence without live tokens has no tile and therefore no segment: its
                // output rows are the zero context
                const size_t base = static_cast<size_t>(b) * tokens_per_req * (p.H * (p.rows / tokens_per_req)) * D;
                const size_t count = static_cast<size_t>(tokens_per_req) * (p.H * (p.rows / tokens_per_req)) * D;
                for (size_t i = 0; i < count; ++i) {
                    if (p.out_dtype == TQ_DTYPE_F32) static_cast<float*>(p.output)[base + i] = 0.f;
                    else static_cast<uint16_t*>(p.output)[base + i] = 0;
                }
            }
        }
        // inclusive scan over the threads' slices (warp shuffles, then the four warp totals)
        uint32_t incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += up;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) nmax = max(nmax, __shfl_xor_sync(0xffffffffu, nmax, o));
        if (lane == 31) {
            sk_scan[warp] = incl;
            sk_scan[kDecWarps + warp] = nmax;
        }
        __syncthreads();
        uint32_t before = 0, total = 0;
#pragma unroll
        for (int w = 0; w < kDecWarps; ++w) {
            if (w < warp) before += sk_scan[w];
            total += sk_scan[w];
            nmax = max(nmax, sk_scan[kDecWarps + w]);
        }
        sk_prefix[tid] = before + incl - mine;   // tiles per head before this thread's slice
        if (tid == 0) sk_prefix[kDecWarps * 32] = total;
        sched.W = static_cast<unsigned long long>(total) * heads_per_seq;   // all tiles of the launch
        // no chunk below one tile per warp, nor so small that the longest head could be cut
        // into more segments than the workspace has record slots for
        const uint32_t cap = p.splits > 1u ? p.splits - 1u : 1u;
        const unsigned long long cmin = max(static_cast<uint32_t>(kDecWarps), (nmax + cap - 1u) / cap);
        const unsigned long long share = (sched.W + gridDim.x - 1ull) / gridDim.x;   // an equal share
        sched.c0 = static_cast<uint32_t>(max(cmin, (share * 17ull + 19ull) / 20ull));
        sched.c1 = static_cast<uint32_t>(max(cmin, (share + 7ull) / 8ull));
        sched.c2 = static_cast<uint32_t>(max(cmin, (share + 15ull) / 16ull));
        if (!begin_chunk(blockIdx.x)) {   // the first chunk of every CTA is dealt statically
            leave();
            return;
        }
    } else {
        // The split is the slowest index of the grid: the hardware hands out CTAs in index
        // order, so all first pieces run before any second piece, and with the graded
        // partition below the pieces that start last are the smallest ones.
        split = p.by_heads_tiles.quotient(blockIdx.x);
        const uint32_t per_split = blockIdx.x - split * (p.items * row_tiles);
        const uint32_t item = p.by_row_tiles.quotient(per_split);
        row_tile = per_split - item * row_tiles;
        seq = p.by_heads.quotient(item);
        head = item - seq * p.H;
    }

#pragma unroll 1
    for (;;) {
        // ---- this segment: (seq, head, row_tile), strips [s0, s1), where its record goes
        uint32_t ctx, s0, s1, seg_count = 1, seg_slot = split;
        bool no_pages = false;
        [[maybe_unused]] int32_t spec_pg[kTileStrips];
        // The sign diagonal and this warp's two raw query rows: requested as early as the
        // segment's (sequence, head, row tile) is known, ahead of everything that waits.
        constexpr int K = D / 32;
        float sgn[K], qraw[2][K];
        auto request_query = [&]() {
            const int rows_now = min(8u, p.rows - row_tile * 8u);
#pragma unroll
            for (int i = 0; i < K; ++i) {
                if constexpr (STREAMK) sgn[i] = prerot ? 1.0f : sk_sgn[lane * K + i];
                else sgn[i] = !prerot && sign_is_negative(p.signs, p.sign_source, lane * K + i) ? -1.0f : 1.0f;
            }
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                const int row = warp * 2 + rr;
#pragma unroll
                for (int i = 0; i < K; ++i) qraw[rr][i] = 0.f;
                if (row < rows_now) {
                    // row = token * G + g of the request's (1 + speculative) query tokens; with one
                    // token per request this is (item * rows + row)
                    const uint32_t row_g = row_tile * 8u + row, grp = p.rows / tokens_per_req;
                    const uint32_t q_tok = row_g / grp, q_g = row_g - q_tok * grp;
                    const size_t qoff = ((static_cast<size_t>(seq) * tokens_per_req + q_tok) * (p.H * grp) +
                                         static_cast<size_t>(head) * grp + q_g) * D + lane * K;
                    const uint16_t* qsrc = p.q + qoff;
#pragma unroll
                    for (int i = 0; i < K; ++i)
                        qraw[rr][i] = prerot ? p.q_f32[qoff + i]
                                             : q_f16 ? __half2float(__ushort_as_half(qsrc[i])) : bf16_bits_to_f32(qsrc[i]);
                }
            }
        };
        if constexpr (!STREAMK) request_query();
        [[maybe_unused]] uint32_t sk_take = 0;
        if constexpr (STREAMK) {
            const uint32_t in_seq = sk_loc / sk_n, t0 = sk_loc - in_seq * sk_n;
            sk_take = min(sk_left, sk_n - t0);
            head = in_seq / row_tiles;
            row_tile = in_seq - head * row_tiles;
            ctx = context_cached(seq);
            s0 = t0 * kTileStrips;
            s1 = min((t0 + sk_take) * kTileStrips, (ctx + kStrip - 1u) / kStrip);
            // the chunks this head's tiles [first, first + n) fall into: one record slot each
            const unsigned long long first = static_cast<unsigned long long>(sk_before) * heads_per_seq +
                                             static_cast<unsigned long long>(in_seq) * sk_n;
            const uint32_t k_first = chunk_of(sched, first);
            seg_count = chunk_of(sched, first + sk_n - 1u) - k_first + 1u;
            seg_slot = cur_chunk - k_first;
        } else {
            // Graded plan: where the piece starts is a launch constant, so the block-table
            // entries of this warp's first tile are requested together with the context length
            // instead of one round trip after it (entries past the sequence are read but not used).
            const bool graded = p.graded != 0u;
            if (graded) {
                const uint32_t first = (p.page_begin + p.cuts[split]) * SP + warp * kTileStrips;
                const int32_t* row = p.table + static_cast<size_t>(seq) * p.table_stride;
#pragma unroll
                for (int ts = 0; ts < kTileStrips; ++ts) {
                    const uint32_t entry = (first + ts) >> sp_shift;
                    spec_pg[ts] = entry < p.table_stride ? __ldg(row + entry) : -1;
                }
            }
            uint32_t page_count;
            if (p.context_lens != nullptr) {
                ctx = context_of(seq);
                page_count = (ctx + p.S - 1u) >> (4u + sp_shift);   // pages hold 16 << sp_shift tokens
            } else {
                ctx = p.fixed_ctx;
                page_count = p.page_count;
            }
            // Ragged batches: a sequence takes only as many of the launch's splits as it has
            // chunks of chunk_pages pages, so CTAs carry similar amounts of work; the splits it
            // does not use fall out of the partition as empty ranges and export the neutral element.
            uint32_t eff_splits = p.splits;
            if (p.chunk_pages != 0u) {
                const uint32_t chunks = p.by_chunk_pages.quotient(page_count + p.chunk_pages - 1u);
                eff_splits = chunks < 1u ? 1u : (chunks < p.splits ? chunks : p.splits);
            }
            // eff_splits <= 32 and page counts stay far below 2^27: one multiply by the tabulated
            // floor(2^32 / d) + 1 is the exact quotient
            uint32_t rb, rc;
            if (graded) {
                rb = p.cuts[split];
                const uint32_t end = min(p.cuts[split + 1u], page_count);
                rc = end > rb ? end - rb : 0u;
            } else {
                const uint32_t width = eff_splits == 1u ? page_count
                                                        : __umulhi(page_count + eff_splits - 1u, kSmallReciprocal[eff_splits]);
                rb = split * width;
                const uint32_t remaining = rb < page_count ? page_count - rb : 0u;
                rc = remaining < width ? remaining : width;
            }
            s0 = (p.page_begin + rb) * SP;
            s1 = s0 + rc * SP;
            const uint32_t live_strips = (ctx + kStrip - 1u) / kStrip;
            if (s1 > live_strips) s1 = live_strips;
            no_pages = rc == 0u;
        }
        const uint32_t item = seq * p.H + head;
        const int rows_here = min(8u, p.rows - row_tile * 8u);
        // A split whose page range is empty takes no part at all; one whose pages all
        // lie past the live tokens still rotates and publishes its query (the rotation
        // does not depend on the cache) and then exports the neutral element
        // (kernels/ops/turboquant/turboquant_paged_decode_attention.cpp:1626-1637).
        const bool empty = s1 <= s0;

        float* rec_base = p.workspace +
                          ((static_cast<size_t>(item) * p.splits + seg_slot) * p.rows_stride + row_tile * 8u) *
                              kRecord;

        // classic grid, one split, an output to write: the CTA holds the head's whole state
        // and finishes it itself -- no record, no workspace, no second kernel
        constexpr bool direct = DIRECT;
        if constexpr (!STREAMK) {
            if (empty) {
                if constexpr (direct) {
                    float* zero = reinterpret_cast<float*>(ring + L::kMergeBytes + L::kRecBytes);
                    for (int i = tid; i < rows_here * D; i += blockDim.x) zero[i] = 0.f;
                    __syncthreads();
                    egress_rows<D>(p, zero, rows_here, seq, head, row_tile, tokens_per_req, tid);
                    return;
                } else {
                    for (int i = tid; i < rows_here * kRecord; i += blockDim.x) {
                        const int c = i % kRecord;
                        rec_base[i] = c < 8 ? kMaskedScore : 0.0f;
                    }
                    if (no_pages || p.q_rot == nullptr) return;
                }
            }
        }

        // ---- the copy machinery of this segment
        const int32_t* table_row = p.table + static_cast<size_t>(seq) * p.table_stride;
        // Block-table entries of the tile whose first strip is `strip` (-1 past the range).
        // The loaded entries are not touched before the copy stage uses them one tile later:
        // any arithmetic on them here would wait out the table read once per tile (measured:
        // 4 % of the kernel).
        auto load_pages = [&](uint32_t strip, int32_t (&pg)[kTileStrips]) {
#pragma unroll
            for (int ts = 0; ts < kTileStrips; ++ts)
                pg[ts] = strip + ts < s1 ? __ldg(table_row + ((strip + ts) >> sp_shift)) : -1;
        };
        const uint8_t* ksrc0;
        const uint8_t* vsrc0;
        const float* ssrc0;
        if constexpr (NZ) {
            // (64-row tile, head) images of 8 KiB inside a page of S * H * 128 bytes
            ksrc0 = p.key_cache + static_cast<size_t>(head) * 8192u + lane * 16;
            vsrc0 = p.value_cache + static_cast<size_t>(head) * 8192u + lane * 16;
            ssrc0 = p.scale_cache + static_cast<size_t>(lane & 15) * p.nz_slot_floats + (lane >> 4) * p.H + head;
        } else {
            ksrc0 = p.key_cache + head * head_block + lane * 16;
            vsrc0 = p.value_cache + head * head_block + lane * 16;
            ssrc0 = p.scale_cache + (lane >> 2) * scale_plane + static_cast<size_t>(head) * p.S + (lane & 3) * 4;
        }
        auto issue = [&](uint32_t strip, uint32_t stage, const int32_t (&pg)[kTileStrips]) {
#pragma unroll
            for (int ts = 0; ts < kTileStrips; ++ts) {
                if (pg[ts] < 0 && strip + ts >= s1) continue;   // warp-uniform: past the range
                // a negative entry under live tokens is as wrong as one past the pool
                uint32_t page = static_cast<uint32_t>(pg[ts]);
                if (page >= p.P) {
                    if (lane == 0) report(p.status, TQ_STATUS_BAD_PAGE);
                    page = 0;
                }
                const uint32_t sip = (strip + ts) & sip_mask;
                const uint32_t dst = my_ring_s + stage * L::kStageBytes + ts * L::kStripStage;
                if constexpr (NZ) {
                    // strip sip of the page: 64-row tile sip / 4, rows 16 (sip % 4) .. of its image
                    const size_t off = static_cast<size_t>(page) * page_stride +
                                       static_cast<size_t>(sip >> 2) * (64u * 128u) * p.H + (sip & 3u) * 512u;
#pragma unroll
                    for (int i = 0; i < kChunksPerLane; ++i) {
                        cp_async16(dst + kdst[i], ksrc0 + off + i * 2048);
                        cp_async16(dst + vdst_nz + i * 512, vsrc0 + off + i * 2048);
                    }
                    cp_async4(dst + 2 * L::kStripBytes + lane * 4,
                              ssrc0 + (static_cast<size_t>(page) * p.S + sip * kStrip) * p.nz_slot_floats);
                } else {
                    const uint8_t* ksrc = ksrc0 + static_cast<size_t>(page) * page_stride + sip * L::kStripBytes;
                    const uint8_t* vsrc = vsrc0 + static_cast<size_t>(page) * page_stride + sip * L::kStripBytes;
#pragma unroll
                    for (int i = 0; i < kChunksPerLane; ++i) {
                        cp_async16(dst + kdst[i], ksrc + i * 512);
                        cp_async16(dst + L::kStripBytes + i * 512 + lane * 16, vsrc + i * 512);
                    }
                    if (lane < 8)
                        cp_async16(dst + 2 * L::kStripBytes + lane * 16,
                                   ssrc0 + static_cast<size_t>(page) * page_stride_scale + sip * kStrip);
                }
            }
        };

        // ---- per-warp pipeline over tiles warp, warp+4, ...: the first tile goes out before
        // the query is rotated wherever its stage does not share bytes with the prologue
        const uint32_t tiles = empty ? 0u : (s1 - s0 + kTileStrips - 1u) / kTileStrips;
        const uint32_t my_tiles = tiles > static_cast<uint32_t>(warp)
                                      ? (tiles - warp + kDecWarps - 1u) / kDecWarps : 0u;
        const uint32_t strip_first = s0 + warp * kTileStrips;   // first strip of this warp's tile 0
        int32_t pg_next[kTileStrips];
        static_assert(kStages == 2, "the prologue below fills one stage ahead");
        // the first tile's entries: requested at the top of the segment under the graded plan
        auto first_pages = [&](int32_t (&pg)[kTileStrips]) {
            if constexpr (!STREAMK) {
                if (p.graded != 0u) {
#pragma unroll
                    for (int ts = 0; ts < kTileStrips; ++ts) pg[ts] = strip_first + ts < s1 ? spec_pg[ts] : -1;
                    return;
                }
            }
            load_pages(strip_first, pg);
        };
        // Every global round trip of the prologue is started before anything waits for one: the
        // draw of the next chunk and a first look at the head's arrival counter (persistent grid,
        // consumed only after the fragments are built), the sign diagonal and this warp's two raw
        // query rows; the block-table entries of the first tile follow, and only then the rotation.
        [[maybe_unused]] unsigned long long drawn = 0;
        [[maybe_unused]] uint32_t seen = 0;
        if constexpr (STREAMK) {
            if (tid == 0) {
                if (sk_take == sk_left) drawn = atomicAdd(p.ticket, 1ull);
                if (seg_count > 1u)
                    seen = *reinterpret_cast<volatile uint32_t*>(p.counters + (static_cast<size_t>(item) * row_tiles + row_tile));
            }
        }
        if constexpr (STREAMK) request_query();
        // (the record-only kernel keeps rotation first: ahead of it the copies measured 2 % slower there)
        const bool early = MODE != kModeRecords && L::early_issue(warp) && !empty;
        // Launched as the programmatic dependent of the step's scatter writer, the CTA has come
        // this far under it; the cache itself is read only once the writer has completed (a no-op
        // after an ordinary launch).
        auto writer_done = [] { asm volatile("griddepcontrol.wait;\n" ::: "memory"); };
        if (early) {
            writer_done();
            first_pages(pg_next);
            issue(strip_first, 0, pg_next);
            cp_async_commit();
            load_pages(strip_first + kTileStep, pg_next);
        }

        // ---- rotate the query rows once: each warp takes two rows through the FP32
        // ingress cascade, scales, rounds to bf16 (the pinned operand) and publishes it.
        // The key contraction runs on the integer tensor path, so every row then becomes
        // fixed point: its entries times the power of two that puts the largest below
        // 2^(8 NL - 1), rounded to an integer of NL 8-bit limbs (NL = 2: 2^-16 of the row
        // maximum, far inside the tolerance of the native path; NL = 3: 2^-24, FP32 grade,
        // for the entry point that is checked against the reference's partial records).
        // The inverse power goes into the per-row score factor together with
        // softmax_scale * log2(e) and the 1/16 of the key operand (see compute_tile).
        // A lane later reads the eight integers of its key word's channels, lanes (r, qd) at
        // channel qd * d/4 + ...: rows are padded by 16 and quarters of a row by 4 words so that
        // the eight lanes one 128-bit access serves together fall into eight different bank groups.
        auto q_index = [](int row, int ch) { return row * (D + 16) + (ch / (D / 4)) * (D / 4 + 4) + ch % (D / 4); };
        {
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                const int row = warp * 2 + rr;
                float v[K];
#pragma unroll
                for (int i = 0; i < K; ++i) v[i] = qraw[rr][i];
                if (!prerot) cascade_ingress<K>(v, sgn, lane);
                float am = 0.f;
#pragma unroll
                for (int i = 0; i < K; ++i) {
                    float val = prerot ? v[i] : v[i] * p.inv_sqrt_len;
                    if (!q_f16 && !prerot) {   // the bf16 operand the reference pins (and publishes)
                        const uint16_t bits = f32_to_bf16_bits(val);
                        val = bf16_bits_to_f32(bits);
                        if constexpr (!STREAMK) {
                            if (p.q_rot != nullptr && row < rows_here)
                                p.q_rot[((static_cast<size_t>(item) * p.splits + split) * p.rows_stride +
                                         row_tile * 8u + row) * D + lane * K + i] = bits;
                        }
                    }
                    v[i] = val;
                    am = fmaxf(am, fabsf(val));
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
                // 2^(top - e) and 2^(e - top) from the exponent field of the row maximum,
                // top = 8 NL - 2; a row below 1e-25 scores as zero
                constexpr int kTop = 8 * NL - 2;
                const bool tiny = !(am >= 1.0e-25f);
                const int e_bits = __float_as_int(am) & 0x7F800000;
                const float up = tiny ? 0.0f : __int_as_float(((254 + kTop) << 23) - e_bits);
                const float down = tiny ? 1.0f : __int_as_float(e_bits - (kTop << 23));
                int qsum = 0;
#pragma unroll
                for (int i = 0; i < K; ++i) {
                    const int fx = __float2int_rn(v[i] * up);
                    qfix[q_index(row, lane * K + i)] = fx;
                    qsum += fx;
                }
                if (midrise) {
                    // sum_c q_c (16 code_c + 8): the half step of every code adds 8 * sum_c q_c to a raw score
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) qsum += __shfl_xor_sync(0xffffffffu, qsum, o);
                    if (lane == 0) row_qsum8[row] = qsum;
                }
                if (lane == 0) row_unscale[row] = down * 0.0625f * p.softmax_scale * kLog2e;
            }
        }
        if constexpr (!STREAMK) {
            if (empty) return;
        }
        __syncthreads();

        // ---- limbs of q_rot^T as B fragments of the integer MMA. Word wi of a key row holds
        // channels qd*(D/4) + wi*8 + n, n = 0..7: the even n feed contraction slots qd*4 + n/2
        // (b0), the odd n slots 16 + qd*4 + n/2 (b1). NZ-tiled source: MMA wi = 2 g + half takes
        // the low (half 0) or high nibbles of column group g, channels 128 half + 32 g + 8 qd + n,
        // n = 0..3 in b0 and 4..7 in b1.
        uint32_t bq[L::kQFragSmem ? 1 : NL][L::kQFragSmem ? 1 : WPT][2];
        // [wi][limb][lane] pairs of registers; every warp holds the same fragments, warp 0 writes them
        uint2* qfrag = reinterpret_cast<uint2*>(smem + L::kBody) + lane;
#pragma unroll
        for (int wi = 0; wi < WPT; ++wi) {
            const int* qr = NZ ? qfix + q_index(r, (wi & 1) * 128 + (wi >> 1) * 32 + qd * 8)
                               : qfix + q_index(r, qd * (D / 4) + wi * 8);
            int qv[8];
#pragma unroll
            for (int n = 0; n < 8; ++n) qv[n] = qr[n];
#pragma unroll
            for (int l = 0; l < NL; ++l)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    // byte e of the word = limb l of channel 2e + h (NZ: 4h + e): three byte permutes
                    const uint32_t pick = static_cast<uint32_t>(l) | (static_cast<uint32_t>(4 + l) << 4);
                    const uint32_t lo = NZ ? __byte_perm(qv[4 * h], qv[4 * h + 1], pick)
                                           : __byte_perm(qv[h], qv[2 + h], pick);
                    const uint32_t hi = NZ ? __byte_perm(qv[4 * h + 2], qv[4 * h + 3], pick)
                                           : __byte_perm(qv[4 + h], qv[6 + h], pick);
                    const uint32_t frag = __byte_perm(lo, hi, 0x5410u);
                    if constexpr (L::kQFragSmem) {
                        if (warp == 0) reinterpret_cast<uint32_t*>(qfrag + (wi * NL + l) * 32)[h] = frag;
                    } else {
                        bq[l][wi][h] = frag;
                    }
                }
        }
        // scores are kept as raw * key_scale; the per-row factor enters inside the exponent
        const float rfac[2] = {row_unscale[qd * 2], row_unscale[qd * 2 + 1]};
        const int qs8[2] = {midrise ? row_qsum8[qd * 2] : 0, midrise ? row_qsum8[qd * 2 + 1] : 0};
        float ps[2] = {0.f, 0.f};   // mid-rise codes: running sum of P (as the value contraction sees it) per row
        if constexpr (STREAMK) {
            if (tid == 0) {   // the two round trips started at the top of the prologue are back by now
                if (sk_take == sk_left) {
                    const unsigned long long t = drawn & ((1ull << 40) - 1ull);
                    sk_chunk = t < 0x7FFFFFFFull - gridDim.x ? gridDim.x + static_cast<uint32_t>(t) : 0xFFFFFFFFu;
                }
                sk_seen = seen;
            }
        }
        __syncthreads();  // everyone is done with the fixed-point query: the ring may overwrite it

        // Online-softmax state for query rows qd*2 and qd*2+1, in units of raw * key_scale.
        float m_run[2] = {kMaskedScore, kMaskedScore}, l_run[2] = {0.f, 0.f};
        float m_fac[2] = {0.f, 0.f};   // m_run * rfac, the exponent offset (0 while m_run is the sentinel)
        float acc[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[mt][i] = 0.f;
        // Running power-of-two normaliser of the value scales: P is carried in f16, so
        // it is kept in [0, 1] by dividing the value scale by the largest seen so far.
        float vnorm = 0.f, inv_vnorm = 0.f;

        if (!early) {
            writer_done();
            first_pages(pg_next);
            issue(strip_first, 0, pg_next);
            cp_async_commit();
            load_pages(strip_first + kTileStep, pg_next);
        }

        // Speculative tokens: query token t of a request sees the context without the last
        // (tokens_per_req - 1 - t) tokens. row_drop[q] is that count for this thread's two rows.
        uint32_t row_drop[2];
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const uint32_t row_g = row_tile * 8u + qd * 2 + q, grp = p.rows / tokens_per_req;
            const uint32_t t = min(row_g / grp, tokens_per_req - 1u);
            row_drop[q] = tokens_per_req - 1u - t;
        }
        const uint32_t drop_max = tokens_per_req - 1u;
        const uint32_t ctx_all = ctx > drop_max ? ctx - drop_max : 0u;   // tokens every row sees

        // One tile: scores^T for its strips, the online-softmax update, then acc^T += V^T P^T.
        // TAIL tiles reach past the split's strips or past the live tokens and mask by
        // overwriting (a dead slot's scale may be a NaN); full tiles carry no masking code.
        auto compute_tile = [&](const uint8_t* st, uint32_t strip_t, auto tail_tag) {
            constexpr bool TAIL = decltype(tail_tag)::value;
            float sc[kTileStrips][4], vs[kTileStrips][2];
            bool live[kTileStrips][2];
            float mx[2] = {kMaskedScore, kMaskedScore};
            float vmax = 0.f;
#pragma unroll
            for (int ts = 0; ts < kTileStrips; ++ts) {
                const uint8_t* ss = st + ts * L::kStripStage;
                const float* scales = reinterpret_cast<const float*>(ss + 2 * L::kStripBytes);
                // A operand: 16 * code as a signed byte. The odd channels of a word are its
                // high nibbles already in place (mask), the even ones move up by four bits.
                int ci[NL][4];
                auto limbs = [&](int wi, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3) {
#pragma unroll
                    for (int l = 0; l < NL; ++l) {
                        uint32_t b0, b1;
                        if constexpr (L::kQFragSmem) {
                            const uint2 fr = qfrag[(wi * NL + l) * 32];
                            b0 = fr.x;
                            b1 = fr.y;
                        } else {
                            b0 = bq[l][wi][0];
                            b1 = bq[l][wi][1];
                        }
                        if (wi == 0)
                            mma_s8_limb(l == NL - 1, ci[l], a0, a1, a2, a3, b0, b1, cinit);
                        else
                            mma_s8_limb(l == NL - 1, ci[l], a0, a1, a2, a3, b0, b1, ci[l]);
                    }
                };
                if constexpr (NZ) {
                    // column group g: bytes 8 qd .. 8 qd + 7 of both token rows; the low nibbles
                    // are channels 32 g + 8 qd + j, the high nibbles channels 128 + 32 g + 8 qd + j
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        const uint2 lo = *reinterpret_cast<const uint2*>(ss + g * 512 + koff_lo[0]);
                        const uint2 hi = *reinterpret_cast<const uint2*>(ss + g * 512 + koff_hi[0]);
                        limbs(2 * g, (lo.x << 4) & 0xF0F0F0F0u, (hi.x << 4) & 0xF0F0F0F0u,
                              (lo.y << 4) & 0xF0F0F0F0u, (hi.y << 4) & 0xF0F0F0F0u);
                        limbs(2 * g + 1, lo.x & 0xF0F0F0F0u, hi.x & 0xF0F0F0F0u, lo.y & 0xF0F0F0F0u,
                              hi.y & 0xF0F0F0F0u);
                    }
                } else {
#pragma unroll
                    for (int w4 = 0; w4 < WPT / 4; ++w4) {
                        const uint4 lo = *reinterpret_cast<const uint4*>(ss + koff_lo[w4]);
                        const uint4 hi = *reinterpret_cast<const uint4*>(ss + koff_hi[w4]);
                        const uint32_t wl[4] = {lo.x, lo.y, lo.z, lo.w}, wh[4] = {hi.x, hi.y, hi.z, hi.w};
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            limbs(w4 * 4 + k, (wl[k] << 4) & 0xF0F0F0F0u, (wh[k] << 4) & 0xF0F0F0F0u,
                                  wl[k] & 0xF0F0F0F0u, wh[k] & 0xF0F0F0F0u);
                    }
                }
                // limbs -> one float per score: sum_l 256^l * c_l
                float c[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if constexpr (NL == 2) {
                        // |c1| * 256 + |c0| < 2^31 at either head size: the two limbs combine in
                        // INT32 and one conversion follows
                        int sum = ci[1][i] * 256 + ci[0][i];
                        if constexpr (EXT) sum += 8 * qs8[i & 1];   // < 2^30 + 2^26
                        c[i] = __int2float_rn(sum);
                        continue;
                    }
                    float f = limb_value(ci[NL - 1][i]);
#pragma unroll
                    for (int l = NL - 2; l >= 0; --l) f = fmaf(f, 256.0f, limb_value(ci[l][i]));
                    if constexpr (EXT) f = fmaf(8.0f, __int2float_rn(qs8[i & 1]), f);   // the sum stays below 2^30
                    c[i] = f;
                }
                const float ks_lo = scales[tok_lo], ks_hi = scales[tok_hi];
                vs[ts][0] = scales[kStrip + tok_lo];
                vs[ts][1] = scales[kStrip + tok_hi];
                sc[ts][0] = c[0] * ks_lo;
                sc[ts][1] = c[1] * ks_lo;
                sc[ts][2] = c[2] * ks_hi;
                sc[ts][3] = c[3] * ks_hi;
                if constexpr (TAIL) {
                    const uint32_t strip = strip_t + ts;
                    live[ts][0] = strip < s1 && strip * kStrip + tok_lo < ctx;
                    live[ts][1] = strip < s1 && strip * kStrip + tok_hi < ctx;
                    if (!live[ts][0]) { sc[ts][0] = sc[ts][1] = kMaskedScore; vs[ts][0] = 0.f; }
                    if (!live[ts][1]) { sc[ts][2] = sc[ts][3] = kMaskedScore; vs[ts][1] = 0.f; }
                    if (tokens_per_req > 1u) {   // the last tokens are hidden from the earlier query tokens
                        const uint32_t t_lo = strip * kStrip + tok_lo, t_hi = strip * kStrip + tok_hi;
#pragma unroll
                        for (int q = 0; q < 2; ++q) {
                            if (t_lo + row_drop[q] >= ctx) sc[ts][q] = kMaskedScore;
                            if (t_hi + row_drop[q] >= ctx) sc[ts][2 + q] = kMaskedScore;
                        }
                    }
                }
                mx[0] = max3(mx[0], sc[ts][0], sc[ts][2]);
                mx[1] = max3(mx[1], sc[ts][1], sc[ts][3]);
                vmax = max3(vmax, fabsf(vs[ts][0]), fabsf(vs[ts][1]));
            }
            // -- online softmax update. m_run and vnorm are uniform over the lanes that share
            // them, so "did anything grow" can be asked of every lane's own four scores first;
            // only a tile that raises a row maximum or the value normaliser pays for the
            // reductions and the rescale of the accumulator (rfac > 0: the maximum can be taken
            // before the per-row factor is applied).
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
                    alpha[q] = ex2f((m_run[q] - m_new) * rfac[q]);
                    m_run[q] = m_new;
                    // a row that has seen no live token yet keeps offset 0: its masked scores must
                    // still give exp2(-huge) = 0, not exp2(0)
                    m_fac[q] = m_new > -1.0e37f ? m_new * rfac[q] : 0.f;
                    l_run[q] *= alpha[q];
                }
                if (vmax > vnorm) {  // warp-uniform: value scales depend on the token only
                    // the power of two above vmax; the ratio old/new is exact
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
                if constexpr (EXT) {
                    ps[0] *= alpha[0];
                    ps[1] *= alpha[1];
                }
            }
            // -- P, then acc^T += V^T P^T
            if constexpr (!PRECISE) {
#pragma unroll
                for (int ts = 0; ts < kTileStrips; ++ts) {
                    if constexpr (TAIL) {
                        if (strip_t + ts >= s1) continue;  // warp-uniform
                    }
                    const uint8_t* ss = st + ts * L::kStripStage;
                    const float vs_lo = vs[ts][0] * inv_vnorm, vs_hi = vs[ts][1] * inv_vnorm;
                    float pw[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float pr = ex2f(fmaf(sc[ts][i], rfac[i & 1], -m_fac[i & 1]));
                        l_run[i & 1] += pr;
                        pw[i] = pr * (i < 2 ? vs_lo : vs_hi);
                    }
                    const uint32_t h0 = pack_f16x2(pw[0], pw[1]), h1 = pack_f16x2(pw[2], pw[3]);
                    const uint32_t bh0 = movmatrix_trans(h0), bh1 = movmatrix_trans(h1);
                    if constexpr (EXT) {
                        if (midrise) {   // the f16 values the MMA multiplies, so that acc and ps stay consistent
                            const float2 f0 = unpack_f16x2(h0), f1 = unpack_f16x2(h1);
                            ps[0] += f0.x + f1.x;
                            ps[1] += f0.y + f1.y;
                        }
                    }
                    if constexpr (NZ) {
                        // Token rows are the contraction index and lie 32 bytes apart in the image:
                        // word r of the four rows whose slots are qd, qd+4, qd+8, qd+12 (tokens t, t+4,
                        // t+1, t+5 of this lane's pairs) carries four packed columns, i.e. channels
                        // 32 g + 4 r + u (low nibbles) and 128 + 32 g + 4 r + u (high), u = 0..3. A byte
                        // permute puts the same column of two tokens 16 bits apart, where the masks
                        // of dq_lo / dq_hi pick both channels' pairs.
                        const uint8_t* vbase = ss + L::kStripBytes + qd * 32 + r * 4;
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            const uint32_t wa = *reinterpret_cast<const uint32_t*>(vbase + g * 512);
                            const uint32_t wb = *reinterpret_cast<const uint32_t*>(vbase + g * 512 + 4 * 32);
                            const uint32_t wc = *reinterpret_cast<const uint32_t*>(vbase + g * 512 + 8 * 32);
                            const uint32_t wd = *reinterpret_cast<const uint32_t*>(vbase + g * 512 + 12 * 32);
#pragma unroll
                            for (int u2 = 0; u2 < 2; ++u2) {
                                const uint32_t y = __byte_perm(wa, wb, u2 ? 0x7632u : 0x5410u);
                                const uint32_t z = __byte_perm(wc, wd, u2 ? 0x7632u : 0x5410u);
#pragma unroll
                                for (int u1 = 0; u1 < 2; ++u1) {
                                    const int mt = g * 4 + u2 * 2 + u1;
                                    const uint32_t ys = u1 ? y >> 8 : y, zs = u1 ? z >> 8 : z;
                                    const uint32_t a0 = dq_lo(ys), a1 = dq_hi(ys), a2 = dq_lo(zs), a3 = dq_hi(zs);
                                    mma_f16_16816(acc[mt], a0, a1, a2, a3, bh0, bh1);
                                }
                            }
                        }
                    } else {
                        const uint8_t* vrow = ss + L::kStripBytes + (2 * r) * 8;
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) {
                            const uint4 v = *reinterpret_cast<const uint4*>(vrow + mt * 128);
                            const uint32_t ya = __byte_perm(v.x, v.y, vsel), yb = __byte_perm(v.z, v.w, vsel);
                            const uint32_t a0 = dq_lo(ya), a2 = dq_hi(ya), a1 = dq_lo(yb), a3 = dq_hi(yb);
                            mma_f16_16816(acc[mt], a0, a1, a2, a3, bh0, bh1);
                        }
                    }
                }
            } else {
                // The wider arithmetic: P as hi + lo halves, and every tile's products summed in
                // an accumulator that starts at zero and joins the running one with an ordinary
                // FP32 addition -- the tensor core's own accumulation is then never more than a
                // few steps deep, so whatever rounding it applies cannot build up over a context.
                uint32_t bh[kTileStrips][2], bl[kTileStrips][2];
                bool on[kTileStrips];
#pragma unroll
                for (int ts = 0; ts < kTileStrips; ++ts) {
                    on[ts] = !(TAIL && strip_t + ts >= s1);   // warp-uniform
                    bh[ts][0] = bh[ts][1] = bl[ts][0] = bl[ts][1] = 0u;
                    if (!on[ts]) continue;
                    const float vs_lo = vs[ts][0] * inv_vnorm, vs_hi = vs[ts][1] * inv_vnorm;
                    float pw[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float pr = ex2f(fmaf(sc[ts][i], rfac[i & 1], -m_fac[i & 1]));
                        l_run[i & 1] += pr;
                        pw[i] = pr * (i < 2 ? vs_lo : vs_hi);
                    }
                    const uint32_t h0 = pack_f16x2(pw[0], pw[1]), h1 = pack_f16x2(pw[2], pw[3]);
                    const float2 f0 = unpack_f16x2(h0), f1 = unpack_f16x2(h1);
                    const uint32_t l0 = pack_f16x2(pw[0] - f0.x, pw[1] - f0.y);
                    const uint32_t l1 = pack_f16x2(pw[2] - f1.x, pw[3] - f1.y);
                    bh[ts][0] = movmatrix_trans(h0);
                    bh[ts][1] = movmatrix_trans(h1);
                    bl[ts][0] = movmatrix_trans(l0);
                    bl[ts][1] = movmatrix_trans(l1);
                    if constexpr (EXT) {
                        if (midrise) {   // the f16 values the MMAs multiply, so that acc and ps stay consistent
                            const float2 g0 = unpack_f16x2(l0), g1 = unpack_f16x2(l1);
                            ps[0] += (f0.x + f1.x) + (g0.x + g1.x);
                            ps[1] += (f0.y + f1.y) + (g0.y + g1.y);
                        }
                    }
                }
                if constexpr (NZ) {
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        float t[4][4];
#pragma unroll
                        for (int u = 0; u < 4; ++u)
#pragma unroll
                            for (int i = 0; i < 4; ++i) t[u][i] = 0.f;
#pragma unroll
                        for (int ts = 0; ts < kTileStrips; ++ts) {
                            if (!on[ts]) continue;
                            const uint8_t* vbase = st + ts * L::kStripStage + L::kStripBytes + qd * 32 + r * 4 + g * 512;
                            const uint32_t wa = *reinterpret_cast<const uint32_t*>(vbase);
                            const uint32_t wb = *reinterpret_cast<const uint32_t*>(vbase + 4 * 32);
                            const uint32_t wc = *reinterpret_cast<const uint32_t*>(vbase + 8 * 32);
                            const uint32_t wd = *reinterpret_cast<const uint32_t*>(vbase + 12 * 32);
#pragma unroll
                            for (int u = 0; u < 4; ++u) {
                                const uint32_t y = __byte_perm(wa, wb, (u & 2) ? 0x7632u : 0x5410u);
                                const uint32_t z = __byte_perm(wc, wd, (u & 2) ? 0x7632u : 0x5410u);
                                const uint32_t ys = (u & 1) ? y >> 8 : y, zs = (u & 1) ? z >> 8 : z;
                                const uint32_t a0 = dq_lo(ys), a1 = dq_hi(ys), a2 = dq_lo(zs), a3 = dq_hi(zs);
                                mma_f16_16816(t[u], a0, a1, a2, a3, bl[ts][0], bl[ts][1]);
                                mma_f16_16816(t[u], a0, a1, a2, a3, bh[ts][0], bh[ts][1]);
                            }
                        }
#pragma unroll
                        for (int u = 0; u < 4; ++u)
#pragma unroll
                            for (int i = 0; i < 4; ++i) acc[g * 4 + u][i] += t[u][i];
                    }
                } else {
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        float t[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                        for (int ts = 0; ts < kTileStrips; ++ts) {
                            if (!on[ts]) continue;
                            const uint8_t* vrow = st + ts * L::kStripStage + L::kStripBytes + (2 * r) * 8;
                            const uint4 v = *reinterpret_cast<const uint4*>(vrow + mt * 128);
                            const uint32_t ya = __byte_perm(v.x, v.y, vsel), yb = __byte_perm(v.z, v.w, vsel);
                            const uint32_t a0 = dq_lo(ya), a2 = dq_hi(ya), a1 = dq_lo(yb), a3 = dq_hi(yb);
                            mma_f16_16816(t, a0, a1, a2, a3, bl[ts][0], bl[ts][1]);
                            mma_f16_16816(t, a0, a1, a2, a3, bh[ts][0], bh[ts][1]);
                        }
#pragma unroll
                        for (int i = 0; i < 4; ++i) acc[mt][i] += t[i];
                    }
                }
            }
        };

        [[maybe_unused]] unsigned long long loop_began = 0;
        if constexpr (STREAMK) {
            if (p.census != nullptr && tid == 0) loop_began = global_timer_ns();
        }
        mark(8);   // prologue: copies of the first tile issued, query rotated, fragments built (first: since launch)
        uint32_t stage = 0;
        uint32_t strip_t = strip_first;   // first strip of the tile being computed
#pragma unroll 1
        for (uint32_t j = 0; j < my_tiles; ++j, strip_t += kTileStep) {
            {
                const uint32_t ahead = strip_t + (kStages - 1) * kTileStep;
                issue(ahead, stage == 0 ? kStages - 1 : stage - 1, pg_next);
                cp_async_commit();
                load_pages(ahead + kTileStep, pg_next);
            }
            cp_async_wait<kStages - 1>();
            uint8_t* st = my_ring + stage * L::kStageBytes;
            if constexpr (NZ) {
                // the stored scale is divided by the codebook gain (IEEE division, as the
                // importer does): every lane finishes the one scale it copied
#pragma unroll
                for (int ts = 0; ts < kTileStrips; ++ts) {
                    float* sv = reinterpret_cast<float*>(st + ts * L::kStripStage + 2 * L::kStripBytes) + lane;
                    *sv = __fdiv_rn(*sv, p.nz_gain);
                }
            }
            __syncwarp();
            if (++stage == kStages) stage = 0;
            if (strip_t + kTileStrips > s1 || (strip_t + kTileStrips) * kStrip > ctx_all)
                compute_tile(st, strip_t, std::true_type{});
            else
                compute_tile(st, strip_t, std::false_type{});
            __syncwarp();
        }
        cp_async_wait<0>();
        if constexpr (STREAMK) {
            if (p.census != nullptr && tid == 0) {
                p.census[kCensusWords * blockIdx.x + 2] += global_timer_ns() - loop_began;
                p.census[kCensusWords * blockIdx.x + 3] += 1ull;
            }
        }
        mark(-1);

        // ---- warp-level l, value normaliser out of acc, merge the warps through shared memory.
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            l_run[q] += __shfl_xor_sync(0xffffffffu, l_run[q], 4);
            l_run[q] += __shfl_xor_sync(0xffffffffu, l_run[q], 8);
            l_run[q] += __shfl_xor_sync(0xffffffffu, l_run[q], 16);
        }
        // mid-rise codes: sum_t P_t (code_t + 0.5) = acc + 0.5 * sum_t P_t, the same for every channel
        float half_p[2] = {0.f, 0.f};
        if constexpr (EXT) {
            if (midrise) {
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    ps[q] += __shfl_xor_sync(0xffffffffu, ps[q], 4);
                    ps[q] += __shfl_xor_sync(0xffffffffu, ps[q], 8);
                    ps[q] += __shfl_xor_sync(0xffffffffu, ps[q], 16);
                    half_p[q] = 0.5f * ps[q];
                }
            }
        }
        __syncthreads();  // every warp is done with its ring; reuse it
        mark(4);   // waiting for the slowest warp of the segment
        // Row pitch d + 4 floats: a lane stores its two adjacent channels of a row as one
        // 8-byte word, and with this pitch the 16 lanes of a half-warp hit 16 different banks pairs.
        constexpr int kPitch = L::kMergePitch;
        float* merge = reinterpret_cast<float*>(ring) + warp * 8 * kPitch;
        if (r == 0) {
            merge[(qd * 2 + 0) * kPitch + 0] = m_run[0];
            merge[(qd * 2 + 0) * kPitch + 1] = l_run[0];
            merge[(qd * 2 + 1) * kPitch + 0] = m_run[1];
            merge[(qd * 2 + 1) * kPitch + 1] = l_run[1];
        }
        if constexpr (NZ) {
            // MMA mt = 4 g + u: row r is channel 32 g + 4 r + u, row r + 8 channel 128 + that
#pragma unroll
            for (int g = 0; g < 4; ++g)
#pragma unroll
                for (int u = 0; u < 4; u += 2) {
                    const int mt = g * 4 + u, ch = g * 32 + 4 * r + u;
                    *reinterpret_cast<float2*>(merge + (qd * 2 + 0) * kPitch + 2 + ch) =
                        make_float2((acc[mt][0] + half_p[0]) * vnorm, (acc[mt + 1][0] + half_p[0]) * vnorm);
                    *reinterpret_cast<float2*>(merge + (qd * 2 + 0) * kPitch + 2 + 128 + ch) =
                        make_float2((acc[mt][2] + half_p[0]) * vnorm, (acc[mt + 1][2] + half_p[0]) * vnorm);
                    *reinterpret_cast<float2*>(merge + (qd * 2 + 1) * kPitch + 2 + ch) =
                        make_float2((acc[mt][1] + half_p[1]) * vnorm, (acc[mt + 1][1] + half_p[1]) * vnorm);
                    *reinterpret_cast<float2*>(merge + (qd * 2 + 1) * kPitch + 2 + 128 + ch) =
                        make_float2((acc[mt][3] + half_p[1]) * vnorm, (acc[mt + 1][3] + half_p[1]) * vnorm);
                }
        } else {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const int ch = mt * 16 + 2 * r;
                *reinterpret_cast<float2*>(merge + (qd * 2 + 0) * kPitch + 2 + ch) =
                    make_float2((acc[mt][0] + half_p[0]) * vnorm, (acc[mt][2] + half_p[0]) * vnorm);
                *reinterpret_cast<float2*>(merge + (qd * 2 + 1) * kPitch + 2 + ch) =
                    make_float2((acc[mt][1] + half_p[1]) * vnorm, (acc[mt][3] + half_p[1]) * vnorm);
            }
        }
        __syncthreads();
        // Inside the kernel m is in units of raw * key_scale; row_unscale turns a difference
        // of such maxima into log2 units, and times ln 2 into the natural units of a record.
        const float* mg = reinterpret_cast<const float*>(ring);
        // element c of the merged record of row q: 0 = m (natural units), 1 = l, 2 + ch = acc[ch]
        auto merged = [&](int q, int c) -> float {
            const float rf = row_unscale[q];
            float mm = kMaskedScore;
#pragma unroll
            for (int w = 0; w < kDecWarps; ++w) mm = fmaxf(mm, mg[(w * 8 + q) * kPitch]);
            if (c == 0) return mm > -1.0e37f ? mm * rf * kLn2 : kMaskedScore;
            float out = 0.f;
#pragma unroll
            for (int w = 0; w < kDecWarps; ++w) {
                const float* rw = mg + (w * 8 + q) * kPitch;
                out += rw[c] * ex2f((rw[0] - mm) * rf);
            }
            return out;
        };
        if constexpr (!STREAMK && !DIRECT) {
            for (int i = tid; i < rows_here * kRecord; i += blockDim.x) {
                const int q = i / kRecord, c = i % kRecord;
                rec_base[i] = merged(q, c < 8 ? 0 : c < 16 ? 1 : 2 + (c - 16));
            }
            return;
        } else {
            constexpr int kRecPitch = L::kRecPitch;
            float* rec = reinterpret_cast<float*>(ring + L::kMergeBytes);            // [8][kRecPitch]
            float* ebuf = reinterpret_cast<float*>(ring + L::kMergeBytes + L::kRecBytes);   // [2][8][D]
            bool finish = true;   // this CTA holds the head's complete state after the next block
            if (seg_count == 1u) {
                for (int i = tid; i < rows_here * kRecPitch; i += blockDim.x)
                    rec[i] = merged(i / kRecPitch, i % kRecPitch);
            } else {
                // several CTAs share this head: publish the record, count the arrival, and let
                // whoever arrives last merge all of them (nobody waits for anybody)
                for (int i = tid; i < rows_here * kRecPitch; i += blockDim.x) {
                    const int q = i / kRecPitch, c = i % kRecPitch;
                    const float v = merged(q, c);
                    float* dst = rec_base + q * kRecord;
                    if (c >= 2) dst[16 + (c - 2)] = v;
                    else
#pragma unroll
                        for (int k = 0; k < 8; ++k) dst[c * 8 + k] = v;
                }
                __threadfence();
                __syncthreads();
                if (tid == 0) {
                    uint32_t* word = p.counters + (static_cast<size_t>(item) * row_tiles + row_tile);
                    uint32_t old = STREAMK ? sk_seen : *reinterpret_cast<volatile uint32_t*>(word), want = 0;
                    bool counted = false;
                    // a word counts for this launch only under its tag; anything else is stale
                    for (int it = 0; it < 64 && !counted; ++it) {
                        want = ((old >> 8) == p.tag && (old & 0xFFu) < seg_count) ? old + 1u : ((p.tag << 8) | 1u);
                        const uint32_t prev = atomicCAS(word, old, want);
                        counted = prev == old;
                        old = prev;
                    }
                    if (!counted) report(p.status, TQ_STATUS_WAIT_EXPIRED);
                    const bool last = counted && (want & 0xFFu) == seg_count;
                    if (last) *reinterpret_cast<volatile uint32_t*>(word) = 0u;   // leave it clean for the next launch
                    sk_last = last ? 1u : 0u;
                }
                __syncthreads();
                finish = sk_last != 0u;
                if (finish) {
                    __threadfence();
                    const float* first = p.workspace +
                                         ((static_cast<size_t>(item) * p.splits) * p.rows_stride + row_tile * 8u) * kRecord;
                    const size_t slot_stride = static_cast<size_t>(p.rows_stride) * kRecord;
                    // weights of the records first: lane k of warp w reads m of record k of rows w
                    // and w + 4; the row maximum and exp(m_k - max) go to shared memory (the egress
                    // buffer is free)
                    float* wgt = ebuf;               // [8][32]
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const int q = warp + 4 * j, k = lane;
                        float mk = kMaskedScore;
                        if (q < rows_here && static_cast<uint32_t>(k) < seg_count)
                            mk = __ldcg(first + q * kRecord + k * slot_stride);
                        float mm = mk;
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, o));
                        wgt[q * 32 + k] = static_cast<uint32_t>(k) < seg_count ? ex2f((mk - mm) * kLog2e) : 0.f;
                        if (k == 0 && q < rows_here) rec[q * kRecPitch] = mm;
                    }
                    __syncthreads();
                    // then l and acc: sixteen records of an element are fetched before the first is
                    // used, so the loads overlap instead of forming a chain of round trips to L2
                    for (int i = tid; i < rows_here * (kRecPitch - 1); i += blockDim.x) {
                        const int q = i / (kRecPitch - 1), c = 1 + i % (kRecPitch - 1);
                        const float* rq = first + q * kRecord + (c == 1 ? 8 : 16 + (c - 2));
                        float out = 0.f;
                        for (uint32_t k0 = 0; k0 < seg_count; k0 += 16u) {
                            float v[16];
#pragma unroll
                            for (int k = 0; k < 16; ++k)
                                v[k] = k0 + k < seg_count ? __ldcg(rq + (k0 + k) * slot_stride) : 0.f;
#pragma unroll
                            for (int k = 0; k < 16; ++k) out = fmaf(v[k], wgt[q * 32 + k0 + k], out);
                        }
                        rec[q * kRecPitch + c] = out;
                    }
                }
            }
            mark(5);   // merge of the warps, record, fence, arrival (and the records of the other segments)
            if (finish) {
                __syncthreads();
                for (int i = tid; i < rows_here * D; i += blockDim.x) {
                    const int q = i / D, c = i % D;
                    const float l = rec[q * kRecPitch + 1], a = rec[q * kRecPitch + 2 + c];
                    ebuf[q * D + c] = l > 0.f ? a / l : 0.f;
                }
                __syncthreads();
                egress_rows<D>(p, ebuf, rows_here, seq, head, row_tile, tokens_per_req, tid);
            }
        }
        if constexpr (STREAMK) {
            mark(6);   // normalise, egress, output
            // ---- next segment of the chunk, or the next chunk off the ticket
            sk_left -= sk_take;
            if (sk_left == 0u) {
                __syncthreads();
                const uint32_t k = sk_chunk;   // drawn at the start of this segment
                if (k == 0xFFFFFFFFu || !begin_chunk(k)) {
                    leave();
                    return;
                }
                mark(7);   // next chunk located
                continue;   // begin_chunk ended on a barrier: the ring and the query buffer are free
            }
            sk_loc += sk_take;
            if (sk_loc == sk_n * heads_per_seq) {
                sk_before += sk_n;
                sk_loc = 0;
                do {   // tiles are left, so a sequence with tiles follows
                    ++seq;
                    if (seq >= batch) {
                        leave();
                        return;
                    }
                    sk_n = tiles_of(context_cached(seq));
                } while (sk_n == 0u);
            }
            __syncthreads();   // the epilogue buffers alias the ring and the prologue's query
            mark(7);
        } else {
            return;
        }
    }
}

// ------------------------------------------------------------------ combine
struct CombineParams {
    const float* workspace;
    const float* signs;
    const void* gate;
    void* output;
    uint32_t rows, rows_stride, splits, output_stage, out_dtype;
    float inv_sqrt_len;
    uint32_t block16;   // egress rotation: 0 the cache's two-level rotation, 1 block-diagonal H16 / 4
                        // (Lloyd-Max variant), 2 diag(s) H_d diag(s) / sqrt(d) (the fused decoder's Pi)
    uint32_t gate_dtype; // TQ_DTYPE_* of `gate`
    uint32_t tokens_per_req, kv_heads;   // output row of (item, row): see out_row below
};

// One CTA per (item, row): merge `splits` records, normalise, optionally rotate
// back with the egress cascade (routines/routine_vector_egress_rotate.hpp:186-277)
// and gate, narrow to bf16. D threads, one channel each.
// MAXK bounds the records per row (16 or kMaxSplits): the record loads are fully unrolled, and
// the narrower instantiation keeps the common case at half the registers.
template <int D, int MAXK>
__global__ void __launch_bounds__(D) tq_combine_kernel(const CombineParams p)
{
    constexpr int kRecord = 16 + D;
    __shared__ float buf[2][D];
    const uint32_t item = blockIdx.x / p.rows, row = blockIdx.x % p.rows;
    const int c = threadIdx.x;
    // (item, row) = (sequence, KV head, query token, head in group) -> row of the [tokens][heads]
    // output; with one query token per request this is blockIdx.x
    const uint32_t grp = p.rows / p.tokens_per_req, o_tok = row / grp, o_g = row - o_tok * grp;
    const uint32_t o_seq = item / p.kv_heads, o_head = item - o_seq * p.kv_heads;
    const size_t out_row = (static_cast<size_t>(o_seq) * p.tokens_per_req + o_tok) * (p.kv_heads * grp) +
                           static_cast<size_t>(o_head) * grp + o_g;
    const float* base = p.workspace + (static_cast<size_t>(item) * p.splits * p.rows_stride + row) * kRecord;
    const size_t split_stride = static_cast<size_t>(p.rows_stride) * kRecord;
    // Launched as the programmatic dependent of the kernel that writes the records, this grid
    // is set up while that kernel's last CTAs still run; the records are read only once that
    // kernel has completed (a no-op after an ordinary launch).
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    // All records are fetched before the first one is merged, so the loads overlap instead
    // of forming a chain of dependent round trips to L2 (at most MAXK records).
    float mk[MAXK], lk[MAXK], ak[MAXK];
#pragma unroll
    for (int k = 0; k < MAXK; ++k)
        if (static_cast<uint32_t>(k) < p.splits) {
            const float* rec = base + k * split_stride;
            mk[k] = rec[0];
            lk[k] = rec[8];
            ak[k] = rec[16 + c];
        }
    float m = kMaskedScore, l = 0.f, a = 0.f;
#pragma unroll
    for (int k = 0; k < MAXK; ++k)
        if (static_cast<uint32_t>(k) < p.splits) {
            const float mn = fmaxf(m, mk[k]);
            const float wa = ex2f((m - mn) * kLog2e), wb = ex2f((mk[k] - mn) * kLog2e);
            l = l * wa + lk[k] * wb;
            a = a * wa + ak[k] * wb;
            m = mn;
        }
    float v = l > 0.f ? a / l : 0.f;
    if (p.output_stage != TQ_OUT_ROTATED) {
        int cur = 0;
        buf[0][c] = p.block16 == 2u ? v * p.signs[c] : v;
        __syncthreads();
        auto stage = [&](int s) {
            const float mine = buf[cur][c], other = buf[cur][c ^ s];
            buf[cur ^ 1][c] = other + ((c & s) ? -mine : mine);
            __syncthreads();
            cur ^= 1;
        };
        if (p.block16 == 1u) {
            for (int s = 1; s < 16; s <<= 1) stage(s);
            v = buf[cur][c] * 0.25f;
        } else if (p.block16 == 2u) {
            // Pi = diag(s) H diag(s) / sqrt(d), an involution (tests/common/fused_decode_opt_fixture.hpp:
            // 104-117): signs went in with the load above, the full butterfly, signs and scale out
            for (int s = 1; s < D; s <<= 1) stage(s);
            v = buf[cur][c] * p.signs[c] * p.inv_sqrt_len;
        } else {
            for (int s = kGroup; s < D; s <<= 1) stage(s);
            buf[cur][c] *= p.signs[c];
            __syncthreads();
            for (int s = 1; s < kGroup; s <<= 1) stage(s);
            v = buf[cur][c] * p.inv_sqrt_len;
        }
        if (p.output_stage == TQ_OUT_GATED)
        {
            const size_t gi = out_row * D + c;
            const float gt = p.gate_dtype == TQ_DTYPE_F32 ? static_cast<const float*>(p.gate)[gi]
                             : p.gate_dtype == TQ_DTYPE_F16 ? __half2float(static_cast<const __half*>(p.gate)[gi])
                                                            : bf16_bits_to_f32(static_cast<const uint16_t*>(p.gate)[gi]);
            v = v / (1.0f + __expf(-gt));
        }
    }
    const size_t at = out_row * D + c;
    if (p.out_dtype == TQ_DTYPE_F32) static_cast<float*>(p.output)[at] = v;
    else if (p.out_dtype == TQ_DTYPE_F16) static_cast<__half*>(p.output)[at] = __float2half_rn(v);
    else static_cast<uint16_t*>(p.output)[at] = f32_to_bf16_bits(v);
}

// Pages of 16, 32, 64 or 128 tokens: the strip walk uses shifts, not divides.
static bool page_size_ok(uint32_t block_size, uint32_t* sp_shift)
{
    const uint32_t sp = block_size / kStrip;
    if (block_size % kStrip != 0 || sp == 0 || (sp & (sp - 1u)) != 0u) return false;
    uint32_t sh = 0;
    while ((1u << sh) < sp) ++sh;
    *sp_shift = sh;
    return true;
}

static bool aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0u; }

// A tag that no earlier launch used (24 bits, never zero): arrival counts of the persistent
// grid are valid only under the tag of their own launch, so the counter words need no
// clearing between launches and may start out as anything.
static uint32_t next_launch_tag()
{
    static std::atomic<uint32_t> serial{0};
    const uint32_t n = serial.fetch_add(1, std::memory_order_relaxed) + 1u;
    const uint32_t tag = (n * 2654435761u) >> 8;
    return tag ? tag : 1u;
}

// Worker census (tq_decode_worker_census): where the persistent grid's CTAs stamp their times.
static std::atomic<unsigned long long*> g_census{nullptr};
static std::atomic<uint32_t> g_census_ctas{0};

template <int D, bool PRECISE, bool EXT, bool NZ, int MODE>
static cudaError_t launch_partial_as(cudaStream_t stream, const DecodeParams& p_in)
{
    constexpr bool STREAMK = MODE == kModePersistent;
    DecodeParams p = p_in;
    // Opt in to the large dynamic shared-memory carve-out once per device. The
    // flags race benignly: setting the attribute twice is harmless.
    static bool configured[64] = {};
    static int sm_count[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return cudaErrorNoDevice;
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(tq_decode_partial_kernel<D, PRECISE, EXT, NZ, MODE>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             DecodeSmem<D>::kTotal);
        if (e != cudaSuccess) return e;
        int sms = 0;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) {
            sm_count[dev] = sms;
            configured[dev] = true;
        }
    }
    uint64_t grid = static_cast<uint64_t>(p.items) * ((p.rows + 7u) / 8u) * p.splits;
    if (grid == 0) return cudaSuccess;
    p.by_heads_tiles = Divider(p.items * ((p.rows + 7u) / 8u));
    p.by_row_tiles = Divider((p.rows + 7u) / 8u);
    p.by_heads = Divider(p.H);
    p.by_chunk_pages = Divider(p.chunk_pages ? p.chunk_pages : 1u);
    const bool equal_pieces = p.graded == 2u;
    p.graded = (!STREAMK && p.chunk_pages != 0u && p.splits > 1u && p.context_lens != nullptr) ? 1u : 0u;
    if (p.graded) {
        // The plan's split count is the number of record slots per head, whatever the head size
        // (the caller sizes its workspace and runs the combine with it). Head size 256 fills
        // fewer of them with longer pieces: its CTAs cost more (twice the rotation and merge) and
        // three are resident per SM instead of four; the slots it leaves out get an empty range
        // and export the neutral record. Measured on ragged batches of 64 (2048..16384 tokens, 16 q /
        // 4 KV heads): 0.7 of the pieces for the native layout (+5 % over all of them), all of them
        // for the NZ-tiled pools read in place.
        int sms = dev >= 0 && dev < 64 ? sm_count[dev] : 0;
        if (sms <= 0) sms = 148;
        uint32_t used = p.splits;
        if (D == 256) {
            if (equal_pieces) {
                const uint32_t fit = static_cast<uint32_t>(3 * sms) / (p.items ? p.items : 1u);
                used = fit < 1u ? 1u : (fit < p.splits ? fit : p.splits);
            } else {
                used = NZ ? p.splits : (p.splits * 7u + 9u) / 10u;   // ceil(0.7 splits)
                if (used < 1u) used = 1u;
            }
        }
        const double n = used, all = static_cast<double>(p.splits) * p.chunk_pages;
        // Graded pieces: widths fall linearly from `hi` to `2 - hi` of the mean, so the long pieces,
        // which amortise a CTA's fixed cost, start first and the short ones fill the end of the
        // launch (the split is the slowest grid index). Measured best on the ragged benchmark
        // batches: 1.75..1.85 at head size 128 (+1.5 % over 1.6), 1.6 at head size 256. The
        // one-wave plan asks for equal pieces (hi = 1).
        const double hi = equal_pieces || used == 1u ? 1.0 : (D == 128 ? 1.8 : 1.6);
        for (uint32_t k = 0; k <= p.splits; ++k)
            p.cuts[k] = k < used ? static_cast<uint32_t>(all * (k * (hi - (hi - 1.0) * (k - 1.0) / (n > 1.0 ? n - 1.0 : 1.0)) / n))
                                 : 0xFFFFFFFFu;
    }
    if (STREAMK) {
        int sms = dev >= 0 && dev < 64 ? sm_count[dev] : 0;
        if (sms <= 0) sms = 148;
        grid = static_cast<uint64_t>(sms) * DecodeSmem<D>::kCtasPerSm;   // one resident wave
    }
    if (grid > 0x7FFFFFFFull) return cudaErrorInvalidValue;
    p.census = STREAMK && grid <= g_census_ctas.load() ? g_census.load() : nullptr;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3(kDecWarps * 32);
    cfg.dynamicSmemBytes = DecodeSmem<D>::kTotal;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = p.follows_writer ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, tq_decode_partial_kernel<D, PRECISE, EXT, NZ, MODE>, p);
}

// The classic grid: one CTA per (sequence, KV head, split, row tile), records only.
template <int D, bool PRECISE, int MODE>
static cudaError_t launch_partial_mode(cudaStream_t stream, const DecodeParams& p)
{
    if constexpr (D == 256) {
        if (p.nz_slot_floats != 0u) return launch_partial_as<D, PRECISE, true, true, MODE>(stream, p);
    }
    if (p.q_f16 != 0u || p.tokens_per_req > 1u || p.q_f32 != nullptr || p.midrise != 0u)
        return launch_partial_as<D, PRECISE, true, false, MODE>(stream, p);
    return launch_partial_as<D, PRECISE, false, false, MODE>(stream, p);
}
template <int D, bool PRECISE>
static cudaError_t launch_partial(cudaStream_t stream, const DecodeParams& p)
{
    // an output to write (and therefore one split): the CTAs finish their heads themselves
    if (p.output != nullptr) return launch_partial_mode<D, PRECISE, kModeDirect>(stream, p);
    return launch_partial_mode<D, PRECISE, kModeRecords>(stream, p);
}

// The persistent grid with the combine folded in (native precision only).
template <int D>
static cudaError_t launch_streamk(cudaStream_t stream, const DecodeParams& p)
{
    return launch_partial_mode<D, false, kModePersistent>(stream, p);
}

}  // namespace tq

using namespace tq;

// Split plan for a launch that leaves the choice to the library. A sequence is cut into
// pieces of `chunk` tokens on average (graded by the launcher: the first piece 1.8, the last
// 0.2 of it at head size 128; 1.6 and 0.4 at head size 256), one CTA per piece and KV head. A CTA costs about 7 us besides its streaming
// (context length and block table, query rotation, merge and record), so pieces should be
// long; the end of the launch is filled by whatever pieces start last, so they should be
// short. Measured on ragged batches of 64 (2048..16384 tokens; 8 KV heads x 128 and 4 x 256):
// best with eight pieces for the longest sequence (head size 256 then fills four fifths of the
// slots with longer pieces, see launch_partial_as). Hence
//   chunk = max(tokens that give 32 CTAs per SM, max_context / 8),
// but no larger than what leaves three pieces per resident CTA slot (small batches need the
// parallelism more: batch 1 at 4096 tokens gets 256-token pieces; 16 sequences of 65 536 tokens
// x 8 heads: 216 us with three graded pieces per slot, 242 us with two), within 256..8192 tokens,
// in steps of 256, at least 1024 once the batch alone has a CTA per SM; the launch's split
// count is what the longest context needs, at most TQ_MAX_SPLITS.
static void decode_plan(uint32_t batch, uint32_t num_kv_heads, uint32_t block_size,
                        uint32_t max_context, uint32_t sm_count, uint32_t* splits,
                        uint32_t* chunk_pages)
{
    *splits = 1;
    *chunk_pages = 0;
    if (batch == 0 || num_kv_heads == 0 || block_size == 0 || max_context <= 256u) return;
    const uint64_t sms = sm_count ? sm_count : 148u;
    const uint64_t items = static_cast<uint64_t>(batch) * num_kv_heads;
    const uint64_t slots = sms * 4u;   // resident CTAs of the decode kernel at head size 128
    const uint64_t work = items * max_context;
    const uint64_t by_load = work / (32ull * sms);
    const uint64_t by_shape = max_context / 8u;
    const uint64_t by_fill = work / (3ull * slots);
    const uint64_t floor_tokens = items >= sms ? 1024 : 256;
    uint64_t chunk = by_load > by_shape ? by_load : by_shape;
    if (chunk > by_fill) chunk = by_fill;
    if (chunk < floor_tokens) chunk = floor_tokens;
    chunk = (chunk + 255u) / 256u * 256u;
    if (chunk > 8192u) chunk = 8192u;
    while ((max_context + chunk - 1u) / chunk > TQ_MAX_SPLITS) chunk += 256u;   // very long contexts
    if (chunk < block_size) chunk = block_size;
    chunk = (chunk + block_size - 1u) / block_size * block_size;
    *splits = static_cast<uint32_t>((max_context + chunk - 1u) / chunk);
    // A launch that fits the resident CTA slots at once gains nothing from pieces of different
    // lengths: its time is that of its longest piece, so they are made equal.
    const bool equal = items * *splits <= slots;
    *chunk_pages = static_cast<uint32_t>(chunk / block_size) | (equal ? kEqualPieces : 0u);
}

// Worker census of the persistent decode grid, after the reference's WorkerMetrics
// (include/turboquant_splitk_contract.hpp:101-118, absolute cycle stamps published per worker):
// while a buffer is registered, every CTA of a persistent decode launch writes ten words at
// device_words[10 * cta]: the global-timer nanosecond of its start, of its leaving (0: no
// work), the nanoseconds its first warp spent inside tile loops, its segment count, and the
// nanoseconds of five boundary phases (see mark() in the kernel). capacity_ctas bounds the
// grid that may write. A process-wide setting
// for measurement runs, not for concurrent use; null switches it off.
extern "C" int tq_decode_worker_census(unsigned long long* device_words, uint32_t capacity_ctas)
{
    g_census_ctas.store(device_words ? capacity_ctas : 0u);
    g_census.store(device_words);
    return TQ_OK;
}

extern "C" uint32_t tq_decode_choose_splits(uint32_t batch, uint32_t num_kv_heads,
                                            uint32_t block_size, uint32_t max_context,
                                            uint32_t sm_count)
{
    uint32_t splits, chunk_pages;
    decode_plan(batch, num_kv_heads, block_size, max_context, sm_count, &splits, &chunk_pages);
    return splits;
}

extern "C" size_t tq_decode_workspace_floats(uint32_t batch, uint32_t num_heads,
                                             uint32_t num_kv_heads, uint32_t head_size,
                                             uint32_t splits)
{
    if (num_kv_heads == 0) return 0;
    const size_t rows = num_heads / num_kv_heads;
    // the partial records, then one arrival counter per (sequence, KV head, 8-row tile) for
    // the launches that fold the combine into the decode kernel
    // ... and, 8-byte aligned behind them, the two 64-bit words of its chunk schedule
    const size_t words = static_cast<size_t>(batch) * num_kv_heads * splits * rows * (16u + head_size) +
                         static_cast<size_t>(batch) * num_kv_heads * ((rows + 7u) / 8u);
    return (words + 1u) / 2u * 2u + 4u;
}

extern "C" int tq_decode_splitk_partials(void* stream, const uint16_t* q, const void* signs,
                                         uint32_t sign_source, const int8_t* key_cache,
                                         const int8_t* value_cache, const float* scale_cache,
                                         const uint32_t* table, uint16_t* q_rot, float* workspace,
                                         uint32_t requests, uint32_t heads, uint32_t rows,
                                         uint32_t head_size, uint32_t block_size,
                                         uint32_t cache_pages, uint32_t seq_pages, uint32_t splits,
                                         uint32_t page_begin, uint32_t page_count, uint32_t seq_len,
                                         float inv_sqrt_len, float softmax_scale, uint32_t* status)
{
    // Geometry rules of the reference launcher
    // (kernels/ops/turboquant/turboquant_paged_decode_attention.cpp:1747-1759).
    if (!requests || !heads || !splits || splits > 16 || !seq_pages || !block_size ||
        block_size % kStrip != 0 || seq_pages > cache_pages || page_begin > seq_pages ||
        page_count > seq_pages - page_begin || rows == 0 || rows > 16 ||
        (head_size != 128 && head_size != 256) ||
        (sign_source != TQ_SIGNS_F32 && sign_source != TQ_SIGNS_TABLES_BF16) ||
        !(softmax_scale > 0.0f) || !(softmax_scale <= 3.0e38f))
        return TQ_ERR_INVALID_ARGUMENT;
    if (seq_len != 0u) {
        if (static_cast<uint64_t>(seq_len) > static_cast<uint64_t>(cache_pages) * block_size)
            return TQ_ERR_INVALID_ARGUMENT;  // seq_len exceeds the allocated cache
        const uint64_t window_end = static_cast<uint64_t>(page_begin + page_count) * block_size;
        if (static_cast<uint64_t>(seq_len) > window_end)
            return TQ_ERR_INVALID_ARGUMENT;  // live tokens past the end of the page window
    }
    if (!q || !signs || !key_cache || !value_cache || !scale_cache || !table || !workspace)
        return TQ_ERR_INVALID_ARGUMENT;
    uint32_t sp_shift = 0;
    if (!page_size_ok(block_size, &sp_shift) || !aligned16(key_cache) || !aligned16(value_cache) ||
        !aligned16(scale_cache))
        return TQ_ERR_INVALID_ARGUMENT;
    DecodeParams p{};
    p.tokens_per_req = 1;
    p.sp_shift = sp_shift;
    p.q = q;
    p.signs = signs;
    p.sign_source = sign_source;
    p.key_cache = reinterpret_cast<const uint8_t*>(key_cache);
    p.value_cache = reinterpret_cast<const uint8_t*>(value_cache);
    p.scale_cache = scale_cache;
    p.table = reinterpret_cast<const int32_t*>(table);
    p.context_lens = nullptr;
    p.q_rot = q_rot;
    p.workspace = workspace;
    p.items = requests * heads;
    p.H = heads;
    p.rows = rows;
    p.rows_stride = 16;
    p.S = block_size;
    p.P = cache_pages;
    p.table_stride = seq_pages;
    p.splits = splits;
    p.page_begin = page_begin;
    p.page_count = page_count;
    p.fixed_ctx = seq_len ? seq_len : seq_pages * block_size;
    p.inv_sqrt_len = inv_sqrt_len;
    p.softmax_scale = softmax_scale;
    p.status = status;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const cudaError_t e = head_size == 128 ? launch_partial<128, true>(s, p) : launch_partial<256, true>(s, p);
    return e == cudaSuccess ? TQ_OK : TQ_ERR_LAUNCH;
}

static int splitk_combine(void* stream, const float* workspace, const float* pi_signs,
                          const void* gate, uint32_t gate_dtype, void* output, uint32_t out_dtype,
                          uint32_t items, uint32_t rows, uint32_t rows_stride, uint32_t head_size,
                          uint32_t splits, uint32_t output_stage, float inv_sqrt_len,
                          uint32_t tokens_per_req = 1, uint32_t kv_heads = 1, uint32_t rotation = ~0u,
                          bool follows_export = false)
{
    if (!rows || rows > rows_stride || !splits || splits > TQ_MAX_SPLITS || output_stage > TQ_OUT_GATED ||
        out_dtype > TQ_DTYPE_F32 || gate_dtype > TQ_DTYPE_F32 ||
        (head_size != 128 && head_size != 256))
        return TQ_ERR_INVALID_ARGUMENT;
    // pi_signs == nullptr selects the block-diagonal H16 / 4 egress of the Lloyd-Max variant
    if (!workspace || !output || (output_stage == TQ_OUT_GATED && !gate))
        return TQ_ERR_INVALID_ARGUMENT;
    if (items == 0) return TQ_OK;
    CombineParams p{workspace, pi_signs, gate, output, rows, rows_stride, splits, output_stage,
                    out_dtype, inv_sqrt_len, rotation != ~0u ? rotation : (pi_signs == nullptr ? 1u : 0u),
                    gate_dtype, tokens_per_req, kv_heads};
    const uint64_t grid = static_cast<uint64_t>(items) * rows;
    if (grid > 0x7FFFFFFFull) return TQ_ERR_INVALID_ARGUMENT;
    // Right behind the export kernel of the same call the combine is its programmatic
    // dependent: the export's CTAs release it as they start, it is scheduled as they drain, and
    // griddepcontrol.wait holds its reads back until the export has completed.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3(head_size);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = follows_export ? 1 : 0;
    cudaError_t e;
    if (head_size == 128)
        e = splits <= 16u ? cudaLaunchKernelEx(&cfg, tq_combine_kernel<128, 16>, p)
                          : cudaLaunchKernelEx(&cfg, tq_combine_kernel<128, kMaxSplits>, p);
    else
        e = splits <= 16u ? cudaLaunchKernelEx(&cfg, tq_combine_kernel<256, 16>, p)
                          : cudaLaunchKernelEx(&cfg, tq_combine_kernel<256, kMaxSplits>, p);
    return e == cudaSuccess ? TQ_OK : TQ_ERR_LAUNCH;
}

extern "C" int tq_splitk_combine(void* stream, const float* workspace, const float* pi_signs,
                                 const float* gate, void* output, uint32_t out_dtype,
                                 uint32_t items, uint32_t rows, uint32_t rows_stride,
                                 uint32_t head_size, uint32_t splits, uint32_t output_stage,
                                 float inv_sqrt_len, uint32_t* /*status*/)
{
    return splitk_combine(stream, workspace, pi_signs, gate, TQ_DTYPE_F32, output, out_dtype, items, rows,
                          rows_stride, head_size, splits, output_stage, inv_sqrt_len);
}

static uint32_t resolve_splits(uint32_t splits, uint32_t batch, uint32_t num_kv_heads,
                               uint32_t block_size, uint32_t max_blocks, uint32_t hint,
                               uint32_t* chunk_pages = nullptr)
{
    if (chunk_pages) *chunk_pages = 0;
    if (splits != 0) return splits;   // explicit: every sequence uses the reference Partition
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess)
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    uint32_t s = 1, c = 0;
    decode_plan(batch, num_kv_heads, block_size, hint ? hint : max_blocks * block_size,
                static_cast<uint32_t>(sms), &s, &c);
    if (chunk_pages) *chunk_pages = c;
    return s;
}

// What the serving entries add to the plain decode.
struct DecodeOptions {
    bool q_f16 = false;                  // FP16 query whose rotation stays FP32
    uint32_t tokens_per_req = 1;         // query tokens per request
    const float* query_rot_f32 = nullptr;  // pre-rotated FP32 query (replaces query and signs)
    uint32_t midrise = 0;                // codes on the uniform mid-rise grid
    uint32_t rotation = ~0u;             // egress rotation of the combine (~0: from pi_signs)
    uint32_t gate_dtype = TQ_DTYPE_F32;
    uint32_t nz_slot_floats = 0;         // != 0: NZ-tiled source pools, floats per slot of the scale records
    float nz_gain = 1.0f;                // the codebook gain those scales are divided by
    bool precise = false;                // 24-bit fixed-point query and P as hi + lo halves (classic grid)
    bool persistent = false;             // one launch: persistent grid, combine folded in
    bool follows_writer = false;         // directly behind the step's scatter writer in the stream
};

// Validates a decode call and fills the kernel parameters (everything but the combine part).
static int decode_params(DecodeParams& p, const uint16_t* query, const int8_t* key_cache,
                         const int8_t* value_cache, const float* scale_cache,
                         const int32_t* block_tables, const int32_t* context_lens,
                         const float* pi_signs, float* workspace, uint32_t batch,
                         uint32_t num_heads, uint32_t num_kv_heads, uint32_t head_size,
                         uint32_t block_size, uint32_t num_blocks, uint32_t max_blocks,
                         uint32_t splits, uint32_t chunk_pages, float inv_sqrt_len,
                         float softmax_scale, uint32_t* status, const DecodeOptions& o,
                         bool needs_workspace = true)
{
    if (!num_heads || !num_kv_heads || num_heads % num_kv_heads != 0 || !block_size ||
        block_size % kStrip != 0 || !num_blocks || !max_blocks || !splits || splits > TQ_MAX_SPLITS ||
        (head_size != 128 && head_size != 256))
        return TQ_ERR_INVALID_ARGUMENT;
    // the kernels take the maximum of raw scores before the positive per-row factor is applied
    if (!(softmax_scale > 0.0f) || !(softmax_scale <= 3.0e38f)) return TQ_ERR_INVALID_ARGUMENT;
    const uint32_t rows = num_heads / num_kv_heads * o.tokens_per_req;
    if (rows > 16 || o.tokens_per_req == 0) return TQ_ERR_INVALID_ARGUMENT;
    if (o.nz_slot_floats != 0u &&
        (head_size != 256 || (block_size != 64 && block_size != 128) || !(o.nz_gain > 0.0f) ||
         o.nz_slot_floats < 2u * num_kv_heads))
        return TQ_ERR_INVALID_ARGUMENT;
    if (batch == 0) return TQ_OK;
    // a pre-rotated FP32 query replaces both the 16-bit query and the sign diagonal
    if ((!query || !pi_signs) && !o.query_rot_f32) return TQ_ERR_INVALID_ARGUMENT;
    if (!key_cache || !value_cache || !scale_cache || !block_tables || !context_lens ||
        (needs_workspace && !workspace))
        return TQ_ERR_INVALID_ARGUMENT;
    uint32_t sp_shift = 0;
    if (!page_size_ok(block_size, &sp_shift) || !aligned16(key_cache) || !aligned16(value_cache) ||
        !aligned16(scale_cache))
        return TQ_ERR_INVALID_ARGUMENT;
    p = DecodeParams{};
    p.sp_shift = sp_shift;
    p.q = query;
    p.q_f32 = o.query_rot_f32;
    p.midrise = o.midrise;
    p.signs = pi_signs;
    p.sign_source = TQ_SIGNS_F32;
    p.key_cache = reinterpret_cast<const uint8_t*>(key_cache);
    p.value_cache = reinterpret_cast<const uint8_t*>(value_cache);
    p.scale_cache = scale_cache;
    p.table = block_tables;
    p.context_lens = context_lens;
    p.follows_writer = o.follows_writer ? 1u : 0u;
    p.q_rot = nullptr;
    p.workspace = workspace;
    p.items = batch * num_kv_heads;
    p.H = num_kv_heads;
    p.rows = rows;
    p.rows_stride = rows;
    p.S = block_size;
    p.P = num_blocks;
    p.table_stride = max_blocks;
    p.splits = splits;
    p.chunk_pages = chunk_pages & ~kEqualPieces;
    p.graded = (chunk_pages & kEqualPieces) ? 2u : 0u;   // 2: equal cuts asked for (see launch_partial_as)
    p.q_f16 = o.q_f16 ? 1u : 0u;
    p.tokens_per_req = o.tokens_per_req;
    p.page_begin = 0;
    p.page_count = 0;
    p.fixed_ctx = 0;
    p.inv_sqrt_len = inv_sqrt_len;
    p.softmax_scale = softmax_scale;
    p.status = status;
    p.nz_slot_floats = o.nz_slot_floats;
    p.nz_gain = o.nz_gain;
    return TQ_OK;
}

// The export stage with its split plan resolved: `splits` partitions per sequence in the
// workspace, of which a sequence uses ceil(pages / chunk_pages) when chunk_pages != 0.
static int decode_export_planned(void* stream, const uint16_t* query, const int8_t* key_cache,
                                 const int8_t* value_cache, const float* scale_cache,
                                 const int32_t* block_tables, const int32_t* context_lens,
                                 const float* pi_signs, float* workspace, uint32_t batch,
                                 uint32_t num_heads, uint32_t num_kv_heads, uint32_t head_size,
                                 uint32_t block_size, uint32_t num_blocks, uint32_t max_blocks,
                                 uint32_t splits, uint32_t chunk_pages, float inv_sqrt_len,
                                 float softmax_scale, uint32_t* status, const DecodeOptions& o = {})
{
    DecodeParams p{};
    const int st = decode_params(p, query, key_cache, value_cache, scale_cache, block_tables,
                                 context_lens, pi_signs, workspace, batch, num_heads, num_kv_heads,
                                 head_size, block_size, num_blocks, max_blocks, splits, chunk_pages,
                                 inv_sqrt_len, softmax_scale, status, o);
    if (st != TQ_OK || batch == 0) return st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e;
    if (o.precise) e = head_size == 128 ? launch_partial<128, true>(s, p) : launch_partial<256, true>(s, p);
    else e = head_size == 128 ? launch_partial<128, false>(s, p) : launch_partial<256, false>(s, p);
    return e == cudaSuccess ? TQ_OK : TQ_ERR_LAUNCH;
}

extern "C" int tq_decode_splitk_export(void* stream, const uint16_t* query,
                                       const int8_t* key_cache, const int8_t* value_cache,
                                       const float* scale_cache, const int32_t* block_tables,
                                       const int32_t* context_lens, const float* pi_signs,
                                       float* workspace, uint32_t batch, uint32_t num_heads,
                                       uint32_t num_kv_heads, uint32_t head_size,
                                       uint32_t block_size, uint32_t num_blocks,
                                       uint32_t max_blocks, uint32_t splits,
                                       uint32_t max_context_hint, float inv_sqrt_len,
                                       float softmax_scale, uint32_t* status)
{
    if (!num_kv_heads || !block_size || splits > TQ_MAX_SPLITS) return TQ_ERR_INVALID_ARGUMENT;
    uint32_t chunk_pages = 0;
    splits = resolve_splits(splits, batch, num_kv_heads, block_size, max_blocks, max_context_hint,
                            &chunk_pages);
    return decode_export_planned(stream, query, key_cache, value_cache, scale_cache, block_tables,
                                 context_lens, pi_signs, workspace, batch, num_heads, num_kv_heads,
                                 head_size, block_size, num_blocks, max_blocks, splits, chunk_pages,
                                 inv_sqrt_len, softmax_scale, status);
}

// One decode call, split plan resolved. The classic grid exports `splits` records per head
// (a plan the library made itself gives every sequence as many as it has chunks; a split
// count the caller fixed keeps the reference's page partition) and the combine kernel merges
// them; one split finishes inside the export kernel. `persistent` selects the single-launch
// persistent grid instead (tq_decode_splitk_persistent).
static int decode_planned(void* stream, const uint16_t* query, const int8_t* key_cache,
                          const int8_t* value_cache, const float* scale_cache,
                          const int32_t* block_tables, const int32_t* context_lens,
                          const float* pi_signs, const void* gate, float* workspace, void* output,
                          uint32_t out_dtype, uint32_t batch, uint32_t num_heads,
                          uint32_t num_kv_heads, uint32_t head_size, uint32_t block_size,
                          uint32_t num_blocks, uint32_t max_blocks, uint32_t splits,
                          uint32_t chunk_pages, uint32_t output_stage, float inv_sqrt_len,
                          float softmax_scale, uint32_t* status, const DecodeOptions& o = {})
{
    if (output_stage > TQ_OUT_GATED || out_dtype > TQ_DTYPE_F32 || o.gate_dtype > TQ_DTYPE_F32 || !output ||
        (output_stage == TQ_OUT_GATED && !gate))
        return TQ_ERR_INVALID_ARGUMENT;
    const uint32_t rotation = o.rotation != ~0u ? o.rotation : (pi_signs == nullptr ? 1u : 0u);
    const bool persistent = o.persistent && splits >= 2u && !o.precise;
    if (persistent || splits == 1u) {
        // one launch: the persistent grid, or (one split) the classic grid whose CTAs hold a
        // head's whole state and write the output themselves without touching the workspace
        DecodeParams p{};
        const int st = decode_params(p, query, key_cache, value_cache, scale_cache, block_tables,
                                     context_lens, pi_signs, workspace, batch, num_heads, num_kv_heads,
                                     head_size, block_size, num_blocks, max_blocks, splits, chunk_pages,
                                     inv_sqrt_len, softmax_scale, status, o, persistent);
        if (st != TQ_OK || batch == 0) return st;
        if (output_stage != TQ_OUT_ROTATED && rotation != 1u && !pi_signs) return TQ_ERR_INVALID_ARGUMENT;
        if (persistent) {
            // the counters follow the records, the schedule words the counters (tq_decode_workspace_floats)
            if ((reinterpret_cast<uintptr_t>(workspace) & 7u) != 0u) return TQ_ERR_INVALID_ARGUMENT;
            const size_t records = static_cast<size_t>(batch) * num_kv_heads * splits * p.rows * (16u + head_size);
            const size_t counters = static_cast<size_t>(batch) * num_kv_heads * ((p.rows + 7u) / 8u);
            p.counters = reinterpret_cast<uint32_t*>(workspace + records);
            p.ticket = reinterpret_cast<unsigned long long*>(workspace + (records + counters + 1u) / 2u * 2u);
            p.tag = next_launch_tag();
        }
        p.egress_signs = pi_signs;
        p.gate = gate;
        p.output = output;
        p.output_stage = output_stage;
        p.out_dtype = out_dtype;
        p.gate_dtype = o.gate_dtype;
        p.rotation = rotation;
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        cudaError_t e;
        if (persistent) e = head_size == 128 ? launch_streamk<128>(s, p) : launch_streamk<256>(s, p);
        else if (o.precise) e = head_size == 128 ? launch_partial<128, true>(s, p) : launch_partial<256, true>(s, p);
        else e = head_size == 128 ? launch_partial<128, false>(s, p) : launch_partial<256, false>(s, p);
        return e == cudaSuccess ? TQ_OK : TQ_ERR_LAUNCH;
    }
    const int st = decode_export_planned(stream, query, key_cache, value_cache, scale_cache,
                                         block_tables, context_lens, pi_signs, workspace, batch,
                                         num_heads, num_kv_heads, head_size, block_size, num_blocks,
                                         max_blocks, splits, chunk_pages, inv_sqrt_len,
                                         softmax_scale, status, o);
    if (st != TQ_OK || batch == 0) return st;
    const uint32_t rows = num_heads / num_kv_heads * o.tokens_per_req;
    return splitk_combine(stream, workspace, pi_signs, gate, o.gate_dtype, output, out_dtype,
                          batch * num_kv_heads, rows, rows, head_size, splits, output_stage,
                          inv_sqrt_len, o.tokens_per_req, num_kv_heads, rotation, true);
}

// Query, gate and output in ONE 16-bit element type, FP16 or BF16, as the raw-query entry of
// the reference's fused decoder takes them (include/turboquant_fused_decode_opt.hpp:118-131,
// :160-169). A BF16 query is rotated and rounded to bf16 exactly as in tq_decode_splitk; an
// FP16 query keeps its FP32 rotation (the fused decoder's rotated image is FP32) and is cut
// to the 16-bit fixed point of the integer MMA directly.
extern "C" int tq_decode_splitk_elem(void* stream, const void* query, const int8_t* key_cache,
                                     const int8_t* value_cache, const float* scale_cache,
                                     const int32_t* block_tables, const int32_t* context_lens,
                                     const float* pi_signs, const void* gate, float* workspace,
                                     void* output, uint32_t elem_dtype, uint32_t batch,
                                     uint32_t num_heads, uint32_t num_kv_heads, uint32_t head_size,
                                     uint32_t block_size, uint32_t num_blocks, uint32_t max_blocks,
                                     uint32_t splits, uint32_t max_context_hint,
                                     uint32_t output_stage, float inv_sqrt_len, float softmax_scale,
                                     uint32_t* status)
{
    if (!num_kv_heads || !block_size || splits > TQ_MAX_SPLITS ||
        (elem_dtype != TQ_DTYPE_BF16 && elem_dtype != TQ_DTYPE_F16))
        return TQ_ERR_INVALID_ARGUMENT;
    uint32_t chunk_pages = 0;
    splits = resolve_splits(splits, batch, num_kv_heads, block_size, max_blocks, max_context_hint,
                            &chunk_pages);
    DecodeOptions o;
    o.gate_dtype = elem_dtype;
    o.q_f16 = elem_dtype == TQ_DTYPE_F16;
    return decode_planned(stream, static_cast<const uint16_t*>(query), key_cache, value_cache, scale_cache,
                          block_tables, context_lens, pi_signs, gate, workspace, output, elem_dtype, batch,
                          num_heads, num_kv_heads, head_size, block_size, num_blocks, max_blocks, splits,
                          chunk_pages, output_stage, inv_sqrt_len, softmax_scale, status, o);
}

extern "C" int tq_decode_splitk(void* stream, const uint16_t* query, const int8_t* key_cache,
                                const int8_t* value_cache, const float* scale_cache,
                                const int32_t* block_tables, const int32_t* context_lens,
                                const float* pi_signs, const float* gate, float* workspace,
                                void* output, uint32_t out_dtype, uint32_t batch, uint32_t num_heads,
                                uint32_t num_kv_heads, uint32_t head_size, uint32_t block_size,
                                uint32_t num_blocks, uint32_t max_blocks, uint32_t splits,
                                uint32_t max_context_hint, uint32_t output_stage,
                                float inv_sqrt_len, float softmax_scale, uint32_t* status)
{
    if (!num_kv_heads || !block_size || splits > TQ_MAX_SPLITS) return TQ_ERR_INVALID_ARGUMENT;
    uint32_t chunk_pages = 0;
    splits = resolve_splits(splits, batch, num_kv_heads, block_size, max_blocks, max_context_hint,
                            &chunk_pages);
    return decode_planned(stream, query, key_cache, value_cache, scale_cache, block_tables,
                          context_lens, pi_signs, gate, workspace, output, out_dtype, batch, num_heads,
                          num_kv_heads, head_size, block_size, num_blocks, max_blocks, splits,
                          chunk_pages, output_stage, inv_sqrt_len, softmax_scale, status);
}

// One decode step of a serving stack as one call: the new token of every sequence is written
// into the cache (tq_reshape_scatter: request r owns token r, slot_mapping[r] its slot, a negative
// slot skips the write), then the batch is decoded over its pages, the new token included
// (context_lens already count it). The decode is launched as the programmatic dependent of the
// writer: its CTAs are scheduled, read their context lengths, block-table entries and queries and
// rotate their queries while the writer still runs, and wait for the writer's completion only
// before their first read of the cache.
extern "C" int tq_reshape_scatter(void* stream, const uint16_t* key, const uint16_t* value,
                                  int8_t* key_cache, int8_t* value_cache, float* scale_cache,
                                  const int32_t* slot_mapping, const float* pi_signs,
                                  const int32_t* cu_seqlens, uint32_t num_requests,
                                  uint32_t num_kv_heads, uint32_t head_size, uint32_t block_size,
                                  uint32_t num_blocks, uint32_t item_begin, uint32_t item_count,
                                  float inv_sqrt_len, uint32_t* status);

extern "C" int tq_decode_step(void* stream, const uint16_t* new_key, const uint16_t* new_value,
                              const int32_t* slot_mapping, const uint16_t* query, int8_t* key_cache,
                              int8_t* value_cache, float* scale_cache, const int32_t* block_tables,
                              const int32_t* context_lens, const float* pi_signs, const float* gate,
                              float* workspace, void* output, uint32_t out_dtype, uint32_t batch,
                              uint32_t num_heads, uint32_t num_kv_heads, uint32_t head_size,
                              uint32_t block_size, uint32_t num_blocks, uint32_t max_blocks,
                              uint32_t splits, uint32_t max_context_hint, uint32_t output_stage,
                              float inv_sqrt_len, float softmax_scale, uint32_t* status)
{
    if (!num_kv_heads || !block_size || splits > TQ_MAX_SPLITS) return TQ_ERR_INVALID_ARGUMENT;
    uint32_t chunk_pages = 0;
    splits = resolve_splits(splits, batch, num_kv_heads, block_size, max_blocks, max_context_hint,
                            &chunk_pages);
    // everything the decode would refuse is refused before the cache is touched
    {
        DecodeParams probe{};
        DecodeOptions o;
        const int st = decode_params(probe, query, key_cache, value_cache, scale_cache, block_tables,
                                     context_lens, pi_signs, workspace, batch, num_heads, num_kv_heads,
                                     head_size, block_size, num_blocks, max_blocks, splits, chunk_pages,
                                     inv_sqrt_len, softmax_scale, status, o, splits > 1u);
        if (st != TQ_OK) return st;
        if (output_stage > TQ_OUT_GATED || out_dtype > TQ_DTYPE_F32 || !output ||
            (output_stage == TQ_OUT_GATED && !gate))
            return TQ_ERR_INVALID_ARGUMENT;
    }
    if (batch == 0) return TQ_OK;
    const int ws = tq_reshape_scatter(stream, new_key, new_value, key_cache, value_cache, scale_cache,
                                      slot_mapping, pi_signs, nullptr, batch, num_kv_heads, head_size,
                                      block_size, num_blocks, 0, batch * num_kv_heads, inv_sqrt_len, status);
    if (ws != TQ_OK) return ws;
    DecodeOptions o;
    o.follows_writer = true;
    return decode_planned(stream, query, key_cache, value_cache, scale_cache, block_tables,
                          context_lens, pi_signs, gate, workspace, output, out_dtype, batch, num_heads,
                          num_kv_heads, head_size, block_size, num_blocks, max_blocks, splits,
                          chunk_pages, output_stage, inv_sqrt_len, softmax_scale, status, o);
}

// Several query tokens per request (a decode step that verifies speculative tokens): the
// query is [batch * tokens_per_req][num_heads][d], token t of a request attends to
// context_lens[b] - (tokens_per_req - 1 - t) tokens, and all tokens_per_req * (num_heads /
// num_kv_heads) <= 16 rows of a KV head share one pass over its pages (the row tile of the
// reference's draft for its GQA decoder, reports/qwen35_turboquant_rfc.md:221-236). The
// workspace holds batch * num_kv_heads * splits * rows * (16 + d) floats.
extern "C" int tq_decode_splitk_mtp(void* stream, const uint16_t* query, const int8_t* key_cache,
                                    const int8_t* value_cache, const float* scale_cache,
                                    const int32_t* block_tables, const int32_t* context_lens,
                                    const float* pi_signs, const float* gate, float* workspace,
                                    void* output, uint32_t out_dtype, uint32_t batch,
                                    uint32_t tokens_per_req, uint32_t num_heads, uint32_t num_kv_heads,
                                    uint32_t head_size, uint32_t block_size, uint32_t num_blocks,
                                    uint32_t max_blocks, uint32_t splits, uint32_t max_context_hint,
                                    uint32_t output_stage, float inv_sqrt_len, float softmax_scale,
                                    uint32_t* status)
{
    if (!num_kv_heads || !block_size || splits > TQ_MAX_SPLITS || tokens_per_req == 0) return TQ_ERR_INVALID_ARGUMENT;
    uint32_t chunk_pages = 0;
    splits = resolve_splits(splits, batch, num_kv_heads, block_size, max_blocks, max_context_hint,
                            &chunk_pages);
    DecodeOptions o;
    o.tokens_per_req = tokens_per_req;
    return decode_planned(stream, query, key_cache, value_cache, scale_cache, block_tables, context_lens,
                          pi_signs, gate, workspace, output, out_dtype, batch, num_heads, num_kv_heads,
                          head_size, block_size, num_blocks, max_blocks, splits, chunk_pages, output_stage,
                          inv_sqrt_len, softmax_scale, status, o);
}

// The pre-rotated entry of the reference's fused decoder (launch_fused_decode_opt,
// include/turboquant_fused_decode_opt.hpp:187-189: `queryRot` is the FP32 rotated image of
// the query) over a cache in this library's native layout. code_grid 0: a nibble is the
// integer c (dequantised value c * scale), the TurboQuant cache; code_grid 1: the uniform
// mid-rise grid of the KV4/FP8 cache, a nibble c stands for (c + 0.5) * scale
// (fused_decode/common/turboquant_mode.h:100-124 with b = c + 8), which is how a cache brought
// over with tq_nz_kv4_import decodes. query_rot is [batch][num_heads][head_size] FP32; nothing
// is rotated or rounded on the way in. Output stages as in the fused decoder's raw-query entry
// (fused_decode/common/turboquant_layout.h:141-150): 0 leaves the context in the rotated basis,
// 1 applies Pi = diag(pi_signs) H diag(pi_signs) / sqrt(head_size) once more (Pi is an
// involution), 2 also divides by 1 + exp(-gate). pi_signs is read by stages 1 and 2 only, gate
// by stage 2 only.
extern "C" int tq_decode_splitk_prerotated(void* stream, const float* query_rot, const int8_t* key_cache,
                                           const int8_t* value_cache, const float* scale_cache,
                                           const int32_t* block_tables, const int32_t* context_lens,
                                           const float* pi_signs, const void* gate, float* workspace,
                                           void* output, uint32_t out_dtype, uint32_t gate_dtype,
                                           uint32_t batch, uint32_t num_heads, uint32_t num_kv_heads,
                                           uint32_t head_size, uint32_t block_size, uint32_t num_blocks,
                                           uint32_t max_blocks, uint32_t splits, uint32_t max_context_hint,
                                           uint32_t code_grid, uint32_t output_stage, float softmax_scale,
                                           uint32_t* status)
{
    if (!num_kv_heads || !block_size || splits > TQ_MAX_SPLITS || code_grid > 1u || (batch != 0 && !query_rot) ||
        output_stage > TQ_OUT_GATED || gate_dtype > TQ_DTYPE_F32 ||
        (output_stage != TQ_OUT_ROTATED && !pi_signs) || (head_size != 128 && head_size != 256))
        return TQ_ERR_INVALID_ARGUMENT;
    uint32_t chunk_pages = 0;
    splits = resolve_splits(splits, batch, num_kv_heads, block_size, max_blocks, max_context_hint,
                            &chunk_pages);
    const float inv_sqrt_len = head_size == 128 ? 0.08838834764831845f : 0.0625f;
    DecodeOptions o;
    o.gate_dtype = gate_dtype;
    o.query_rot_f32 = query_rot;
    o.midrise = code_grid;
    o.rotation = 2u;
    return decode_planned(stream, nullptr, key_cache, value_cache, scale_cache, block_tables, context_lens,
                          pi_signs, gate, workspace, output, out_dtype, batch, num_heads, num_kv_heads,
                          head_size, block_size, num_blocks, max_blocks, splits, chunk_pages,
                          output_stage, inv_sqrt_len, softmax_scale, status, o);
}

// The same decode over native planes whose codes index a 16-level table instead of a uniform
// grid: the read side of the fused decoder's Lloyd-Max toggle (DecodeUnpack::kLloydMaxLut,
// kernels/ops/turboquant/fused_decode/common/turboquant_mode.h:181-206,:252-263), whose cache
// keeps the KV4/FP8 storage (bin b as the signed nibble b - 8) and reconstructs
// levels16[b] * scale with gain 1. The pools are imported once with tq_nz_kv4_import(gain = 1);
// the export runs on the table-lookup kernel of the Lloyd-Max variant (a non-uniform codebook
// has no integer grid for the s8 key path), the merge and the output stages are those of
// tq_decode_splitk_prerotated. splits 1..16, 0 = the library's choice capped at 16; at most 8
// query heads per KV head.
extern "C" int tq_decode_levels_export(void* stream, const float* query_rot, const float* levels16,
                                       const int8_t* key_cache, const int8_t* value_cache,
                                       const float* scale_cache, const int32_t* block_tables,
                                       const int32_t* context_lens, float* workspace, uint32_t batch,
                                       uint32_t num_heads, uint32_t num_kv_heads, uint32_t head_size,
                                       uint32_t block_size, uint32_t num_blocks, uint32_t max_blocks,
                                       uint32_t splits, float softmax_scale, uint32_t* status);

extern "C" int tq_decode_splitk_levels(void* stream, const float* query_rot, const float* levels16,
                                       const int8_t* key_cache, const int8_t* value_cache,
                                       const float* scale_cache, const int32_t* block_tables,
                                       const int32_t* context_lens, const float* pi_signs, const void* gate,
                                       float* workspace, void* output, uint32_t out_dtype, uint32_t gate_dtype,
                                       uint32_t batch, uint32_t num_heads, uint32_t num_kv_heads,
                                       uint32_t head_size, uint32_t block_size, uint32_t num_blocks,
                                       uint32_t max_blocks, uint32_t splits, uint32_t max_context_hint,
                                       uint32_t output_stage, float softmax_scale, uint32_t* status)
{
    if (!num_kv_heads || !num_heads || num_heads % num_kv_heads != 0 || !block_size || splits > 16u ||
        output_stage > TQ_OUT_GATED || gate_dtype > TQ_DTYPE_F32 || out_dtype > TQ_DTYPE_F32 ||
        (output_stage != TQ_OUT_ROTATED && !pi_signs) || (output_stage == TQ_OUT_GATED && !gate) ||
        (head_size != 128 && head_size != 256) || (batch != 0 && (!output || !workspace)))
        return TQ_ERR_INVALID_ARGUMENT;
    if (splits == 0u) {
        splits = resolve_splits(0, batch, num_kv_heads, block_size, max_blocks, max_context_hint);
        if (splits > 16u) splits = 16u;
    }
    const int st = tq_decode_levels_export(stream, query_rot, levels16, key_cache, value_cache, scale_cache,
                                           block_tables, context_lens, workspace, batch, num_heads, num_kv_heads,
                                           head_size, block_size, num_blocks, max_blocks, splits, softmax_scale,
                                           status);
    if (st != TQ_OK || batch == 0) return st;
    const uint32_t rows = num_heads / num_kv_heads;
    const float inv_sqrt_len = head_size == 128 ? 0.08838834764831845f : 0.0625f;
    return splitk_combine(stream, workspace, pi_signs, gate, gate_dtype, output, out_dtype, batch * num_kv_heads,
                          rows, rows, head_size, splits, output_stage, inv_sqrt_len, 1, num_kv_heads, 2u);
}

// tq_decode_splitk as ONE launch: a persistent grid (one resident wave of CTAs) over the
// batch's 48-token tiles, flattened sequence by sequence and head by head and cut into chunks
// by a schedule every CTA can evaluate (85 % of an equal share dealt statically, the rest taken
// in eighths and sixteenths of a share from an atomic ticket); a CTA walks the (sequence, KV
// head) segments of its chunks, publishes one record per segment, counts its arrival at the
// head, and the CTA that arrives last merges the head's records and writes the output -- no
// second kernel, nobody waits for anybody. `splits` is the number of record slots per head the
// workspace holds (2..TQ_MAX_SPLITS, 0 = TQ_MAX_SPLITS); size it with
// tq_decode_workspace_floats. Measured on B200 the segment boundaries (about 12 us each:
// rotation, record, fence, arrival, draw) cost more than a hardware-scheduled CTA's, so on
// the ragged benchmark batch this entry runs at about 0.85 of tq_decode_splitk's rate; it is
// the choice where one graph node or one launch matters more.
extern "C" int tq_decode_splitk_persistent(void* stream, const uint16_t* query, const int8_t* key_cache,
                                           const int8_t* value_cache, const float* scale_cache,
                                           const int32_t* block_tables, const int32_t* context_lens,
                                           const float* pi_signs, const float* gate, float* workspace,
                                           void* output, uint32_t out_dtype, uint32_t batch,
                                           uint32_t num_heads, uint32_t num_kv_heads, uint32_t head_size,
                                           uint32_t block_size, uint32_t num_blocks, uint32_t max_blocks,
                                           uint32_t splits, uint32_t output_stage, float inv_sqrt_len,
                                           float softmax_scale, uint32_t* status)
{
    if (!num_kv_heads || !block_size || splits == 1u || splits > TQ_MAX_SPLITS) return TQ_ERR_INVALID_ARGUMENT;
    DecodeOptions o;
    o.persistent = true;
    return decode_planned(stream, query, key_cache, value_cache, scale_cache, block_tables,
                          context_lens, pi_signs, gate, workspace, output, out_dtype, batch, num_heads,
                          num_kv_heads, head_size, block_size, num_blocks, max_blocks,
                          splits ? splits : TQ_MAX_SPLITS, 0u, output_stage, inv_sqrt_len, softmax_scale,
                          status, o);
}

// tq_decode_splitk with the wider arithmetic of the reference-contract entry: the query as a
// 24-bit fixed point (three limbs) and P as a hi + lo pair of halves, so the error no longer
// scales with the magnitude of the values. For callers whose values are far from unit
// variance. Classic grid and combine kernel; about half the speed of tq_decode_splitk.
extern "C" int tq_decode_splitk_precise(void* stream, const uint16_t* query, const int8_t* key_cache,
                                        const int8_t* value_cache, const float* scale_cache,
                                        const int32_t* block_tables, const int32_t* context_lens,
                                        const float* pi_signs, const float* gate, float* workspace,
                                        void* output, uint32_t out_dtype, uint32_t batch,
                                        uint32_t num_heads, uint32_t num_kv_heads, uint32_t head_size,
                                        uint32_t block_size, uint32_t num_blocks, uint32_t max_blocks,
                                        uint32_t splits, uint32_t max_context_hint,
                                        uint32_t output_stage, float inv_sqrt_len, float softmax_scale,
                                        uint32_t* status)
{
    if (!num_kv_heads || !block_size || splits > TQ_MAX_SPLITS) return TQ_ERR_INVALID_ARGUMENT;
    uint32_t chunk_pages = 0;
    splits = resolve_splits(splits, batch, num_kv_heads, block_size, max_blocks, max_context_hint,
                            &chunk_pages);
    DecodeOptions o;
    o.precise = true;
    return decode_planned(stream, query, key_cache, value_cache, scale_cache, block_tables,
                          context_lens, pi_signs, gate, workspace, output, out_dtype, batch, num_heads,
                          num_kv_heads, head_size, block_size, num_blocks, max_blocks, splits,
                          chunk_pages, output_stage, inv_sqrt_len, softmax_scale, status, o);
}

// Decode over the fused decoder's KV4 cache where it lies: nz_key / nz_value are its NZ-tiled
// packed pools and nz_scales its per-slot scale records (see tq_nz_kv4_import for the format),
// read in place -- no second pool, no re-tiling pass. The strips of a 64-row tile are staged
// with their rows permuted so that both contractions read them without bank conflicts; keys
// feed the integer MMA as they are (a fixed permutation of the contraction index, applied to
// the query fragments once), and the token pairs the value contraction needs are put together
// from the words of two token rows with one byte permute per four channels. The stored scale
// is divided by `gain` on the way in (IEEE division, as the importer does), so records and
// outputs equal those of tq_nz_kv4_import followed by tq_decode_splitk_prerotated bit for
// bit. Head size 256, pages of 64 or 128 slots. num_blocks 0 = unknown (page numbers are then
// not range-checked). precise != 0 selects the wider arithmetic of tq_decode_splitk_precise.
// Other arguments as for tq_decode_splitk_prerotated.
extern "C" int tq_decode_splitk_nz(void* stream, const float* query_rot, const uint8_t* nz_key,
                                   const uint8_t* nz_value, const float* nz_scales,
                                   const int32_t* block_tables, const int32_t* context_lens,
                                   const float* pi_signs, const void* gate, float* workspace,
                                   void* output, uint32_t out_dtype, uint32_t gate_dtype, uint32_t batch,
                                   uint32_t num_heads, uint32_t num_kv_heads, uint32_t block_size,
                                   uint32_t num_blocks, uint32_t max_blocks, uint32_t splits,
                                   uint32_t max_context_hint, uint32_t code_grid, uint32_t output_stage,
                                   float gain, float inv_sqrt_len, float softmax_scale, uint32_t precise,
                                   uint32_t* status)
{
    if (!num_kv_heads || (block_size != 64 && block_size != 128) || splits > TQ_MAX_SPLITS || code_grid > 1u ||
        (batch != 0 && !query_rot) || output_stage > TQ_OUT_GATED || gate_dtype > TQ_DTYPE_F32 ||
        (output_stage != TQ_OUT_ROTATED && !pi_signs) || !(gain > 0.0f))
        return TQ_ERR_INVALID_ARGUMENT;
    uint32_t chunk_pages = 0;
    splits = resolve_splits(splits, batch, num_kv_heads, block_size, max_blocks, max_context_hint,
                            &chunk_pages);
    DecodeOptions o;
    o.gate_dtype = gate_dtype;
    o.query_rot_f32 = query_rot;
    o.midrise = code_grid;
    o.rotation = 2u;
    o.nz_slot_floats = (2u * num_kv_heads + 7u) / 8u * 8u;
    o.nz_gain = gain;
    o.precise = precise != 0u;
    return decode_planned(stream, nullptr, reinterpret_cast<const int8_t*>(nz_key),
                          reinterpret_cast<const int8_t*>(nz_value), nz_scales, block_tables, context_lens,
                          pi_signs, gate, workspace, output, out_dtype, batch, num_heads, num_kv_heads, 256,
                          block_size, num_blocks ? num_blocks : 0x7FFFFFFFu, max_blocks, splits, chunk_pages,
                          output_stage, inv_sqrt_len, softmax_scale, status, o);
}

// ------------------------------------------------- decode without a caller workspace
// Split-K partials normally live in a workspace the caller allocates. Some hosts have
// no way to provide one: a serving process that handed every free byte of HBM to its
// KV-cache pool at start-up (a later cudaMalloc simply fails), or an attention backend
// embedded in a runtime whose allocator it may not call from the launch path. For
// them the partials go into this fixed array, which every GPU that loads the library
// carries until the process exits: 8 MiB, enough for e.g. 64 sequences x 8 KV heads
// x 4 record slots x 4 query rows per KV head at head size 128 (a launch that leaves the
// split plan to the library asks for up to 32 slots per head: 8 such sequences).
static __device__ __align__(256) float g_static_workspace[TQ_STATIC_WORKSPACE_FLOATS];

// In host code `g_static_workspace` is only a handle for the device symbol, not a
// device address: the address is looked up once per device, with that device current.
// The per-device slot is an atomic: threads that race on a device's first call each make
// the query and store the same address. The cached address belongs to the device's primary
// context; a host that destroys that context (cudaDeviceReset) must not call this again
// from the same process image, the slot is not re-validated.
static float* static_workspace_address(int* status)
{
    static std::atomic<float*> address[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        (void)cudaGetLastError();
        *status = TQ_ERR_NO_DEVICE;
        return nullptr;
    }
    float* cached = address[dev].load(std::memory_order_acquire);
    if (cached == nullptr) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_static_workspace) != cudaSuccess || ptr == nullptr) {
            (void)cudaGetLastError();   // leave no sticky-looking error behind for the caller
            *status = TQ_ERR_LAUNCH;
            return nullptr;
        }
        cached = static_cast<float*>(ptr);
        address[dev].store(cached, std::memory_order_release);
    }
    *status = TQ_OK;
    return cached;
}

extern "C" int tq_decode_splitk_static(void* stream, const uint16_t* query, const int8_t* key_cache,
                                       const int8_t* value_cache, const float* scale_cache,
                                       const int32_t* block_tables, const int32_t* context_lens,
                                       const float* pi_signs, const float* gate, void* output,
                                       uint32_t out_dtype, uint32_t batch, uint32_t num_heads,
                                       uint32_t num_kv_heads, uint32_t head_size,
                                       uint32_t block_size, uint32_t num_blocks,
                                       uint32_t max_blocks, uint32_t splits,
                                       uint32_t max_context_hint, uint32_t output_stage,
                                       float inv_sqrt_len, float softmax_scale, uint32_t* status)
{
    // geometry first, so that nonsense is refused as nonsense and not as "too large"
    if (!num_kv_heads || !num_heads || num_heads % num_kv_heads != 0 || num_heads / num_kv_heads > 16 ||
        !block_size || block_size % kStrip != 0 || splits > TQ_MAX_SPLITS ||
        (head_size != 128 && head_size != 256))
        return TQ_ERR_INVALID_ARGUMENT;
    // Resolve the split count first: it decides how much of the array the launch needs.
    uint32_t chunk_pages = 0;
    splits = resolve_splits(splits, batch, num_kv_heads, block_size, max_blocks, max_context_hint,
                            &chunk_pages);
    const size_t need = tq_decode_workspace_floats(batch, num_heads, num_kv_heads, head_size, splits);
    if (need > static_cast<size_t>(TQ_STATIC_WORKSPACE_FLOATS)) return TQ_ERR_WORKSPACE_TOO_SMALL;
    int st = TQ_OK;
    float* workspace = static_workspace_address(&st);
    if (workspace == nullptr) return st;
    // Every record that is merged is written by this launch first, and the arrival counters
    // behind the records are valid only under the launch's own tag, so nothing in the array
    // has to start at zero.
    return decode_planned(stream, query, key_cache, value_cache, scale_cache, block_tables,
                          context_lens, pi_signs, gate, workspace, output, out_dtype, batch, num_heads,
                          num_kv_heads, head_size, block_size, num_blocks, max_blocks, splits,
                          chunk_pages, output_stage, inv_sqrt_len, softmax_scale, status);
}

// kernels/ops/turboquant/turboquant_paged_decode_attention.cpp:1727-1766. The
// reference decoder is compiled for d = 256 and 16 packed query rows per head;
// pi_table is its 16 resident bf16 blocks, of which only the sign diagonal is
// data (the 1/sqrt(d) magnitude of its entries is the constant 1/16).
extern "C" void launch_turboquant_paged_decode_splitk_aic(
    void* stream, uint16_t* q, uint16_t* pi_table, int8_t* key, int8_t* value, float* scales,
    uint32_t* table, uint16_t* qrot, float* workspace, uint32_t requests, uint32_t heads,
    uint32_t block_size, uint32_t cache_pages, uint32_t seq_pages, uint32_t splits,
    uint32_t page_begin, uint32_t page_count, uint32_t seq_len)
{
    if (block_size > 128u) throw std::invalid_argument("invalid AIC temporal split geometry");
    const int st = tq_decode_splitk_partials(stream, q, pi_table, TQ_SIGNS_TABLES_BF16, key, value,
                                             scales, table, qrot, workspace, requests, heads, 16,
                                             256, block_size, cache_pages, seq_pages, splits,
                                             page_begin, page_count, seq_len, 0.0625f, 1.0f,
                                             nullptr);
    if (st == TQ_ERR_INVALID_ARGUMENT)
        throw std::invalid_argument("invalid AIC temporal split geometry");
    if (st != TQ_OK) throw std::runtime_error("paged_decode_splitk_aic: launch failed");
}
