// reshape_and_cache, aligned writer for head size 256 on the 5th-generation tensor core
// (tcgen05) with the accumulators in tensor memory.
//
// What is computed is what the warp-MMA writer computes (tq_ingest.cu; reference:
// tests/common/turboquant_oracle.hpp:357-449,
// kernels/ops/turboquant/turboquant_reshape_and_cache_a8.cpp:714-744,:1083-1226):
//   y = M x,  M = (H_8 (x) I32) diag(s) (I_8 (x) H32)      256 x 256, entries +-1
//   absmax = max(1, max|y|), scale = 2^(e-2) * inv_sqrt_len, q = rint_even(min(y 2^(2-e), 7))
//
// How. H_8 = H_2 (x) H_4, so with x = (x_lo, x_hi) split at channel 128
//   a = M_0 x_lo,  b = M_1 x_hi,  y_lo = a + b,  y_hi = a - b,
// where M_h = (H_4 (x) I32) diag(s[128 h ..]) (I_4 (x) H32) is the 128 x 128 matrix of the
// head-size-128 writer over one half of the sign diagonal: two 128 x 128 x 128 products per
// 128-token tile into two accumulators (half the multiply-adds of the dense 256 x 256 form), and
// one add and one subtract per pair of outputs in the epilogue. Otherwise the plan of
// tq_ingest_umma.cu: M_0 and M_1 built once per persistent CTA in shared memory (K-major, 128-byte
// swizzle), tiles fetched by TMA, key plane read out per token, value plane per channel from the
// products with the operands swapped, INT32 accumulators preset to the bit pattern of 1.5 * 2^23.
// Two accumulators of 128 columns per group leave room for two groups per SM, so a group is
// eight warps: warp w reads lane quarter w & 3 (the rows) and column half w >> 2 of both
// accumulators, and the two halves of a row exchange their absmax through shared memory.
// Every wait on a barrier is bounded by a clock budget (see tq_ingest_umma.cu).
#include <type_traits>

#include "tq_umma.cuh"

namespace tq {
namespace {

constexpr int kTileTokens = 128;
constexpr int kGroups = 2;                   // independent groups per CTA, one tile each
constexpr int kGroupThreads = 256;           // eight warps
constexpr int kThreads = kGroups * kGroupThreads;
constexpr uint32_t kAccCols = 128;           // one 128 x 128 accumulator
constexpr uint32_t kGroupCols = 2 * kAccCols;   // a, then b
constexpr uint32_t kTmemCols = kGroups * kGroupCols;

template <bool BF16>
struct Cfg {
    static constexpr int kElem = BF16 ? 2 : 1;
    static constexpr int kHalfRowBytes = 128 * kElem;        // 128 channels of one token
    static constexpr int kBlocksHalf = kHalfRowBytes / 128;  // 128-byte-wide K blocks per half row
    static constexpr int kBlockBytes = 128 * 128;            // 128 rows of one K block
    static constexpr int kHalfBytes = kBlocksHalf * kBlockBytes;   // x_lo, x_hi, M_0, M_1: each this size
    static constexpr int kTileBytes = 2 * kHalfBytes;
    static constexpr int kKSteps = kHalfRowBytes / 32;       // one MMA contracts 32 bytes of K
    // per group: 128 inverse scales, 2 x 128 absmax halves, 8 strip offsets, 2 barriers
    static constexpr int kSmallBytes = 3 * kTileTokens * 4 + 8 * 8 + 64;
    static constexpr int kUsed = 2 * kHalfBytes + kGroups * (kTileBytes + kSmallBytes) + 64;
    static constexpr int kSmem = kUsed + 1024;               // slack for aligning the tiles
};

#define TQ_W8(v, o) "=r"(v[o]), "=r"(v[o + 1]), "=r"(v[o + 2]), "=r"(v[o + 3]), "=r"(v[o + 4]), \
                    "=r"(v[o + 5]), "=r"(v[o + 6]), "=r"(v[o + 7])
#define TQ_RW8(v, o) "+r"(v[o]), "+r"(v[o + 1]), "+r"(v[o + 2]), "+r"(v[o + 3]), "+r"(v[o + 4]), \
                     "+r"(v[o + 5]), "+r"(v[o + 6]), "+r"(v[o + 7])
// 32 lanes x 16 columns: lane i of the warp receives columns col .. col + 15 of its row.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : TQ_W8(v, 0), TQ_W8(v, 8) : "r"(taddr) : "memory");
}
// 32 lanes x 32 columns, the low 16 bits of each: register j holds columns 2j and 2j + 1.
__device__ __forceinline__ void tmem_ld16_low16(uint32_t taddr, uint32_t (&v)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.pack::16b.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : TQ_W8(v, 0), TQ_W8(v, 8) : "r"(taddr) : "memory");
}
// The wait for the loads into both arrays; naming them as in-out operands keeps every use behind it.
__device__ __forceinline__ void tmem_arrived2(uint32_t (&a)[16], uint32_t (&b)[16])
{
    asm volatile("tcgen05.wait::ld.sync.aligned;\n"
                 : TQ_RW8(a, 0), TQ_RW8(a, 8), TQ_RW8(b, 0), TQ_RW8(b, 8) :: "memory");
}
#undef TQ_W8
#undef TQ_RW8
// The same 32-bit value into 16 columns of every lane of the warp's quarter.
__device__ __forceinline__ void tmem_fill16(uint32_t taddr, uint32_t x)
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1};\n"
        ::"r"(taddr), "r"(x) : "memory");
}

struct TileId {
    uint32_t tok_tile, head;
};
__device__ __forceinline__ TileId tile_of(const IngestParams& p, uint32_t item)
{
    TileId id;
    id.tok_tile = fast_div(2u * item, p.div_mul, p.div_shift);   // item / H with the 2H divider
    id.head = item - id.tok_tile * p.H;
    return id;
}

// All 256 threads of one group (named barrier 1 + group).
__device__ __forceinline__ void group_sync(int group)
{
    asm volatile("bar.sync %0, %1;\n" ::"r"(group + 1), "r"(kGroupThreads) : "memory");
}

// The same barrier carrying a vote: true for every thread of the group if any of them says so.
// The decision to leave the item loop must be one decision per group, or the next barrier hangs.
__device__ __forceinline__ bool group_sync_any(int group, bool mine)
{
    uint32_t any;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %3, 0;\n\t"
        "bar.red.or.pred q, %1, %2, p;\n\tselp.u32 %0, 1, 0, q;\n\t}\n"
        : "=r"(any) : "r"(group + 1), "r"(kGroupThreads), "r"(mine ? 1u : 0u) : "memory");
    return any != 0u;
}

template <bool BF16>
__global__ void __launch_bounds__(kThreads, 1)
tq_ingest_umma256_kernel(const IngestParams p, const __grid_constant__ CUtensorMap key_map,
                         const __grid_constant__ CUtensorMap value_map)
{
    using C = Cfg<BF16>;
    extern __shared__ uint8_t smem_raw[];
    // tiles on a 1024-byte boundary: the swizzle is a function of address bits 4..9
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~uintptr_t(1023));
    const int group = threadIdx.x / kGroupThreads, tid = threadIdx.x % kGroupThreads;
    const int warp = tid >> 5, lane = tid & 31;
    const int quarter = warp & 3, half = warp >> 2;   // tensor-memory lane quarter, column half
    const int row = quarter * 32 + lane;              // token (plain products) or channel (swapped)
    uint8_t* m_tiles = base;                          // M_0, then M_1
    uint8_t* x_tile = base + 2 * C::kHalfBytes + group * C::kTileBytes;   // x_lo blocks, then x_hi blocks
    uint8_t* small = base + 2 * C::kHalfBytes + kGroups * C::kTileBytes + group * C::kSmallBytes;
    float* inv_s = reinterpret_cast<float*>(small);   // per token: 2^(2-e)
    float* amax_s = inv_s + kTileTokens;              // [2][128]: each column half's absmax of the row
    unsigned long long* strip_off = reinterpret_cast<unsigned long long*>(small + 3 * kTileTokens * 4);  // [8]
    uint64_t* mbar = reinterpret_cast<uint64_t*>(strip_off + 8);   // [0]: products done, [1]: tile landed
    uint32_t* shared_words = reinterpret_cast<uint32_t*>(base + 2 * C::kHalfBytes + kGroups * C::kTileBytes +
                                                         kGroups * C::kSmallBytes);
    uint32_t* tmem_slot = shared_words;
    volatile uint32_t* abort_flag = shared_words + 1;

    const uint32_t items = ((p.num_strips + 7u) / 8u) * p.H;
    const uint32_t num_tokens = p.num_strips * kStrip;

    // ---- one-time set-up: barriers, tensor memory, the two rotation matrices
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(smem_addr(mbar)));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(smem_addr(mbar + 1)));
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        if (group == 0) *abort_flag = 0u;
    }
    if (threadIdx.x < 32) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_addr(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    {
        // Row r of M_h: output channel c1*32 + c0 against input channel g*32 + i (both inside the
        // half) is H4[c1][g] * s[128 h + g*32 + c0] * H32[c0][i]; true = -1. Thread t writes half a
        // row: row t & 127 of matrix t >> 8, chunk half (t >> 7) & 1.
        const unsigned r = threadIdx.x & 127u, hsel = threadIdx.x >> 8, part = (threadIdx.x >> 7) & 1u;
        const unsigned c1 = r >> 5, c0 = r & 31u;
        bool gneg[4];
#pragma unroll
        for (int g = 0; g < 4; ++g)
            gneg[g] = hneg(c1, g) != sign_is_negative(p.signs, p.sign_source, hsel * 128 + g * kGroup + c0);
        constexpr int kPerChunk = 16 / C::kElem;   // elements in a 16-byte chunk
        constexpr int kChunks = C::kHalfRowBytes / 16;
        uint8_t* m_tile = m_tiles + hsel * C::kHalfBytes;
#pragma unroll 1
        for (int q = part * (kChunks / 2); q < (part + 1) * (kChunks / 2); ++q) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t word = 0;
#pragma unroll
                for (int b = 0; b < 4 / C::kElem; ++b) {
                    const unsigned in = q * kPerChunk + j * (4 / C::kElem) + b;
                    const bool neg = gneg[in >> 5] != hneg(c0, in & 31u);
                    if constexpr (BF16) word |= (neg ? 0xBF80u : 0x3F80u) << (16 * b);
                    else word |= (neg ? 0xFFu : 0x01u) << (8 * b);
                }
                w[j] = word;
            }
            const int blk = q >> 3, cq = q & 7;
            *reinterpret_cast<uint4*>(m_tile + blk * C::kBlockBytes + r * 128 + ((cq ^ (r & 7)) << 4)) =
                make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
    fence_async_smem();
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_group = tmem_base + static_cast<uint32_t>(group) * kGroupCols;
    // this thread's 64 columns of accumulator a; b lies kAccCols further on
    const uint32_t acc = tmem_group + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(half) * 64u;
    const uint32_t mbar_s = smem_addr(mbar), tma_bar_s = smem_addr(mbar + 1);
    const uint32_t x_tile_s = smem_addr(x_tile), m_tiles_s = smem_addr(m_tiles);
    const uint64_t desc_x = umma_desc(x_tile_s), desc_m = umma_desc(m_tiles_s);

    // Thread 0 of the group keeps the books of what it has in flight towards this CTA's shared and
    // tensor memory; nothing new is issued once a wait has run out.
    uint32_t parity = 0, tma_parity = 0, mma_pending_parity = 0;
    bool healthy = true, mma_pending = false, tma_pending = false;
    auto load_tile = [&](uint32_t item, uint32_t plane) {
        if (tid != 0 || !healthy) return;
        const TileId id = tile_of(p, item);
        const CUtensorMap* map = plane == 0 ? &key_map : &value_map;
        mbar_expect_tx(tma_bar_s, C::kTileBytes);
#pragma unroll
        for (int blk = 0; blk < 2 * C::kBlocksHalf; ++blk)
            tma_load_2d(x_tile_s + blk * C::kBlockBytes, map,
                        static_cast<int>(id.head * 256u + blk * (128 / C::kElem)),
                        static_cast<int>(id.tok_tile * kTileTokens), tma_bar_s);
        tma_pending = true;
    };

    auto bounded_wait = [&](uint32_t bar, uint32_t par, long long budget, bool watch_abort) {
        return bounded_mbar_wait(bar, par, budget, watch_abort ? abort_flag : nullptr);
    };
    // The two products a and b into the group's accumulators, then the bounded wait for them.
    // transposed = false: D[token][channel] = X_h M_h^T; true: D'[channel][token] = M_h X_h^T.
    auto product = [&](bool transposed, bool fresh_tile) {
        if constexpr (!BF16) tmem_wait_st();   // the refill of the columns (see refill) is in place
        fence_before_sync();
        group_sync(group);
        if (tid == 0 && healthy) {
            bool landed = true;
            if (fresh_tile) {
                landed = bounded_wait(tma_bar_s, tma_parity, p.wait_budget, false);
                if (landed) {
                    tma_pending = false;
                    tma_parity ^= 1u;
                }
            }
            if (landed) {
                fence_after_sync();
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint64_t dx0 = desc_x + ((h * C::kHalfBytes) >> 4), dm0 = desc_m + ((h * C::kHalfBytes) >> 4);
#pragma unroll
                    for (int k = 0; k < C::kKSteps; ++k) {
                        const uint32_t off16 = ((k >> 2) * C::kBlockBytes + (k & 3) * 32) >> 4;
                        const uint64_t dx = dx0 + off16, dm = dm0 + off16;
                        umma<BF16>(tmem_group + h * kAccCols, transposed ? dm : dx, transposed ? dx : dm,
                                   (!BF16 || k > 0) ? 1u : 0u);
                    }
                }
                umma_commit(mbar_s);
                mma_pending = true;
                mma_pending_parity = parity;
            } else {
                healthy = false;
                *abort_flag = 1u;
            }
        }
        const bool done = healthy && bounded_wait(mbar_s, parity, p.wait_budget, true);
        if (done && tid == 0) mma_pending = false;
        if (!done || *abort_flag != 0u) {
            healthy = false;
            *abort_flag = 1u;
            report(p.status, TQ_STATUS_WAIT_EXPIRED);
        }
        parity ^= 1u;
        fence_after_sync();
    };

    // INT32 accumulators start at the bit pattern of 1.5 * 2^23: set once here and again, chunk by
    // chunk, by whoever reads a product for the last time.
    auto refill = [&](uint32_t col) {
        if constexpr (!BF16) {
            tmem_fill16(acc + col, kBiasBits);
            tmem_fill16(acc + kAccCols + col, kBiasBits);
        }
    };
#pragma unroll
    for (int c = 0; c < 4; ++c) refill(c * 16);

    const uint32_t item_step = gridDim.x * kGroups;
    uint32_t item = blockIdx.x * kGroups + group;
    if (item < items) load_tile(item, 0);
    int32_t slot = -1;
    bool strip_ok = false, tok_live = false;
    uint32_t head = 0;
    size_t block_off = 0, scale_at = 0;
    const size_t plane_scales = static_cast<size_t>(p.P) * p.H * p.S;
    const float2 minus1 = make_float2(-1.0f, -1.0f), minus2bias = make_float2(-2.0f * kBias, -2.0f * kBias);

    // y_lo and y_hi of two adjacent columns out of the raw accumulator words. int8: a' = B + a and
    // b' = B + b with B = 1.5 * 2^23; b' - 2B, a' + (b' - 2B) and a' - b' are all exact in FP32.
    auto combine = [&](uint32_t a0, uint32_t a1, uint32_t b0, uint32_t b1, float2& lo, float2& hi) {
        const float2 a = make_float2(__uint_as_float(a0), __uint_as_float(a1));
        const float2 b = make_float2(__uint_as_float(b0), __uint_as_float(b1));
        if constexpr (BF16) lo = __fadd2_rn(a, b);
        else lo = __fadd2_rn(a, __fadd2_rn(b, minus2bias));
        hi = __ffma2_rn(b, minus1, a);
    };

    auto do_plane = [&](auto plane_tag) -> bool {
        constexpr uint32_t kPlane = decltype(plane_tag)::value;
        if constexpr (kPlane == 0) {
            const TileId id = tile_of(p, item);
            const uint32_t tok = id.tok_tile * kTileTokens + row;
            head = id.head;
            tok_live = tok < num_tokens;
            slot = -1;   // a volatile load: it must not sink below the product's wait
            if (tok_live) asm volatile("ld.global.nc.s32 %0, [%1];\n" : "=r"(slot) : "l"(p.slots + tok));
        }

        product(false, true);
        // the tile is consumed: the item's value tile takes its place
        if constexpr (kPlane == 0) load_tile(item, 1);

        if constexpr (kPlane == 0) {
            const int32_t slot0 = __shfl_sync(0xffffffffu, slot, lane & 16);
            const bool run_ok = slot == slot0 + (lane & 15);
            const uint32_t votes = __ballot_sync(0xffffffffu, run_ok);
            const bool strip_live = __shfl_sync(0xffffffffu, tok_live ? 1 : 0, lane & 16) != 0;
            const uint32_t slot_page = fast_div(static_cast<uint32_t>(slot0), p.page_mul, p.page_shift);
            strip_ok = strip_live && ((votes >> (lane & 16)) & 0xFFFFu) == 0xFFFFu && slot0 >= 0 &&
                       (slot0 % kStrip) == 0 && slot_page < p.P;
            if (strip_live && !strip_ok && (lane & 15) == 0 && half == 0) report(p.status, TQ_STATUS_BAD_SLOT);
            const uint32_t page = strip_ok ? slot_page : 0u;
            const uint32_t tok_in_page = strip_ok ? static_cast<uint32_t>(slot0) - slot_page * p.S : 0u;
            // byte offset of the strip's (page, head) block in either code plane
            block_off = (static_cast<size_t>(page) * p.H + head) * (static_cast<size_t>(p.S) * 128u) +
                        static_cast<size_t>(tok_in_page / kStrip) * 2048u;
            scale_at = (static_cast<size_t>(page) * p.H + head) * p.S + tok_in_page + (lane & 15);
        }

        // ---- pass 1 over this thread's 64 columns of D[token][.]: absmax of y_lo and y_hi there
        uint32_t a0[16], b0[16], a1[16], b1[16];
        float amax;
        if constexpr (BF16) {
            float m0 = 0.0f, m1 = 0.0f;
            auto fold = [&](const uint32_t (&va)[16], const uint32_t (&vb)[16]) {
#pragma unroll
                for (int j = 0; j < 16; j += 2) {
                    float2 lo, hi;
                    combine(va[j], va[j + 1], vb[j], vb[j + 1], lo, hi);
                    m0 = max3f(m0, fabsf(lo.x), fabsf(lo.y));
                    m1 = max3f(m1, fabsf(hi.x), fabsf(hi.y));
                }
            };
            tmem_ld16(acc + 0, a0);
            tmem_ld16(acc + kAccCols + 0, b0);
            tmem_arrived2(a0, b0);
            tmem_ld16(acc + 16, a1);
            tmem_ld16(acc + kAccCols + 16, b1);
            fold(a0, b0);
            tmem_arrived2(a1, b1);
            tmem_ld16(acc + 32, a0);
            tmem_ld16(acc + kAccCols + 32, b0);
            fold(a1, b1);
            tmem_arrived2(a0, b0);
            tmem_ld16(acc + 48, a1);
            tmem_ld16(acc + kAccCols + 48, b1);
            fold(a0, b0);
            tmem_arrived2(a1, b1);
            fold(a1, b1);
            amax = fmaxf(m0, m1);
        } else {
            // the sums a and b as signed 16-bit pairs, 32 columns per read. a + b can reach +32768 only
            // as exactly that value, which wraps to -32768 and still reads as 32768 below.
            uint32_t top2 = 0x80008000u, bottom2 = 0x7FFF7FFFu;
            auto fold = [&](const uint32_t (&va)[16], const uint32_t (&vb)[16]) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const uint32_t s = __vadd2(va[j], vb[j]), d = __vsub2(va[j], vb[j]);
                    top2 = __vimax3_s16x2(top2, s, d);
                    bottom2 = __vimin3_s16x2(bottom2, s, d);
                }
            };
            tmem_ld16_low16(acc + 0, a0);
            tmem_ld16_low16(acc + kAccCols + 0, b0);
            tmem_arrived2(a0, b0);
            tmem_ld16_low16(acc + 32, a1);
            tmem_ld16_low16(acc + kAccCols + 32, b1);
            fold(a0, b0);
            tmem_arrived2(a1, b1);
            fold(a1, b1);
            const int top = max(static_cast<int>(static_cast<int16_t>(top2 & 0xFFFFu)),
                                static_cast<int>(static_cast<int16_t>(top2 >> 16)));
            const int bottom = min(static_cast<int>(static_cast<int16_t>(bottom2 & 0xFFFFu)),
                                   static_cast<int>(static_cast<int16_t>(bottom2 >> 16)));
            amax = static_cast<float>(max(top, -bottom));
        }
        // the row's other 64 columns belong to the warp four further on
        amax_s[half * kTileTokens + row] = amax;
        if constexpr (kPlane == 0) {   // first chunk of pass 2, requested under the exchange
            tmem_ld16(acc + 0, a0);
            tmem_ld16(acc + kAccCols + 0, b0);
        }
        group_sync(group);
        amax = fmaxf(fmaxf(amax, amax_s[(half ^ 1) * kTileTokens + row]), 1.0f);   // the writer floors absmax at 1
        const int pow_bits = (__float_as_int(amax) & 0x7F800000) - (2 << 23);
        const float inv = __int_as_float((254 << 23) - pow_bits);
        if (half == 0 && strip_ok && healthy)
            p.scale_cache[scale_at + (kPlane ? plane_scales : 0)] = __int_as_float(pow_bits) * p.inv_sqrt_len;
        const float2 magic2 = make_float2(kMagic, kMagic);

        if constexpr (kPlane == 0) {
            // ---- key page: the token's row of 128 bytes; this thread's columns are channels
            // 64 half .. of y_lo (bytes 32 half ..) and 128 + 64 half .. of y_hi (bytes 64 + 32 half ..)
            uint2* dst = reinterpret_cast<uint2*>(p.key_cache + block_off + static_cast<size_t>(lane & 15) * 128u +
                                                  static_cast<size_t>(half) * 32u);
            const float2 inv2 = make_float2(inv, inv);
            const bool store = strip_ok && healthy;
            auto emit = [&](const uint32_t (&va)[16], const uint32_t (&vb)[16], int c) {
                float rl[16], rh[16];
#pragma unroll
                for (int j = 0; j < 16; j += 2) {
                    float2 lo, hi;
                    combine(va[j], va[j + 1], vb[j], vb[j + 1], lo, hi);
                    const float2 l = __ffma2_rn(lo, inv2, magic2), h = __ffma2_rn(hi, inv2, magic2);
                    rl[j] = l.x;
                    rl[j + 1] = l.y;
                    rh[j] = h.x;
                    rh[j + 1] = h.y;
                }
                const float (&rl0)[8] = *reinterpret_cast<const float (*)[8]>(rl);
                const float (&rl1)[8] = *reinterpret_cast<const float (*)[8]>(rl + 8);
                const float (&rh0)[8] = *reinterpret_cast<const float (*)[8]>(rh);
                const float (&rh1)[8] = *reinterpret_cast<const float (*)[8]>(rh + 8);
                const uint2 wl = make_uint2(pack8(rl0), pack8(rl1)), wh = make_uint2(pack8(rh0), pack8(rh1));
                if (store) {
                    __stcs(dst + c, wl);
                    __stcs(dst + 8 + c, wh);   // 64 bytes further on
                }
            };
            tmem_arrived2(a0, b0);
            tmem_ld16(acc + 16, a1);
            tmem_ld16(acc + kAccCols + 16, b1);
            refill(0);
            emit(a0, b0, 0);
            tmem_arrived2(a1, b1);
            tmem_ld16(acc + 32, a0);
            tmem_ld16(acc + kAccCols + 32, b0);
            refill(16);
            emit(a1, b1, 1);
            tmem_arrived2(a0, b0);
            tmem_ld16(acc + 48, a1);
            tmem_ld16(acc + kAccCols + 48, b1);
            refill(32);
            emit(a0, b0, 2);
            tmem_arrived2(a1, b1);
            refill(48);
            emit(a1, b1, 3);
        } else {
            // ---- value page: publish the per-token constants, swap the operands, then work per
            // channel: this thread is channel `row` of y_lo and 128 + row of y_hi, tokens 64 half ..
#pragma unroll
            for (int c = 0; c < 4; ++c) refill(c * 16);   // pass 1 was the only pass over these products
            if (half == 0) {
                inv_s[row] = inv;
                if ((lane & 15) == 0)
                    strip_off[row >> 4] = strip_ok ? static_cast<unsigned long long>(block_off) : ~0ull;
            }
            product(true, false);   // its barrier also publishes the constants and ends pass 1's reads
            if (item + item_step < items) load_tile(item + item_step, 0);
            const bool store = healthy;
            auto emit = [&](const uint32_t (&va)[16], const uint32_t (&vb)[16], int c) {
                const int s = half * 4 + c;   // the strip of these 16 tokens
                const unsigned long long off = strip_off[s];
                float rl[16], rh[16];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float4 iv = *reinterpret_cast<const float4*>(inv_s + s * 16 + q * 4);
                    const float2 i01 = make_float2(iv.x, iv.y), i23 = make_float2(iv.z, iv.w);
                    float2 lo, hi;
                    combine(va[q * 4], va[q * 4 + 1], vb[q * 4], vb[q * 4 + 1], lo, hi);
                    float2 l = __ffma2_rn(lo, i01, magic2), h = __ffma2_rn(hi, i01, magic2);
                    rl[q * 4] = l.x;
                    rl[q * 4 + 1] = l.y;
                    rh[q * 4] = h.x;
                    rh[q * 4 + 1] = h.y;
                    combine(va[q * 4 + 2], va[q * 4 + 3], vb[q * 4 + 2], vb[q * 4 + 3], lo, hi);
                    l = __ffma2_rn(lo, i23, magic2);
                    h = __ffma2_rn(hi, i23, magic2);
                    rl[q * 4 + 2] = l.x;
                    rl[q * 4 + 3] = l.y;
                    rh[q * 4 + 2] = h.x;
                    rh[q * 4 + 3] = h.y;
                }
                const float (&rl0)[8] = *reinterpret_cast<const float (*)[8]>(rl);
                const float (&rl1)[8] = *reinterpret_cast<const float (*)[8]>(rl + 8);
                const float (&rh0)[8] = *reinterpret_cast<const float (*)[8]>(rh);
                const float (&rh1)[8] = *reinterpret_cast<const float (*)[8]>(rh + 8);
                const uint2 wl = make_uint2(pack8(rl0), pack8(rl1)), wh = make_uint2(pack8(rh0), pack8(rh1));
                if (store && off != ~0ull) {
                    uint8_t* blk = p.value_cache + off;
                    __stcs(reinterpret_cast<uint2*>(blk + static_cast<size_t>(row) * 8u), wl);
                    __stcs(reinterpret_cast<uint2*>(blk + static_cast<size_t>(128 + row) * 8u), wh);
                }
            };
            tmem_ld16(acc + 0, a0);
            tmem_ld16(acc + kAccCols + 0, b0);
            tmem_arrived2(a0, b0);
            tmem_ld16(acc + 16, a1);
            tmem_ld16(acc + kAccCols + 16, b1);
            refill(0);
            emit(a0, b0, 0);
            tmem_arrived2(a1, b1);
            tmem_ld16(acc + 32, a0);
            tmem_ld16(acc + kAccCols + 32, b0);
            refill(16);
            emit(a1, b1, 1);
            tmem_arrived2(a0, b0);
            tmem_ld16(acc + 48, a1);
            tmem_ld16(acc + kAccCols + 48, b1);
            refill(32);
            emit(a0, b0, 2);
            tmem_arrived2(a1, b1);
            refill(48);
            emit(a1, b1, 3);
        }
        // every read of tensor memory and of the per-token constants is done before the
        // group's next products overwrite them
        fence_before_sync();
        return !group_sync_any(group, !healthy || *abort_flag != 0u);
    };
#pragma unroll 1
    for (; item < items; item += item_step) {
        if (!do_plane(std::integral_constant<uint32_t, 0>{})) break;
        if (!do_plane(std::integral_constant<uint32_t, 1>{})) break;
    }
    // After a wait ran out (here or in the other group) a tile fetch or a product chain may still
    // be on its way into this CTA's shared and tensor memory: thread 0 gives each the full budget
    // to finish before the memory goes back to the SM.
    if (tid == 0) {
        if (tma_pending) bounded_wait(tma_bar_s, tma_parity, kWaitBudget, false);
        if (mma_pending) bounded_wait(mbar_s, mma_pending_parity, kWaitBudget, false);
    }
    fence_before_sync();
    __syncthreads();
    if (threadIdx.x < 32)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
}

// The activation tensor [num_tokens][H * 256] as a 2-D map whose box is 128 rows of one
// 128-byte K block, stored with the 128-byte swizzle the MMA descriptors expect.
template <bool BF16>
bool activation_map(CUtensorMap* map, const void* base, uint32_t num_tokens, uint32_t H)
{
    const EncodeTiled fn = encode_tiled();
    if (fn == nullptr) return false;
    constexpr uint32_t elem = BF16 ? 2 : 1;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(H) * 256u, num_tokens};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(H) * 256u * elem};
    const cuuint32_t box[2] = {128u / elem, kTileTokens};
    const cuuint32_t estr[2] = {1u, 1u};
    return fn(map, BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
              const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <bool BF16>
cudaError_t launch(cudaStream_t stream, const IngestParams& p)
{
    using C = Cfg<BF16>;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) != cudaSuccess) return cudaErrorNoDevice;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    static bool configured[64] = {};   // benign race: the attribute is idempotent
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(tq_ingest_umma256_kernel<BF16>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    const uint64_t tiles = static_cast<uint64_t>((p.num_strips + 7u) / 8u) * p.H;   // (tile, head) items
    if (tiles == 0) return cudaSuccess;
    alignas(64) CUtensorMap key_map, value_map;
    if (!activation_map<BF16>(&key_map, p.key, p.num_strips * kStrip, p.H) ||
        !activation_map<BF16>(&value_map, p.value, p.num_strips * kStrip, p.H))
        return cudaErrorNotSupported;
    const uint32_t resident = static_cast<uint32_t>(sms);   // persistent: one CTA per SM
    const uint64_t wanted = (tiles + kGroups - 1) / kGroups;
    const uint32_t blocks = wanted < resident ? static_cast<uint32_t>(wanted) : resident;
    tq_ingest_umma256_kernel<BF16><<<blocks, kThreads, C::kSmem, stream>>>(p, key_map, value_map);
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_ingest_umma256(cudaStream_t stream, const IngestParams& p, bool bf16)
{
    return bf16 ? launch<true>(stream, p) : launch<false>(stream, p);
}

}  // namespace tq
