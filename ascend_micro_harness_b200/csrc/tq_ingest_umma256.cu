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
// one add and one subtract per pair of outputs in the epilogue. M_0 and M_1 are built once per
// persistent CTA in shared memory (K-major, 128-byte swizzle); INT32 sums get the bit pattern of
// 1.5 * 2^23 added on the way out of tensor memory, as in tq_ingest_umma.cu.
// Two accumulators of 128 columns are half of an SM's tensor memory, so there are two sets and the
// kernel is a pipeline: one lane issues the products (per item the key plane, D[token][channel], then
// the value plane with the operands swapped, D'[channel][token]) into alternating sets, one lane of
// another warp fetches the tiles by TMA as their buffers come free, and sixteen warps read the sets
// out: warp w takes lane quarter w & 3 (the rows) and column quarter w >> 2 of both accumulators.
// Key plane: a row is a token; the four warps that hold it exchange their absmax through shared
// memory. Value plane: a column is a token; its absmax is a maximum down the column, over a warp's
// rows by a warp reduction and over the lane quarters through shared memory -- no product of its
// own for the scales.
// Every wait on a barrier is bounded by a clock budget (see tq_ingest_umma.cu).
#include <type_traits>

#include "tq_umma.cuh"

namespace tq {
namespace {

constexpr int kTileTokens = 128;
constexpr int kEpiWarps = 16;                // warp w: lane quarter w & 3 (rows), column quarter w >> 2
constexpr int kEpiThreads = kEpiWarps * 32;
constexpr int kThreads = kEpiThreads + 64;   // + one warp whose first lane issues the products, one whose first lane fetches tiles
constexpr uint32_t kAccCols = 128;           // one 128 x 128 accumulator
constexpr uint32_t kSetCols = 2 * kAccCols;  // a, then b
constexpr uint32_t kTmemCols = 2 * kSetCols; // two sets: one is read out while the other is written

template <bool BF16>
struct Cfg {
    static constexpr int kElem = BF16 ? 2 : 1;
    static constexpr int kHalfRowBytes = 128 * kElem;        // 128 channels of one token
    static constexpr int kBlocksHalf = kHalfRowBytes / 128;  // 128-byte-wide K blocks per half row
    static constexpr int kBlockBytes = 128 * 128;            // 128 rows of one K block
    static constexpr int kHalfBytes = kBlocksHalf * kBlockBytes;   // x_lo, x_hi, M_0, M_1: each this size
    static constexpr int kTileBytes = 2 * kHalfBytes;
    static constexpr int kKSteps = kHalfRowBytes / 32;       // one MMA contracts 32 bytes of K
    // Tile buffers: 0 the key tile, 1 the value tile of the item in flight. Measured and dropped:
    // a second item's tiles in flight for int8, whose tiles are half the size (3.31 against 3.33 TB/s:
    // int8 waits on its epilogue, not on tiles), and halves of a tile fetched and given back
    // separately (bf16 4.94 against 5.30 TB/s: the extra commit between the two chains of a product
    // holds the second chain back).
    static constexpr int kTileBufs = 2;
    // 128 inverse scales, 2 x 4 x 128 absmax quarters, 8 strip offsets, 8 barriers
    static constexpr int kSmallBytes = 9 * kTileTokens * 4 + 8 * 8 + 8 * 8;
    static constexpr int kUsed = 2 * kHalfBytes + kTileBufs * kTileBytes + kSmallBytes + 64;
    static constexpr int kSmem = kUsed + 1024;               // slack for aligning the tiles
};

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

// All 512 epilogue threads (named barrier 1); the producer warps take no part.
__device__ __forceinline__ void epi_sync()
{
    asm volatile("bar.sync 1, %0;\n" ::"r"(kEpiThreads) : "memory");
}
// The same barrier carrying a
// vote: true for every epilogue thread if any of them says so. The
// decision to leave the item loop must be one decision for all of them, or the next barrier hangs.
__device__ __forceinline__ bool epi_sync_any(bool mine)
{
    uint32_t any;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %2, 0;\n\t"
        "bar.red.or.pred q, 1, %1, p;\n\tselp.u32 %0, 1, 0, q;\n\t}\n"
        : "=r"(any) : "r"(kEpiThreads), "r"(mine ? 1u : 0u) : "memory");
    return any != 0u;
}
// The four warps that share a lane quarter, i.e. the same 32 rows (named barrier 2 + quarter).
__device__ __forceinline__ void rows_sync(int quarter)
{
    asm volatile("bar.sync %0, 128;\n" ::"r"(quarter + 2) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t mbar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(mbar) : "memory");
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
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool producer = warp >= kEpiWarps;     // warp 16: products, warp 17: tile fetches
    const int quarter = warp & 3, cq = (warp >> 2) & 3;   // tensor-memory lane quarter, column quarter
    const int row = quarter * 32 + lane;                  // token (plain products) or channel (swapped)
    uint8_t* m_tiles = base;                              // M_0, then M_1
    uint8_t* x_tiles = base + 2 * C::kHalfBytes;          // per buffer: x_lo blocks, then x_hi blocks
    uint8_t* small = x_tiles + C::kTileBufs * C::kTileBytes;
    float* inv_s = reinterpret_cast<float*>(small);       // per token: 2^(2-e)
    float* amax_s = inv_s + kTileTokens;                  // [2 planes][4 quarters][128]
    unsigned long long* strip_off = reinterpret_cast<unsigned long long*>(small + 9 * kTileTokens * 4);  // [8]
    // [0..1]: tile buffer landed, [2..3]: tile buffer consumed, [4..5]: accumulator set written,
    // [6..7]: accumulator set read out
    uint64_t* mbar = reinterpret_cast<uint64_t*>(strip_off + 8);
    uint32_t* shared_words = reinterpret_cast<uint32_t*>(mbar + 8);
    uint32_t* tmem_slot = shared_words;
    volatile uint32_t* abort_flag = shared_words + 1;
    volatile uint32_t* fetched = shared_words + 2;   // [2]: tile fetches issued per buffer (written by the fetching lane)

    const uint32_t items = ((p.num_strips + 7u) / 8u) * p.H;
    const uint32_t num_tokens = p.num_strips * kStrip;

    // ---- one-time set-up: barriers, tensor memory, the two rotation matrices
    if (threadIdx.x == 0) {
#pragma unroll
        for (int i = 0; i < 6; ++i)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(smem_addr(mbar + i)));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_addr(mbar + 6)), "r"(kEpiWarps));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_addr(mbar + 7)), "r"(kEpiWarps));
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        *abort_flag = 0u;
        fetched[0] = 0u;
        fetched[1] = 0u;
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_addr(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    if (!producer) {
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
            const int blk = q >> 3, cq16 = q & 7;
            *reinterpret_cast<uint4*>(m_tile + blk * C::kBlockBytes + r * 128 + ((cq16 ^ (r & 7)) << 4)) =
                make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
    fence_async_smem();
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    // this thread's 32 columns of accumulator a in set 0; b lies kAccCols further on, set 1 kSetCols
    const uint32_t acc0 = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(cq) * 32u;
    const uint32_t bar_s = smem_addr(mbar);
    auto bar_of = [&](int i) { return bar_s + 8u * static_cast<uint32_t>(i); };
    const uint32_t item_step = gridDim.x;

    if (producer) {
        const uint32_t x_tiles_s = smem_addr(x_tiles);
        bool healthy = true;
        auto wait = [&](uint32_t bar, uint32_t par) {
            if (!healthy) return;
            if (!bounded_mbar_wait(bar, par, p.wait_budget, abort_flag)) {
                healthy = false;
                *abort_flag = 1u;
                report(p.status, TQ_STATUS_WAIT_EXPIRED);
            }
        };
        uint32_t landed_par = 0, landed_seen[2] = {0, 0};   // the issuing lane's view of the tile barriers
        if (warp == kEpiWarps + 1 && lane == 0) {
            // ---- tile fetches: a buffer (0: key tile, 1: value tile) is fetched again, for the CTA's
            // next item, as soon as the last product reading it has completed
            uint32_t consumed_par = 0, count[2] = {0, 0};
            auto fetch = [&](uint32_t item, uint32_t buf) {
                if (!healthy) return;
                const TileId id = tile_of(p, item);
                const CUtensorMap* map = buf == 0 ? &key_map : &value_map;
                const uint32_t bar = bar_of(buf), dst = x_tiles_s + buf * C::kTileBytes;
                mbar_expect_tx(bar, C::kTileBytes);
#pragma unroll
                for (int blk = 0; blk < 2 * C::kBlocksHalf; ++blk)
                    tma_load_2d(dst + blk * C::kBlockBytes, map,
                                static_cast<int>(id.head * 256u + blk * (128 / C::kElem)),
                                static_cast<int>(id.tok_tile * kTileTokens), bar);
                fetched[buf] = ++count[buf];
            };
            uint32_t item = blockIdx.x;
            if (item < items) {
                fetch(item, 0);
                fetch(item, 1);
            }
            for (; item + item_step < items && healthy; item += item_step) {
#pragma unroll
                for (uint32_t buf = 0; buf < 2; ++buf) {
                    wait(bar_of(2 + buf), (consumed_par >> buf) & 1u);
                    consumed_par ^= 1u << buf;
                    fetch(item + item_step, buf);
                }
            }
        }
        uint32_t n = 0, commits = 0;
        if (warp == kEpiWarps && lane == 0) {
            // ---- products. Product n writes accumulator set n & 1; per item the key plane, then the
            // value plane with the operands swapped; an accumulator set is written again as soon as
            // the epilogue warps have read it out.
            const uint64_t desc_x = umma_desc(x_tiles_s), desc_m = umma_desc(smem_addr(m_tiles));
            // transposed = false: D[token][channel] = X_h M_h^T; true: D'[channel][token] = M_h X_h^T
            auto product = [&](bool transposed, uint32_t buf, bool fresh, bool last_use) {
                if (fresh) {
                    wait(bar_of(buf), (landed_par >> buf) & 1u);
                    if (healthy) {
                        landed_par ^= 1u << buf;
                        ++landed_seen[buf];
                    }
                }
                const uint32_t set = n & 1u;
                wait(bar_of(6 + set), ((n >> 1) & 1u) ^ 1u);   // the set has been read out (passes at once the first time)
                if (healthy) {
                    fence_after_sync();
                    const uint32_t tmem_set = tmem_base + set * kSetCols;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint64_t dx0 = desc_x + ((buf * C::kTileBytes + h * C::kHalfBytes) >> 4);
                        const uint64_t dm0 = desc_m + ((h * C::kHalfBytes) >> 4);
#pragma unroll
                        for (int k = 0; k < C::kKSteps; ++k) {
                            const uint32_t off16 = ((k >> 2) * C::kBlockBytes + (k & 3) * 32) >> 4;
                            const uint64_t dx = dx0 + off16, dm = dm0 + off16;
                            umma<BF16>(tmem_set + h * kAccCols, transposed ? dm : dx, transposed ? dx : dm, k > 0 ? 1u : 0u);
                        }
                    }
                    umma_commit(bar_of(4 + set));
                    if (last_use) umma_commit(bar_of(2 + buf));
                    ++commits;
                }
                ++n;
            };
            for (uint32_t item = blockIdx.x; item < items && healthy; item += item_step) {
                product(false, 0, true, true);    // key plane, per token
                product(true, 1, true, true);     // value plane, per channel
            }
        }
        // Both lanes are through (the other lanes of the two warps have nothing to do): whatever is
        // still on its way into this CTA's shared and tensor memory gets the full budget to finish
        // before the memory goes back to the SM -- the fetches the issuing lane has not seen land,
        // and the last product chain (its commit also covers every earlier one).
        asm volatile("bar.sync 6, 64;\n" ::: "memory");
        if (warp == kEpiWarps && lane == 0) {
#pragma unroll
            for (uint32_t buf = 0; buf < 2; ++buf)
                if (fetched[buf] != landed_seen[buf])
                    bounded_mbar_wait(bar_of(buf), (landed_par >> buf) & 1u, kWaitBudget, nullptr);
            if (commits != 0u) {
                const uint32_t last = n - 1u;
                bounded_mbar_wait(bar_of(4 + (last & 1u)), (last >> 1) & 1u, kWaitBudget, nullptr);
            }
        }
    } else {
        // ---- epilogue warps
        bool healthy = true;
        uint32_t m = 0;   // product counter, in step with the producer's
        // wait for product m, return the address of this thread's columns in its set
        auto await_product = [&]() -> uint32_t {
            const uint32_t set = m & 1u;
            if (healthy && !bounded_mbar_wait(bar_of(4 + set), (m >> 1) & 1u, p.wait_budget, abort_flag)) {
                healthy = false;
                *abort_flag = 1u;
                report(p.status, TQ_STATUS_WAIT_EXPIRED);
            }
            fence_after_sync();
            return acc0 + set * kSetCols;
        };
        // this warp is done with product m's accumulators
        auto release_product = [&]() {
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_of(6 + (m & 1u)));
            ++m;
        };

        int32_t slot = -1;
        bool strip_ok = false, tok_live = false;
        uint32_t head = 0;
        size_t block_off = 0, scale_at = 0;
        const size_t plane_scales = static_cast<size_t>(p.P) * p.H * p.S;
        const float2 minus1 = make_float2(-1.0f, -1.0f), minus2bias = make_float2(-2.0f * kBias, -2.0f * kBias);
        const float2 magic2 = make_float2(kMagic, kMagic);

        // y_lo and y_hi of two adjacent columns out of the raw accumulator words. int8: a' = B + a and
        // b' = B + b with B = 1.5 * 2^23; b' - 2B, a' + (b' - 2B) and a' - b' are all exact in FP32.
        auto combine = [&](uint32_t a0, uint32_t a1, uint32_t b0, uint32_t b1, float2& lo, float2& hi) {
            const float2 a = make_float2(__uint_as_float(a0), __uint_as_float(a1));
            const float2 b = make_float2(__uint_as_float(b0), __uint_as_float(b1));
            if constexpr (BF16) lo = __fadd2_rn(a, b);
            else lo = __fadd2_rn(a, __fadd2_rn(b, minus2bias));
            hi = __ffma2_rn(b, minus1, a);
        };
        // This thread's 32 columns of both accumulators of the set at `acc`, read out in one go and
        // turned in place into y_lo (in va) and y_hi (in vb); the set is handed back to the issuing
        // lane at once, so the next product into it runs under everything that follows.
        auto take_product = [&](uint32_t acc, uint32_t (&va)[32], uint32_t (&vb)[32]) {
            tmem_ld32(acc, va);
            tmem_ld32(acc + kAccCols, vb);
            tmem_arrived(va);
            tmem_arrived(vb);
            if constexpr (!BF16) {
                // INT32 sums (|sum| <= 2^14) onto the bit pattern of 1.5 * 2^23: read as a float that is
                // 12582912 + sum exactly, no integer-to-float conversion
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    va[j] += kBiasBits;
                    vb[j] += kBiasBits;
                }
            }
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
                float2 lo, hi;
                combine(va[j], va[j + 1], vb[j], vb[j + 1], lo, hi);
                va[j] = __float_as_uint(lo.x);
                va[j + 1] = __float_as_uint(lo.y);
                vb[j] = __float_as_uint(hi.x);
                vb[j + 1] = __float_as_uint(hi.y);
            }
            release_product();
        };
        // the row's absmax over all four column quarters (a barrier of the four warps that hold the row inside)
        auto row_absmax = [&](float mine, int plane) -> float {
            float* ex = amax_s + plane * 4 * kTileTokens;
            ex[cq * kTileTokens + row] = mine;
            rows_sync(quarter);
            const float m01 = fmaxf(ex[row], ex[kTileTokens + row]);
            const float m23 = fmaxf(ex[2 * kTileTokens + row], ex[3 * kTileTokens + row]);
            return fmaxf(fmaxf(m01, m23), 1.0f);   // the writer floors absmax at 1
        };

#pragma unroll 1
        for (uint32_t item = blockIdx.x; item < items; item += item_step) {
            uint32_t va[32], vb[32];
            // ---- where this thread's token of the tile goes (requested before anything waits)
            {
                const TileId id = tile_of(p, item);
                const uint32_t tok = id.tok_tile * kTileTokens + row;
                head = id.head;
                tok_live = tok < num_tokens;
                slot = -1;   // a volatile load: it must not sink below the product's wait
                if (tok_live) asm volatile("ld.global.nc.s32 %0, [%1];\n" : "=r"(slot) : "l"(p.slots + tok));
            }
            // ================= key plane: a row is a token
            take_product(await_product(), va, vb);
            {
                const int32_t slot0 = __shfl_sync(0xffffffffu, slot, lane & 16);
                const bool run_ok = slot == slot0 + (lane & 15);
                const uint32_t votes = __ballot_sync(0xffffffffu, run_ok);
                const bool strip_live = __shfl_sync(0xffffffffu, tok_live ? 1 : 0, lane & 16) != 0;
                const uint32_t slot_page = fast_div(static_cast<uint32_t>(slot0), p.page_mul, p.page_shift);
                strip_ok = strip_live && ((votes >> (lane & 16)) & 0xFFFFu) == 0xFFFFu && slot0 >= 0 &&
                           (slot0 % kStrip) == 0 && slot_page < p.P;
                if (strip_live && !strip_ok && (lane & 15) == 0 && cq == 0) report(p.status, TQ_STATUS_BAD_SLOT);
                const uint32_t page = strip_ok ? slot_page : 0u;
                const uint32_t tok_in_page = strip_ok ? static_cast<uint32_t>(slot0) - slot_page * p.S : 0u;
                // byte offset of the strip's (page, head) block in either code plane
                block_off = (static_cast<size_t>(page) * p.H + head) * (static_cast<size_t>(p.S) * 128u) +
                            static_cast<size_t>(tok_in_page / kStrip) * 2048u;
                scale_at = (static_cast<size_t>(page) * p.H + head) * p.S + tok_in_page + (lane & 15);
            }
            {
                float m0 = 0.0f, m1 = 0.0f;
#pragma unroll
                for (int j = 0; j < 32; j += 2) {
                    m0 = max3f(m0, fabsf(__uint_as_float(va[j])), fabsf(__uint_as_float(va[j + 1])));
                    m1 = max3f(m1, fabsf(__uint_as_float(vb[j])), fabsf(__uint_as_float(vb[j + 1])));
                }
                const float amax = row_absmax(fmaxf(m0, m1), 0);
                const int pow_bits = (__float_as_int(amax) & 0x7F800000) - (2 << 23);
                const float inv = __int_as_float((254 << 23) - pow_bits);
                if (cq == 0 && strip_ok && healthy)
                    p.scale_cache[scale_at] = __int_as_float(pow_bits) * p.inv_sqrt_len;
                // the token's row of 128 bytes; this thread's columns are channels 32 cq .. of y_lo
                // (bytes 16 cq ..) and 128 + 32 cq .. of y_hi (bytes 64 + 16 cq ..)
                uint4* dst = reinterpret_cast<uint4*>(p.key_cache + block_off + static_cast<size_t>(lane & 15) * 128u +
                                                      static_cast<size_t>(cq) * 16u);
                const float2 inv2 = make_float2(inv, inv);
                uint32_t wl[4], wh[4];
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    float rl[8], rh[8];
#pragma unroll
                    for (int e = 0; e < 8; e += 2) {
                        const float2 l = __ffma2_rn(make_float2(__uint_as_float(va[g * 8 + e]), __uint_as_float(va[g * 8 + e + 1])),
                                                    inv2, magic2);
                        const float2 h = __ffma2_rn(make_float2(__uint_as_float(vb[g * 8 + e]), __uint_as_float(vb[g * 8 + e + 1])),
                                                    inv2, magic2);
                        rl[e] = l.x;
                        rl[e + 1] = l.y;
                        rh[e] = h.x;
                        rh[e + 1] = h.y;
                    }
                    wl[g] = pack8(rl);
                    wh[g] = pack8(rh);
                }
                if (strip_ok && healthy) {
                    __stcs(dst, make_uint4(wl[0], wl[1], wl[2], wl[3]));
                    __stcs(dst + 4, make_uint4(wh[0], wh[1], wh[2], wh[3]));   // 64 bytes further on
                }
            }
            // ================= value plane: one product, with the operands swapped. This thread is
            // channel `row` of y_lo and 128 + row of y_hi, tokens 32 cq .. (two strips). A token's
            // absmax is the maximum down a column: over the warp's 32 rows by a warp reduction (lane t
            // keeps column t's), over the four lane quarters and both accumulators through shared memory.
            take_product(await_product(), va, vb);
            {
                float kept = 0.0f;
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const float v = fmaxf(fabsf(__uint_as_float(va[j])), fabsf(__uint_as_float(vb[j])));
                    const uint32_t mx = __reduce_max_sync(0xffffffffu, __float_as_uint(v));
                    if (lane == j) kept = __uint_as_float(mx);
                }
                float* part = amax_s + 4 * kTileTokens;   // [4 lane quarters][128 tokens]
                part[quarter * kTileTokens + cq * 32 + lane] = kept;
            }
            // every quarter's share is in; also the one place where the epilogue warps agree to stop
            if (epi_sync_any(!healthy || *abort_flag != 0u)) break;
            if (cq == 0) {
                // token `row`: the thread that placed it in the key plane finishes its scale
                const float* part = amax_s + 4 * kTileTokens;
                const float m01 = fmaxf(part[row], part[kTileTokens + row]);
                const float m23 = fmaxf(part[2 * kTileTokens + row], part[3 * kTileTokens + row]);
                const float amax_v = fmaxf(fmaxf(m01, m23), 1.0f);   // the writer floors absmax at 1
                const int pow_bits = (__float_as_int(amax_v) & 0x7F800000) - (2 << 23);
                inv_s[row] = __int_as_float((254 << 23) - pow_bits);
                if ((lane & 15) == 0)
                    strip_off[row >> 4] = strip_ok ? static_cast<unsigned long long>(block_off) : ~0ull;
                if (strip_ok && healthy)
                    p.scale_cache[scale_at + plane_scales] = __int_as_float(pow_bits) * p.inv_sqrt_len;
            }
            epi_sync();   // publishes the per-token constants
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int s = cq * 2 + c;   // the strip of tokens 32 cq + 16 c ..
                const unsigned long long off = strip_off[s];
                uint32_t wl[2], wh[2];
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    float rl[8], rh[8];
#pragma unroll
                    for (int q = 0; q < 2; ++q) {
                        const int t = c * 16 + g * 8 + q * 4;
                        const float4 iv = *reinterpret_cast<const float4*>(inv_s + cq * 32 + t);
                        const float2 i01 = make_float2(iv.x, iv.y), i23 = make_float2(iv.z, iv.w);
                        const float2 l0 = __ffma2_rn(make_float2(__uint_as_float(va[t]), __uint_as_float(va[t + 1])), i01, magic2);
                        const float2 l1 = __ffma2_rn(make_float2(__uint_as_float(va[t + 2]), __uint_as_float(va[t + 3])), i23, magic2);
                        const float2 h0 = __ffma2_rn(make_float2(__uint_as_float(vb[t]), __uint_as_float(vb[t + 1])), i01, magic2);
                        const float2 h1 = __ffma2_rn(make_float2(__uint_as_float(vb[t + 2]), __uint_as_float(vb[t + 3])), i23, magic2);
                        rl[q * 4] = l0.x;
                        rl[q * 4 + 1] = l0.y;
                        rl[q * 4 + 2] = l1.x;
                        rl[q * 4 + 3] = l1.y;
                        rh[q * 4] = h0.x;
                        rh[q * 4 + 1] = h0.y;
                        rh[q * 4 + 2] = h1.x;
                        rh[q * 4 + 3] = h1.y;
                    }
                    wl[g] = pack8(rl);
                    wh[g] = pack8(rh);
                }
                if (healthy && off != ~0ull) {
                    uint8_t* blk = p.value_cache + off;
                    __stcs(reinterpret_cast<uint2*>(blk + static_cast<size_t>(row) * 8u), make_uint2(wl[0], wl[1]));
                    __stcs(reinterpret_cast<uint2*>(blk + static_cast<size_t>(128 + row) * 8u), make_uint2(wh[0], wh[1]));
                }
            }
        }
    }
    fence_before_sync();
    __syncthreads();
    if (warp == 0)
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
    const uint32_t blocks = tiles < resident ? static_cast<uint32_t>(tiles) : resident;
    tq_ingest_umma256_kernel<BF16><<<blocks, kThreads, C::kSmem, stream>>>(p, key_map, value_map);
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_ingest_umma256(cudaStream_t stream, const IngestParams& p, bool bf16)
{
    return bf16 ? launch<true>(stream, p) : launch<false>(stream, p);
}

}  // namespace tq
