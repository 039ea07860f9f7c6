// reshape_and_cache, aligned writer for head size 128 on the 5th-generation tensor
// core (tcgen05) with the accumulator in tensor memory.
//
// What is computed is what the warp-MMA writer computes (tq_ingest.cu; reference:
// tests/common/turboquant_oracle.hpp:357-449,
// kernels/ops/turboquant/turboquant_reshape_and_cache_a8.cpp:714-744,:1083-1226):
//   y = M x,  M = (H_4 (x) I32) diag(s) (I_4 (x) H32)      128 x 128, entries +-1
//   absmax = max(1, max|y|), scale = 2^(e-2) * inv_sqrt_len, q = rint_even(min(y 2^(2-e), 7))
//
// How: M is a dense +-1 matrix, so a tile of 128 tokens of one (plane, head) is ONE
// 128 x 128 x 128 tensor-core product instead of MMAs plus register butterflies:
//   * a persistent CTA builds M once in shared memory (K-major, 128-byte swizzle); its two
//     groups of 128 threads then walk tiles independently, each with its own tile buffer,
//     128 tensor-memory columns, completion barriers and named CTA barrier. The activations
//     of a group's next tile are fetched by TMA (one 128-row x 128-byte box per K block,
//     hardware 128-byte swizzle, rows past the last token filled with zeros) as soon as the
//     tensor core has consumed the current ones; four groups share an SM, so one group's
//     waits are another's work;
//   * key plane:   D[token][channel] = X M^T  -- a thread reads its token's 128 rotated
//     channels out of tensor memory, so absmax, scale, rounding and the packing of the
//     token's 64-byte page row are all thread-local;
//   * value plane: the same product gives the per-token scales; then the product with the
//     operands swapped, D'[channel][token] = M X^T (same two shared-memory tiles, same
//     tensor-memory columns), hands every thread one channel with its 128 tokens: the 8
//     bytes a channel owns in each channel-major 16-token strip are thread-local too, and
//     a warp's stores are 256 contiguous bytes;
//   * int8 tiles accumulate in INT32; a sum read out of tensor memory gets the bit pattern of
//     1.5 * 2^23 added, so that as a float it is 12582912 + y exactly and no integer-to-float
//     conversion is issued; bf16 tiles accumulate in FP32 (exact for integer-valued inputs).
// Every wait on the tensor core's completion barrier is bounded by a clock budget; when it
// runs out the kernel stops storing, reports TQ_STATUS_WAIT_EXPIRED, frees its tensor
// memory and returns.
#include <type_traits>

#include "tq_umma.cuh"

namespace tq {
namespace {

constexpr int kTileTokens = 128;
constexpr int kGroups = 2;                   // independent 128-thread groups per CTA, one tile each
constexpr int kGroupThreads = 128;
constexpr int kThreads = kGroups * kGroupThreads;
constexpr uint32_t kGroupCols = 128;         // one 128 x 128 FP32/INT32 accumulator per group
constexpr uint32_t kTmemCols = kGroups * kGroupCols;
template <bool BF16>
struct Cfg {
    static constexpr int kElem = BF16 ? 2 : 1;
    static constexpr int kRowBytes = 128 * kElem;        // one token row of one head
    static constexpr int kBlocks = kRowBytes / 128;      // 128-byte-wide K blocks per row
    static constexpr int kBlockBytes = 128 * 128;        // 128 rows of one K block
    static constexpr int kTileBytes = kBlocks * kBlockBytes;
    static constexpr int kKSteps = kRowBytes / 32;       // one MMA contracts 32 bytes of K
    // Per CTA: M once; per group one activation tile, the per-token quantiser constants,
    // the strip offsets and a barrier; 1 KiB of slack for aligning the tiles. Two CTAs per
    // SM: 2 x 256 tensor-memory columns is all an SM has, so the request is padded to
    // 80 KiB and a third CTA can never land on an SM and stall in its allocation.
    static constexpr int kCtasPerSm = 2;
    // int8 tiles are half the size: a group keeps the key tile and the value tile of an item in
    // buffers of their own and fetches each a whole item ahead; bf16 has room for one buffer
    static constexpr int kTileBufs = BF16 ? 1 : 2;
    static constexpr int kSmallBytes = 2 * kTileTokens * 4 + 8 * 8 + 64;
    static constexpr int kGroupBytes = kTileBufs * kTileBytes + kSmallBytes;
    static constexpr int kUsed = kTileBytes + kGroups * kGroupBytes + 64;
    static constexpr int kSmem = (kUsed + 1024) > 80 * 1024 ? (kUsed + 1024) : 80 * 1024;
};

// Work is dealt out as (128-token tile, head) items; a group does the key plane and then
// the value plane of its item, so every group carries the same mix of the cheaper key
// tiles and the dearer value tiles whatever the grid size. Unit u of a group is plane
// u & 1 of its (u >> 1)-th item.
struct TileId {
    uint32_t tok_tile, plane, head;
};
__device__ __forceinline__ TileId tile_of(const IngestParams& p, uint32_t item, uint32_t plane)
{
    TileId id;
    id.tok_tile = fast_div(2u * item, p.div_mul, p.div_shift);   // item / H with the 2H divider
    id.head = item - id.tok_tile * p.H;
    id.plane = plane;
    return id;
}

// All 128 threads of one group (named barrier 1 + group).
__device__ __forceinline__ void group_sync(int group)
{
    asm volatile("bar.sync %0, %1;\n" ::"r"(group + 1), "r"(kGroupThreads) : "memory");
}

// The same barrier carrying a vote: true for every thread of the group if any of them says so.
// Leaving the item loop must be one decision per group, or the group's next barrier would hang.
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
__global__ void __launch_bounds__(kThreads, Cfg<BF16>::kCtasPerSm)
tq_ingest_umma_kernel(const IngestParams p, const __grid_constant__ CUtensorMap key_map,
                      const __grid_constant__ CUtensorMap value_map)
{
    using C = Cfg<BF16>;
    extern __shared__ uint8_t smem_raw[];
    // tiles on a 1024-byte boundary: the swizzle is a function of address bits 4..9
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~uintptr_t(1023));
    const int group = threadIdx.x / kGroupThreads, tid = threadIdx.x % kGroupThreads;
    const int warp = tid >> 5, lane = tid & 31;   // warp within the group = its tensor-memory lane quarter
    uint8_t* m_tile = base;
    uint8_t* x_tile = base + C::kTileBytes + group * (C::kTileBufs * C::kTileBytes);
    uint8_t* small = base + (1 + kGroups * C::kTileBufs) * C::kTileBytes + group * C::kSmallBytes;
    float* inv_s = reinterpret_cast<float*>(small);   // per token: 2^(2-e)
    unsigned long long* strip_off = reinterpret_cast<unsigned long long*>(small + 2 * kTileTokens * 4);  // [8]
    uint64_t* mbar = reinterpret_cast<uint64_t*>(strip_off + 8);   // [0]: products done, [1 + b]: tile buffer b landed
    uint32_t* shared_words = reinterpret_cast<uint32_t*>(base + (1 + kGroups * C::kTileBufs) * C::kTileBytes +
                                                         kGroups * C::kSmallBytes);
    uint32_t* tmem_slot = shared_words;
    volatile uint32_t* abort_flag = shared_words + 1;

    const uint32_t items = ((p.num_strips + 7u) / 8u) * p.H;
    const uint32_t num_tokens = p.num_strips * kStrip;
    const size_t row_pitch = static_cast<size_t>(p.H) * C::kRowBytes;         // bytes between tokens

    // ---- one-time set-up: barriers, tensor memory, the rotation matrix
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(smem_addr(mbar)));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(smem_addr(mbar + 1)));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(smem_addr(mbar + 2)));
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        if (group == 0) *abort_flag = 0u;
    }
    if (threadIdx.x < 32) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_addr(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    {
        // Row `tid` of M: output channel c1*32 + c0 against input channel g*32 + i is
        // H4[c1][g] * s[g*32 + c0] * H32[c0][i]; true = -1. Each group writes half the row.
        const unsigned c1 = tid >> 5, c0 = tid & 31;
        bool gneg[4];
#pragma unroll
        for (int g = 0; g < 4; ++g)
            gneg[g] = hneg(c1, g) != sign_is_negative(p.signs, p.sign_source, g * kGroup + c0);
        constexpr int kPerChunk = 16 / C::kElem;   // elements in a 16-byte chunk
        constexpr int kChunks = C::kRowBytes / 16;
#pragma unroll 1
        for (int q = group * (kChunks / kGroups); q < (group + 1) * (kChunks / kGroups); ++q) {
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
            *reinterpret_cast<uint4*>(m_tile + blk * C::kBlockBytes + tid * 128 + ((cq ^ (tid & 7)) << 4)) =
                make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
    fence_async_smem();
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_group = tmem_base + static_cast<uint32_t>(group) * kGroupCols;
    const uint32_t acc = tmem_group + (static_cast<uint32_t>(warp * 32) << 16);   // this warp's lanes
    const uint32_t mbar_s = smem_addr(mbar), tma_bar_s = smem_addr(mbar + 1);
    const uint32_t x_tile_s = smem_addr(x_tile), m_tile_s = smem_addr(m_tile);
    const uint64_t desc_x = umma_desc(x_tile_s), desc_m = umma_desc(m_tile_s);

    // The group's thread 0 fetches a tile: one box per 128-byte K block, rows = the tile's 128
    // tokens (past the end of the tensor: zeros, never stored), x = the head's first channel.
    // Thread 0 of the group keeps the books of what it has in flight towards this CTA's shared
    // and tensor memory: a tile fetch whose barrier phase nobody has seen complete, a chain of
    // products whose commit nobody has seen arrive. Nothing new is issued once a wait has run out.
    // Tile buffer of a plane: with two buffers the key tile lives in 0 and the value tile in 1.
    // Bit b of tma_parity / tma_pending is the state of buffer b's barrier.
    uint32_t parity = 0, tma_parity = 0, tma_pending = 0, mma_pending_parity = 0;
    bool healthy = true, mma_pending = false;
    auto buffer_of = [](uint32_t plane) { return C::kTileBufs == 2 ? plane : 0u; };
    auto load_tile = [&](uint32_t item, uint32_t plane) {
        if (tid != 0 || !healthy) return;
        const TileId id = tile_of(p, item, plane);
        const CUtensorMap* map = plane == 0 ? &key_map : &value_map;
        const uint32_t buf = buffer_of(plane), bar = tma_bar_s + 8u * buf, dst = x_tile_s + buf * C::kTileBytes;
        mbar_expect_tx(bar, C::kTileBytes);
#pragma unroll
        for (int blk = 0; blk < C::kBlocks; ++blk)
            tma_load_2d(dst + blk * C::kBlockBytes, map,
                        static_cast<int>(id.head * 128u + blk * (128 / C::kElem)),
                        static_cast<int>(id.tok_tile * kTileTokens), bar);
        tma_pending |= 1u << buf;
    };

    auto bounded_wait = [&](uint32_t bar, uint32_t par, long long budget, bool watch_abort) {
        return bounded_mbar_wait(bar, par, budget, watch_abort ? abort_flag : nullptr);
    };
    // One product into the accumulator columns, then the bounded wait for it.
    // transposed = false: D[token][channel] = X M^T; true: D'[channel][token] = M X^T.
    auto product = [&](bool transposed, bool fresh_tile, uint32_t buf) {
        fence_before_sync();
        group_sync(group);
        if (tid == 0 && healthy) {
            bool landed = true;
            if (fresh_tile) {   // the TMA boxes of this tile have landed (same proxy as the MMA reads)
                landed = bounded_wait(tma_bar_s + 8u * buf, (tma_parity >> buf) & 1u, p.wait_budget, false);
                if (landed) {
                    tma_pending &= ~(1u << buf);
                    tma_parity ^= 1u << buf;
                }
            }
            if (landed) {
                fence_after_sync();
                // descriptors of the K-steps differ from the tile's first one only in the address
                // field (16-byte units in the low bits, no carry out of it below 256 KiB): one add each
                // instead of building them anew, which cost the issuing thread most of its time here
                const uint64_t dx0 = desc_x + ((buf * C::kTileBytes) >> 4);
#pragma unroll
                for (int k = 0; k < C::kKSteps; ++k) {
                    const uint32_t off16 = ((k >> 2) * C::kBlockBytes + (k & 3) * 32) >> 4;
                    const uint64_t dx = dx0 + off16, dm = desc_m + off16;
                    umma<BF16>(tmem_group, transposed ? dm : dx, transposed ? dx : dm, k > 0 ? 1u : 0u);
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

    // An INT32 sum read out of tensor memory gets the bit pattern of 1.5 * 2^23 added, so that as a
    // float it is 12582912 + sum exactly: no integer-to-float conversion. (Presetting the columns to
    // that pattern instead, so that the sums come out ready, measured slower: the stores into tensor
    // memory each need as many registers as columns and a wait before the next product.)
    auto biased = [](uint32_t (&v)[32]) {
        if constexpr (!BF16) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += kBiasBits;
        }
    };

    const uint32_t item_step = gridDim.x * kGroups;
    uint32_t item = blockIdx.x * kGroups + group;
    if (item < items) {
        load_tile(item, 0);
        if (C::kTileBufs == 2) load_tile(item, 1);
    }
    int32_t slot = -1;
    bool strip_ok = false, tok_live = false;
    uint32_t page = 0, tok_in_page = 0, head = 0;
    size_t block_off = 0, scale_at = 0;
    const size_t plane_scales = static_cast<size_t>(p.P) * p.H * p.S;

    // One plane of one item; the plane is a compile-time tag, so that an item is a straight run
    // of key-plane code and value-plane code with one loop turn per item (a turn of this long
    // loop costs the group some hundreds of cycles). Returns false once a wait has run out.
    auto do_plane = [&](auto plane_tag) -> bool {
        constexpr uint32_t kPlane = decltype(plane_tag)::value;
        // ---- this thread's token of the tile: its slot is requested before anything waits
        if constexpr (kPlane == 0) {
            const TileId id = tile_of(p, item, 0);
            const uint32_t tok = id.tok_tile * kTileTokens + tid;
            head = id.head;
            tok_live = tok < num_tokens;
            slot = -1;   // a volatile load: it must not sink below the product's wait
            if (tok_live) asm volatile("ld.global.nc.s32 %0, [%1];\n" : "=r"(slot) : "l"(p.slots + tok));
        }

        product(false, true, buffer_of(kPlane));
        // the tile is consumed: with one buffer the item's value tile takes its place, with two
        // the next item's key tile does (the value tile stays for the transposed product)
        if constexpr (kPlane == 0) {
            if (C::kTileBufs == 1) load_tile(item, 1);
            else if (item + item_step < items) load_tile(item + item_step, 0);
        }

        // Where the strip goes is the same for both planes of an item: worked out in the key
        // plane (a bad strip is reported once), kept for the value plane.
        if constexpr (kPlane == 0) {
            const int32_t slot0 = __shfl_sync(0xffffffffu, slot, lane & 16);
            const bool run_ok = slot == slot0 + (lane & 15);
            const uint32_t votes = __ballot_sync(0xffffffffu, run_ok);
            const bool strip_live = __shfl_sync(0xffffffffu, tok_live ? 1 : 0, lane & 16) != 0;
            // page = slot0 / S by the precomputed multiplier: a hardware-free division costs this
            // thread hundreds of cycles per tile
            const uint32_t slot_page = fast_div(static_cast<uint32_t>(slot0), p.page_mul, p.page_shift);
            strip_ok = strip_live && ((votes >> (lane & 16)) & 0xFFFFu) == 0xFFFFu && slot0 >= 0 &&
                       (slot0 % kStrip) == 0 && slot_page < p.P;
            if (strip_live && !strip_ok && (lane & 15) == 0) report(p.status, TQ_STATUS_BAD_SLOT);
            page = strip_ok ? slot_page : 0u;
            tok_in_page = strip_ok ? static_cast<uint32_t>(slot0) - slot_page * p.S : 0u;
            // byte offset of the strip's (page, head) block in either code plane
            block_off = (static_cast<size_t>(page) * p.H + head) * (static_cast<size_t>(p.S) * 64u) +
                        static_cast<size_t>(tok_in_page / kStrip) * 1024u;
            // this thread's scale of the key plane; the value plane's lies P * H * S floats on
            scale_at = (static_cast<size_t>(page) * p.H + head) * p.S + tok_in_page + (lane & 15);
        }

        // ---- pass 1 over D[token][.]: absmax of the token, its power-of-two scale.
        // Tensor-memory reads run one 32-column chunk ahead of the arithmetic.
        uint32_t va[32], vb[32];
        float amax;
        if constexpr (BF16) {
            float hi0 = 0.0f, hi1 = 0.0f;
            auto fold = [&](const uint32_t (&v)[32]) {
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    hi0 = max3f(hi0, fabsf(__uint_as_float(v[j])), fabsf(__uint_as_float(v[j + 1])));
                    hi1 = max3f(hi1, fabsf(__uint_as_float(v[j + 2])), fabsf(__uint_as_float(v[j + 3])));
                }
            };
            tmem_ld32(acc + 0, va);
            tmem_arrived(va);
            tmem_ld32(acc + 32, vb);
            fold(va);
            tmem_arrived(vb);
            tmem_ld32(acc + 64, va);
            fold(vb);
            tmem_arrived(va);
            tmem_ld32(acc + 96, vb);
            fold(va);
            tmem_arrived(vb);
            if constexpr (kPlane == 0) tmem_ld32(acc + 0, va);   // first chunk of pass 2
            fold(vb);
            amax = fmaxf(hi0, hi1);
        } else {
            // the sums as signed 16-bit pairs, 64 columns per read: two-lane maximum and minimum
            uint32_t hi0 = 0x80008000u, hi1 = hi0, lo0 = 0x7FFF7FFFu, lo1 = lo0;
            auto fold = [&](const uint32_t (&v)[32]) {
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    hi0 = __vimax3_s16x2(hi0, v[j], v[j + 1]);
                    hi1 = __vimax3_s16x2(hi1, v[j + 2], v[j + 3]);
                    lo0 = __vimin3_s16x2(lo0, v[j], v[j + 1]);
                    lo1 = __vimin3_s16x2(lo1, v[j + 2], v[j + 3]);
                }
            };
            tmem_ld32_low16(acc + 0, va);
            tmem_arrived(va);
            tmem_ld32_low16(acc + 64, vb);
            fold(va);
            tmem_arrived(vb);
            if constexpr (kPlane == 0) tmem_ld32(acc + 0, va);   // first chunk of pass 2
            fold(vb);
            const uint32_t hi = __vmaxs2(hi0, hi1), lo = __vmins2(lo0, lo1);
            const int top = max(static_cast<int>(static_cast<int16_t>(hi & 0xFFFFu)),
                                static_cast<int>(static_cast<int16_t>(hi >> 16)));
            const int bottom = min(static_cast<int>(static_cast<int16_t>(lo & 0xFFFFu)),
                                   static_cast<int>(static_cast<int16_t>(lo >> 16)));
            amax = static_cast<float>(max(top, -bottom));
        }
        amax = fmaxf(amax, 1.0f);   // the writer floors absmax at 1
        const int pow_bits = (__float_as_int(amax) & 0x7F800000) - (2 << 23);
        const float inv = __int_as_float((254 << 23) - pow_bits);
        // rounding addend: r = y * inv + (1.5 * 2^23 + 8); an int8 accumulator carries the
        // extra 1.5 * 2^23, taken off again here (all terms are integers below 2^26: exact)
        const float addend = BF16 ? kMagic : kMagic - kBias * inv;
        if (strip_ok && healthy)
            p.scale_cache[scale_at + (kPlane ? plane_scales : 0)] = __int_as_float(pow_bits) * p.inv_sqrt_len;

        if constexpr (kPlane == 0) {
            // ---- key page: the token's row, 32 channels (16 bytes) per tensor-memory read
            uint4* dst = reinterpret_cast<uint4*>(p.key_cache + block_off + static_cast<size_t>(lane & 15) * 64u);
            const float2 inv2 = make_float2(inv, inv), add2 = make_float2(addend, addend);
            const bool store = strip_ok && healthy;
            auto emit = [&](const uint32_t (&v)[32], int c) {
                uint32_t w[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float r[8];
#pragma unroll
                    for (int e = 0; e < 8; e += 2) {
                        const float2 rr = __ffma2_rn(make_float2(__uint_as_float(v[j * 8 + e]),
                                                                 __uint_as_float(v[j * 8 + e + 1])),
                                                     inv2, add2);
                        r[e] = rr.x;
                        r[e + 1] = rr.y;
                    }
                    w[j] = pack8(r);
                }
                if (store) __stcs(dst + c, make_uint4(w[0], w[1], w[2], w[3]));
            };
            tmem_arrived(va);
            tmem_ld32(acc + 32, vb);
            biased(va);
            emit(va, 0);
            tmem_arrived(vb);
            tmem_ld32(acc + 64, va);
            biased(vb);
            emit(vb, 1);
            tmem_arrived(va);
            tmem_ld32(acc + 96, vb);
            biased(va);
            emit(va, 2);
            tmem_arrived(vb);
            biased(vb);
            emit(vb, 3);
        } else {
            // ---- value page: publish the per-token constants, swap the operands, then
            // work per channel
            inv_s[tid] = inv;
            if ((lane & 15) == 0)
                strip_off[tid >> 4] = strip_ok ? static_cast<unsigned long long>(block_off) : ~0ull;
            product(true, false, buffer_of(1));   // its barrier also publishes the constants and ends pass 1's reads
            if (item + item_step < items) load_tile(item + item_step, C::kTileBufs == 1 ? 0 : 1);
            const bool store = healthy;
            // 32 tokens = two strips per tensor-memory read, as many independent chains in
            // flight as in the key plane; a strip's constants (16 scales, its offset) are read
            // where they are used and the compiler moves the reads up as far as registers allow
            auto emit = [&](const uint32_t (&v)[32], int s0) {
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int s = s0 + half;
                    const unsigned long long off = strip_off[s];
                    uint32_t w[2];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const float4 i0 = *reinterpret_cast<const float4*>(inv_s + s * 16 + h * 8);
                        const float4 i1 = *reinterpret_cast<const float4*>(inv_s + s * 16 + h * 8 + 4);
                        const float iv[8] = {i0.x, i0.y, i0.z, i0.w, i1.x, i1.y, i1.z, i1.w};
                        float r[8];
#pragma unroll
                        for (int e = 0; e < 8; e += 2) {
                            // an int8 sum carries the float offset 1.5 * 2^23: taken off first
                            // (exact), so that the one rounding happens in the multiply-add as in the
                            // key plane
                            float2 y = make_float2(__uint_as_float(v[half * 16 + h * 8 + e]),
                                                   __uint_as_float(v[half * 16 + h * 8 + e + 1]));
                            if constexpr (!BF16) y = __fadd2_rn(y, make_float2(-kBias, -kBias));
                            const float2 rr = __ffma2_rn(y, make_float2(iv[e], iv[e + 1]), make_float2(kMagic, kMagic));
                            r[e] = rr.x;
                            r[e + 1] = rr.y;
                        }
                        w[h] = pack8(r);
                    }
                    if (store && off != ~0ull)
                        __stcs(reinterpret_cast<uint2*>(p.value_cache + off + static_cast<size_t>(tid) * 8u),
                               make_uint2(w[0], w[1]));
                }
            };
            tmem_ld32(acc + 0, va);
            tmem_arrived(va);
            tmem_ld32(acc + 32, vb);
            biased(va);
            emit(va, 0);
            tmem_arrived(vb);
            tmem_ld32(acc + 64, va);
            biased(vb);
            emit(vb, 2);
            tmem_arrived(va);
            tmem_ld32(acc + 96, vb);
            biased(va);
            emit(va, 4);
            tmem_arrived(vb);
            biased(vb);
            emit(vb, 6);
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
    // After a wait ran out (here or in the other group) a tile fetch or a product chain may
    // still be on its way into this CTA's shared and tensor memory: thread 0 gives each the
    // full budget to finish before the memory goes back to the SM.
    if (tid == 0) {
#pragma unroll
        for (uint32_t buf = 0; buf < C::kTileBufs; ++buf)
            if ((tma_pending >> buf) & 1u)
                bounded_wait(tma_bar_s + 8u * buf, (tma_parity >> buf) & 1u, kWaitBudget, false);
        if (mma_pending) bounded_wait(mbar_s, mma_pending_parity, kWaitBudget, false);
    }
    fence_before_sync();
    __syncthreads();
    if (threadIdx.x < 32)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
}

// The activation tensor [num_tokens][H * 128] as a 2-D map whose box is 128 rows of one
// 128-byte K block, stored with the 128-byte swizzle the MMA descriptors expect.
template <bool BF16>
bool activation_map(CUtensorMap* map, const void* base, uint32_t num_tokens, uint32_t H)
{
    const EncodeTiled fn = encode_tiled();
    if (fn == nullptr) return false;
    constexpr uint32_t elem = BF16 ? 2 : 1;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(H) * 128u, num_tokens};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(H) * 128u * elem};
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
        cudaError_t e = cudaFuncSetAttribute(tq_ingest_umma_kernel<BF16>,
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
    const uint32_t resident = static_cast<uint32_t>(sms) * C::kCtasPerSm;   // persistent: one resident wave
    const uint64_t wanted = (tiles + kGroups - 1) / kGroups;
    const uint32_t blocks = wanted < resident ? static_cast<uint32_t>(wanted) : resident;
    tq_ingest_umma_kernel<BF16><<<blocks, kThreads, C::kSmem, stream>>>(p, key_map, value_map);
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_ingest_umma(cudaStream_t stream, const IngestParams& p, bool bf16)
{
    return bf16 ? launch<true>(stream, p) : launch<false>(stream, p);
}

}  // namespace tq
