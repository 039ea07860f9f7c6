// tcgen05 / tensor-memory / TMA primitives shared by the two tensor-core writers
// (tq_ingest_umma.cu: head size 128, tq_ingest_umma256.cu: head size 256).
#pragma once

#include <cuda.h>   // CUtensorMap and the encode entry point's signature; nothing is linked from libcuda

#include "tq_ingest.cuh"

namespace tq {
namespace {

constexpr long long kWaitBudget = kIngestWaitBudget;   // clock cycles, about a second
constexpr uint32_t kSuspendHintNs = 20000u;       // one poll may sleep this long before it returns

constexpr float kBias = 12582912.0f;         // 1.5 * 2^23
constexpr uint32_t kBiasBits = 0x4B400000u;
constexpr float kMagic = 12582920.0f;        // 1.5 * 2^23 + 8

// Instruction descriptor of a 128 x 128 product: D format (1 = F32, 2 = S32) at bit 4, A and B
// format (kind::f16: 1 = BF16; kind::i8: 1 = INT8) at bits 7 and 10, both operands K-major,
// N / 8 at bit 17, M / 16 at bit 24
template <bool BF16>
constexpr uint32_t kIdesc128 = ((BF16 ? 1u : 2u) << 4) | (1u << 7) | (1u << 10) | ((128u >> 3) << 17) |
                               ((128u >> 4) << 24);

__device__ __forceinline__ uint32_t smem_addr(const void* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// Shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr)
{
    return static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) |
           (1ull << 46) | (2ull << 61);
}

template <bool BF16>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                     uint32_t accumulate)
{
    const uint32_t z = 0;
    if constexpr (BF16)
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}\n"
            ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(kIdesc128<BF16>), "r"(accumulate),
              "r"(z), "r"(z), "r"(z), "r"(z) : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}\n"
            ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(kIdesc128<BF16>), "r"(accumulate),
              "r"(z), "r"(z), "r"(z), "r"(z) : "memory");
}

__device__ __forceinline__ void umma_commit(uint32_t mbar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n"
                 ::"r"(mbar) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t mbar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(ok) : "r"(mbar), "r"(parity), "r"(kSuspendHintNs) : "memory");
    return ok != 0;
}

// A wait on a barrier phase for at most `budget` clock cycles; a budget of zero gives up
// without looking, and a raised abort flag (when one is watched) ends the wait early: the awaited
// work may then never have been issued. (Out of line it cost 4 %: the calls sit in the hot loop.)
__device__ __forceinline__ bool bounded_mbar_wait(uint32_t bar, uint32_t par, long long budget,
                                               const volatile uint32_t* abort_flag)
{
    if (budget <= 0) return false;
    bool done = mbar_try_wait(bar, par);
    if (!done) {
        const long long t0 = clock64();
        do {
            done = mbar_try_wait(bar, par);
        } while (!done && clock64() - t0 < budget && !(abort_flag != nullptr && *abort_flag != 0u));
    }
    return done;
}

#define TQ_W8(v, o) "=r"(v[o]), "=r"(v[o + 1]), "=r"(v[o + 2]), "=r"(v[o + 3]), "=r"(v[o + 4]), \
                    "=r"(v[o + 5]), "=r"(v[o + 6]), "=r"(v[o + 7])
#define TQ_RW8(v, o) "+r"(v[o]), "+r"(v[o + 1]), "+r"(v[o + 2]), "+r"(v[o + 3]), "+r"(v[o + 4]), \
                     "+r"(v[o + 5]), "+r"(v[o + 6]), "+r"(v[o + 7])

// 32 lanes x 32 columns: lane i of the warp receives columns col .. of its row. The
// load is asynchronous; tmem_arrived() is the wait, and it names the registers as in-out
// operands so that no use of them can be scheduled ahead of it.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : TQ_W8(v, 0), TQ_W8(v, 8), TQ_W8(v, 16), TQ_W8(v, 24)
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_arrived(uint32_t (&v)[32])
{
    asm volatile("tcgen05.wait::ld.sync.aligned;\n"
                 : TQ_RW8(v, 0), TQ_RW8(v, 8), TQ_RW8(v, 16), TQ_RW8(v, 24)
                 :: "memory");
}
// 32 lanes x 64 columns, the low 16 bits of each: register j holds columns 2j (low half) and
// 2j + 1 (high half). An INT32 accumulator on top of 1.5 * 2^23 keeps the sum itself, as a
// signed 16-bit number, in its low half (|sum| <= 128 * 128).
__device__ __forceinline__ void tmem_ld32_low16(uint32_t taddr, uint32_t (&v)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.pack::16b.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : TQ_W8(v, 0), TQ_W8(v, 8), TQ_W8(v, 16), TQ_W8(v, 24)
        : "r"(taddr) : "memory");
}
#undef TQ_W8
#undef TQ_RW8
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

// The same 32-bit value into 32 columns of every lane of the warp's quarter.
__device__ __forceinline__ void tmem_fill32(uint32_t taddr, uint32_t x)
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, "
        "%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1};\n"
        ::"r"(taddr), "r"(x) : "memory");
}

__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

// One 2-D box of the activation tensor into shared memory; completion is counted in bytes
// on `mbar`. No multicast: the box goes to this CTA only.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t mbar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(mbar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t mbar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(mbar), "r"(bytes) : "memory");
}

// Three-input maximum.
__device__ __forceinline__ float max3f(float a, float b, float c)
{
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
// cuTensorMapEncodeTiled through the runtime's entry-point lookup (no link against libcuda).
using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                 CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                 CUtensorMapFloatOOBfill);
EncodeTiled encode_tiled()
{
    static EncodeTiled fn = [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            ptr = nullptr;
        return reinterpret_cast<EncodeTiled>(ptr);
    }();
    return fn;
}

}  // namespace
}  // namespace tq
