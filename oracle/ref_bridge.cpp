// Bridge to the reference project's own CPU golden models. TEST INFRASTRUCTURE ONLY.
//
// This translation unit contains no arithmetic of its own. It includes the
// reference's headers from where they lie in a checkout of
// fxslava/ascend-micro-harness (passed with -I at build time, see the Makefile
// beside this file) and re-exports a few of their entry points through a C ABI
// so that the restatement in tq_oracle.cpp, and through it the CUDA kernels,
// can be pinned against the reference's own code and fixtures:
//
//   tests/common/turboquant_oracle.hpp          aligned reshape_and_cache writer
//   tests/common/turboquant_scatter_oracle.hpp  1..16-token scatter writer
//   tests/common/aic_splitk_decode_fixture.hpp  split-K decode fixture + FP64 oracle
//   include/turboquant_splitk_contract.hpp      Partition, workspace ABI
//   include/routines/routine_vector_lloydmax_quantize.hpp  Lloyd-Max codebook
//   tests/common/fused_decode_opt_fixture.hpp   KV4/FP8 NZ-tiled cache fixture + FP64 oracle
//   tests/common/single_token_decode_oracle.hpp 6-row single-token decode fixture + golden model
//   include/turboquant_fused_decode_opt.hpp     Launch / Buffers layout (checked against include/tq_b200.h)
//
// The resulting library lives under oracle/_ref/ and is never linked into the
// product. ref_writer_reference is also the reference-compiled CPU leg the benchmark
// times for reshape_and_cache.

#include <tests/common/aic_splitk_decode_fixture.hpp>
#include <tests/common/turboquant_oracle.hpp>
#include <tests/common/turboquant_scatter_oracle.hpp>
#include <include/routines/routine_vector_lloydmax_quantize.hpp>
#include <include/sim_micro_testbed.hpp>
#include <tests/common/lloydmax_oracle.hpp>
#include <tests/cpu/icdf_fixture.hpp>
#include <tests/common/fused_decode_opt_fixture.hpp>
#include <tests/common/single_token_decode_oracle.hpp>

#define TQ_B200_NO_REFERENCE_LAUNCHERS
#include "../include/tq_b200.h"

#include <cstddef>
#include <cstdint>
#include <cstring>
#include <memory>
#include <thread>
#include <vector>

extern "C" {

// ------------------------------------------------------------ aligned writer
int ref_writer_pi_sign(int channel) { return tq_oracle::pi_sign(channel); }

void ref_writer_build_tables(int head_size, std::int8_t* out)
{
    tq_oracle::Shape s;
    s.head_size = head_size;
    const auto t = tq_oracle::build_tables(s);
    std::memcpy(out, t.data(), t.size());
}

// The reference fixture generator: activations (int8 [T][H*d]) and the
// fragmented strip -> page 2s+1 slot mapping.
void ref_writer_fixture(int num_tokens, int num_kv_heads, int head_size, int block_size,
                        std::int8_t* key, std::int8_t* value, std::int32_t* slots)
{
    tq_oracle::Shape s;
    s.num_tokens = num_tokens;
    s.num_kv_heads = num_kv_heads;
    s.head_size = head_size;
    s.block_size = block_size;
    s.num_blocks = tq_oracle::fragmented_num_blocks(num_tokens / block_size);
    std::vector<std::int8_t> k, v;
    tq_oracle::build_activations(s, k, v);
    std::memcpy(key, k.data(), k.size());
    std::memcpy(value, v.data(), v.size());
    const auto sl = tq_oracle::build_slot_mapping(s);
    std::memcpy(slots, sl.data(), sl.size() * sizeof(std::int32_t));
}

// compute_oracle_reference over caller activations. Cache images are written in
// full (pages no strip owns are zero); page_written gets one flag per page.
// Returns bad_slot_strip. `threads` > 1 splits the strips across host threads,
// each thread running the reference function on its own contiguous share.
int ref_writer_reference(int num_tokens, int num_kv_heads, int head_size, int block_size,
                         int num_blocks, const std::int8_t* key, const std::int8_t* value,
                         const std::int32_t* slots, std::int8_t* key_cache,
                         std::int8_t* value_cache, float* scale_cache, char* page_written,
                         int threads)
{
    const int strips = num_tokens / block_size;
    if (threads <= 1 || strips <= 1) {
        const auto ref = tq_oracle::compute_oracle_reference(
            num_tokens, num_kv_heads, head_size, block_size, num_blocks, key, value, slots);
        std::memcpy(key_cache, ref.key_cache.data(), ref.key_cache.size());
        std::memcpy(value_cache, ref.value_cache.data(), ref.value_cache.size());
        std::memcpy(scale_cache, ref.scale_cache.data(), ref.scale_cache.size() * sizeof(float));
        if (page_written) std::memcpy(page_written, ref.page_written.data(), ref.page_written.size());
        return ref.bad_slot_strip;
    }
    // One call per strip range; every call sees the whole cache geometry and
    // only its own tokens, so the merged images equal the single-call result.
    threads = std::min(threads, strips);
    std::vector<int> bad(threads, -1);
    std::vector<std::thread> pool;
    const std::size_t row = static_cast<std::size_t>(num_kv_heads) * head_size;
    tq_oracle::Shape shape;
    shape.num_tokens = num_tokens;
    shape.num_kv_heads = num_kv_heads;
    shape.head_size = head_size;
    shape.block_size = block_size;
    shape.num_blocks = num_blocks;
    std::memset(key_cache, 0, shape.cache_bytes());
    std::memset(value_cache, 0, shape.cache_bytes());
    std::memset(scale_cache, 0, shape.scale_floats() * sizeof(float));
    if (page_written) std::memset(page_written, 0, num_blocks);
    for (int t = 0; t < threads; ++t)
        pool.emplace_back([&, t]() {
            const int s0 = static_cast<int>(static_cast<long long>(strips) * t / threads);
            const int s1 = static_cast<int>(static_cast<long long>(strips) * (t + 1) / threads);
            if (s1 <= s0) return;
            const int tokens = (s1 - s0) * block_size;
            const auto ref = tq_oracle::compute_oracle_reference(
                tokens, num_kv_heads, head_size, block_size, num_blocks,
                key + static_cast<std::size_t>(s0) * block_size * row,
                value + static_cast<std::size_t>(s0) * block_size * row,
                slots + static_cast<std::size_t>(s0) * block_size);
            if (ref.bad_slot_strip >= 0) bad[t] = s0 + ref.bad_slot_strip;
            for (int page = 0; page < num_blocks; ++page) {
                if (!ref.page_written[page]) continue;
                const std::size_t off = ref.page_offset(page), n = shape.page_bytes();
                std::memcpy(key_cache + off, ref.key_cache.data() + off, n);
                std::memcpy(value_cache + off, ref.value_cache.data() + off, n);
                for (int plane = 0; plane < 2; ++plane) {
                    const std::size_t so = ref.scale_offset(plane, page, 0);
                    std::memcpy(scale_cache + so, ref.scale_cache.data() + so,
                                sizeof(float) * num_kv_heads * block_size);
                }
                if (page_written) page_written[page] = 1;
            }
        });
    for (auto& th : pool) th.join();
    for (int b : bad)
        if (b >= 0) return b;
    return -1;
}

// Audit of the reference fixture (tq_oracle::audit_reference): returns 1 when
// Audit::ok() holds for the fixture of this many tokens at the given geometry.
int ref_writer_fixture_audit_ok(int num_tokens, int num_kv_heads, int head_size, int block_size)
{
    tq_oracle::Shape s;
    s.num_tokens = num_tokens;
    s.num_kv_heads = num_kv_heads;
    s.head_size = head_size;
    s.block_size = block_size;
    s.num_blocks = tq_oracle::fragmented_num_blocks(num_tokens / block_size);
    std::vector<std::int8_t> k, v;
    tq_oracle::build_activations(s, k, v);
    const auto slots = tq_oracle::build_slot_mapping(s);
    const auto ref = tq_oracle::compute_oracle_reference(s, k.data(), v.data(), slots.data());
    return tq_oracle::audit_reference(ref).ok() ? 1 : 0;
}

// ------------------------------------------------------------ scatter writer
// The scatter oracle is hard-wired to head_size 256 (rot_oracle::kChannels).
// tokens = one per request; slot per token; activations from tq_scatter::activation.
// prior caches in, updated caches out (in place).
int ref_scatter_reference(int num_requests, int num_kv_heads, int block_size, int num_blocks,
                          const std::int32_t* slots, const std::int32_t* cu_seqlens,
                          int zero_token, std::int8_t* key_cache, std::int8_t* value_cache,
                          float* scale_cache, std::uint16_t* key_out, std::uint16_t* value_out)
{
    tq_scatter::Shape s;
    s.num_requests = num_requests;
    s.num_kv_heads = num_kv_heads;
    s.head_size = 256;
    s.block_size = block_size;
    s.num_blocks = num_blocks;
    if (!s.valid()) return -1;
    std::vector<tq_scatter::TokenPlan> plans;
    for (int r = 0; r < num_requests; ++r) {
        const int b = cu_seqlens ? cu_seqlens[r] : r, e = cu_seqlens ? cu_seqlens[r + 1] : r + 1;
        for (int t = b; t < e; ++t) plans.push_back(tq_scatter::plan_token(s, r, t, slots[t]));
    }
    const auto signs = rot_oracle::canonical_signs();
    std::vector<std::int8_t> pk(key_cache, key_cache + s.cache_bytes());
    std::vector<std::int8_t> pv(value_cache, value_cache + s.cache_bytes());
    std::vector<float> ps(scale_cache, scale_cache + s.scale_floats());
    const auto ref = tq_scatter::compute_reference(s, plans, signs, zero_token, pk, pv, ps);
    std::memcpy(key_cache, ref.key_cache.data(), ref.key_cache.size());
    std::memcpy(value_cache, ref.value_cache.data(), ref.value_cache.size());
    std::memcpy(scale_cache, ref.scale_cache.data(), ref.scale_cache.size() * sizeof(float));
    // The bf16 activation rows the device would read, [tokens][H*256].
    const std::size_t row = static_cast<std::size_t>(num_kv_heads) * 256;
    for (const auto& p : plans)
        for (int h = 0; h < num_kv_heads; ++h)
            for (int c = 0; c < 256; ++c) {
                const std::size_t at = static_cast<std::size_t>(p.token_index) * row + h * 256 + c;
                key_out[at] = tq_scatter::float_to_bf16_rne(
                    tq_scatter::activation(p.request, 0, h, p.token_index, c, zero_token));
                value_out[at] = tq_scatter::float_to_bf16_rne(
                    tq_scatter::activation(p.request, 1, h, p.token_index, c, zero_token));
            }
    return ref.zero_rows;
}

// -------------------------------------------------------------------- decode
struct RefDecodeFixture {
    std::unique_ptr<splitk_decode_test::Fixture> f;
    std::vector<std::uint16_t> raw_q;
};

// splitk_decode_test::Fixture(n, batch, heads, rows, page, live, fill); fill
// 0 = zero, 1 = dirty, 2 = NaN canary. rows must be 16 for the AIC helpers.
void* ref_decode_fixture_new(int n, int batch, int heads, int rows, int page_tokens, int live,
                             int fill)
{
    auto* h = new RefDecodeFixture;
    h->f.reset(new splitk_decode_test::Fixture(
        n, batch, heads, rows, page_tokens, live,
        static_cast<splitk_decode_test::TailFill>(fill)));
    if (rows == splitk_decode_test::kAicRows) h->raw_q = splitk_decode_test::AicRawQuery(*h->f);
    return h;
}
void ref_decode_fixture_free(void* p) { delete static_cast<RefDecodeFixture*>(p); }

// dims: tokens, seq_len, pages, requests, heads, rows, page_tokens
void ref_decode_fixture_dims(void* p, int* dims)
{
    const auto& f = *static_cast<RefDecodeFixture*>(p)->f;
    const int v[7] = {f.tokens, f.seq_len, f.pages, f.requests, f.heads, f.rows, f.page_tokens};
    std::memcpy(dims, v, sizeof v);
}
// which: 0 q_rot(bf16) 1 key 2 value 3 scales 4 gate 5 signs 6 table 7 expected 8 raw_q(bf16)
std::size_t ref_decode_fixture_get(void* p, int which, void* out)
{
    auto* h = static_cast<RefDecodeFixture*>(p);
    const auto& f = *h->f;
    const void* src = nullptr;
    std::size_t n = 0;
    switch (which) {
    case 0: src = f.q.data(); n = f.q.size() * 2; break;
    case 1: src = f.key.data(); n = f.key.size(); break;
    case 2: src = f.value.data(); n = f.value.size(); break;
    case 3: src = f.scales.data(); n = f.scales.size() * 4; break;
    case 4: src = f.gate.data(); n = f.gate.size() * 4; break;
    case 5: src = f.signs.data(); n = f.signs.size() * 4; break;
    case 6: src = f.table.data(); n = f.table.size() * 4; break;
    case 7: src = f.expected.data(); n = f.expected.size() * 4; break;
    case 8: src = h->raw_q.data(); n = h->raw_q.size() * 2; break;
    default: return 0;
    }
    if (out) std::memcpy(out, src, n);
    return n;
}
// ReferenceAicPartial over logical pages [begin, begin+pages): m[16], l[16], acc[16*256].
void ref_decode_aic_partial(void* p, int request, int head, unsigned begin, unsigned pages,
                            double* m, double* l, double* acc)
{
    const auto& f = *static_cast<RefDecodeFixture*>(p)->f;
    const auto r = splitk_decode_test::ReferenceAicPartial(f, request, head, begin, pages);
    std::memcpy(m, r.m.data(), r.m.size() * 8);
    std::memcpy(l, r.l.data(), r.l.size() * 8);
    std::memcpy(acc, r.acc.data(), r.acc.size() * 8);
}
// The 16 resident bf16 rotation blocks the AIC decoder is handed (row-major).
void ref_decode_rotation_table(std::uint16_t* out)
{
    const auto t = paged_decode::BuildRotationTable();
    std::memcpy(out, t.row_major.data(), t.row_major.size() * 2);
}
int ref_decode_pi_sign(int channel) { return paged_decode::PiSign(channel); }

void ref_partition(unsigned pages, unsigned splits, unsigned split, unsigned* begin,
                   unsigned* count)
{
    const auto r = turboquant_splitk::Partition(pages, splits, split);
    *begin = r.begin;
    *count = r.count;
}
unsigned long long ref_workspace_floats(unsigned requests, unsigned heads, unsigned splits)
{
    return turboquant_splitk::WorkspaceFloats(requests, heads, splits);
}

// ----------------------------------------------------------------- Lloyd-Max
void ref_lloydmax4_tables(float* centroids16, float* thresholds15)
{
    std::memcpy(centroids16, ascend_micro::LloydMaxCodebook<4>::centroids, 16 * 4);
    std::memcpy(thresholds15, ascend_micro::LloydMaxCodebook<4>::thresholds, 15 * 4);
}
unsigned ref_lloydmax4_code(float x) { return ascend_micro::lloydmax_code<4>(x); }
// the reference's probe fixture (normalised Hadamard of Box-Muller normals, optional
// threshold-boundary probes) and its packing
void ref_lloydmax_fixture(unsigned n, unsigned rows, int boundaries, float* out)
{
    const auto x = lloyd::fixture(n, rows, boundaries != 0, 4);
    std::memcpy(out, x.data(), x.size() * sizeof(float));
}
void ref_lloydmax4_pack(const float* x, unsigned n, std::uint8_t* out)
{
    std::vector<unsigned> q(n);
    for (unsigned i = 0; i < n; ++i) q[i] = ascend_micro::lloydmax_code<4>(x[i]);
    const auto bytes = lloyd::pack(q, 4);
    std::memcpy(out, bytes.data(), bytes.size());
}

// ------------------------------------------------------------------ ICDF int4
// The probe fixture (tests/cpu/icdf_fixture.hpp:178-245): `tiles` tiles of 1024 FP16/BF16
// inputs and the 512 packed oracle bytes of each.
void ref_icdf_fixture(int bf16, unsigned tiles, std::uint16_t* in_bits, std::uint8_t* packed)
{
    const auto fx = icdf::make_fixture(bf16 != 0, tiles);
    std::memcpy(in_bits, fx.in_bits.data(), fx.in_bits.size() * 2);
    std::memcpy(packed, fx.oracle_packed.data(), fx.oracle_packed.size());
}

// ---------------------------------------------------------------- Hadamard 16
void ref_hadamard16(const std::uint16_t* x_f16, float* y)
{
    const auto r = ascend_micro::sim::golden_hadamard16(x_f16);
    std::memcpy(y, r.data(), 256 * sizeof(float));
}

// ------------------------------------------- fused decoder: KV4/FP8 NZ-tiled cache
// fused_decode_opt_test::Fixture(context, requests, kv_heads, group_heads, page_tokens)
// (tests/common/fused_decode_opt_fixture.hpp:247-318). Head size 256.
void* ref_fused_fixture_new(int context, int requests, int kv_heads, int group_heads, int page_tokens)
{
    return new fused_decode_opt_test::Fixture(context, requests, kv_heads, group_heads, page_tokens);
}
void ref_fused_fixture_free(void* p) { delete static_cast<fused_decode_opt_test::Fixture*>(p); }
// dims: pages per request, physical pages
void ref_fused_fixture_dims(void* p, int* dims)
{
    const auto& f = *static_cast<fused_decode_opt_test::Fixture*>(p);
    dims[0] = f.pages;
    dims[1] = f.physical_pages;
}
// which: 0 query (f32, pre-rotated) 1 key 2 value 3 scales 4 table 5 lengths 6 expected
std::size_t ref_fused_fixture_get(void* p, int which, void* out)
{
    const auto& f = *static_cast<fused_decode_opt_test::Fixture*>(p);
    const void* src = nullptr;
    std::size_t n = 0;
    switch (which) {
    case 0: src = f.query.data(); n = f.query.size() * 4; break;
    case 1: src = f.key.data(); n = f.key.size(); break;
    case 2: src = f.value.data(); n = f.value.size(); break;
    case 3: src = f.scales.data(); n = f.scales.size() * 4; break;
    case 4: src = f.table.data(); n = f.table.size() * 4; break;
    case 5: src = f.lengths.data(); n = f.lengths.size() * 4; break;
    case 6: src = f.expected.data(); n = f.expected.size() * 4; break;
    default: return 0;
    }
    if (out) std::memcpy(out, src, n);
    return n;
}
// The fused decoder's Pi = diag(s) H diag(s) / sqrt(D) (fixture :104-186), its sign vector, the
// expected output row under an output stage and the fixture's gate logits (FP16 bits).
float ref_fused_sign(int channel) { return fused_decode_opt_test::RawQueryBasis::sign_at(channel); }
void ref_fused_pi_apply(const float* x, float* y)
{
    const fused_decode_opt_test::RawQueryBasis basis;
    const auto r = basis.apply(x);
    std::memcpy(y, r.data(), r.size() * sizeof(float));
}
void ref_fused_expected_row(void* p, std::size_t row, unsigned stage, float* out)
{
    const auto& f = *static_cast<fused_decode_opt_test::Fixture*>(p);
    const fused_decode_opt_test::RawQueryBasis basis;
    const auto r = f.expected_row(basis, row, stage);
    std::memcpy(out, r.data(), r.size() * sizeof(float));
}
void ref_fused_raw_query_bits(void* p, std::uint16_t* out)
{
    const auto& f = *static_cast<fused_decode_opt_test::Fixture*>(p);
    const fused_decode_opt_test::RawQueryBasis basis;
    const auto q = f.raw_query(basis);
    std::memcpy(out, q.data(), q.size() * 2);
}
void ref_fused_gate_bits(void* p, std::uint16_t* out)
{
    const auto& f = *static_cast<fused_decode_opt_test::Fixture*>(p);
    const auto g = f.gate_logits();
    std::memcpy(out, g.data(), g.size() * 2);
}
// The e4m3-rounded Lloyd-Max codebook the fused decoder's KV4/FP8 mode can be switched to
// (turboquant_mode.h:181-206): levels by bin index, the midpoint thresholds, the gain (1).
void ref_kv4_lloydmax_lut(float* levels16, float* thresholds15, float* gain)
{
    using T = vllm_ascend::turboquant::TurboQuantLloydMaxTraits<vllm_ascend::turboquant::TurboQuantMode::KV4_FP8>;
    for (int i = 0; i < T::kLevels; ++i) levels16[i] = T::kCentroids[i];
    for (int i = 0; i < T::kThresholdCount; ++i) thresholds15[i] = T::kThresholds[i];
    *gain = T::kGain;
}
float ref_kv4_gain() { return vllm_ascend::turboquant::TurboQuantModeTraits<vllm_ascend::turboquant::TurboQuantMode::KV4_FP8>::kGain; }
std::uint64_t ref_nz_tiled_packed_byte(std::uint64_t slot, std::uint64_t head, std::uint64_t column,
                                       std::uint64_t H, std::uint64_t packed)
{
    return vllm_ascend::turboquant::NzTiledPackedByte(slot, head, column, H, packed);
}


// ------------------------------------------------- single-token decode fixture
// tests/common/single_token_decode_oracle.hpp: one request, 4 KV heads x 6 query rows, head
// size 256, pages of 128 tokens, `pages` <= 8 logical pages through the reference's block
// table. The caller pre-fills the caches (canaries); only mapped strips are written.
//   q_raw  bf16 [4][6][256], the original-basis query rows (exact small integers)
//   key, value  9 * 4 * 8 * 2048 bytes each; scales float[2 * 9 * 4 * 128]; table int32[pages]
void ref_single_token_fixture(int pages, std::uint16_t* q_raw, std::uint8_t* key, std::uint8_t* value,
                              float* scales, std::int32_t* table)
{
    namespace st = single_token_decode;
    namespace pd = paged_decode;
    for (int head = 0; head < st::kKvHeads; ++head)
        for (int row = 0; row < st::kRows; ++row)
            for (int c = 0; c < st::kHeadSize; ++c)
                q_raw[(head * st::kRows + row) * st::kHeadSize + c] = ascend_micro::sim::float_to_bfloat16_rne(
                    pd::QueryEntry(st::QueryRowOf(head, row), c));
    for (int page = 0; page < pages; ++page) {
        const int block = pd::BlockTableEntry(page);
        table[page] = block;
        for (int head = 0; head < st::kKvHeads; ++head)
            for (int strip = 0; strip < st::kStripsPerPage; ++strip) {
                const int global = page * st::kStripsPerPage + strip;
                std::uint8_t* ks = key + pd::KeyStripOffset(block, head, strip);
                std::uint8_t* vs = value + pd::ValueStripOffset(block, head, strip);
                for (int t = 0; t < st::kKeys; ++t)
                    for (int c = 0; c < st::kHeadSize; ++c) {
                        pd::PackNibble(ks, pd::KeyNibbleIndex(t, c), st::KeyNibbleAt(head, global, t, c));
                        pd::PackNibble(vs, pd::ValueNibbleIndex(c, t), st::ValueNibbleAt(head, global, c, t));
                    }
                for (int t = 0; t < st::kKeys; ++t) {
                    const int in_page = strip * st::kKeys + t;
                    scales[pd::ScaleOffset(0, block, head, in_page)] = st::KeyScale(head, global, t);
                    scales[pd::ScaleOffset(1, block, head, in_page)] = st::ValueScaleAt(head, global, t);
                }
            }
    }
}
// GoldenDecode of one head over the first `pages` pages: m[6], l[6], acc / rotated / context [6][256],
// q_rot[6][256] (the bf16 image of the rotated query, as floats).
void ref_single_token_golden(int head, int pages, float* m, float* l, float* acc, float* rotated,
                             float* context, float* q_rot)
{
    namespace st = single_token_decode;
    std::vector<int> strips;
    for (int g = 0; g < pages * st::kStripsPerPage; ++g) strips.push_back(g);
    const auto gs = st::GoldenDecode(head, strips);
    std::memcpy(m, gs.m.data(), gs.m.size() * 4);
    std::memcpy(l, gs.l.data(), gs.l.size() * 4);
    std::memcpy(acc, gs.acc.data(), gs.acc.size() * 4);
    std::memcpy(rotated, gs.rotated.data(), gs.rotated.size() * 4);
    std::memcpy(context, gs.context.data(), gs.context.size() * 4);
    for (int row = 0; row < st::kRows; ++row)
        for (int c = 0; c < st::kHeadSize; ++c) q_rot[row * st::kHeadSize + c] = st::QRotEntry(head, row, c);
}
// gate logits of the fixture, [4][6][256]
void ref_single_token_gate(float* gate)
{
    namespace st = single_token_decode;
    for (int head = 0; head < st::kKvHeads; ++head)
        for (int row = 0; row < st::kRows; ++row)
            for (int c = 0; c < st::kHeadSize; ++c)
                gate[(head * st::kRows + row) * st::kHeadSize + c] =
                    paged_decode::GateEntry(head, st::QueryRowOf(head, row), c);
}

// ------------------------------------------- layout of the fused decoder's descriptors
// 1 when tq_fused_launch / tq_fused_buffers / tq_fused_raw_query_buffers of include/tq_b200.h
// have the size and field offsets of the reference's Launch / Buffers / RawQueryBuffers.
int ref_fused_descriptor_layout_matches()
{
    namespace fd = ascend_micro::fused_decode_opt;
#define TQ_SAME(T, U, f) (offsetof(T, f) == offsetof(U, f))
    static_assert(sizeof(tq_fused_launch) == sizeof(fd::Launch), "Launch size");
    static_assert(sizeof(tq_fused_buffers) == sizeof(fd::Buffers), "Buffers size");
    static_assert(sizeof(tq_fused_raw_query_buffers) == sizeof(fd::RawQueryBuffers), "RawQueryBuffers size");
    static_assert(TQ_SAME(tq_fused_launch, fd::Launch, grid) && TQ_SAME(tq_fused_launch, fd::Launch, tokens) &&
                  TQ_SAME(tq_fused_launch, fd::Launch, heads) && TQ_SAME(tq_fused_launch, fd::Launch, kv_heads) &&
                  TQ_SAME(tq_fused_launch, fd::Launch, head_size) && TQ_SAME(tq_fused_launch, fd::Launch, block_size) &&
                  TQ_SAME(tq_fused_launch, fd::Launch, max_blocks) && TQ_SAME(tq_fused_launch, fd::Launch, splits) &&
                  TQ_SAME(tq_fused_launch, fd::Launch, heads_per_task) &&
                  TQ_SAME(tq_fused_launch, fd::Launch, tasks_per_block) &&
                  TQ_SAME(tq_fused_launch, fd::Launch, reduce_tasks_per_block) &&
                  TQ_SAME(tq_fused_launch, fd::Launch, fused_context_limit) && TQ_SAME(tq_fused_launch, fd::Launch, scale) &&
                  TQ_SAME(tq_fused_launch, fd::Launch, inv_sqrt_len) &&
                  TQ_SAME(tq_fused_launch, fd::Launch, prologue_vectors_per_block) &&
                  TQ_SAME(tq_fused_launch, fd::Launch, prologue_cube_chunk_vectors) &&
                  TQ_SAME(tq_fused_launch, fd::Launch, output_stage) && TQ_SAME(tq_fused_launch, fd::Launch, element_type) &&
                  TQ_SAME(tq_fused_launch, fd::Launch, probe_page) && TQ_SAME(tq_fused_launch, fd::Launch, probe_tile),
                  "Launch fields");
    static_assert(TQ_SAME(tq_fused_buffers, fd::Buffers, query) && TQ_SAME(tq_fused_buffers, fd::Buffers, key) &&
                  TQ_SAME(tq_fused_buffers, fd::Buffers, value) && TQ_SAME(tq_fused_buffers, fd::Buffers, scales) &&
                  TQ_SAME(tq_fused_buffers, fd::Buffers, block_table) &&
                  TQ_SAME(tq_fused_buffers, fd::Buffers, context_lengths) &&
                  TQ_SAME(tq_fused_buffers, fd::Buffers, mode_tables) && TQ_SAME(tq_fused_buffers, fd::Buffers, workspace) &&
                  TQ_SAME(tq_fused_buffers, fd::Buffers, output) && TQ_SAME(tq_fused_buffers, fd::Buffers, tiling),
                  "Buffers fields");
    static_assert(TQ_SAME(tq_fused_raw_query_buffers, fd::RawQueryBuffers, raw_query) &&
                  TQ_SAME(tq_fused_raw_query_buffers, fd::RawQueryBuffers, pi_signs) &&
                  TQ_SAME(tq_fused_raw_query_buffers, fd::RawQueryBuffers, rot_tables) &&
                  TQ_SAME(tq_fused_raw_query_buffers, fd::RawQueryBuffers, h16) &&
                  TQ_SAME(tq_fused_raw_query_buffers, fd::RawQueryBuffers, gate) &&
                  TQ_SAME(tq_fused_raw_query_buffers, fd::RawQueryBuffers, decode),
                  "RawQueryBuffers fields");
#undef TQ_SAME
    return 1;
}

}  // extern "C"
