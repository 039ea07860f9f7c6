// The reference project's launcher symbols, forwarding to the engine's tq_*
// entry points. Same names, same argument order, same error behaviour: a
// refused geometry throws std::invalid_argument out of the extern "C" function
// exactly as the AscendC launchers do, so the reference's C++ harnesses
// (tests/npu/turboquant_npu_common.hpp, tests/npu/turboquant_splitk_rigs.hpp)
// behave identically when linked against this library.
#include <cstdint>
#include <stdexcept>
#include <string>

#include "../../include/tq_b200.h"

namespace {
void throw_on(int status, const char* who)
{
    if (status == TQ_OK) return;
    if (status == TQ_ERR_PARTIAL_STRIP)
        throw std::invalid_argument(std::string(who) +
                                    ": numTokens must be a whole number of tokensPerCore strips; "
                                    "a partial trailing strip would be dropped");
    if (status == TQ_ERR_INVALID_ARGUMENT)
        throw std::invalid_argument(std::string(who) + ": " + tq_status_string(status));
    throw std::runtime_error(std::string(who) + ": " + tq_status_string(status));
}
}  // namespace

extern "C" const char* tq_version(void) { return "tq_b200 0.1 (sm_100a)"; }

extern "C" const char* tq_status_string(int status)
{
    switch (status) {
    case TQ_OK: return "ok";
    case TQ_ERR_INVALID_ARGUMENT: return "invalid geometry or null operand";
    case TQ_ERR_PARTIAL_STRIP: return "num_tokens is not a whole number of 16-token strips";
    case TQ_ERR_LAUNCH: return "the CUDA runtime refused the launch";
    case TQ_ERR_NO_DEVICE: return "no usable CUDA device";
    case TQ_ERR_WORKSPACE_TOO_SMALL:
        return "the launch needs more split-K workspace than the built-in array holds";
    default: return "unknown status";
    }
}

// pi_signs is unread by the aligned writers of the reference as well: the sign
// diagonal reaches them folded into `tables`
// (kernels/ops/turboquant/turboquant_reshape_and_cache_a8.cpp:1470-1475).
// reuse_mode4_flags selects between two Ascend cross-core flag policies and has
// no meaning here. tokens_per_core must be the 16-token strip.
extern "C" void launch_turboquant_reshape_and_cache_a8(
    void* stream, const int8_t* key, const int8_t* value, int8_t* key_cache, int8_t* value_cache,
    float* scale_cache, const int32_t* slot_mapping, const float* /*pi_signs*/,
    const int32_t* tables, uint32_t num_tokens, uint32_t num_kv_heads, uint32_t head_size,
    uint32_t block_size, uint32_t num_blocks, uint32_t tokens_per_core, float inv_sqrt_len,
    bool /*reuse_mode4_flags*/)
{
    if (tokens_per_core == 0 || num_tokens % tokens_per_core != 0)
        throw_on(TQ_ERR_PARTIAL_STRIP, "reshape_and_cache_a8");
    if (tokens_per_core % 16 != 0) throw_on(TQ_ERR_INVALID_ARGUMENT, "reshape_and_cache_a8");
    throw_on(tq_reshape_and_cache(stream, key, value, key_cache, value_cache, scale_cache,
                                  slot_mapping, tables, TQ_SIGNS_TABLES_I8, TQ_IN_INT8, num_tokens,
                                  num_kv_heads, head_size, block_size, num_blocks, inv_sqrt_len,
                                  nullptr),
             "reshape_and_cache_a8");
}

extern "C" void launch_turboquant_reshape_and_cache_bf16(
    void* stream, const uint16_t* key, const uint16_t* value, int8_t* key_cache,
    int8_t* value_cache, float* scale_cache, const int32_t* slot_mapping,
    const float* /*pi_signs*/, const int32_t* tables, uint32_t num_tokens, uint32_t num_kv_heads,
    uint32_t head_size, uint32_t block_size, uint32_t num_blocks, uint32_t tokens_per_core,
    float inv_sqrt_len, bool reuse_mode4_flags)
{
    if (tokens_per_core == 0 || num_tokens % tokens_per_core != 0)
        throw_on(TQ_ERR_PARTIAL_STRIP, "reshape_and_cache_bf16");
    // The reference's fallback entry point runs one strip per block and refuses
    // anything else (turboquant_reshape_and_cache_bf16.cpp:2034-2039).
    if (!reuse_mode4_flags && tokens_per_core != block_size)
        throw std::invalid_argument(
            "reshape_and_cache_bf16: the mode-4 single-shot fallback runs one strip per block; "
            "tokensPerCore must equal blockSize for it");
    if (tokens_per_core % 16 != 0) throw_on(TQ_ERR_INVALID_ARGUMENT, "reshape_and_cache_bf16");
    throw_on(tq_reshape_and_cache(stream, key, value, key_cache, value_cache, scale_cache,
                                  slot_mapping, tables, TQ_SIGNS_TABLES_BF16, TQ_IN_BF16,
                                  num_tokens, num_kv_heads, head_size, block_size, num_blocks,
                                  inv_sqrt_len, nullptr),
             "reshape_and_cache_bf16");
}

// ------------------------------------------------------------- fused decoder entries
// launch_fused_decode_opt / launch_fused_decode_opt_raw_query of the reference
// (include/turboquant_fused_decode_opt.hpp:172-180; the AscendC launchers are
// kernels/ops/turboquant/vllm_integration_layer/op_kernel/turboquant_fused_decode.cpp:1193-1307).
// The cache is the fused decoder's own KV4 format (NZ-tiled packed planes, per-slot scale
// records) and is read where it lies. tq_fused_launch / tq_fused_buffers /
// tq_fused_raw_query_buffers mirror the reference's Launch / Buffers / RawQueryBuffers field
// for field. What has no meaning off the Ascend part is accepted and ignored -- grid,
// heads_per_task, tasks_per_block, reduce_tasks_per_block, fused_context_limit,
// prologue_* (sizes of per-core work shares), mode_tables, rot_tables, h16 (constant pools of
// the vector and Cube services), the contents of the tiling descriptors -- but the refusals
// stay: a null descriptor, a null tiling buffer, an unknown element type, a geometry
// valid_launch rejects or an output stage above 2 throw std::invalid_argument.
namespace {
// include/turboquant_fused_decode_opt.hpp:76-105, restated
bool fused_valid_launch(uint32_t grid, uint32_t tokens, uint32_t heads, uint32_t kv_heads, uint32_t dim,
                        uint32_t block_size, uint32_t max_blocks, uint32_t splits, uint32_t heads_per_task,
                        uint32_t tasks_per_block, uint32_t reduce_tasks_per_block)
{
    if (!grid || grid > 32 || !tokens || !kv_heads || kv_heads > 4 || !heads || heads % kv_heads ||
        dim != 256 || !block_size || block_size % 64 || !max_blocks || !splits || splits > 8 ||
        !heads_per_task || heads_per_task > 16 || !tasks_per_block || !reduce_tasks_per_block)
        return false;
    if (block_size & (block_size - 1)) return false;
    const uint32_t group = heads / kv_heads;
    const uint32_t chunk = heads_per_task < group ? heads_per_task : group;
    const uint64_t tasks = uint64_t{tokens} * kv_heads * splits * ((uint64_t{group} + chunk - 1) / chunk);
    return tasks <= UINT32_MAX && uint64_t{grid} * tasks_per_block >= tasks &&
           uint64_t{tokens} * heads <= UINT32_MAX && uint64_t{grid} * tasks_per_block <= UINT32_MAX &&
           uint64_t{grid} * reduce_tasks_per_block <= UINT32_MAX &&
           uint64_t{grid} * reduce_tasks_per_block >= uint64_t{tokens} * heads;
}

// TurboQuantModeTraits<KV4_FP8>::kGain (fused_decode/common/turboquant_mode.h:113)
constexpr float kKv4Gain = 2.9832882881f;

uint32_t fused_elem(uint32_t element_type)
{
    // AscendType: 0 = FP16, 1 = BF16 (include/turboquant_fused_decode_opt.hpp:134-142)
    if (element_type == 0u) return TQ_DTYPE_F16;
    if (element_type == 1u) return TQ_DTYPE_BF16;
    throw std::invalid_argument("fused decode launch with no kernel instance for its element type");
}

void fused_decode(void* stream, const tq_fused_launch* c, const tq_fused_buffers* b, const float* pi_signs,
                  const void* gate, uint32_t output_stage, const char* who)
{
    if (!b->tiling) throw std::invalid_argument("fused decode launch without host tiling descriptors");
    if (!fused_valid_launch(c->grid, c->tokens, c->heads, c->kv_heads, c->head_size, c->block_size,
                            c->max_blocks, c->splits, c->heads_per_task, c->tasks_per_block,
                            c->reduce_tasks_per_block))
        throw std::invalid_argument("unsupported fused decode geometry or incomplete task coverage");
    const uint32_t elem = fused_elem(c->element_type);
    // The partial records take requests * heads * splits * (256 + 16) floats of the workspace,
    // the layout the reference's rig sizes it for; the split count is the caller's, so the
    // classic grid and the combine kernel serve the call. The wider arithmetic keeps the
    // output within the reference rig's 1-ULP budget.
    throw_on(tq_decode_splitk_nz(stream, static_cast<const float*>(b->query),
                                 static_cast<const uint8_t*>(b->key), static_cast<const uint8_t*>(b->value),
                                 static_cast<const float*>(b->scales),
                                 static_cast<const int32_t*>(b->block_table),
                                 static_cast<const int32_t*>(b->context_lengths), pi_signs, gate,
                                 static_cast<float*>(b->workspace), b->output, elem, elem, c->tokens, c->heads,
                                 c->kv_heads, c->block_size, 0u, c->max_blocks, c->splits, 0u, 1u, output_stage,
                                 kKv4Gain, c->inv_sqrt_len, c->scale, 1u, nullptr),
             who);
}
}  // namespace

extern "C" void launch_fused_decode_opt(void* stream, const tq_fused_launch* launch,
                                        const tq_fused_buffers* buffers)
{
    if (!launch || !buffers) throw std::invalid_argument("null fused decode launch descriptor");
    fused_elem(launch->element_type);
    fused_decode(stream, launch, buffers, nullptr, nullptr, TQ_OUT_ROTATED, "fused_decode_opt");
}

extern "C" void launch_fused_decode_opt_raw_query(void* stream, const tq_fused_launch* launch,
                                                  const tq_fused_raw_query_buffers* buffers)
{
    if (!launch || !buffers) throw std::invalid_argument("null fused decode raw-query launch descriptor");
    const uint32_t elem = fused_elem(launch->element_type);
    if (!buffers->decode.tiling) throw std::invalid_argument("fused decode launch without host tiling descriptors");
    if (uint64_t{launch->grid} * launch->prologue_vectors_per_block < uint64_t{launch->tokens} * launch->heads ||
        (launch->prologue_cube_chunk_vectors != 0 && launch->prologue_cube_chunk_vectors != 16) ||
        launch->output_stage > 2)
        throw std::invalid_argument("unsupported raw query basis tiling");
    if (!fused_valid_launch(launch->grid, launch->tokens, launch->heads, launch->kv_heads, launch->head_size,
                            launch->block_size, launch->max_blocks, launch->splits, launch->heads_per_task,
                            launch->tasks_per_block, launch->reduce_tasks_per_block))
        throw std::invalid_argument("unsupported fused decode geometry or incomplete task coverage");
    // the prologue: Pi(raw query) into the FP32 query buffer the decode then reads
    throw_on(tq_rotate_query_pi(stream, static_cast<const uint16_t*>(buffers->raw_query), elem,
                                static_cast<const float*>(buffers->pi_signs),
                                static_cast<float*>(buffers->decode.query), launch->tokens * launch->heads,
                                launch->head_size),
             "fused_decode_opt_raw_query");
    fused_decode(stream, launch, &buffers->decode, static_cast<const float*>(buffers->pi_signs), buffers->gate,
                 launch->output_stage, "fused_decode_opt_raw_query");
}

// ------------------------------------------------------- the Lloyd-Max writer entry
// vllm_ascend::turboquant_reshape_and_cache_impl is the launcher of the BF16 Vector writer the
// reference vendors as its comparison kernel (kernels/ops/turboquant/baseline/
// turboquant_paged_attention.cpp:754; called by tests/npu/bench/
// bench_turboquant_reshape_and_cache.cpp:82-91): RMS scale and 16-level Lloyd-Max codes, one
// 16-token strip per block. It is served by this library's writer of that cache variant
// (tq_reshape_and_cache_lloydmax: same quantiser definition, block-diagonal rotation, this
// library's page layout), so the reference's ingest benchmark links and times all three of
// its rows here. The reference's harness never checks this kernel's bytes. block_dim,
// pi_signs and tables (the Ascend codec's constant pool) are not read.
namespace vllm_ascend {
enum struct AscendType { FP16 = 0, BF16 = 1, FP32 = 2 };   // kernels/ops/turboquant/baseline/types.h

void turboquant_reshape_and_cache_impl(AscendType type, void* stream, uint32_t /*block_dim*/, void* key,
                                       void* value, void* key_cache, void* value_cache, void* scale_cache,
                                       void* slot_mapping, void* /*pi_signs*/, void* /*tables*/,
                                       uint32_t num_tokens, uint32_t num_kv_heads, uint32_t head_size,
                                       uint32_t block_size, uint32_t num_blocks, uint32_t tokens_per_core,
                                       float inv_sqrt_len)
{
    if (type != AscendType::BF16) throw std::invalid_argument("reshape_and_cache baseline: bf16 activations only");
    if (tokens_per_core == 0 || num_tokens % tokens_per_core != 0)
        throw_on(TQ_ERR_PARTIAL_STRIP, "reshape_and_cache baseline");
    throw_on(tq_reshape_and_cache_lloydmax(stream, key, value, static_cast<int8_t*>(key_cache),
                                           static_cast<int8_t*>(value_cache), static_cast<float*>(scale_cache),
                                           static_cast<const int32_t*>(slot_mapping), TQ_IN_BF16, num_tokens,
                                           num_kv_heads, head_size, block_size, num_blocks, inv_sqrt_len, nullptr),
             "reshape_and_cache baseline");
}
}  // namespace vllm_ascend
