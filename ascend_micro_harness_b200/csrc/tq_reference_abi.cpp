// The reference project's launcher symbols, forwarding to the engine's tq_*
// entry points. Same names, same argument order, same error behaviour: a
// refused geometry throws std::invalid_argument out of the extern "C" function
// exactly as the AscendC launchers do, so the reference's C++ harnesses
// (tests/npu/turboquant_npu_common.hpp, tests/npu/turboquant_splitk_rigs.hpp)
// behave identically when linked against this library.
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
