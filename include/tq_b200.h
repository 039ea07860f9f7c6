/* tq_b200 -- C ABI of the B200-native TurboQuant KV-cache engine.
 *
 * Two families of entry points live in libtq_b200.so:
 *
 *   tq_*      the engine's own interface: status-returning, never throws.
 *   launch_*  the operator surface of fxslava/ascend-micro-harness, symbol for
 *             symbol and argument for argument, so that project's C++ host
 *             code links against this library unchanged. Like the originals
 *             they return void and report a refused geometry by throwing
 *             std::invalid_argument across the boundary.
 *
 * Conventions shared by every entry point (they are the reference launchers'
 * conventions): `stream` is an opaque stream handle (here a cudaStream_t, may
 * be null for the default stream); every pointer except `stream` is DEVICE
 * memory owned by the caller; nothing is allocated, nothing synchronises, the
 * call returns once the work is queued on the stream.
 *
 * Cache formats (reference: reports/qwen35_turboquant_rfc.md:104-115 and
 * tests/common/turboquant_oracle.hpp:31-38), P pages of S tokens, H KV heads,
 * head size d, strip height 16:
 *   key_cache, value_cache : int8[P*H*S*d/2], two signed INT4 codes per byte,
 *       low nibble first.
 *       key   nibble index = ((page*H + head)*S + token)*d + channel
 *       value nibble index = ((page*H + head)*S)*d + (token/16)*(16*d)
 *                            + channel*16 + token%16
 *   scale_cache : float[2*P*H*S], index ((kv*P + page)*H + head)*S + token,
 *       kv 0 = key plane, 1 = value plane.
 */
#ifndef TQ_B200_H
#define TQ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------ status codes */
#define TQ_OK 0
#define TQ_ERR_INVALID_ARGUMENT 1 /* geometry the kernels do not serve          */
#define TQ_ERR_PARTIAL_STRIP 2    /* num_tokens not a whole number of strips    */
#define TQ_ERR_LAUNCH 3           /* the CUDA runtime refused the launch        */
#define TQ_ERR_NO_DEVICE 4        /* no CUDA device / kernel image unusable     */
#define TQ_ERR_WORKSPACE_TOO_SMALL 5 /* the launch needs more than the built-in workspace holds */

/* Bits a kernel ORs into the optional device status word. */
#define TQ_STATUS_BAD_SLOT 0x1u     /* a strip's slots break the one-strip-one-page run */
#define TQ_STATUS_BAD_PAGE 0x2u     /* a page index left the cache                      */
#define TQ_STATUS_WAIT_EXPIRED 0x4u /* a bounded wait on a copy ran out                 */

/* Activation element type of reshape_and_cache. */
#define TQ_IN_INT8 0u
#define TQ_IN_BF16 1u

/* Where the rotation's sign diagonal comes from. The rotation is
 *   M = (H_{d/32} (x) I32) diag(s) (I_{d/32} (x) H32)
 * (kernels/ops/turboquant/turboquant_reshape_and_cache_a8.cpp:42-54); only s is
 * data. TABLES_* read it out of the reference's resident 32x32 blocks
 * (tests/common/turboquant_oracle.hpp:146-171): block g, row c0, column 0. */
#define TQ_SIGNS_F32 0u         /* float[d], negative = -1                      */
#define TQ_SIGNS_TABLES_I8 1u   /* int8  2*(d/32) row-major 32x32 blocks         */
#define TQ_SIGNS_TABLES_BF16 2u /* the same blocks widened to bf16               */

/* Decode output stages (kernels/ops/turboquant/fused_decode/common/turboquant_layout.h:139-147). */
#define TQ_OUT_ROTATED 0u   /* acc / l, still in the cache's rotated basis      */
#define TQ_OUT_UNROTATED 1u /* (acc / l) Pi                                     */
#define TQ_OUT_GATED 2u     /* stage 1 divided by 1 + exp(-gate)                */

/* Most record slots per (sequence, KV head) a decode workspace can be asked to hold: the
 * largest split count the tq_* decode entries accept (the reference-contract entries keep the
 * reference's own limits, 16 and 8). */
#define TQ_MAX_SPLITS 32u

/* Element type of the decode output. */
#define TQ_DTYPE_BF16 0u
#define TQ_DTYPE_F16 1u
#define TQ_DTYPE_F32 2u

const char* tq_version(void);
const char* tq_status_string(int status);

/* ------------------------------------------------------- reshape_and_cache
 * Aligned writer: num_tokens is a whole number of 16-token strips and each
 * strip fills 16 consecutive slots starting on a strip boundary of one page.
 * Replaces launch_turboquant_reshape_and_cache_{a8,bf16}
 * (kernels/ops/turboquant/turboquant_reshape_and_cache_a8.cpp:1578-1630,
 *  kernels/ops/turboquant/turboquant_reshape_and_cache_bf16.cpp:1993-2059).
 * key/value: [num_tokens][H*d] int8 or bf16. status may be null. */
int tq_reshape_and_cache(void* stream, const void* key, const void* value, int8_t* key_cache,
                         int8_t* value_cache, float* scale_cache, const int32_t* slot_mapping,
                         const void* signs, uint32_t sign_source, uint32_t in_dtype,
                         uint32_t num_tokens, uint32_t num_kv_heads, uint32_t head_size,
                         uint32_t block_size, uint32_t num_blocks, float inv_sqrt_len,
                         uint32_t* status);

/* tq_reshape_and_cache runs on the tcgen05 kernels (tensor-core products into tensor memory,
 * one kernel per head size), and on the warp-MMA kernel where the driver cannot encode a tensor
 * map. The two entries below force one or the other for any head size and element type: same
 * arguments, same bytes out. The tcgen05 entry returns TQ_ERR_LAUNCH where the warp-MMA kernel
 * would have had to step in. */
int tq_reshape_and_cache_warp_mma(void* stream, const void* key, const void* value,
                                  int8_t* key_cache, int8_t* value_cache, float* scale_cache,
                                  const int32_t* slot_mapping, const void* signs,
                                  uint32_t sign_source, uint32_t in_dtype, uint32_t num_tokens,
                                  uint32_t num_kv_heads, uint32_t head_size, uint32_t block_size,
                                  uint32_t num_blocks, float inv_sqrt_len, uint32_t* status);
int tq_reshape_and_cache_tcgen05(void* stream, const void* key, const void* value,
                                 int8_t* key_cache, int8_t* value_cache, float* scale_cache,
                                 const int32_t* slot_mapping, const void* signs,
                                 uint32_t sign_source, uint32_t in_dtype, uint32_t num_tokens,
                                 uint32_t num_kv_heads, uint32_t head_size, uint32_t block_size,
                                 uint32_t num_blocks, float inv_sqrt_len, uint32_t* status);

/* Every wait inside the tcgen05 writer (on a tile fetch, on a tensor-core product) is bounded:
 * when `cycles` clock cycles have passed the kernel reports TQ_STATUS_WAIT_EXPIRED, stores
 * nothing more, lets what it has in flight finish and returns. The default is about a second;
 * zero makes every wait give up at once (what the tests use to walk that path); a negative
 * value restores the default. Process-wide, read at each launch. */
void tq_ingest_set_wait_budget(long long cycles);

/* The aligned writer over ragged requests (bf16): request b owns tokens cu_seqlens[b] ..
 * cu_seqlens[b+1] and the strips strip_begin[b] .. strip_begin[b+1] (the caller's prefix sum
 * of ceil(length / 16); both arrays have num_requests + 1 device entries, total_strips =
 * strip_begin[num_requests]). A strip never straddles a request boundary; the last strip of
 * a request may hold n < 16 tokens: the key plane then receives n rows, the scale planes n
 * entries, the value plane the whole channel-major strip with the missing tokens as zeros
 * (so the 16 - n slots after the tail, which belong to the request's current page, are
 * overwritten in the value plane). Each strip's slots must be consecutive and start on a
 * strip boundary of a page. Follows the design note reports/qwen35_turboquant_rfc.md:564-650
 * for the reference's aligned writer. */
int tq_reshape_and_cache_varlen(void* stream, const uint16_t* key, const uint16_t* value,
                                int8_t* key_cache, int8_t* value_cache, float* scale_cache,
                                const int32_t* slot_mapping, const float* pi_signs,
                                const int32_t* cu_seqlens, const int32_t* strip_begin,
                                uint32_t num_requests, uint32_t total_strips, uint32_t num_kv_heads,
                                uint32_t head_size, uint32_t block_size, uint32_t num_blocks,
                                float inv_sqrt_len, uint32_t* status);

/* Scatter writer: 1..16 bf16 tokens per request at arbitrary slots, key rows
 * written whole, value strips read-modify-written so unowned nibbles survive.
 * Replaces launch_turboquant_reshape_scatter_aiv
 * (kernels/ops/turboquant/vllm_integration_layer/op_adapter/turboquant_torch_adpt.h:40-46).
 * cu_seqlens may be null (request r owns token r); slot < 0 = padded token. */
int tq_reshape_scatter(void* stream, const uint16_t* key, const uint16_t* value,
                       int8_t* key_cache, int8_t* value_cache, float* scale_cache,
                       const int32_t* slot_mapping, const float* pi_signs,
                       const int32_t* cu_seqlens, uint32_t num_requests, uint32_t num_kv_heads,
                       uint32_t head_size, uint32_t block_size, uint32_t num_blocks,
                       uint32_t item_begin, uint32_t item_count, float inv_sqrt_len,
                       uint32_t* status);

/* ------------------------------------------------------ paged split-K decode
 * One decode step for `batch` sequences: rotate each query once, stream the
 * sequence's packed pages through shared memory, online softmax per split,
 * log-sum-exp merge of the per-split (m, l, acc) partials through `workspace`.
 * The surface is the query / block_tables / context_lens one of
 * include/turboquant_fused_decode_opt.hpp:149-158 over the strip cache of the
 * AIC decoder (kernels/ops/turboquant/turboquant_paged_decode_attention.cpp:1727-1766).
 *
 *   query         bf16 [batch][num_heads][d], original basis
 *   block_tables  int32 [batch][max_blocks], logical -> physical page
 *   context_lens  int32 [batch], live tokens per sequence
 *   pi_signs      float [d]
 *   gate          float [batch][num_heads][d], read only by TQ_OUT_GATED
 *   workspace     float [tq_decode_workspace_floats(...)]; always required (a launch
 *                 that resolves to one split still writes its records there)
 *   output        [batch][num_heads][d] of out_dtype (TQ_DTYPE_*)
 *   splits        1..TQ_MAX_SPLITS, or 0 to choose from context lengths and SM count;
 *                 max_context_hint (0 = max_blocks*block_size) feeds that choice
 *                 since context_lens lives on the device
 *   softmax_scale multiplies every score (the AIC decoder uses 1) */
int tq_decode_splitk(void* stream, const uint16_t* query, const int8_t* key_cache,
                     const int8_t* value_cache, const float* scale_cache,
                     const int32_t* block_tables, const int32_t* context_lens,
                     const float* pi_signs, const float* gate, float* workspace,
                     void* output, uint32_t out_dtype, uint32_t batch, uint32_t num_heads,
                     uint32_t num_kv_heads, uint32_t head_size, uint32_t block_size,
                     uint32_t num_blocks, uint32_t max_blocks, uint32_t splits,
                     uint32_t max_context_hint, uint32_t output_stage, float inv_sqrt_len,
                     float softmax_scale, uint32_t* status);

/* One decode step of a serving stack as one call (the fused step the benchmark times): the new
 * token of every sequence is written into the cache as tq_reshape_scatter does (request r owns row r
 * of new_key / new_value, bf16 [batch][num_kv_heads*d]; slot_mapping[r] is its slot, a negative slot
 * skips the write), then the batch is decoded exactly as by tq_decode_splitk; context_lens already
 * count the new token. The decode is launched as the programmatic dependent of the writer, so its
 * set-up (context lengths, block tables, query rotation) runs under the writer and only its
 * first read of the cache waits for the writer's completion. Same refusals as the two calls; a
 * decode the library would refuse leaves the cache untouched. */
int tq_decode_step(void* stream, const uint16_t* new_key, const uint16_t* new_value,
                   const int32_t* slot_mapping, const uint16_t* query, int8_t* key_cache,
                   int8_t* value_cache, float* scale_cache, const int32_t* block_tables,
                   const int32_t* context_lens, const float* pi_signs, const float* gate,
                   float* workspace, void* output, uint32_t out_dtype, uint32_t batch,
                   uint32_t num_heads, uint32_t num_kv_heads, uint32_t head_size,
                   uint32_t block_size, uint32_t num_blocks, uint32_t max_blocks, uint32_t splits,
                   uint32_t max_context_hint, uint32_t output_stage, float inv_sqrt_len,
                   float softmax_scale, uint32_t* status);

/* tq_decode_splitk as one launch: a persistent grid over the batch's tiles with the
 * log-sum-exp merge folded in (the CTA that finishes a head's last outstanding segment merges
 * its records; no CTA waits for another). `splits` is the number of record slots per head the
 * workspace holds, 2..TQ_MAX_SPLITS (0 = TQ_MAX_SPLITS); workspace as tq_decode_workspace_floats
 * sizes it, 8-byte aligned. Other arguments as for tq_decode_splitk. Slower than
 * tq_decode_splitk on ragged batches (segment boundaries cost more than hardware-scheduled
 * CTAs); meant for callers to whom a single launch matters. The reference has no counterpart:
 * its fused decoder merges after a grid-wide barrier
 * (kernels/ops/turboquant/vllm_integration_layer/op_kernel/turboquant_fused_decode.cpp:1084). */
int tq_decode_splitk_persistent(void* stream, const uint16_t* query, const int8_t* key_cache,
                                const int8_t* value_cache, const float* scale_cache,
                                const int32_t* block_tables, const int32_t* context_lens,
                                const float* pi_signs, const float* gate, float* workspace,
                                void* output, uint32_t out_dtype, uint32_t batch, uint32_t num_heads,
                                uint32_t num_kv_heads, uint32_t head_size, uint32_t block_size,
                                uint32_t num_blocks, uint32_t max_blocks, uint32_t splits,
                                uint32_t output_stage, float inv_sqrt_len, float softmax_scale,
                                uint32_t* status);

/* tq_decode_splitk with a 24-bit fixed-point query and the softmax weights carried as a
 * hi + lo pair of halves (the arithmetic of tq_decode_splitk_partials, whose records are held
 * to the reference rig's tolerances, tests/npu/turboquant_splitk_rigs.hpp:144-215): the error
 * no longer grows with the magnitude of the cached values. Same arguments. */
int tq_decode_splitk_precise(void* stream, const uint16_t* query, const int8_t* key_cache,
                             const int8_t* value_cache, const float* scale_cache,
                             const int32_t* block_tables, const int32_t* context_lens,
                             const float* pi_signs, const float* gate, float* workspace,
                             void* output, uint32_t out_dtype, uint32_t batch, uint32_t num_heads,
                             uint32_t num_kv_heads, uint32_t head_size, uint32_t block_size,
                             uint32_t num_blocks, uint32_t max_blocks, uint32_t splits,
                             uint32_t max_context_hint, uint32_t output_stage, float inv_sqrt_len,
                             float softmax_scale, uint32_t* status);

/* The first half of tq_decode_splitk on its own: every (sequence, KV head, split)
 * exports its partial record into `workspace`, nothing is merged. Followed by
 * tq_splitk_combine(items = batch*num_kv_heads, rows = rows_stride =
 * num_heads/num_kv_heads) it is tq_decode_splitk. `splits` must be resolved by
 * the caller (tq_decode_choose_splits) when the combine is called separately. */
int tq_decode_splitk_export(void* stream, const uint16_t* query, const int8_t* key_cache,
                            const int8_t* value_cache, const float* scale_cache,
                            const int32_t* block_tables, const int32_t* context_lens,
                            const float* pi_signs, float* workspace, uint32_t batch,
                            uint32_t num_heads, uint32_t num_kv_heads, uint32_t head_size,
                            uint32_t block_size, uint32_t num_blocks, uint32_t max_blocks,
                            uint32_t splits, uint32_t max_context_hint, float inv_sqrt_len,
                            float softmax_scale, uint32_t* status);

/* Worker census of the persistent decode grid (tq_decode_splitk_persistent), after the
 * reference's WorkerMetrics (include/turboquant_splitk_contract.hpp:101-118): while a device
 * buffer of 10 * capacity_ctas 64-bit words is registered, CTA c of such a launch stores in
 * words 10c .. 10c + 8: the global-timer nanosecond at which it started, the one at which it
 * left (0: it never had work), the nanoseconds its first warp spent inside tile loops, the
 * number of segments it served, and the nanoseconds spent waiting for its slowest warp,
 * merging + publishing + counting arrivals, finishing heads, locating the next chunk, and in
 * segment prologues. Process-wide, for measurement runs only; pass NULL to switch it off. */
int tq_decode_worker_census(unsigned long long* device_words, uint32_t capacity_ctas);

/* Split count the launcher would pick for splits == 0 (1..TQ_MAX_SPLITS): what to size the
 * workspace with. The plan cuts work into chunks of a power-of-two number of tokens (256..8192,
 * about 32 CTAs per SM); a sequence uses as many splits as it has chunks. */
uint32_t tq_decode_choose_splits(uint32_t batch, uint32_t num_kv_heads, uint32_t block_size,
                                 uint32_t max_context, uint32_t sm_count);

/* Floats of workspace a decode launch with this many splits needs:
 * batch * num_kv_heads * splits partitions of (num_heads/num_kv_heads) rows,
 * each row {m x8, l x8, acc[d]}, the record of
 * include/turboquant_splitk_contract.hpp:23-27 with kChannels -> head_size,
 * followed by one 32-bit arrival counter per (sequence, KV head, 8-row tile)
 * and two 64-bit words of chunk schedule for tq_decode_splitk_persistent, which
 * merges inside the decode kernel (none of these needs initialisation; that entry
 * wants the workspace 8-byte aligned). For splits == 0 size it with
 * tq_decode_choose_splits. */
size_t tq_decode_workspace_floats(uint32_t batch, uint32_t num_heads, uint32_t num_kv_heads,
                                  uint32_t head_size, uint32_t splits);

/* tq_decode_splitk for callers that cannot hand over a workspace. It has no
 * counterpart in the reference. Meant for hosts that cannot allocate device memory
 * when a decode step is launched: a serving process whose KV-cache pool took all
 * free HBM at start-up, or a backend that must not call its host runtime's allocator
 * from the launch path. The split-K partials go into a fixed 8 MiB array inside the
 * library (TQ_STATIC_WORKSPACE_FLOATS floats, resident on every GPU that loads the
 * library until the process exits); the call itself allocates and frees nothing.
 *   - Limit: tq_decode_workspace_floats(batch, num_heads, num_kv_heads, head_size, splits)
 *     must not exceed TQ_STATIC_WORKSPACE_FLOATS; otherwise TQ_ERR_WORKSPACE_TOO_SMALL is
 *     returned and nothing runs. With splits == 0 the limit is checked against the record
 *     slots the launcher picks (tq_decode_choose_splits, up to TQ_MAX_SPLITS per head); a
 *     caller close to the limit passes an explicit split count instead.
 *   - The first call on each device looks up the array's device address (one CUDA
 *     runtime query, made with that device current). Make that first call before any
 *     stream capture begins.
 *   - All calls share the one array and it keeps whatever the last call left in it.
 *     Nothing needs clearing (each launch writes every record it later reads, and its
 *     counters are valid only under the launch's own tag), but two
 *     calls whose kernels can overlap on the GPU -- different streams, no ordering --
 *     race on it: keep calls on one device ordered.
 * Arguments are those of tq_decode_splitk without `workspace`. */
#define TQ_STATIC_WORKSPACE_FLOATS (2u * 1024u * 1024u)
int tq_decode_splitk_static(void* stream, const uint16_t* query, const int8_t* key_cache,
                            const int8_t* value_cache, const float* scale_cache,
                            const int32_t* block_tables, const int32_t* context_lens,
                            const float* pi_signs, const float* gate, void* output,
                            uint32_t out_dtype, uint32_t batch, uint32_t num_heads,
                            uint32_t num_kv_heads, uint32_t head_size, uint32_t block_size,
                            uint32_t num_blocks, uint32_t max_blocks, uint32_t splits,
                            uint32_t max_context_hint, uint32_t output_stage,
                            float inv_sqrt_len, float softmax_scale, uint32_t* status);

/* Per-split export only, no merge: the contract of
 * launch_turboquant_paged_decode_splitk_aic (16 query rows per KV head, records
 * of 16 + d floats, partitions of 16 rows; q_rot may be null). */
int tq_decode_splitk_partials(void* stream, const uint16_t* q, const void* signs,
                              uint32_t sign_source, const int8_t* key_cache,
                              const int8_t* value_cache, const float* scale_cache,
                              const uint32_t* table, uint16_t* q_rot, float* workspace,
                              uint32_t requests, uint32_t heads, uint32_t rows,
                              uint32_t head_size, uint32_t block_size, uint32_t cache_pages,
                              uint32_t seq_pages, uint32_t splits, uint32_t page_begin,
                              uint32_t page_count, uint32_t seq_len, float inv_sqrt_len,
                              float softmax_scale, uint32_t* status);

/* Log-sum-exp merge of `splits` partitions per (item,row) and the egress
 * (routines/routine_probe_l2_atomic_sync.hpp:467-498;
 *  routines/routine_vector_egress_rotate.hpp:186-277). Records as above. */
int tq_splitk_combine(void* stream, const float* workspace, const float* pi_signs,
                      const float* gate, void* output, uint32_t out_dtype, uint32_t items,
                      uint32_t rows, uint32_t rows_stride, uint32_t head_size, uint32_t splits,
                      uint32_t output_stage, float inv_sqrt_len, uint32_t* status);

/* tq_decode_splitk with query, gate and output in ONE 16-bit element type (TQ_DTYPE_BF16 or
 * TQ_DTYPE_F16), the form the raw-query entry of the reference's fused decoder takes them in
 * (include/turboquant_fused_decode_opt.hpp:118-131,:160-169: raw_query and gate are the element
 * type, output_stage 0 / 1 / 2). A BF16 query is rotated and rounded to bf16 as in
 * tq_decode_splitk; an FP16 query keeps its FP32 rotation, as the fused decoder's rotated
 * image is FP32. gate is read only by TQ_OUT_GATED. */
int tq_decode_splitk_elem(void* stream, const void* query, const int8_t* key_cache,
                          const int8_t* value_cache, const float* scale_cache,
                          const int32_t* block_tables, const int32_t* context_lens,
                          const float* pi_signs, const void* gate, float* workspace, void* output,
                          uint32_t elem_dtype, uint32_t batch, uint32_t num_heads,
                          uint32_t num_kv_heads, uint32_t head_size, uint32_t block_size,
                          uint32_t num_blocks, uint32_t max_blocks, uint32_t splits,
                          uint32_t max_context_hint, uint32_t output_stage, float inv_sqrt_len,
                          float softmax_scale, uint32_t* status);

/* Several query tokens per request (a step that verifies speculative tokens): query is
 * [batch * tokens_per_req][num_heads][d], token t of request b attends to
 * context_lens[b] - (tokens_per_req - 1 - t) tokens, output and gate are laid out like the
 * query. All tokens_per_req * (num_heads / num_kv_heads) <= 16 rows of a KV head share one
 * pass over its pages -- the row tile the reference drafts for its GQA decoder
 * (reports/qwen35_turboquant_rfc.md:221-236). workspace: batch * num_kv_heads * splits * rows *
 * (16 + d) floats with rows = tokens_per_req * num_heads / num_kv_heads. */
int tq_decode_splitk_mtp(void* stream, const uint16_t* query, const int8_t* key_cache,
                         const int8_t* value_cache, const float* scale_cache,
                         const int32_t* block_tables, const int32_t* context_lens,
                         const float* pi_signs, const float* gate, float* workspace, void* output,
                         uint32_t out_dtype, uint32_t batch, uint32_t tokens_per_req,
                         uint32_t num_heads, uint32_t num_kv_heads, uint32_t head_size,
                         uint32_t block_size, uint32_t num_blocks, uint32_t max_blocks,
                         uint32_t splits, uint32_t max_context_hint, uint32_t output_stage,
                         float inv_sqrt_len, float softmax_scale, uint32_t* status);

/* ------------------------------------------- caches of the reference's fused decoder
 * The reference's fused decoder (include/turboquant_fused_decode_opt.hpp) keeps a second
 * cache format, KV4/FP8: head size 256, pages of 64 or 128 slots, packed planes NZ-tiled
 * (NzTiledPackedByte, kernels/ops/turboquant/fused_decode/common/turboquant_layout.h:80-92),
 * byte `column` = channel `column` (bits 3:0) | channel `column + 128` (bits 7:4), a nibble c
 * (two's complement) standing for (c + 0.5) * scale / gain -- the uniform mid-rise grid of
 * fused_decode/common/turboquant_mode.h:100-124 -- and ceil(2 H / 8) * 8 scale floats per slot,
 * key scales first (fused_decode/common/turboquant_common.h:62-65). Such a cache is read in
 * two steps: tq_nz_kv4_import re-tiles it into the native pools (codes copied bit for bit,
 * scale_cache = scale / gain), tq_decode_splitk_prerotated decodes those with code_grid 1. */

/* nz_key, nz_value: num_blocks * block_size * num_kv_heads * 128 bytes; nz_scales:
 * num_blocks * block_size * ceil(2 num_kv_heads / 8) * 8 floats; key_cache, value_cache,
 * scale_cache: native pools for head size 256 and the same page geometry. block_size 64 or
 * 128. gain: 2.9832882881 for KV4/FP8 (TurboQuantModeTraits<KV4_FP8>::kGain). */
int tq_nz_kv4_import(void* stream, const uint8_t* nz_key, const uint8_t* nz_value,
                     const float* nz_scales, int8_t* key_cache, int8_t* value_cache,
                     float* scale_cache, uint32_t num_kv_heads, uint32_t block_size,
                     uint32_t num_blocks, float gain);

/* The pre-rotated entry (launch_fused_decode_opt, include/turboquant_fused_decode_opt.hpp:
 * 187-189): query_rot is the FP32 rotated image [batch][num_heads][head_size] of the query,
 * nothing is rotated or rounded on the way in. code_grid 0: nibble c decodes to c * scale (the
 * TurboQuant cache); 1: to (c + 0.5) * scale (an imported KV4/FP8 cache). Output stages as in
 * the fused decoder's raw-query entry (fused_decode/common/turboquant_layout.h:141-150):
 * TQ_OUT_ROTATED leaves the context in the rotated basis; TQ_OUT_UNROTATED applies
 * Pi = diag(pi_signs) H diag(pi_signs) / sqrt(head_size) once more (an involution, so this is
 * the original basis); TQ_OUT_GATED also divides by 1 + exp(-gate). pi_signs (head_size
 * floats, +-1) is read by the last two stages only, gate ([batch][num_heads][head_size] of
 * gate_dtype) by the last only. Workspace, splits, max_context_hint, status as for
 * tq_decode_splitk. */
int tq_decode_splitk_prerotated(void* stream, const float* query_rot, const int8_t* key_cache,
                                const int8_t* value_cache, const float* scale_cache,
                                const int32_t* block_tables, const int32_t* context_lens,
                                const float* pi_signs, const void* gate, float* workspace,
                                void* output, uint32_t out_dtype, uint32_t gate_dtype, uint32_t batch,
                                uint32_t num_heads, uint32_t num_kv_heads, uint32_t head_size,
                                uint32_t block_size, uint32_t num_blocks, uint32_t max_blocks,
                                uint32_t splits, uint32_t max_context_hint, uint32_t code_grid,
                                uint32_t output_stage, float softmax_scale, uint32_t* status);

/* The fused decoder's KV4/FP8 cache written on its Lloyd-Max codebook (DecodeUnpack::kLloydMaxLut,
 * kernels/ops/turboquant/fused_decode/common/turboquant_mode.h:181-206,:252-263): same storage (bin b
 * as the signed nibble b - 8), value = levels16[b] * scale, gain 1. Import the pools once with
 * tq_nz_kv4_import(gain = 1), then decode with this entry: query_rot FP32 [batch][num_heads][d] in the
 * cache's basis, levels16 a HOST array of 16 floats by bin index (the reference's table:
 * -2.75 -2 -1.625 -1.25 -0.9375 -0.6875 -0.375 -0.125 and their mirror images), output stages as in
 * tq_decode_splitk_prerotated. splits 1..16 (0 = the library's choice, at most 16); at most 8 query heads per
 * KV head; workspace tq_decode_workspace_floats(batch, num_heads, num_kv_heads, d, 16). Runs on the
 * table-lookup kernel of the Lloyd-Max variant (about a third of the uniform grid's rate). */
int tq_decode_splitk_levels(void* stream, const float* query_rot, const float* levels16,
                            const int8_t* key_cache, const int8_t* value_cache, const float* scale_cache,
                            const int32_t* block_tables, const int32_t* context_lens,
                            const float* pi_signs, const void* gate, float* workspace, void* output,
                            uint32_t out_dtype, uint32_t gate_dtype, uint32_t batch, uint32_t num_heads,
                            uint32_t num_kv_heads, uint32_t head_size, uint32_t block_size,
                            uint32_t num_blocks, uint32_t max_blocks, uint32_t splits,
                            uint32_t max_context_hint, uint32_t output_stage, float softmax_scale,
                            uint32_t* status);

/* The same decode over the NZ-tiled pools themselves: no import, no second pool. nz_key,
 * nz_value and nz_scales are the fused decoder's buffers as described above (head size 256,
 * block_size 64 or 128); each stored scale is divided by `gain` on the way in, exactly as
 * tq_nz_kv4_import does, so the results equal import + tq_decode_splitk_prerotated bit for
 * bit. This is what launch_fused_decode_opt[_raw_query] run. num_blocks 0 = unknown (page
 * numbers are not range-checked); inv_sqrt_len scales the egress rotation of stages 1 and 2;
 * precise != 0 selects the arithmetic of tq_decode_splitk_precise. */
int tq_decode_splitk_nz(void* stream, const float* query_rot, const uint8_t* nz_key,
                        const uint8_t* nz_value, const float* nz_scales, const int32_t* block_tables,
                        const int32_t* context_lens, const float* pi_signs, const void* gate,
                        float* workspace, void* output, uint32_t out_dtype, uint32_t gate_dtype,
                        uint32_t batch, uint32_t num_heads, uint32_t num_kv_heads, uint32_t block_size,
                        uint32_t num_blocks, uint32_t max_blocks, uint32_t splits,
                        uint32_t max_context_hint, uint32_t code_grid, uint32_t output_stage, float gain,
                        float inv_sqrt_len, float softmax_scale, uint32_t precise, uint32_t* status);

/* Pi q for `rows` FP16 or BF16 (elem_dtype) query vectors of head_size 128 or 256, FP32 out: the
 * rotated image tq_decode_splitk_prerotated takes, Pi = diag(pi_signs) H diag(pi_signs) /
 * sqrt(head_size) -- the prologue of the fused decoder's raw-query entry
 * (include/turboquant_fused_decode_opt.hpp:160-169; tests/common/fused_decode_opt_fixture.hpp:104-117). */
int tq_rotate_query_pi(void* stream, const uint16_t* query, uint32_t elem_dtype, const float* pi_signs,
                       float* query_rot, uint32_t rows, uint32_t head_size);

/* ------------------------------------------------------- stand-alone routines
 * The reference's single-purpose routines that its cache operators do not call. */

/* Q_rot = Q Pi^T for `rows` bf16 vectors of head_size 128 or 256, rounded to bf16: the rotated
 * operand the decoders pin (routines/routine_cube_decode_score.hpp:202-223;
 * tests/common/paged_decode_oracle.hpp:486-515). tq_decode_* rotate inside the kernel; this
 * is the stand-alone form of the same arithmetic. */
int tq_rotate_query(void* stream, const uint16_t* query, const float* pi_signs, uint16_t* query_rot,
                    uint32_t rows, uint32_t head_size, float inv_sqrt_len);

/* Y = X x H16 on `tiles` 16x16 tiles, X FP16 row-major, H16[k][c] = (-1)^popcount(k & c),
 * FP32 accumulation; y is float, half or bf16 by out_dtype (TQ_DTYPE_*). Replaces
 * cube_hadamard16 (routines/routine_cube_hadamard16.hpp:32-84; golden model
 * include/sim_micro_testbed.hpp:181-198). */
int tq_hadamard16(void* stream, const uint16_t* x_f16, void* y, uint32_t out_dtype, uint32_t tiles);

/* 16-level Lloyd-Max codec for N(0,1)-scaled inputs: code = number of thresholds <= x
 * (equality to the upper bin), unsigned codes packed low nibble first; recon (may be null) =
 * centroid of the code. count a multiple of 8. Replaces lloydmax_quantize_vf
 * (include/routines/routine_vector_lloydmax_quantize.hpp:18-38,:190-219;
 * tests/common/lloydmax_oracle.hpp:65-69). */
int tq_lloydmax4_quantize(void* stream, const float* x, uint8_t* packed, float* recon, size_t count);

/* Inverse-CDF int4 quantiser: y = 14 sigmoid(x) - 7, round to nearest even, saturate to
 * [-8, 7], two's-complement nibbles packed low first. x is FP16 or BF16 (TQ_DTYPE_F16 /
 * TQ_DTYPE_BF16), count a multiple of 8. Replaces icdf_quantize_vf
 * (routines/routine_vector_icdf_quantize.hpp:95-132; oracle tests/cpu/icdf_fixture.hpp:124-142). */
int tq_icdf_quantize(void* stream, const uint16_t* x, uint32_t in_dtype, uint8_t* packed, size_t count);

/* ---------------------------------------------------- Lloyd-Max cache variant
 * The ingest and decode built from those routines: block-diagonal 16x16 Hadamard rotation,
 * per-token RMS scale (kernels/ops/turboquant/baseline/common/turboquant_codec_950.h:194-207),
 * 16-level Lloyd-Max codes, in the same planes and page layout as the power-of-two cache.
 * The reference pins the stages, not this composite; integer-valued inputs determine every
 * scale bit and code (sums of squares are taken in FP64). */
int tq_reshape_and_cache_lloydmax(void* stream, const void* key, const void* value,
                                  int8_t* key_cache, int8_t* value_cache, float* scale_cache,
                                  const int32_t* slot_mapping, uint32_t in_dtype, uint32_t num_tokens,
                                  uint32_t num_kv_heads, uint32_t head_size, uint32_t block_size,
                                  uint32_t num_blocks, float inv_sqrt_len, uint32_t* status);

/* Split-K partial records of a decode over a Lloyd-Max cache, same workspace layout as
 * tq_decode_splitk_export (rows per record = num_heads / num_kv_heads, at most 8). Merge them
 * with tq_splitk_combine, passing pi_signs = NULL: that selects the block-diagonal egress. */
int tq_decode_lloydmax_export(void* stream, const uint16_t* query, const int8_t* key_cache,
                              const int8_t* value_cache, const float* scale_cache,
                              const int32_t* block_tables, const int32_t* context_lens,
                              float* workspace, uint32_t batch, uint32_t num_heads,
                              uint32_t num_kv_heads, uint32_t head_size, uint32_t block_size,
                              uint32_t num_blocks, uint32_t max_blocks, uint32_t splits,
                              float softmax_scale, uint32_t* status);

/* ------------------------------------------------- fused decoder descriptors
 * Field-for-field mirrors of ascend_micro::fused_decode_opt::Launch, Buffers and
 * RawQueryBuffers (include/turboquant_fused_decode_opt.hpp:108-133,:149-170), so that a
 * caller built against the reference's header passes its own structs unchanged. */
typedef struct tq_fused_launch {
    uint32_t grid, tokens, heads, kv_heads;
    uint32_t head_size, block_size, max_blocks;
    uint32_t splits, heads_per_task, tasks_per_block;
    uint32_t reduce_tasks_per_block, fused_context_limit;
    float scale, inv_sqrt_len;
    uint32_t prologue_vectors_per_block, prologue_cube_chunk_vectors;
    uint32_t output_stage;
    uint32_t element_type; /* 0 = FP16, 1 = BF16 query / gate / output elements */
    uint32_t probe_page, probe_tile;
} tq_fused_launch;

typedef struct tq_fused_buffers {
    void *query, *key, *value, *scales, *block_table, *context_lengths;
    void *mode_tables, *workspace, *output;
    void* tiling;
} tq_fused_buffers;

typedef struct tq_fused_raw_query_buffers {
    void *raw_query, *pi_signs, *rot_tables, *h16, *gate;
    tq_fused_buffers decode;
} tq_fused_raw_query_buffers;

#ifdef __cplusplus
} /* extern "C" */
#endif

/* ------------------------------------------------ reference-named launchers
 * Declared for C++ callers only: they throw std::invalid_argument. Signatures
 * are those of the reference (file:line beside each). A translation unit that also
 * includes the reference's own headers defines TQ_B200_NO_REFERENCE_LAUNCHERS first:
 * the symbols are the same, the C++ parameter types of the two declarations are not. */
#if defined(__cplusplus) && !defined(TQ_B200_NO_REFERENCE_LAUNCHERS)
extern "C" {
/* kernels/ops/turboquant/turboquant_reshape_and_cache_a8.cpp:1578-1585 */
void launch_turboquant_reshape_and_cache_a8(
    void* stream, const int8_t* key, const int8_t* value, int8_t* key_cache, int8_t* value_cache,
    float* scale_cache, const int32_t* slot_mapping, const float* pi_signs, const int32_t* tables,
    uint32_t num_tokens, uint32_t num_kv_heads, uint32_t head_size, uint32_t block_size,
    uint32_t num_blocks, uint32_t tokens_per_core, float inv_sqrt_len, bool reuse_mode4_flags);
/* kernels/ops/turboquant/turboquant_reshape_and_cache_bf16.cpp:1993-2000 */
void launch_turboquant_reshape_and_cache_bf16(
    void* stream, const uint16_t* key, const uint16_t* value, int8_t* key_cache,
    int8_t* value_cache, float* scale_cache, const int32_t* slot_mapping, const float* pi_signs,
    const int32_t* tables, uint32_t num_tokens, uint32_t num_kv_heads, uint32_t head_size,
    uint32_t block_size, uint32_t num_blocks, uint32_t tokens_per_core, float inv_sqrt_len,
    bool reuse_mode4_flags);
/* kernels/ops/turboquant/turboquant_reshape_scatter_aiv.cpp:760-766 */
void launch_turboquant_reshape_scatter_aiv(
    void* stream, uint32_t block_dim, uint16_t* key, uint16_t* value, int8_t* key_cache,
    int8_t* value_cache, float* scale_cache, int32_t* slot_mapping, float* pi_signs,
    int32_t* cu_seqlens, int32_t* launch_probe, uint32_t num_requests, uint32_t num_kv_heads,
    uint32_t head_size, uint32_t block_size, uint32_t num_blocks, uint32_t item_begin,
    uint32_t item_count, float inv_sqrt_len);
/* kernels/ops/turboquant/turboquant_paged_decode_attention.cpp:1727-1745 */
void launch_turboquant_paged_decode_splitk_aic(
    void* stream, uint16_t* q, uint16_t* pi_table, int8_t* key, int8_t* value, float* scales,
    uint32_t* table, uint16_t* qrot, float* workspace, uint32_t requests, uint32_t heads,
    uint32_t block_size, uint32_t cache_pages, uint32_t seq_pages, uint32_t splits,
    uint32_t page_begin, uint32_t page_count, uint32_t seq_len);
/* include/turboquant_fused_decode_opt.hpp:172-174: the pre-rotated entry. buffers->query is the
 * FP32 rotated query [tokens][heads][256]; key / value / scales the KV4 NZ-tiled cache;
 * workspace at least tokens * heads * splits * 272 floats; output [tokens][heads][256] of the
 * launch's element type, context in the rotated basis. */
void launch_fused_decode_opt(void* stream, const tq_fused_launch* launch, const tq_fused_buffers* buffers);
/* include/turboquant_fused_decode_opt.hpp:178-180: the raw-query entry. raw_query and gate are
 * of the launch's element type, pi_signs float[256]; decode.query is WRITTEN (Pi raw_query,
 * FP32) and then read; launch->output_stage 0 / 1 / 2. */
void launch_fused_decode_opt_raw_query(void* stream, const tq_fused_launch* launch,
                                       const tq_fused_raw_query_buffers* buffers);
}
#endif

#endif /* TQ_B200_H */
