"""Host-side mirror of the operator surface over the C ABI. torch supplies device
memory and streams only; every computation happens in libtq_b200.so."""
from __future__ import annotations

import ctypes

import torch

from ._lib import TqError, load_library

SIGNS_F32, SIGNS_TABLES_I8, SIGNS_TABLES_BF16 = 0, 1, 2
OUT_ROTATED, OUT_UNROTATED, OUT_GATED = 0, 1, 2
STATUS_BAD_SLOT, STATUS_BAD_PAGE, STATUS_WAIT_EXPIRED = 1, 2, 4
MAX_SPLITS = 32


def _ptr(t):
    if t is None:
        return None
    if not t.is_cuda:
        raise ValueError("the engine takes device tensors only")
    if not t.is_contiguous():
        raise ValueError("the engine takes contiguous tensors only")
    return t.data_ptr()


def _stream(stream, device=None):
    s = torch.cuda.current_stream(device) if stream is None else stream
    return s.cuda_stream


def _out_dtype(t):
    return {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}[t.dtype]


def _check(status, what):
    if status != 0:
        raise TqError(status, what)


_I32 = (torch.int32,)
_F32 = (torch.float32,)
_BYTES = (torch.uint8, torch.int8)
_BF16 = (torch.bfloat16,)
_ELEM16 = (torch.bfloat16, torch.float16)
_ANYF = (torch.bfloat16, torch.float16, torch.float32)


class _Call:
    """Operand checks of one entry point. The library reads raw pointers: a tensor on another
    GPU than the launch's, or of another element type than the kernel assumes (an int64 block
    table, a float16 query where bfloat16 bits are read), would be misread without any error,
    so both are refused here. Used as a context manager it makes the operands' device current,
    because the library launches on the current device."""

    def __init__(self, what):
        self.what, self.device = what, None

    def take(self, name, t, dtypes, optional=False):
        if t is None:
            if optional:
                return self
            raise ValueError(f"{self.what}: {name} is required")
        if not isinstance(t, torch.Tensor) or not t.is_cuda:
            raise ValueError(f"{self.what}: {name} must be a CUDA tensor")
        if t.dtype not in dtypes:
            want = " or ".join(str(d).replace("torch.", "") for d in dtypes)
            raise ValueError(f"{self.what}: {name} must be {want}, got {str(t.dtype).replace('torch.', '')}")
        if self.device is None:
            self.device = t.device
        elif t.device != self.device:
            raise ValueError(f"{self.what}: {name} is on {t.device}, the other operands on {self.device}")
        return self

    def caches(self, key_cache, value_cache, scale_cache):
        return (self.take("key_cache", key_cache, _BYTES).take("value_cache", value_cache, _BYTES)
                .take("scale_cache", scale_cache, _F32))

    def __enter__(self):
        self._guard = torch.cuda.device(self.device)
        self._guard.__enter__()
        return self

    def __exit__(self, *exc):
        return self._guard.__exit__(*exc)


def _sm_count(device=None):
    if torch.cuda.is_available():
        return torch.cuda.get_device_properties(device if device is not None else torch.cuda.current_device()
                                                ).multi_processor_count
    return 148


def _need_workspace(call, workspace, batch, num_heads, num_kv_heads, head_size, block_size, max_blocks,
                    splits, max_context_hint, rows_factor=1, always=False):
    """The split count the launch will use and the check that `workspace` holds its records:
    resolved exactly as the library resolves it (same hint, the device's own SM count). A
    launch that resolves to one split writes the output directly and takes no workspace."""
    n = splits if splits else choose_splits(batch, num_kv_heads, block_size,
                                            max_context_hint if max_context_hint else max_blocks * block_size,
                                            _sm_count(call.device))
    if n == 1 and not always:
        call.take("workspace", workspace, _F32, optional=True)
        return n
    need = decode_workspace_floats(batch, num_heads * rows_factor, num_kv_heads, head_size, n)
    call.take("workspace", workspace, _F32)
    if workspace.numel() < need:
        raise ValueError(f"{call.what}: workspace holds {workspace.numel()} floats, the launch needs {need} "
                         f"({n} splits)")
    return n


def reshape_and_cache(key, value, key_cache, value_cache, scale_cache, slot_mapping, signs, *,
                      num_kv_heads, head_size, block_size, num_blocks, inv_sqrt_len,
                      sign_source=SIGNS_F32, status=None, stream=None, warp_mma=False, tcgen05=False):
    """Aligned writer (reference: launch_turboquant_reshape_and_cache_{a8,bf16}).
    key/value: [T, H*d] int8 or bfloat16. Runs on the tcgen05 kernels (the warp-MMA kernel where the
    driver cannot encode a tensor map); warp_mma=True or tcgen05=True forces one of them."""
    lib = load_library()
    call = _Call("reshape_and_cache").take("key", key, (torch.int8, torch.bfloat16))
    call.take("value", value, (key.dtype,)).caches(key_cache, value_cache, scale_cache)
    call.take("slot_mapping", slot_mapping, _I32).take("status", status, _I32, optional=True)
    call.take("signs", signs, {SIGNS_F32: _F32, SIGNS_TABLES_I8: (torch.int8, torch.int32),
                               SIGNS_TABLES_BF16: (torch.bfloat16, torch.int32, torch.int16)}[sign_source])
    in_dtype = {torch.int8: 0, torch.bfloat16: 1}[key.dtype]
    num_tokens = key.numel() // (num_kv_heads * head_size)
    if warp_mma and tcgen05:
        raise ValueError("reshape_and_cache: warp_mma and tcgen05 exclude each other")
    fn = (lib.tq_reshape_and_cache_warp_mma if warp_mma else
          lib.tq_reshape_and_cache_tcgen05 if tcgen05 else lib.tq_reshape_and_cache)
    with call:
        _check(fn(
            _stream(stream, call.device), _ptr(key), _ptr(value), _ptr(key_cache), _ptr(value_cache),
            _ptr(scale_cache), _ptr(slot_mapping), _ptr(signs), sign_source, in_dtype, num_tokens,
            num_kv_heads, head_size, block_size, num_blocks, inv_sqrt_len, _ptr(status)),
            "tq_reshape_and_cache")


def set_ingest_wait_budget(cycles):
    """Clock cycles one wait inside the tcgen05 writer may take before the launch reports
    STATUS_WAIT_EXPIRED and stops storing. 0: every wait gives up at once; negative: the default
    (about a second). Process-wide."""
    load_library().tq_ingest_set_wait_budget(int(cycles))


def reshape_and_cache_varlen(key, value, key_cache, value_cache, scale_cache, slot_mapping, signs,
                             cu_seqlens, *, num_kv_heads, head_size, block_size, num_blocks,
                             inv_sqrt_len, status=None, stream=None):
    """Aligned writer over ragged requests. cu_seqlens: host sequence of num_requests + 1 token
    offsets; the strips' prefix sum is formed here and uploaded with it."""
    lib = load_library()
    cu = [int(c) for c in cu_seqlens]
    begin = [0]
    for a, b in zip(cu[:-1], cu[1:]):
        begin.append(begin[-1] + (b - a + 15) // 16)
    call = _Call("reshape_and_cache_varlen").take("key", key, _BF16).take("value", value, _BF16)
    call.caches(key_cache, value_cache, scale_cache).take("slot_mapping", slot_mapping, _I32)
    call.take("signs", signs, _F32).take("status", status, _I32, optional=True)
    dev = key.device
    cu_d = torch.tensor(cu, dtype=torch.int32, device=dev)
    begin_d = torch.tensor(begin, dtype=torch.int32, device=dev)
    with call:
        _check(lib.tq_reshape_and_cache_varlen(
            _stream(stream, dev), _ptr(key), _ptr(value), _ptr(key_cache), _ptr(value_cache),
            _ptr(scale_cache), _ptr(slot_mapping), _ptr(signs), _ptr(cu_d), _ptr(begin_d), len(cu) - 1,
            begin[-1], num_kv_heads, head_size, block_size, num_blocks, inv_sqrt_len, _ptr(status)),
            "tq_reshape_and_cache_varlen")


def reshape_scatter(key, value, key_cache, value_cache, scale_cache, slot_mapping, pi_signs,
                    cu_seqlens, *, num_requests, num_kv_heads, head_size, block_size, num_blocks,
                    inv_sqrt_len, item_begin=0, item_count=None, status=None, stream=None):
    """Scatter writer (reference: launch_turboquant_reshape_scatter_aiv)."""
    lib = load_library()
    if item_count is None:
        item_count = num_requests * num_kv_heads
    call = _Call("reshape_scatter").take("key", key, _BF16).take("value", value, _BF16)
    call.caches(key_cache, value_cache, scale_cache).take("slot_mapping", slot_mapping, _I32)
    call.take("pi_signs", pi_signs, _F32).take("cu_seqlens", cu_seqlens, _I32, optional=True)
    call.take("status", status, _I32, optional=True)
    with call:
        _check(lib.tq_reshape_scatter(
            _stream(stream, call.device), _ptr(key), _ptr(value), _ptr(key_cache), _ptr(value_cache),
            _ptr(scale_cache), _ptr(slot_mapping), _ptr(pi_signs), _ptr(cu_seqlens), num_requests,
            num_kv_heads, head_size, block_size, num_blocks, item_begin, item_count, inv_sqrt_len,
            _ptr(status)), "tq_reshape_scatter")


def decode_workspace_floats(batch, num_heads, num_kv_heads, head_size, splits):
    return load_library().tq_decode_workspace_floats(batch, num_heads, num_kv_heads, head_size,
                                                     splits)


def worker_census(words=None):
    """Registers (or, with None, removes) the int64 device tensor in which the CTAs of persistent
    decode launches stamp four words each: start and end in nanoseconds of the global timer, the
    nanoseconds the first warp spent in tile loops, the segments served."""
    lib = load_library()
    if words is None:
        _check(lib.tq_decode_worker_census(None, 0), "tq_decode_worker_census")
        return
    call = _Call("worker_census").take("words", words, (torch.int64,))
    _check(lib.tq_decode_worker_census(_ptr(words), words.numel() // 10), "tq_decode_worker_census")


def choose_splits(batch, num_kv_heads, block_size, max_context, sm_count=None):
    """The split count a launch with splits=0 resolves to (sm_count: the launching device's)."""
    return load_library().tq_decode_choose_splits(batch, num_kv_heads, block_size, max_context,
                                                  _sm_count() if sm_count is None else sm_count)


def _decode_operands(call, key_cache, value_cache, scale_cache, block_tables, context_lens, pi_signs, output,
                     gate, status, gate_dtypes=_F32, signs_optional=False):
    call.caches(key_cache, value_cache, scale_cache).take("block_tables", block_tables, _I32)
    call.take("context_lens", context_lens, _I32).take("pi_signs", pi_signs, _F32, optional=signs_optional)
    call.take("output", output, _ANYF).take("gate", gate, gate_dtypes, optional=True)
    call.take("status", status, _I32, optional=True)


def decode_splitk(query, key_cache, value_cache, scale_cache, block_tables, context_lens,
                  pi_signs, output, *, num_heads, num_kv_heads, head_size, block_size, num_blocks,
                  inv_sqrt_len, softmax_scale=1.0, splits=0, max_context_hint=0, workspace=None,
                  gate=None, output_stage=OUT_ROTATED, status=None, stream=None, precise=False,
                  persistent=False):
    """Paged split-K decode over query / block_tables / context_lens. query bfloat16, gate
    float32. precise=True selects the wider arithmetic (24-bit query, hi + lo softmax weights);
    persistent=True the single-launch persistent grid, where `splits` is the number of record
    slots per head the workspace holds (0 = 32)."""
    lib = load_library()
    call = _Call("decode_splitk").take("query", query, _BF16)
    _decode_operands(call, key_cache, value_cache, scale_cache, block_tables, context_lens, pi_signs, output,
                     gate, status)
    batch = query.numel() // (num_heads * head_size)
    max_blocks = block_tables.shape[-1]
    if persistent:
        slots = splits if splits else MAX_SPLITS
        _need_workspace(call, workspace, batch, num_heads, num_kv_heads, head_size, block_size, max_blocks,
                        slots, max_context_hint, always=True)
        with call:
            _check(lib.tq_decode_splitk_persistent(
                _stream(stream, call.device), _ptr(query), _ptr(key_cache), _ptr(value_cache), _ptr(scale_cache),
                _ptr(block_tables), _ptr(context_lens), _ptr(pi_signs), _ptr(gate), _ptr(workspace),
                _ptr(output), _out_dtype(output), batch, num_heads, num_kv_heads, head_size, block_size,
                num_blocks, max_blocks, splits, output_stage, inv_sqrt_len, softmax_scale, _ptr(status)),
                "tq_decode_splitk_persistent")
        return
    _need_workspace(call, workspace, batch, num_heads, num_kv_heads, head_size, block_size, max_blocks, splits,
                    max_context_hint)
    fn, name = ((lib.tq_decode_splitk_precise, "tq_decode_splitk_precise") if precise
                else (lib.tq_decode_splitk, "tq_decode_splitk"))
    with call:
        _check(fn(
            _stream(stream, call.device), _ptr(query), _ptr(key_cache), _ptr(value_cache), _ptr(scale_cache),
            _ptr(block_tables), _ptr(context_lens), _ptr(pi_signs), _ptr(gate), _ptr(workspace),
            _ptr(output), _out_dtype(output), batch, num_heads, num_kv_heads, head_size, block_size,
            num_blocks, max_blocks, splits, max_context_hint, output_stage, inv_sqrt_len, softmax_scale,
            _ptr(status)), name)


def decode_step(new_key, new_value, slot_mapping, query, key_cache, value_cache, scale_cache, block_tables,
                context_lens, pi_signs, output, *, num_heads, num_kv_heads, head_size, block_size, num_blocks,
                inv_sqrt_len, softmax_scale=1.0, splits=0, max_context_hint=0, workspace=None, gate=None,
                output_stage=OUT_ROTATED, status=None, stream=None):
    """One decode step as one call: scatter-write the new token of every sequence (new_key / new_value
    bfloat16 [batch, num_kv_heads * head_size], slot_mapping int32 [batch]), then decode_splitk over the
    batch, the decode scheduled under the writer (programmatic dependent launch)."""
    lib = load_library()
    call = _Call("decode_step").take("new_key", new_key, _BF16).take("new_value", new_value, _BF16)
    call.take("slot_mapping", slot_mapping, _I32).take("query", query, _BF16)
    _decode_operands(call, key_cache, value_cache, scale_cache, block_tables, context_lens, pi_signs, output,
                     gate, status)
    batch = query.numel() // (num_heads * head_size)
    if new_key.numel() != batch * num_kv_heads * head_size or slot_mapping.numel() != batch:
        raise ValueError("decode_step: one new token per sequence: new_key [batch, num_kv_heads * head_size], "
                         "slot_mapping [batch]")
    max_blocks = block_tables.shape[-1]
    _need_workspace(call, workspace, batch, num_heads, num_kv_heads, head_size, block_size, max_blocks, splits,
                    max_context_hint)
    with call:
        _check(lib.tq_decode_step(
            _stream(stream, call.device), _ptr(new_key), _ptr(new_value), _ptr(slot_mapping), _ptr(query),
            _ptr(key_cache), _ptr(value_cache), _ptr(scale_cache), _ptr(block_tables), _ptr(context_lens),
            _ptr(pi_signs), _ptr(gate), _ptr(workspace), _ptr(output), _out_dtype(output), batch, num_heads,
            num_kv_heads, head_size, block_size, num_blocks, max_blocks, splits, max_context_hint, output_stage,
            inv_sqrt_len, softmax_scale, _ptr(status)), "tq_decode_step")


def decode_splitk_elem(query, key_cache, value_cache, scale_cache, block_tables, context_lens,
                       pi_signs, output, *, num_heads, num_kv_heads, head_size, block_size, num_blocks,
                       inv_sqrt_len, softmax_scale=1.0, splits=0, max_context_hint=0, workspace=None,
                       gate=None, output_stage=OUT_ROTATED, status=None, stream=None):
    """decode_splitk with query, gate and output all bfloat16 or all float16."""
    lib = load_library()
    call = _Call("decode_splitk_elem").take("query", query, _ELEM16)
    if output.dtype != query.dtype or (gate is not None and gate.dtype != query.dtype):
        raise ValueError("query, gate and output share one element type")
    _decode_operands(call, key_cache, value_cache, scale_cache, block_tables, context_lens, pi_signs, output,
                     gate, status, gate_dtypes=_ELEM16)
    batch = query.numel() // (num_heads * head_size)
    _need_workspace(call, workspace, batch, num_heads, num_kv_heads, head_size, block_size,
                    block_tables.shape[-1], splits, max_context_hint)
    with call:
        _check(lib.tq_decode_splitk_elem(
            _stream(stream, call.device), _ptr(query), _ptr(key_cache), _ptr(value_cache), _ptr(scale_cache),
            _ptr(block_tables), _ptr(context_lens), _ptr(pi_signs), _ptr(gate), _ptr(workspace),
            _ptr(output), _out_dtype(query), batch, num_heads, num_kv_heads, head_size, block_size,
            num_blocks, block_tables.shape[-1], splits, max_context_hint, output_stage, inv_sqrt_len,
            softmax_scale, _ptr(status)), "tq_decode_splitk_elem")


def decode_splitk_mtp(query, key_cache, value_cache, scale_cache, block_tables, context_lens, pi_signs,
                      output, *, tokens_per_req, num_heads, num_kv_heads, head_size, block_size, num_blocks,
                      inv_sqrt_len, softmax_scale=1.0, splits=0, max_context_hint=0, workspace=None,
                      gate=None, output_stage=OUT_ROTATED, status=None, stream=None):
    """decode_splitk with tokens_per_req query tokens per request (speculative decoding):
    query/output are [batch * tokens_per_req, num_heads, d]; token t sees the context without
    its last tokens_per_req - 1 - t tokens."""
    lib = load_library()
    call = _Call("decode_splitk_mtp").take("query", query, _BF16)
    _decode_operands(call, key_cache, value_cache, scale_cache, block_tables, context_lens, pi_signs, output,
                     gate, status)
    batch = query.numel() // (num_heads * head_size * tokens_per_req)
    _need_workspace(call, workspace, batch, num_heads, num_kv_heads, head_size, block_size,
                    block_tables.shape[-1], splits, max_context_hint, rows_factor=tokens_per_req)
    with call:
        _check(lib.tq_decode_splitk_mtp(
            _stream(stream, call.device), _ptr(query), _ptr(key_cache), _ptr(value_cache), _ptr(scale_cache),
            _ptr(block_tables), _ptr(context_lens), _ptr(pi_signs), _ptr(gate), _ptr(workspace),
            _ptr(output), _out_dtype(output), batch, tokens_per_req, num_heads, num_kv_heads, head_size,
            block_size, num_blocks, block_tables.shape[-1], splits, max_context_hint, output_stage,
            inv_sqrt_len, softmax_scale, _ptr(status)), "tq_decode_splitk_mtp")


KV4_FP8_GAIN = 2.9832882881   # TurboQuantModeTraits<KV4_FP8>::kGain of the reference's fused decoder
GRID_INTEGER, GRID_MIDRISE = 0, 1


def nz_kv4_import(nz_key, nz_value, nz_scales, key_cache, value_cache, scale_cache, *, num_kv_heads,
                  block_size, num_blocks, gain=KV4_FP8_GAIN, stream=None):
    """Re-tiles a KV4/FP8 cache of the reference's fused decoder (NZ-tiled packed planes, head
    size 256, per-slot scale records) into the native pools; codes are copied bit for bit and
    scale_cache receives scale / gain. Decode the result with decode_splitk_prerotated(...,
    code_grid=GRID_MIDRISE), or skip the import and decode the source with decode_splitk_nz."""
    lib = load_library()
    call = _Call("nz_kv4_import").take("nz_key", nz_key, _BYTES).take("nz_value", nz_value, _BYTES)
    call.take("nz_scales", nz_scales, _F32).caches(key_cache, value_cache, scale_cache)
    with call:
        _check(lib.tq_nz_kv4_import(_stream(stream, call.device), _ptr(nz_key), _ptr(nz_value), _ptr(nz_scales),
                                    _ptr(key_cache), _ptr(value_cache), _ptr(scale_cache), num_kv_heads,
                                    block_size, num_blocks, gain), "tq_nz_kv4_import")


def rotate_query_pi(query, pi_signs, query_rot, *, head_size, stream=None):
    """query_rot (float32) = Pi query for float16/bfloat16 rows, Pi = diag(s) H diag(s) / sqrt(d): the
    raw-query prologue of the fused decoder, feeding decode_splitk_prerotated."""
    lib = load_library()
    call = _Call("rotate_query_pi").take("query", query, _ELEM16).take("pi_signs", pi_signs, _F32)
    call.take("query_rot", query_rot, _F32)
    with call:
        _check(lib.tq_rotate_query_pi(_stream(stream, call.device), _ptr(query), _out_dtype(query),
                                      _ptr(pi_signs), _ptr(query_rot), query.numel() // head_size, head_size),
               "tq_rotate_query_pi")


def decode_splitk_prerotated(query_rot, key_cache, value_cache, scale_cache, block_tables, context_lens,
                             output, *, num_heads, num_kv_heads, head_size, block_size, num_blocks,
                             softmax_scale=1.0, splits=0, max_context_hint=0, workspace=None,
                             code_grid=GRID_INTEGER, pi_signs=None, gate=None, output_stage=OUT_ROTATED,
                             status=None, stream=None):
    """Decode with an FP32 query that is already in the cache's rotated basis (the fused
    decoder's pre-rotated entry). code_grid=GRID_MIDRISE reads a nibble c as (c + 0.5) * scale,
    the grid of an imported KV4/FP8 cache. output_stage OUT_UNROTATED applies
    Pi = diag(pi_signs) H diag(pi_signs) / sqrt(head_size) to the context, OUT_GATED also the
    sigmoid gate (float32, float16 or bfloat16)."""
    lib = load_library()
    call = _Call("decode_splitk_prerotated").take("query_rot", query_rot, _F32)
    _decode_operands(call, key_cache, value_cache, scale_cache, block_tables, context_lens, pi_signs, output,
                     gate, status, gate_dtypes=_ANYF, signs_optional=True)
    batch = query_rot.numel() // (num_heads * head_size)
    _need_workspace(call, workspace, batch, num_heads, num_kv_heads, head_size, block_size,
                    block_tables.shape[-1], splits, max_context_hint)
    with call:
        _check(lib.tq_decode_splitk_prerotated(
            _stream(stream, call.device), _ptr(query_rot), _ptr(key_cache), _ptr(value_cache),
            _ptr(scale_cache), _ptr(block_tables), _ptr(context_lens), _ptr(pi_signs), _ptr(gate),
            _ptr(workspace), _ptr(output), _out_dtype(output), _out_dtype(gate) if gate is not None else 2,
            batch, num_heads, num_kv_heads, head_size, block_size, num_blocks, block_tables.shape[-1], splits,
            max_context_hint, code_grid, output_stage, softmax_scale, _ptr(status)),
            "tq_decode_splitk_prerotated")


def decode_splitk_levels(query_rot, levels, key_cache, value_cache, scale_cache, block_tables, context_lens, output,
                         *, num_heads, num_kv_heads, head_size, block_size, num_blocks, softmax_scale=1.0, splits=0,
                         max_context_hint=0, workspace=None, pi_signs=None, gate=None, output_stage=OUT_ROTATED,
                         status=None, stream=None):
    """Decode over native planes whose codes index a 16-level table (the fused decoder's Lloyd-Max toggle after
    nz_kv4_import with gain 1): `levels` is a host sequence of 16 floats by bin index, query_rot float32 in the
    cache's basis. Output stages as decode_splitk_prerotated; at most 16 splits and 8 query heads per KV head."""
    lib = load_library()
    lv = (ctypes.c_float * 16)(*[float(x) for x in levels])
    call = _Call("decode_splitk_levels").take("query_rot", query_rot, _F32)
    _decode_operands(call, key_cache, value_cache, scale_cache, block_tables, context_lens, pi_signs, output,
                     gate, status, gate_dtypes=_ANYF, signs_optional=True)
    batch = query_rot.numel() // (num_heads * head_size)
    need = decode_workspace_floats(batch, num_heads, num_kv_heads, head_size, splits if splits else 16)
    if workspace is None or workspace.numel() < need:
        raise ValueError(f"decode_splitk_levels: workspace of {need} floats needed")
    call.take("workspace", workspace, _F32)
    with call:
        _check(lib.tq_decode_splitk_levels(
            _stream(stream, call.device), _ptr(query_rot), ctypes.cast(lv, ctypes.c_void_p), _ptr(key_cache),
            _ptr(value_cache), _ptr(scale_cache), _ptr(block_tables), _ptr(context_lens), _ptr(pi_signs), _ptr(gate),
            _ptr(workspace), _ptr(output), _out_dtype(output), _out_dtype(gate) if gate is not None else 2, batch,
            num_heads, num_kv_heads, head_size, block_size, num_blocks, block_tables.shape[-1], splits,
            max_context_hint, output_stage, softmax_scale, _ptr(status)), "tq_decode_splitk_levels")


def decode_splitk_nz(query_rot, nz_key, nz_value, nz_scales, block_tables, context_lens, output, *, num_heads,
                     num_kv_heads, block_size, num_blocks=0, softmax_scale=1.0, splits=0, max_context_hint=0,
                     workspace=None, code_grid=GRID_MIDRISE, pi_signs=None, gate=None,
                     output_stage=OUT_ROTATED, gain=KV4_FP8_GAIN, inv_sqrt_len=0.0625, precise=False,
                     status=None, stream=None):
    """decode_splitk_prerotated over the fused decoder's NZ-tiled KV4 pools where they lie (head
    size 256, pages of 64 or 128 slots): no import, no second pool. Same results, bit for bit,
    as nz_kv4_import followed by decode_splitk_prerotated."""
    lib = load_library()
    call = _Call("decode_splitk_nz").take("query_rot", query_rot, _F32)
    _decode_operands(call, nz_key, nz_value, nz_scales, block_tables, context_lens, pi_signs, output, gate,
                     status, gate_dtypes=_ANYF, signs_optional=True)
    batch = query_rot.numel() // (num_heads * 256)
    _need_workspace(call, workspace, batch, num_heads, num_kv_heads, 256, block_size, block_tables.shape[-1],
                    splits, max_context_hint)
    with call:
        _check(lib.tq_decode_splitk_nz(
            _stream(stream, call.device), _ptr(query_rot), _ptr(nz_key), _ptr(nz_value), _ptr(nz_scales),
            _ptr(block_tables), _ptr(context_lens), _ptr(pi_signs), _ptr(gate), _ptr(workspace), _ptr(output),
            _out_dtype(output), _out_dtype(gate) if gate is not None else 2, batch, num_heads, num_kv_heads,
            block_size, num_blocks, block_tables.shape[-1], splits, max_context_hint, code_grid, output_stage,
            gain, inv_sqrt_len, softmax_scale, 1 if precise else 0, _ptr(status)), "tq_decode_splitk_nz")


STATIC_WORKSPACE_FLOATS = 2 * 1024 * 1024


def decode_splitk_static(query, key_cache, value_cache, scale_cache, block_tables, context_lens,
                         pi_signs, output, *, num_heads, num_kv_heads, head_size, block_size,
                         num_blocks, inv_sqrt_len, softmax_scale=1.0, splits=0, max_context_hint=0,
                         gate=None, output_stage=OUT_ROTATED, status=None, stream=None):
    """decode_splitk for callers that cannot allocate device memory at launch time (all HBM
    already given to a cache pool, or an allocator they may not call): the split-K partials
    go into the library's own fixed 8 MiB array. Raises TqError(5) when the launch needs more
    than STATIC_WORKSPACE_FLOATS floats. Calls on one device share that array: keep them
    ordered, and make the first call on a device before any stream capture."""
    lib = load_library()
    call = _Call("decode_splitk_static").take("query", query, _BF16)
    _decode_operands(call, key_cache, value_cache, scale_cache, block_tables, context_lens, pi_signs, output,
                     gate, status)
    batch = query.numel() // (num_heads * head_size)
    with call:
        _check(lib.tq_decode_splitk_static(
            _stream(stream, call.device), _ptr(query), _ptr(key_cache), _ptr(value_cache), _ptr(scale_cache),
            _ptr(block_tables), _ptr(context_lens), _ptr(pi_signs), _ptr(gate), _ptr(output),
            _out_dtype(output), batch, num_heads, num_kv_heads, head_size, block_size, num_blocks,
            block_tables.shape[-1], splits, max_context_hint, output_stage, inv_sqrt_len,
            softmax_scale, _ptr(status)), "tq_decode_splitk_static")


def decode_splitk_export(query, key_cache, value_cache, scale_cache, block_tables, context_lens,
                         pi_signs, workspace, *, num_heads, num_kv_heads, head_size, block_size,
                         num_blocks, inv_sqrt_len, splits, softmax_scale=1.0, max_context_hint=0,
                         status=None, stream=None):
    """The export half of decode_splitk: per-split partial records into the workspace."""
    lib = load_library()
    call = _Call("decode_splitk_export").take("query", query, _BF16)
    call.caches(key_cache, value_cache, scale_cache).take("block_tables", block_tables, _I32)
    call.take("context_lens", context_lens, _I32).take("pi_signs", pi_signs, _F32)
    call.take("status", status, _I32, optional=True)
    batch = query.numel() // (num_heads * head_size)
    _need_workspace(call, workspace, batch, num_heads, num_kv_heads, head_size, block_size,
                    block_tables.shape[-1], splits, max_context_hint, always=True)
    with call:
        _check(lib.tq_decode_splitk_export(
            _stream(stream, call.device), _ptr(query), _ptr(key_cache), _ptr(value_cache), _ptr(scale_cache),
            _ptr(block_tables), _ptr(context_lens), _ptr(pi_signs), _ptr(workspace), batch, num_heads,
            num_kv_heads, head_size, block_size, num_blocks, block_tables.shape[-1], splits,
            max_context_hint, inv_sqrt_len, softmax_scale, _ptr(status)), "tq_decode_splitk_export")


def decode_splitk_partials(q, signs, key_cache, value_cache, scale_cache, table, q_rot,
                           workspace, *, requests, heads, rows, head_size, block_size,
                           cache_pages, seq_pages, splits, page_begin, page_count, seq_len,
                           inv_sqrt_len, softmax_scale=1.0, sign_source=SIGNS_F32, status=None,
                           stream=None):
    lib = load_library()
    call = _Call("decode_splitk_partials").take("q", q, _BF16).caches(key_cache, value_cache, scale_cache)
    call.take("table", table, _I32).take("q_rot", q_rot, (torch.bfloat16, torch.int16, torch.uint16), optional=True)
    call.take("workspace", workspace, _F32).take("status", status, _I32, optional=True)
    call.take("signs", signs, _F32 if sign_source == SIGNS_F32 else (torch.bfloat16, torch.int16, torch.int32))
    if workspace.numel() < requests * heads * splits * 16 * (16 + head_size):
        raise ValueError("decode_splitk_partials: workspace too small for the 16-row records of this launch")
    with call:
        _check(lib.tq_decode_splitk_partials(
            _stream(stream, call.device), _ptr(q), _ptr(signs), sign_source, _ptr(key_cache), _ptr(value_cache),
            _ptr(scale_cache), _ptr(table), _ptr(q_rot), _ptr(workspace), requests, heads, rows,
            head_size, block_size, cache_pages, seq_pages, splits, page_begin, page_count, seq_len,
            inv_sqrt_len, softmax_scale, _ptr(status)), "tq_decode_splitk_partials")


def splitk_combine(workspace, pi_signs, gate, output, *, items, rows, rows_stride, head_size,
                   splits, output_stage, inv_sqrt_len, status=None, stream=None):
    lib = load_library()
    call = _Call("splitk_combine").take("workspace", workspace, _F32).take("pi_signs", pi_signs, _F32, optional=True)
    call.take("gate", gate, _F32, optional=True).take("output", output, _ANYF)
    if workspace.numel() < items * splits * rows_stride * (16 + head_size):
        raise ValueError("splitk_combine: workspace smaller than the records the merge reads")
    with call:
        _check(lib.tq_splitk_combine(
            _stream(stream, call.device), _ptr(workspace), _ptr(pi_signs), _ptr(gate), _ptr(output),
            _out_dtype(output), items, rows,
            rows_stride, head_size, splits, output_stage, inv_sqrt_len, _ptr(status)),
            "tq_splitk_combine")


def rotate_query(query, pi_signs, query_rot, *, head_size, inv_sqrt_len, stream=None):
    """query_rot = bf16(Pi query) for every head_size-long bf16 vector of `query`."""
    lib = load_library()
    call = _Call("rotate_query").take("query", query, _BF16).take("pi_signs", pi_signs, _F32)
    call.take("query_rot", query_rot, _BF16)
    with call:
        _check(lib.tq_rotate_query(_stream(stream, call.device), _ptr(query), _ptr(pi_signs), _ptr(query_rot),
                                   query.numel() // head_size, head_size, inv_sqrt_len), "tq_rotate_query")


# ------------------------------------------------------------ stand-alone routines
def hadamard16(x_f16, out):
    """Y = X x H16 on 16x16 FP16 tiles (reference: cube_hadamard16); out float32/float16/bfloat16."""
    lib = load_library()
    call = _Call("hadamard16").take("x_f16", x_f16, (torch.float16,)).take("out", out, _ANYF)
    with call:
        _check(lib.tq_hadamard16(_stream(None, call.device), _ptr(x_f16), _ptr(out), _out_dtype(out),
                                 x_f16.numel() // 256), "tq_hadamard16")


def lloydmax4_quantize(x, packed, recon=None):
    """16-level Lloyd-Max codes of float32 x, packed low nibble first; recon = centroids."""
    lib = load_library()
    call = _Call("lloydmax4_quantize").take("x", x, _F32).take("packed", packed, _BYTES)
    call.take("recon", recon, _F32, optional=True)
    with call:
        _check(lib.tq_lloydmax4_quantize(_stream(None, call.device), _ptr(x), _ptr(packed), _ptr(recon),
                                         x.numel()), "tq_lloydmax4_quantize")


def icdf_quantize(x, packed):
    """int4 codes of 14 sigmoid(x) - 7 for float16 / bfloat16 x, packed low nibble first."""
    lib = load_library()
    call = _Call("icdf_quantize").take("x", x, _ELEM16).take("packed", packed, _BYTES)
    with call:
        _check(lib.tq_icdf_quantize(_stream(None, call.device), _ptr(x), _out_dtype(x), _ptr(packed),
                                    x.numel()), "tq_icdf_quantize")


# --------------------------------------------------------- Lloyd-Max cache variant
def reshape_and_cache_lloydmax(key, value, key_cache, value_cache, scale_cache, slot_mapping, *,
                               num_kv_heads, head_size, block_size, num_blocks, inv_sqrt_len,
                               status=None, stream=None):
    """Aligned writer of the variant: block-diagonal H16, RMS scale, Lloyd-Max codes."""
    lib = load_library()
    call = _Call("reshape_and_cache_lloydmax").take("key", key, (torch.int8, torch.bfloat16))
    call.take("value", value, (key.dtype,)).caches(key_cache, value_cache, scale_cache)
    call.take("slot_mapping", slot_mapping, _I32).take("status", status, _I32, optional=True)
    in_dtype = {torch.int8: 0, torch.bfloat16: 1}[key.dtype]
    num_tokens = key.numel() // (num_kv_heads * head_size)
    with call:
        _check(lib.tq_reshape_and_cache_lloydmax(
            _stream(stream, call.device), _ptr(key), _ptr(value), _ptr(key_cache), _ptr(value_cache),
            _ptr(scale_cache), _ptr(slot_mapping), in_dtype, num_tokens, num_kv_heads, head_size,
            block_size, num_blocks, inv_sqrt_len, _ptr(status)), "tq_reshape_and_cache_lloydmax")


def decode_lloydmax(query, key_cache, value_cache, scale_cache, block_tables, context_lens, output,
                    workspace, *, num_heads, num_kv_heads, head_size, block_size, num_blocks, splits,
                    softmax_scale=1.0, output_stage=OUT_ROTATED, status=None, stream=None):
    """Paged split-K decode over a Lloyd-Max cache: export + combine."""
    lib = load_library()
    call = _Call("decode_lloydmax").take("query", query, _BF16)
    _decode_operands(call, key_cache, value_cache, scale_cache, block_tables, context_lens, None, output,
                     None, status, signs_optional=True)
    batch = query.numel() // (num_heads * head_size)
    rows = num_heads // num_kv_heads
    call.take("workspace", workspace, _F32)
    if workspace.numel() < batch * num_kv_heads * splits * rows * (16 + head_size):
        raise ValueError("decode_lloydmax: workspace too small for the records of this launch")
    with call:
        _check(lib.tq_decode_lloydmax_export(
            _stream(stream, call.device), _ptr(query), _ptr(key_cache), _ptr(value_cache), _ptr(scale_cache),
            _ptr(block_tables), _ptr(context_lens), _ptr(workspace), batch, num_heads, num_kv_heads,
            head_size, block_size, num_blocks, block_tables.shape[-1], splits, softmax_scale,
            _ptr(status)), "tq_decode_lloydmax_export")
        _check(lib.tq_splitk_combine(
            _stream(stream, call.device), _ptr(workspace), None, None, _ptr(output), _out_dtype(output),
            batch * num_kv_heads, rows, rows, head_size, splits, output_stage, 0.0, _ptr(status)),
            "tq_splitk_combine")
