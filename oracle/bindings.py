"""ctypes bindings for the CPU oracle. TEST INFRASTRUCTURE ONLY.

Only the test suite, the smoke check and the CPU-baseline leg of the benchmark
may import this module; the product path never does. `Oracle` wraps
libtq_oracle.so (the restatement in tq_oracle.cpp); `Reference` wraps
_ref/libtq_ref.so (the reference project's own headers compiled in place) and is
only available where that library has been built.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "libtq_oracle.so")
REF_SO = os.path.join(HERE, "_ref", "libtq_ref.so")


def reference_root():
    """A checkout of the reference project: $TQ_REFERENCE_ROOT, else a directory named
    `reference` beside this repository; None when neither is there."""
    for cand in (os.environ.get("TQ_REFERENCE_ROOT"), os.path.join(HERE, "..", "..", "reference")):
        if cand and os.path.exists(os.path.join(cand, "tests", "common", "turboquant_oracle.hpp")):
            return os.path.abspath(cand)
    return None


def build(ref_root=None) -> None:
    """Compile the oracle (and the reference bridge when the reference is present)."""
    ref_root = ref_root or reference_root()
    cmd = ["make", "-C", HERE] + ([f"REF={ref_root}"] if ref_root else [])
    subprocess.run(cmd, check=True, capture_output=True)


def _p(a, t=C.c_void_p):
    return None if a is None else a.ctypes.data_as(t)


def _c(a, dtype):
    return np.ascontiguousarray(a, dtype=dtype)


def bf16_from_f32(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even narrowing of float32 to bf16 bit patterns (uint16)."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)
    return r


def f32_from_bf16(x: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(x, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


class Oracle:
    def __init__(self, path: str = ORACLE_SO):
        if not os.path.exists(path):
            build()
        self.lib = C.CDLL(path)
        L = self.lib
        L.tqo_pi_sign_writer.restype = C.c_int
        L.tqo_pi_sign_decode.restype = C.c_int
        L.tqo_reshape_and_cache.restype = C.c_int
        L.tqo_reshape_scatter.restype = C.c_int
        L.tqo_hardware_threads.restype = C.c_int

    # ------------------------------------------------------------ rotation
    def writer_signs(self, d):
        return np.array([self.lib.tqo_pi_sign_writer(c) for c in range(d)], dtype=np.int32)

    def decode_signs(self, d):
        return np.array([self.lib.tqo_pi_sign_decode(c) for c in range(d)], dtype=np.int32)

    def build_tables_i8(self, signs):
        signs = _c(signs, np.int32)
        d = signs.size
        out = np.zeros(2 * (d // 32) * 32 * 32, dtype=np.int8)
        self.lib.tqo_build_tables_i8(C.c_int(d), _p(signs), _p(out))
        return out

    def rotate_int(self, signs, x, dense=False):
        signs = _c(signs, np.int32)
        x = _c(x, np.int64)
        y = np.zeros_like(x)
        fn = self.lib.tqo_rotate_dense_int if dense else self.lib.tqo_rotate_int
        fn(C.c_int(x.size), _p(signs), _p(x), _p(y))
        return y

    def butterfly_f32(self, signs, x, ingress=True, scale=1.0):
        signs = _c(signs, np.float32)
        x = _c(x, np.float32)
        y = np.zeros_like(x)
        self.lib.tqo_butterfly_f32(C.c_int(x.size), _p(signs), _p(x), _p(y),
                                   C.c_int(1 if ingress else 0), C.c_float(scale))
        return y

    def rotate_query_bf16(self, q_bf16, signs, inv_sqrt_len):
        q = _c(q_bf16, np.uint16)
        d = q.shape[-1]
        rows = q.size // d
        out = np.zeros_like(q)
        self.lib.tqo_rotate_query_bf16(C.c_int(rows), C.c_int(d), _p(_c(signs, np.float32)),
                                       C.c_float(inv_sqrt_len), _p(q), _p(out))
        return out

    # ------------------------------------------------------------- writers
    def reshape_and_cache(self, key, value, slots, signs, H, d, S, P, inv_sqrt_len,
                          key_cache=None, value_cache=None, scale_cache=None, threads=1):
        """Aligned writer. key/value: int8 or bf16-bits (uint16) [T][H*d]."""
        dtype = 0 if key.dtype == np.int8 else 1
        key = np.ascontiguousarray(key)
        value = np.ascontiguousarray(value)
        T = key.size // (H * d)
        nbytes = P * H * S * d // 2
        kc = np.zeros(nbytes, np.uint8) if key_cache is None else key_cache
        vc = np.zeros(nbytes, np.uint8) if value_cache is None else value_cache
        sc = np.zeros(2 * P * H * S, np.float32) if scale_cache is None else scale_cache
        pw = np.zeros(P, np.uint8)
        bad = self.lib.tqo_reshape_and_cache(
            C.c_int(dtype), _p(key), _p(value), _p(_c(slots, np.int32)), _p(_c(signs, np.int32)),
            C.c_int(T), C.c_int(H), C.c_int(d), C.c_int(S), C.c_int(P), C.c_float(inv_sqrt_len),
            _p(kc), _p(vc), _p(sc), _p(pw), C.c_int(threads))
        return kc, vc, sc, pw, bad

    def reshape_and_cache_varlen(self, key, value, slots, signs, cu_seqlens, H, d, S, P, inv_sqrt_len,
                                 key_cache, value_cache, scale_cache):
        """Aligned writer over ragged requests (bf16 bits), in place on the given caches."""
        cu = _c(cu_seqlens, np.int32)
        return self.lib.tqo_reshape_and_cache_varlen(
            _p(_c(key, np.uint16)), _p(_c(value, np.uint16)), _p(_c(slots, np.int32)),
            _p(_c(signs, np.int32)), _p(cu), C.c_int(cu.size - 1), C.c_int(H), C.c_int(d), C.c_int(S),
            C.c_int(P), C.c_float(inv_sqrt_len), _p(key_cache), _p(value_cache), _p(scale_cache))

    def reshape_scatter(self, key, value, slots, signs, cu_seqlens, num_requests, H, d, S, P,
                        inv_sqrt_len, key_cache, value_cache, scale_cache):
        """Scatter writer, in place on the given caches. key/value bf16 bits [tokens][H*d]."""
        rc = self.lib.tqo_reshape_scatter(
            _p(_c(key, np.uint16)), _p(_c(value, np.uint16)), _p(_c(slots, np.int32)),
            _p(_c(signs, np.float32)), _p(None if cu_seqlens is None else _c(cu_seqlens, np.int32)),
            C.c_int(num_requests), C.c_int(H), C.c_int(d), C.c_int(S), C.c_int(P),
            C.c_float(inv_sqrt_len), _p(key_cache), _p(value_cache), _p(scale_cache))
        return rc

    # -------------------------------------------------------------- decode
    def partition(self, pages, splits, split):
        b, n = C.c_uint32(), C.c_uint32()
        self.lib.tqo_partition(C.c_uint32(pages), C.c_uint32(splits), C.c_uint32(split),
                               C.byref(b), C.byref(n))
        return b.value, n.value

    def decode_partial(self, q_rot, key_cache, value_cache, scale_cache, block_table, H, head, d,
                       S, P, ctx_len, tok_begin, tok_end, softmax_scale=1.0):
        q_rot = _c(q_rot, np.uint16)
        rows = q_rot.size // d
        m = np.zeros(rows)
        l = np.zeros(rows)
        acc = np.zeros((rows, d))
        self.lib.tqo_decode_partial(
            _p(q_rot), C.c_int(rows), _p(key_cache), _p(value_cache),
            _p(_c(scale_cache, np.float32)), _p(_c(block_table, np.int32)), C.c_int(H),
            C.c_int(head), C.c_int(d), C.c_int(S), C.c_int(P), C.c_int(ctx_len),
            C.c_int(tok_begin), C.c_int(tok_end), C.c_float(softmax_scale), _p(m), _p(l), _p(acc))
        return m, l, acc

    def lse_merge(self, states):
        """states: list of (m, l, acc[d]) -> merged (m, l, acc)."""
        d = states[0][2].size
        m, l = C.c_double(-3.0e38), C.c_double(0.0)
        acc = np.zeros(d)
        for (m2, l2, a2) in states:
            self.lib.tqo_lse_merge(C.c_int(d), C.byref(m), C.byref(l), _p(acc), C.c_double(m2),
                                   C.c_double(l2), _p(_c(a2, np.float64)))
        return m.value, l.value, acc

    def decode(self, q, key_cache, value_cache, scale_cache, block_tables, context_lens, signs,
               Hq, Hkv, d, S, P, inv_sqrt_len, softmax_scale=1.0, output_stage=0, gate=None,
               threads=1, q_f16=False):
        """q: bf16 bits, or FP16 bits with q_f16=True (rotation then stays FP32)."""
        q = _c(q, np.uint16)
        B = q.size // (Hq * d)
        bt = _c(block_tables, np.int32)
        out = np.zeros((B, Hq, d))
        fn = self.lib.tqo_decode_f16q if q_f16 else self.lib.tqo_decode
        fn(
            _p(q), _p(key_cache), _p(value_cache), _p(_c(scale_cache, np.float32)), _p(bt),
            _p(_c(context_lens, np.int32)), _p(_c(signs, np.float32)),
            _p(None if gate is None else _c(gate, np.float32)), C.c_int(B), C.c_int(Hq),
            C.c_int(Hkv), C.c_int(d), C.c_int(S), C.c_int(P), C.c_int(bt.shape[-1]),
            C.c_float(inv_sqrt_len), C.c_float(softmax_scale), C.c_int(output_stage), _p(out),
            C.c_int(threads))
        return out

    def hardware_threads(self):
        return self.lib.tqo_hardware_threads()

    # ------------------------------------------------------------ routines
    def hadamard16(self, x_f16):
        """Y = X x H16 per 16x16 tile; x_f16: FP16 bits [tiles][16][16] -> float32."""
        x = _c(x_f16, np.uint16)
        y = np.zeros(x.size, np.float32)
        self.lib.tqo_hadamard16(_p(x), _p(y), C.c_int(x.size // 256))
        return y.reshape(-1, 16, 16)

    def lloydmax4_tables(self):
        c, t = np.zeros(16, np.float32), np.zeros(15, np.float32)
        self.lib.tqo_lloydmax4_tables(_p(c), _p(t))
        return c, t

    def lloydmax4_quantize(self, x):
        """-> (packed bytes, centroid reconstruction)."""
        x = _c(x, np.float32).reshape(-1)
        packed = np.zeros(x.size // 2, np.uint8)
        recon = np.zeros(x.size, np.float32)
        self.lib.tqo_lloydmax4_quantize(_p(x), _p(packed), _p(recon), C.c_longlong(x.size))
        return packed, recon

    def icdf_quantize(self, x_bits, bf16):
        x = _c(x_bits, np.uint16).reshape(-1)
        packed = np.zeros(x.size // 2, np.uint8)
        self.lib.tqo_icdf_quantize(_p(x), C.c_int(1 if bf16 else 0), _p(packed), C.c_longlong(x.size))
        return packed

    def reshape_and_cache_lm(self, key, value, slots, H, d, S, P, inv_sqrt_len, key_cache=None,
                             value_cache=None, scale_cache=None):
        """Aligned writer, block-diagonal H16 + RMS scale + Lloyd-Max codes."""
        dtype = 0 if key.dtype == np.int8 else 1
        key, value = np.ascontiguousarray(key), np.ascontiguousarray(value)
        T = key.size // (H * d)
        nbytes = P * H * S * d // 2
        kc = np.zeros(nbytes, np.uint8) if key_cache is None else key_cache
        vc = np.zeros(nbytes, np.uint8) if value_cache is None else value_cache
        sc = np.zeros(2 * P * H * S, np.float32) if scale_cache is None else scale_cache
        bad = self.lib.tqo_reshape_and_cache_lm(
            C.c_int(dtype), _p(key), _p(value), _p(_c(slots, np.int32)), C.c_int(T), C.c_int(H),
            C.c_int(d), C.c_int(S), C.c_int(P), C.c_float(inv_sqrt_len), _p(kc), _p(vc), _p(sc))
        return kc, vc, sc, bad

    def lm_rotate_query_bf16(self, q, d):
        q = _c(q, np.uint16)
        out = np.zeros_like(q)
        self.lib.tqo_lm_rotate_query_bf16(C.c_int(q.size // d), C.c_int(d), _p(q), _p(out))
        return out

    def decode_lm(self, q, key_cache, value_cache, scale_cache, block_tables, context_lens, Hq,
                  Hkv, d, S, P, softmax_scale=1.0, output_stage=0, threads=1):
        q = _c(q, np.uint16)
        B = q.size // (Hq * d)
        bt = _c(block_tables, np.int32)
        out = np.zeros((B, Hq, d))
        self.lib.tqo_decode_lm(
            _p(q), _p(key_cache), _p(value_cache), _p(_c(scale_cache, np.float32)), _p(bt),
            _p(_c(context_lens, np.int32)), C.c_int(B), C.c_int(Hq), C.c_int(Hkv), C.c_int(d),
            C.c_int(S), C.c_int(P), C.c_int(bt.shape[-1]), C.c_float(softmax_scale),
            C.c_int(output_stage), _p(out), C.c_int(threads))
        return out

    # ---- NZ-tiled KV4/FP8 cache (the fused decoder's format; head size 256)
    KV4_GAIN = 2.9832882881

    def nz_tiled_packed_byte(self, slot, head, column, H, packed=128):
        self.lib.tqo_nz_tiled_packed_byte.restype = C.c_size_t
        return self.lib.tqo_nz_tiled_packed_byte(C.c_size_t(slot), C.c_size_t(head), C.c_size_t(column),
                                                 C.c_size_t(H), C.c_size_t(packed))

    def nz_kv4_import(self, nz_key, nz_value, nz_scales, H, S, P, gain=KV4_GAIN):
        """NZ-tiled pool -> (key_cache, value_cache, scale_cache) in the native layout."""
        kc = np.zeros(P * H * S * 128, np.uint8)
        vc = np.zeros_like(kc)
        sc = np.zeros(2 * P * H * S, np.float32)
        rc = self.lib.tqo_nz_kv4_import(_p(_c(nz_key, np.uint8)), _p(_c(nz_value, np.uint8)),
                                        _p(_c(nz_scales, np.float32)), C.c_int(H), C.c_int(S),
                                        C.c_int(P), C.c_float(gain), _p(kc), _p(vc), _p(sc))
        assert rc == 0
        return kc, vc, sc

    def signed_hadamard(self, x, signs):
        """Pi x with Pi = diag(s) H diag(s) / sqrt(d), rows of x."""
        x = _c(x, np.float32)
        d = x.shape[-1]
        y = np.zeros_like(x)
        self.lib.tqo_signed_hadamard(C.c_int(d), _p(_c(signs, np.float32)), _p(x), _p(y), C.c_int(x.size // d))
        return y

    def nz_kv4_decode(self, q_rot, nz_key, nz_value, nz_scales, block_tables, context_lens, Hq, H, S,
                      softmax_scale=0.0625, gain=KV4_GAIN):
        q = _c(q_rot, np.float32)
        B = q.size // (Hq * 256)
        bt = _c(block_tables, np.int32).reshape(B, -1)
        out = np.zeros((B, Hq, 256), np.float32)
        self.lib.tqo_nz_kv4_decode(_p(q), _p(_c(nz_key, np.uint8)), _p(_c(nz_value, np.uint8)),
                                   _p(_c(nz_scales, np.float32)), _p(bt),
                                   _p(_c(context_lens, np.int32)), C.c_int(B), C.c_int(Hq), C.c_int(H),
                                   C.c_int(S), C.c_int(bt.shape[1]), C.c_float(softmax_scale),
                                   C.c_float(gain), _p(out))
        return out


    def kv4_lloydmax_lut(self):
        out = np.zeros(16, np.float32)
        self.lib.tqo_kv4_lloydmax_lut(_p(out))
        return out

    def nz_kv4_decode_lut(self, q_rot, nz_key, nz_value, nz_scales, block_tables, context_lens, Hq, H, S,
                          softmax_scale=0.0625, levels=None):
        """nz_kv4_decode over a cache written on the Lloyd-Max codebook (levels by bin index, gain 1)."""
        q = _c(q_rot, np.float32)
        B = q.size // (Hq * 256)
        bt = _c(block_tables, np.int32).reshape(B, -1)
        lv = _c(self.kv4_lloydmax_lut() if levels is None else levels, np.float32)
        out = np.zeros((B, Hq, 256), np.float32)
        self.lib.tqo_nz_kv4_decode_lut(_p(q), _p(_c(nz_key, np.uint8)), _p(_c(nz_value, np.uint8)),
                                       _p(_c(nz_scales, np.float32)), _p(bt),
                                       _p(_c(context_lens, np.int32)), C.c_int(B), C.c_int(Hq), C.c_int(H),
                                       C.c_int(S), C.c_int(bt.shape[1]), C.c_float(softmax_scale), _p(lv), _p(out))
        return out


class Reference:
    """The reference project's own golden models (oracle/_ref/libtq_ref.so)."""

    @staticmethod
    def available() -> bool:
        return os.path.exists(REF_SO)

    def __init__(self, path: str = REF_SO):
        self.lib = C.CDLL(path)
        L = self.lib
        L.ref_writer_reference.restype = C.c_int
        L.ref_scatter_reference.restype = C.c_int
        L.ref_decode_fixture_new.restype = C.c_void_p
        L.ref_decode_fixture_get.restype = C.c_size_t
        L.ref_workspace_floats.restype = C.c_ulonglong
        L.ref_lloydmax4_code.restype = C.c_uint

    def writer_signs(self, d):
        return np.array([self.lib.ref_writer_pi_sign(c) for c in range(d)], dtype=np.int32)

    def writer_tables(self, d):
        out = np.zeros(2 * (d // 32) * 1024, np.int8)
        self.lib.ref_writer_build_tables(C.c_int(d), _p(out))
        return out

    def writer_fixture(self, T, H, d, S=16):
        key = np.zeros(T * H * d, np.int8)
        value = np.zeros_like(key)
        slots = np.zeros(T, np.int32)
        self.lib.ref_writer_fixture(C.c_int(T), C.c_int(H), C.c_int(d), C.c_int(S), _p(key),
                                    _p(value), _p(slots))
        return key, value, slots, 2 * (T // S) + 2

    def writer_reference(self, key, value, slots, H, d, S, P, threads=1):
        key = _c(key, np.int8)
        T = key.size // (H * d)
        kc = np.zeros(P * H * S * d // 2, np.uint8)
        vc = np.zeros_like(kc)
        sc = np.zeros(2 * P * H * S, np.float32)
        pw = np.zeros(P, np.uint8)
        bad = self.lib.ref_writer_reference(
            C.c_int(T), C.c_int(H), C.c_int(d), C.c_int(S), C.c_int(P), _p(key),
            _p(_c(value, np.int8)), _p(_c(slots, np.int32)), _p(kc), _p(vc), _p(sc), _p(pw),
            C.c_int(threads))
        return kc, vc, sc, pw, bad

    def writer_fixture_audit_ok(self, T, H, d, S=16):
        return bool(self.lib.ref_writer_fixture_audit_ok(C.c_int(T), C.c_int(H), C.c_int(d),
                                                         C.c_int(S)))

    def scatter_reference(self, num_requests, H, S, P, slots, cu_seqlens, zero_token, key_cache,
                          value_cache, scale_cache):
        """In place on the caches; returns (zero_rows, key_bf16, value_bf16)."""
        slots = _c(slots, np.int32)
        T = slots.size
        k = np.zeros(T * H * 256, np.uint16)
        v = np.zeros_like(k)
        rc = self.lib.ref_scatter_reference(
            C.c_int(num_requests), C.c_int(H), C.c_int(S), C.c_int(P), _p(slots),
            _p(None if cu_seqlens is None else _c(cu_seqlens, np.int32)), C.c_int(zero_token),
            _p(key_cache), _p(value_cache), _p(scale_cache), _p(k), _p(v))
        return rc, k, v

    def fused_fixture(self, context, requests, kv_heads, group_heads, page_tokens):
        return RefFusedFixture(self, context, requests, kv_heads, group_heads, page_tokens)

    def fused_signs(self, d=256):
        self.lib.ref_fused_sign.restype = C.c_float
        return np.array([self.lib.ref_fused_sign(C.c_int(c)) for c in range(d)], np.float32)

    def fused_pi_apply(self, x):
        x = _c(x, np.float32)
        y = np.zeros(256, np.float32)
        self.lib.ref_fused_pi_apply(_p(x), _p(y))
        return y

    def kv4_gain(self):
        self.lib.ref_kv4_gain.restype = C.c_float
        return float(self.lib.ref_kv4_gain())

    def nz_tiled_packed_byte(self, slot, head, column, H, packed=128):
        self.lib.ref_nz_tiled_packed_byte.restype = C.c_uint64
        return self.lib.ref_nz_tiled_packed_byte(C.c_uint64(slot), C.c_uint64(head), C.c_uint64(column),
                                                 C.c_uint64(H), C.c_uint64(packed))

    def decode_fixture(self, n, batch, heads, rows, page_tokens, live=-1, fill=1):
        h = self.lib.ref_decode_fixture_new(C.c_int(n), C.c_int(batch), C.c_int(heads),
                                            C.c_int(rows), C.c_int(page_tokens), C.c_int(live),
                                            C.c_int(fill))
        return RefDecodeFixture(self, C.c_void_p(h))

    def single_token_fixture(self, pages):
        """The reference's 6-row single-token decode fixture (1 request, 4 KV heads x 6 query
        rows, head size 256, 128-token pages, `pages` <= 8): raw bf16 query [4][6][256], the
        strip cache (unmapped pages keep 0xAA bytes / NaN scales), the block table."""
        q = np.zeros(4 * 6 * 256, np.uint16)
        key = np.full(9 * 4 * 8 * 2048, 0xAA, np.uint8)
        value = np.full_like(key, 0xAA)
        scales = np.full(2 * 9 * 4 * 128, np.nan, np.float32)
        table = np.zeros(pages, np.int32)
        self.lib.ref_single_token_fixture(C.c_int(pages), _p(q), _p(key), _p(value), _p(scales), _p(table))
        gate = np.zeros(4 * 6 * 256, np.float32)
        self.lib.ref_single_token_gate(_p(gate))
        return dict(q=q.reshape(4, 6, 256), key=key, value=value, scales=scales, table=table,
                    gate=gate.reshape(4, 6, 256))

    def single_token_golden(self, head, pages):
        """GoldenDecode of the fixture for one KV head: m, l [6]; acc, rotated, context, q_rot [6][256]."""
        m, l = np.zeros(6, np.float32), np.zeros(6, np.float32)
        arrs = [np.zeros((6, 256), np.float32) for _ in range(4)]
        self.lib.ref_single_token_golden(C.c_int(head), C.c_int(pages), _p(m), _p(l), *[_p(a) for a in arrs])
        return dict(m=m, l=l, acc=arrs[0], rotated=arrs[1], context=arrs[2], q_rot=arrs[3])

    def kv4_lloydmax_lut(self):
        """(levels[16], thresholds[15], gain) of TurboQuantLloydMaxTraits<KV4_FP8>."""
        levels, thr, gain = np.zeros(16, np.float32), np.zeros(15, np.float32), np.zeros(1, np.float32)
        self.lib.ref_kv4_lloydmax_lut(_p(levels), _p(thr), _p(gain))
        return levels, thr, float(gain[0])

    def fused_descriptor_layout_matches(self):
        return bool(self.lib.ref_fused_descriptor_layout_matches())

    def rotation_table_bf16(self):
        out = np.zeros(16 * 1024, np.uint16)
        self.lib.ref_decode_rotation_table(_p(out))
        return out

    def decode_signs(self, d=256):
        return np.array([self.lib.ref_decode_pi_sign(c) for c in range(d)], dtype=np.int32)

    def partition(self, pages, splits, split):
        b, n = C.c_uint(), C.c_uint()
        self.lib.ref_partition(C.c_uint(pages), C.c_uint(splits), C.c_uint(split), C.byref(b),
                               C.byref(n))
        return b.value, n.value

    def workspace_floats(self, requests, heads, splits):
        return self.lib.ref_workspace_floats(C.c_uint(requests), C.c_uint(heads), C.c_uint(splits))

    def lloydmax4_tables(self):
        c = np.zeros(16, np.float32)
        t = np.zeros(15, np.float32)
        self.lib.ref_lloydmax4_tables(_p(c), _p(t))
        return c, t

    def lloydmax4_code(self, x):
        return self.lib.ref_lloydmax4_code(C.c_float(x))

    def lloydmax_fixture(self, n, rows, boundaries):
        out = np.zeros(n * rows, np.float32)
        self.lib.ref_lloydmax_fixture(C.c_uint(n), C.c_uint(rows), C.c_int(1 if boundaries else 0), _p(out))
        return out

    def lloydmax4_pack(self, x):
        x = _c(x, np.float32)
        out = np.zeros(x.size // 2, np.uint8)
        self.lib.ref_lloydmax4_pack(_p(x), C.c_uint(x.size), _p(out))
        return out

    def hadamard16(self, x_f16):
        x = _c(x_f16, np.uint16)
        y = np.zeros(256, np.float32)
        self.lib.ref_hadamard16(_p(x), _p(y))
        return y.reshape(16, 16)

    def icdf_fixture(self, bf16, tiles):
        bits = np.zeros(tiles * 1024, np.uint16)
        packed = np.zeros(tiles * 512, np.uint8)
        self.lib.ref_icdf_fixture(C.c_int(1 if bf16 else 0), C.c_uint(tiles), _p(bits), _p(packed))
        return bits, packed


class RefFusedFixture:
    """fused_decode_opt_test::Fixture: a KV4/FP8 NZ-tiled cache with its FP64 expected output."""
    _KINDS = {"query": (0, np.float32), "key": (1, np.uint8), "value": (2, np.uint8),
              "scales": (3, np.float32), "table": (4, np.int32), "lengths": (5, np.int32),
              "expected": (6, np.float32)}

    def __init__(self, ref, context, requests, kv_heads, group_heads, page_tokens):
        self.ref = ref
        ref.lib.ref_fused_fixture_new.restype = C.c_void_p
        ref.lib.ref_fused_fixture_get.restype = C.c_size_t
        self.h = C.c_void_p(ref.lib.ref_fused_fixture_new(C.c_int(context), C.c_int(requests),
                                                          C.c_int(kv_heads), C.c_int(group_heads),
                                                          C.c_int(page_tokens)))
        dims = (C.c_int * 2)()
        ref.lib.ref_fused_fixture_dims(self.h, dims)
        self.pages, self.physical_pages = list(dims)
        self.context, self.requests, self.kv_heads = context, requests, kv_heads
        self.group_heads, self.page_tokens = group_heads, page_tokens

    def get(self, name):
        which, dt = self._KINDS[name]
        n = self.ref.lib.ref_fused_fixture_get(self.h, C.c_int(which), None)
        out = np.zeros(n // np.dtype(dt).itemsize, dt)
        if n:
            self.ref.lib.ref_fused_fixture_get(self.h, C.c_int(which), _p(out))
        return out

    def expected_row(self, row, stage):
        out = np.zeros(256, np.float32)
        self.ref.lib.ref_fused_expected_row(self.h, C.c_size_t(row), C.c_uint(stage), _p(out))
        return out

    def raw_query_f16_bits(self):
        out = np.zeros(self.requests * self.kv_heads * self.group_heads * 256, np.uint16)
        self.ref.lib.ref_fused_raw_query_bits(self.h, _p(out))
        return out

    def gate_f16_bits(self):
        out = np.zeros(self.requests * self.kv_heads * self.group_heads * 256, np.uint16)
        self.ref.lib.ref_fused_gate_bits(self.h, _p(out))
        return out

    def __del__(self):
        try:
            self.ref.lib.ref_fused_fixture_free(self.h)
        except Exception:
            pass


class RefDecodeFixture:
    _KINDS = {"q_rot": (0, np.uint16), "key": (1, np.uint8), "value": (2, np.uint8),
              "scales": (3, np.float32), "gate": (4, np.float32), "signs": (5, np.float32),
              "table": (6, np.uint32), "expected": (7, np.float32), "raw_q": (8, np.uint16)}

    def __init__(self, ref, handle):
        self.ref, self.h = ref, handle
        dims = (C.c_int * 7)()
        ref.lib.ref_decode_fixture_dims(self.h, dims)
        (self.tokens, self.seq_len, self.pages, self.requests, self.heads, self.rows,
         self.page_tokens) = list(dims)

    def get(self, name):
        which, dt = self._KINDS[name]
        n = self.ref.lib.ref_decode_fixture_get(self.h, C.c_int(which), None)
        out = np.zeros(n // np.dtype(dt).itemsize, dt)
        if n:
            self.ref.lib.ref_decode_fixture_get(self.h, C.c_int(which), _p(out))
        return out

    def aic_partial(self, request, head, begin, pages):
        m = np.zeros(16)
        l = np.zeros(16)
        acc = np.zeros((16, 256))
        self.ref.lib.ref_decode_aic_partial(self.h, C.c_int(request), C.c_int(head),
                                            C.c_uint(begin), C.c_uint(pages), _p(m), _p(l), _p(acc))
        return m, l, acc

    def __del__(self):
        try:
            self.ref.lib.ref_decode_fixture_free(self.h)
        except Exception:
            pass
