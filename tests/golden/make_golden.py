"""Generates the golden vectors under tests/golden/ from the reference project's own
golden models (oracle/_ref/libtq_ref.so, built by oracle/Makefile from a checkout of
the reference). Run from the repository root:  python tests/golden/make_golden.py
The vectors pin the CPU oracle where the reference checkout is not available."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle.bindings import Reference  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    r = Reference()
    # aligned writer: reference geometry (4 heads x 256, 3 strips) and the d=128 shapes
    for name, (T, H, d) in {"writer_h4_d256_t48": (48, 4, 256), "writer_h1_d128_t16": (16, 1, 128),
                            "writer_h8_d128_t32": (32, 8, 128)}.items():
        key, value, slots, P = r.writer_fixture(T, H, d)
        kc, vc, sc, pw, bad = r.writer_reference(key, value, slots, H, d, 16, P)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), key=key, value=value, slots=slots,
                            signs=r.writer_signs(d), tables=r.writer_tables(d), key_cache=kc,
                            value_cache=vc, scale_bits=sc.view(np.uint32), page_written=pw,
                            geometry=np.array([T, H, d, 16, P]), bad=np.array([bad]))
    # scatter writer (d = 256 in the reference), with its all-zero token
    H, S, P = 2, 16, 6
    rng = np.random.default_rng(1)
    cu = np.array([0, 3, 8], np.int32)
    slots = np.array([32, 33, 34, 70, 71, 72, -1, 90], np.int32)
    kc = rng.integers(0, 256, P * H * S * 128, dtype=np.uint8)
    vc = rng.integers(0, 256, P * H * S * 128, dtype=np.uint8)
    sc = rng.standard_normal(2 * P * H * S).astype(np.float32)
    ekc, evc, esc = kc.copy(), vc.copy(), sc.copy()
    zero_rows, kb, vb = r.scatter_reference(2, H, S, P, slots, cu, 1, ekc, evc, esc)
    np.savez_compressed(os.path.join(HERE, "scatter_h2_d256.npz"), key=kb, value=vb, slots=slots,
                        cu_seqlens=cu, signs=r.writer_signs(256), prior_key=kc, prior_value=vc,
                        prior_scale=sc, key_cache=ekc, value_cache=evc,
                        scale_bits=esc.view(np.uint32), geometry=np.array([2, H, 256, S, P]),
                        zero_rows=np.array([zero_rows]))
    # split-K decode fixture: 2 pages of 128 tokens, 1 request x 2 heads, 16 rows; whole and tail
    for name, live, fill in (("decode_aic_p2", -1, 1), ("decode_aic_p2_tail", 150, 2)):
        f = r.decode_fixture(256, 1, 2, 16, 128, live, fill)
        parts = {}
        for head in range(2):
            for (b, c) in ((0, 2), (0, 1), (1, 1)):
                m, l, acc = f.aic_partial(0, head, b, c)
                parts[f"m_h{head}_b{b}_c{c}"] = m
                parts[f"l_h{head}_b{b}_c{c}"] = l
                parts[f"acc_h{head}_b{b}_c{c}"] = acc
        np.savez_compressed(os.path.join(HERE, name + ".npz"), q_rot=f.get("q_rot"),
                            raw_q=f.get("raw_q"), key=f.get("key"), value=f.get("value"),
                            scale_bits=f.get("scales").view(np.uint32), table=f.get("table"),
                            signs=r.decode_signs(), rotation_table=r.rotation_table_bf16(),
                            dims=np.array([f.tokens, f.seq_len, f.pages, f.requests, f.heads, f.rows,
                                           f.page_tokens]), **parts)
    # full-context expected (6 rows per head, gate, un-rotation): 1 request x 4 heads, 3 pages
    f = r.decode_fixture(384, 1, 4, 6, 128, -1, 1)
    np.savez_compressed(os.path.join(HERE, "decode_full_p3.npz"), q_rot=f.get("q_rot"),
                        key=f.get("key"), value=f.get("value"),
                        scale_bits=f.get("scales").view(np.uint32), table=f.get("table"),
                        gate=f.get("gate"), expected=f.get("expected"), signs=r.decode_signs(),
                        dims=np.array([f.tokens, f.seq_len, f.pages, f.requests, f.heads, f.rows,
                                       f.page_tokens]))
    # the 6-row single-token decode fixture over two pages, with its golden state per KV head
    st = r.single_token_fixture(2)
    gold = {f"{k}_h{h}": v for h in range(4) for k, v in r.single_token_golden(h, 2).items()}
    np.savez_compressed(os.path.join(HERE, "single_token_p2.npz"), q=st["q"], key=st["key"], value=st["value"],
                        scale_bits=st["scales"].view(np.uint32), table=st["table"], gate=st["gate"],
                        signs=r.decode_signs(), **gold)
    # partition table and Lloyd-Max codebook
    part = np.array([[p, k, s, *r.partition(p, k, s)] for p in (1, 3, 4, 5, 7, 8, 100)
                     for k in (1, 2, 4, 8, 16) for s in range(k)], np.int64)
    c, t = r.lloydmax4_tables()
    np.savez_compressed(os.path.join(HERE, "contract.npz"), partition=part, lloydmax4_centroids=c,
                        lloydmax4_thresholds=t,
                        workspace_floats=np.array([r.workspace_floats(3, 4, 8)]))
    # the stand-alone routines: the reference's Lloyd-Max probe fixture with its packed codes,
    # dyadic Hadamard tiles through golden_hadamard16, the ICDF probe fixture with its oracle bytes
    lm_x = r.lloydmax_fixture(128, 4, True)
    rng = np.random.default_rng(16)
    h16_x = (rng.integers(-64, 65, size=(6, 16, 16)) / 8).astype(np.float16)
    h16_y = np.stack([r.hadamard16(h16_x[i].view(np.uint16)) for i in range(6)])
    f16_bits, f16_packed = r.icdf_fixture(False, 2)
    bf16_bits, bf16_packed = r.icdf_fixture(True, 2)
    np.savez_compressed(os.path.join(HERE, "routines.npz"), lm_x=lm_x, lm_packed=r.lloydmax4_pack(lm_x),
                        lm_centroids=c, lm_thresholds=t, h16_x=h16_x.view(np.uint16), h16_y=h16_y,
                        icdf_f16_bits=f16_bits, icdf_f16_packed=f16_packed,
                        icdf_bf16_bits=bf16_bits, icdf_bf16_packed=bf16_packed)
    # the fused decoder's KV4/FP8 NZ-tiled cache fixture (ragged context, two page sizes) with
    # its FP64 expected output, and a table of NzTiledPackedByte values
    for name, (n, b, h, g, S) in {"fused_kv4_s64": (200, 2, 2, 4, 64), "fused_kv4_s128": (300, 1, 3, 2, 128)}.items():
        fx = r.fused_fixture(n, b, h, g, S)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), query=fx.get("query"), key=fx.get("key"),
                            value=fx.get("value"), scale_bits=fx.get("scales").view(np.uint32),
                            table=fx.get("table")[:b * fx.pages].reshape(b, fx.pages),
                            lengths=fx.get("lengths")[:b], expected=fx.get("expected"),
                            dims=np.array([n, b, h, g, S, fx.pages, fx.physical_pages]),
                            gain=np.float32(r.kv4_gain()), pi_signs=r.fused_signs(),
                            gate_f16_bits=fx.gate_f16_bits(), raw_query_f16_bits=fx.raw_query_f16_bits(),
                            expected_unrotated=np.stack([fx.expected_row(i, 1) for i in range(b * h * g)]),
                            expected_gated=np.stack([fx.expected_row(i, 2) for i in range(b * h * g)]),
                            nz_bytes=np.array([[slot, head, col, H, r.nz_tiled_packed_byte(slot, head, col, H)]
                                               for H in (1, 3) for slot in (0, 1, 63, 64, 127)
                                               for head in range(H) for col in (0, 31, 32, 127)], np.int64))
    for fn in sorted(os.listdir(HERE)):
        if fn.endswith(".npz"):
            print(fn, os.path.getsize(os.path.join(HERE, fn)))


if __name__ == "__main__":
    main()
