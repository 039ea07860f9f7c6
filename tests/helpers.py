"""Seeded synthetic inputs and small utilities shared by the tests."""
from __future__ import annotations

import math

import numpy as np

from oracle.bindings import bf16_from_f32, f32_from_bf16  # noqa: F401


def inv_sqrt_len(d: int) -> float:
    """1/sqrt(d) rounded the way the reference host computes it (float arithmetic)."""
    return float(np.float32(1.0) / np.sqrt(np.float32(d)))


def int8_activations(rng, T, H, d):
    """int8 K and V uniform in [-127, 127] (the single-strip int8 case of the benchmark configurations)."""
    k = rng.integers(-127, 128, size=(T, H * d), dtype=np.int64).astype(np.int8)
    v = rng.integers(-127, 128, size=(T, H * d), dtype=np.int64).astype(np.int8)
    return k, v


def gaussian_outlier_activations(rng, T, H, d, integer=False):
    """N(0,1) with 1% of elements x20 (the bf16 prefill case of the benchmark configurations), as bf16 bit patterns.
    integer=True rounds the same draws (x16, clipped to [-127, 127]) to integers so
    the result is bit-checkable."""
    out = []
    for _ in range(2):
        x = rng.standard_normal((T, H * d)).astype(np.float32)
        mask = rng.random((T, H * d)) < 0.01
        x = np.where(mask, x * 20.0, x).astype(np.float32)
        if integer:
            x = np.clip(np.rint(x * 16.0), -127, 127).astype(np.float32)
        out.append(bf16_from_f32(x))
    return out[0], out[1]


def page_permutation_slots(rng, strips, S=16, num_blocks=None):
    """strip s -> page perm[s]; returns (slots int32[T], num_blocks)."""
    P = strips if num_blocks is None else num_blocks
    perm = rng.permutation(P)[:strips]
    slots = (perm[:, None] * S + np.arange(16)[None, :]).astype(np.int32).reshape(-1)
    return slots, P


def fragmented_slots(strips, S=16):
    """strip s -> page 2s+1, P = 2*strips+2 (reference fixture mapping)."""
    pages = 2 * np.arange(strips) + 1
    slots = (pages[:, None] * S + np.arange(16)[None, :]).astype(np.int32).reshape(-1)
    return slots, 2 * strips + 2


def random_signs(rng, d):
    return np.where(rng.random(d) < 0.5, -1, 1).astype(np.int32)


def build_cache_from_gaussian(oracle, rng, ctx_lens, Hkv, d, S=16, extra_pages=3, outliers=False):
    """A paged 4-bit cache for a batch of sequences, written by the oracle's aligned
    writer from N(0,1) bf16 K/V, with shuffled block tables. Returns a dict."""
    B = len(ctx_lens)
    SP = S // 16
    pages_per_seq = [(c + S - 1) // S for c in ctx_lens]
    total_pages = sum(pages_per_seq) + extra_pages
    max_blocks = max(max(pages_per_seq), 1)
    perm = rng.permutation(total_pages)
    tables = np.zeros((B, max_blocks), np.int32)
    signs = random_signs(rng, d)
    kc = np.full(total_pages * Hkv * S * d // 2, 0xAA, np.uint8)
    vc = np.full_like(kc, 0xAA)
    sc = np.full(2 * total_pages * Hkv * S, np.nan, np.float32)
    at = 0
    for b in range(B):
        n = pages_per_seq[b]
        tables[b, :n] = perm[at:at + n]
        at += n
        if n == 0:
            continue
        T = n * S
        x = rng.standard_normal((2, T, Hkv * d)).astype(np.float32)
        if outliers:
            x = np.where(rng.random(x.shape) < 0.01, x * 20.0, x).astype(np.float32)
        kb, vb = bf16_from_f32(x[0]), bf16_from_f32(x[1])
        # strip s of the sequence -> slots of its page
        strips = T // 16
        slots = np.zeros(T, np.int32)
        for s in range(strips):
            page = tables[b, s // SP]
            slots[s * 16:(s + 1) * 16] = page * S + (s % SP) * 16 + np.arange(16)
        _write_aligned(oracle, kb, vb, slots, signs, Hkv, d, S, total_pages, kc, vc, sc)
    return dict(key_cache=kc, value_cache=vc, scale_cache=sc, block_tables=tables,
                context_lens=np.asarray(ctx_lens, np.int32), signs=signs, num_blocks=total_pages,
                max_blocks=max_blocks)


def _write_aligned(oracle, kb, vb, slots, signs, H, d, S, P, kc, vc, sc):
    if S == 16:
        oracle.reshape_and_cache(kb, vb, slots, signs, H, d, S, P, inv_sqrt_len(d), kc, vc, sc,
                                 threads=8)
    else:
        # pages larger than a strip: use the scatter oracle token by token
        T = slots.size
        oracle.reshape_scatter(kb, vb, slots, signs.astype(np.float32), None, T, H, d, S, P,
                               inv_sqrt_len(d), kc, vc, sc)
