"""The C-ABI library: it loads, exports every symbol include/tq_b200.h declares, and its
host-side logic (split choice, workspace sizing, geometry refusal) behaves as specified.
No kernel is launched here."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "tq_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b((?:tq|launch)_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    import ascend_micro_harness_b200 as tq
    lib = tq.load_library()
    names = declared_symbols()
    assert len(names) >= 13
    for n in names:
        assert hasattr(lib, n), f"libtq_b200.so does not export {n}"
    from ascend_micro_harness_b200 import _lib
    assert set(names) == set(_lib.SIGNATURES), "Python signature table and header disagree"
    assert b"sm_100a" in lib.tq_version()


def test_acl_shim_exports_the_sixteen_calls():
    path = os.path.join(ROOT, "ascend_micro_harness_b200", "libtq_acl_shim.so")
    if not os.path.exists(path):
        from ascend_micro_harness_b200 import build
        build.build_acl_shim()
    lib = C.CDLL(path)
    for n in ("aclInit aclFinalize aclrtSetDevice aclrtResetDevice aclrtCreateStream aclrtDestroyStream "
              "aclrtSynchronizeStream aclrtMalloc aclrtFree aclrtMemcpy aclrtMemset aclrtCreateEvent "
              "aclrtDestroyEvent aclrtRecordEvent aclrtSynchronizeEvent aclrtEventElapsedTime").split():
        assert hasattr(lib, n)


def test_split_choice():
    """The plan cuts a sequence into pieces of 256..8192 tokens (steps of 256): eight for the
    longest sequence, more tokens per piece when the batch alone fills the machine, fewer when it
    is too small to; the launch's split count is what the longest context needs, at most
    TQ_MAX_SPLITS = 32. (Head size 256 launches use somewhat longer pieces, so never more splits
    than this chooser, which sizes the workspace, reports.)"""
    import ascend_micro_harness_b200 as tq
    choose = lambda b, h, s, c: tq.choose_splits(b, h, s, c, 148)
    assert choose(64, 8, 16, 256) == 1             # short contexts run un-split
    assert choose(1, 8, 16, 4096) == 16            # one sequence: fill the machine
    assert choose(1, 8, 16, 1024) == 4             # ... but keep 256 tokens per piece
    assert choose(64, 8, 16, 16384) == 8           # ragged batch: 2048-token pieces
    assert choose(64, 4, 16, 16384) == 8           # ... whatever the number of KV heads
    assert choose(64, 8, 16, 32768) == 8
    assert choose(4096, 8, 16, 32768) == 4         # plenty of sequences: 8192-token pieces
    assert choose(16, 8, 16, 65536) == 14          # few long sequences: three pieces per resident CTA slot
    assert choose(1, 8, 16, 1 << 20) == 32         # one very long sequence: as many as the records allow
    for b in (1, 3, 64, 1000):
        for ctx in (1, 600, 5000, 70000, 1 << 20):
            s = choose(b, 8, 16, ctx)
            assert 1 <= s <= 32 and s <= max(1, (ctx + 15) // 16)


def test_workspace_sizing():
    import ascend_micro_harness_b200 as tq
    # the records, then one arrival counter per (sequence, KV head, 8-row tile)
    # ... and, 8-byte aligned behind them, two 64-bit words of chunk schedule
    assert tq.decode_workspace_floats(64, 32, 8, 128, 4) == 64 * 8 * 4 * 4 * (16 + 128) + 64 * 8 + 4
    assert tq.decode_workspace_floats(2, 64, 4, 256, 8) == 2 * 4 * 8 * 16 * 272 + 2 * 4 * 2 + 4
    assert tq.decode_workspace_floats(1, 1, 1, 128, 1) == 144 + 1 + 1 + 4      # padded to an even word count


def test_geometry_is_refused_before_any_launch():
    from ascend_micro_harness_b200._lib import load_library
    lib = load_library()
    p = C.c_void_p(16)   # never dereferenced: every call below is refused on the host
    # 24 tokens is not a whole number of strips (reference: a8.cpp:1606-1609)
    assert lib.tq_reshape_and_cache(None, p, p, p, p, p, p, p, 0, 0, 24, 1, 128, 16, 4, 0.1, None) == 2
    assert lib.tq_reshape_and_cache(None, p, p, p, p, p, p, p, 0, 0, 32, 1, 96, 16, 4, 0.1, None) == 1
    assert lib.tq_reshape_and_cache(None, p, p, p, p, p, p, p, 0, 0, 32, 1, 128, 24, 4, 0.1, None) == 1
    assert lib.tq_reshape_and_cache(None, p, p, p, p, p, p, p, 0, 0, 0, 1, 128, 16, 4, 0.1, None) == 0
    # decode: heads not a multiple of KV heads; 33 splits; bad head size
    args = [None, p, p, p, p, p, p, p, p, p, p, 0]
    assert lib.tq_decode_splitk(*args, 2, 30, 8, 128, 16, 8, 4, 1, 0, 0, 0.1, 1.0, None) == 1
    assert lib.tq_decode_splitk(*args, 2, 32, 8, 128, 16, 8, 4, 33, 0, 0, 0.1, 1.0, None) == 1
    assert lib.tq_decode_splitk(*args, 2, 32, 8, 64, 16, 8, 4, 1, 0, 0, 0.1, 1.0, None) == 1
    # AIC contract: page window past the sequence, seq_len past the window
    # (reference: turboquant_paged_decode_attention.cpp:1747-1759)
    part = [None, p, p, 2, p, p, p, p, p, p]
    assert lib.tq_decode_splitk_partials(*part, 1, 1, 16, 256, 128, 8, 4, 2, 3, 2, 0, 0.0625, 1.0, None) == 1
    assert lib.tq_decode_splitk_partials(*part, 1, 1, 16, 256, 128, 8, 4, 2, 0, 2, 300, 0.0625, 1.0, None) == 1
    assert lib.tq_decode_splitk_partials(*part, 1, 1, 16, 256, 128, 8, 4, 17, 0, 2, 0, 0.0625, 1.0, None) == 1
    assert lib.tq_status_string(2).decode().startswith("num_tokens")
    # the softmax scale is a positive finite factor (the kernels take maxima of raw scores)
    for bad in (0.0, -0.5, float("nan"), float("inf")):
        assert lib.tq_decode_splitk(*args, 2, 32, 8, 128, 16, 8, 4, 2, 0, 0, 0.1, bad, None) == 1
        assert lib.tq_decode_splitk_precise(*args, 2, 32, 8, 128, 16, 8, 4, 2, 0, 0, 0.1, bad, None) == 1
        assert lib.tq_decode_splitk_partials(*part, 1, 1, 16, 256, 128, 8, 4, 2, 0, 2, 0, 0.0625, bad, None) == 1
    # the persistent entry takes 2..32 record slots per head (0 = 32), never one
    pers = [None, p, p, p, p, p, p, p, p, p, p, 0]
    assert lib.tq_decode_splitk_persistent(*pers, 2, 32, 8, 128, 16, 8, 4, 1, 0, 0.1, 1.0, None) == 1
    assert lib.tq_decode_splitk_persistent(*pers, 2, 32, 8, 128, 16, 8, 4, 33, 0, 0.1, 1.0, None) == 1
    assert lib.tq_decode_splitk_persistent(*pers, 0, 32, 8, 128, 16, 8, 4, 0, 0, 0.1, 1.0, None) == 0
    misaligned = [None, p, p, p, p, p, p, p, p, C.c_void_p(20), p, 0]
    assert lib.tq_decode_splitk_persistent(*misaligned, 2, 32, 8, 128, 16, 8, 4, 4, 0, 0.1, 1.0, None) == 1
    # one split needs no workspace; more than one does
    noworkspace = [None, p, p, p, p, p, p, p, p, None, p, 0]
    assert lib.tq_decode_splitk(*noworkspace, 0, 32, 8, 128, 16, 8, 4, 1, 0, 0, 0.1, 1.0, None) == 0
    assert lib.tq_decode_splitk(*noworkspace, 2, 32, 8, 128, 16, 8, 4, 2, 0, 0, 0.1, 1.0, None) == 1


def test_nz_entry_and_static_entry_refuse_bad_geometry_on_the_host():
    from ascend_micro_harness_b200._lib import load_library
    lib = load_library()
    p = C.c_void_p(16)   # never dereferenced
    nz = [None, p, p, p, p, p, p, p, p, p, p, 1, 1]
    tail = (2.98, 0.0625, 0.0625, 0, None)
    assert lib.tq_decode_splitk_nz(*nz, 2, 16, 4, 32, 0, 4, 2, 0, 1, 0, *tail) == 1      # pages are 64 or 128 slots
    assert lib.tq_decode_splitk_nz(*nz, 2, 16, 4, 64, 0, 4, 33, 0, 1, 0, *tail) == 1     # 33 splits
    assert lib.tq_decode_splitk_nz(*nz, 2, 16, 4, 64, 0, 4, 2, 0, 2, 0, *tail) == 1      # no such code grid
    assert lib.tq_decode_splitk_nz(*nz, 2, 18, 4, 64, 0, 4, 2, 0, 1, 0, *tail) == 1      # heads % KV heads
    assert lib.tq_decode_splitk_nz(*nz, 2, 16, 4, 64, 0, 4, 2, 0, 1, 0, 0.0, 0.0625, 0.0625, 0, None) == 1   # gain
    assert lib.tq_decode_splitk_nz(*nz, 0, 16, 4, 64, 0, 4, 2, 0, 1, 0, *tail) == 0      # empty batch
    st = [None, p, p, p, p, p, p, p, p, p, 0]
    assert lib.tq_decode_splitk_static(*st, 1 << 20, 17, 1, 128, 16, 8, 4, 16, 0, 0, 0.1, 1.0, None) == 1   # 17 rows
    assert lib.tq_decode_splitk_static(*st, 1 << 20, 16, 1, 96, 16, 8, 4, 16, 0, 0, 0.1, 1.0, None) == 1    # head size
    assert lib.tq_decode_splitk_static(*st, 1 << 20, 16, 1, 128, 16, 8, 4, 16, 0, 0, 0.1, 1.0, None) == 5   # too large


def test_routine_and_lloydmax_entries_refuse_bad_arguments_on_the_host():
    from ascend_micro_harness_b200._lib import load_library
    lib = load_library()
    p = C.c_void_p(16)   # never dereferenced
    assert lib.tq_hadamard16(None, p, p, 3, 4) == 1               # no such output type
    assert lib.tq_hadamard16(None, p, p, 2, 0) == 0               # nothing to do
    assert lib.tq_lloydmax4_quantize(None, p, p, None, 12) == 1   # not a multiple of 8
    assert lib.tq_lloydmax4_quantize(None, C.c_void_p(20), p, None, 16) == 1   # x not 16-byte aligned
    assert lib.tq_icdf_quantize(None, p, 2, p, 16) == 1           # float32 input is not served
    assert lib.tq_icdf_quantize(None, p, 1, p, 0) == 0
    lm = [None, p, p, p, p, p, p]
    assert lib.tq_reshape_and_cache_lloydmax(*lm, 1, 24, 1, 128, 16, 4, 0.1, None) == 2   # partial strip
    assert lib.tq_reshape_and_cache_lloydmax(*lm, 1, 32, 1, 64, 16, 4, 0.1, None) == 1    # head size
    assert lib.tq_reshape_and_cache_lloydmax(*lm, 2, 32, 1, 128, 16, 4, 0.1, None) == 1   # dtype
    dec = [None, p, p, p, p, p, p, p]
    assert lib.tq_decode_lloydmax_export(*dec, 1, 48, 4, 128, 16, 8, 4, 2, 1.0, None) == 1  # 12 rows per KV head
    assert lib.tq_decode_lloydmax_export(*dec, 1, 32, 8, 128, 16, 8, 4, 17, 1.0, None) == 1  # 17 splits
    assert lib.tq_decode_lloydmax_export(*dec, 0, 32, 8, 128, 16, 8, 4, 2, 1.0, None) == 0   # empty batch


def test_varlen_writer_refuses_bad_geometry_on_the_host():
    from ascend_micro_harness_b200._lib import load_library
    lib = load_library()
    p = C.c_void_p(16)
    args = [None, p, p, p, p, p, p, p, p, p]
    assert lib.tq_reshape_and_cache_varlen(*args, 2, 3, 1, 96, 16, 4, 0.1, None) == 1    # head size
    assert lib.tq_reshape_and_cache_varlen(*args, 2, 3, 1, 128, 24, 4, 0.1, None) == 1   # page not strips
    assert lib.tq_reshape_and_cache_varlen(*args, 0, 0, 1, 128, 16, 4, 0.1, None) == 0   # nothing to do
    bad = [None, C.c_void_p(8), p, p, p, p, p, p, p, p]
    assert lib.tq_reshape_and_cache_varlen(*bad, 2, 3, 1, 128, 16, 4, 0.1, None) == 1    # key not aligned


def test_kv4_import_and_prerotated_decode_refuse_bad_arguments_on_the_host():
    from ascend_micro_harness_b200._lib import load_library
    lib = load_library()
    p = C.c_void_p(16)   # never dereferenced
    imp = [None, p, p, p, p, p, p]
    assert lib.tq_nz_kv4_import(*imp, 2, 32, 4, 2.98) == 1     # pages are 64 or 128 slots
    assert lib.tq_nz_kv4_import(*imp, 0, 64, 4, 2.98) == 1     # no KV head
    assert lib.tq_nz_kv4_import(*imp, 2, 64, 4, 0.0) == 1      # the gain divides the scales
    assert lib.tq_nz_kv4_import(*imp, 2, 128, 0, 2.98) == 0    # nothing to import
    bad = [None, C.c_void_p(8), p, p, p, p, p]
    assert lib.tq_nz_kv4_import(*bad, 2, 64, 4, 2.98) == 1     # packed plane not 16-byte aligned
    dec = [None, p, p, p, p, p, p, p, p, p, p, 0, 2]
    assert lib.tq_decode_splitk_prerotated(*dec, 2, 32, 8, 256, 64, 8, 4, 1, 0, 2, 0, 0.0625, None) == 1   # no such grid
    assert lib.tq_decode_splitk_prerotated(*dec, 2, 32, 8, 256, 64, 8, 4, 33, 0, 1, 0, 0.0625, None) == 1  # 33 splits
    assert lib.tq_decode_splitk_prerotated(*dec, 2, 30, 8, 256, 64, 8, 4, 1, 0, 1, 0, 0.0625, None) == 1   # heads % KV heads
    assert lib.tq_decode_splitk_prerotated(*dec, 2, 32, 8, 256, 64, 8, 4, 1, 0, 1, 3, 0.0625, None) == 1   # no such stage
    assert lib.tq_decode_splitk_prerotated(*dec, 0, 32, 8, 256, 64, 8, 4, 1, 0, 1, 0, 0.0625, None) == 0   # empty batch
    nullq = [None, None, p, p, p, p, p, p, p, p, p, 0, 2]
    assert lib.tq_decode_splitk_prerotated(*nullq, 2, 32, 8, 256, 64, 8, 4, 1, 0, 1, 0, 0.0625, None) == 1
    nosign = [None, p, p, p, p, p, p, None, p, p, p, 0, 2]   # un-rotation asked for without the sign diagonal
    assert lib.tq_decode_splitk_prerotated(*nosign, 2, 32, 8, 256, 64, 8, 4, 1, 0, 1, 1, 0.0625, None) == 1
    assert lib.tq_rotate_query_pi(None, p, 2, p, p, 4, 256) == 1     # the raw query is 16-bit
    assert lib.tq_rotate_query_pi(None, p, 1, p, p, 4, 64) == 1      # head size
    assert lib.tq_rotate_query_pi(None, p, 1, p, p, 0, 256) == 0     # no rows


def test_ctypes_table_matches_the_header_argument_counts():
    """Every function include/tq_b200.h declares takes as many arguments as the loader's table gives it
    (a wrong count would only show when the function is first called on a GPU)."""
    import re
    from ascend_micro_harness_b200._lib import SIGNATURES
    text = open(os.path.join(ROOT, "include", "tq_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    seen = 0
    for m in re.finditer(r"\b(\w+)\s*\(([^;{}]*?)\)\s*;", text):
        name, args = m.group(1), m.group(2)
        if name in SIGNATURES and SIGNATURES[name][1] is not None:
            n = len([a for a in args.split(",") if a.strip() and a.strip() != "void"])
            assert n == len(SIGNATURES[name][1]), name
            seen += 1
    assert seen >= 25
