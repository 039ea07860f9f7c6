"""B200-native TurboQuant KV-cache engine: paged 4-bit reshape_and_cache and
split-K decode attention as hand-written sm_100a kernels behind a C ABI
(include/tq_b200.h). This package is the thin Python host layer the tests and
the benchmark use; the product is libtq_b200.so."""
from ._lib import load_library, library_path, TqError  # noqa: F401
from .engine import (  # noqa: F401
    reshape_and_cache, reshape_and_cache_varlen, reshape_scatter, set_ingest_wait_budget, decode_splitk, decode_step, decode_splitk_elem, decode_splitk_mtp, decode_splitk_prerotated, decode_splitk_nz, decode_splitk_levels, rotate_query_pi, nz_kv4_import, KV4_FP8_GAIN, GRID_INTEGER, GRID_MIDRISE, decode_splitk_static, STATIC_WORKSPACE_FLOATS, decode_splitk_export, decode_splitk_partials, splitk_combine,
    decode_workspace_floats, choose_splits, worker_census, MAX_SPLITS, SIGNS_F32, SIGNS_TABLES_I8, SIGNS_TABLES_BF16,
    OUT_ROTATED, OUT_UNROTATED, OUT_GATED, STATUS_BAD_SLOT, STATUS_BAD_PAGE, STATUS_WAIT_EXPIRED,
    rotate_query, hadamard16, lloydmax4_quantize, icdf_quantize, reshape_and_cache_lloydmax, decode_lloydmax,
)
