"""ctypes binding of libhira_b200.so (the C ABI declared in include/hira_b200.h).

The library is the only compute path: there is no CPU or PyTorch fallback.  If it
has not been built, loading raises with the build command.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parent / "libhira_b200.so"

HIRA_OK = 0
HIRA_ERR_ARG, HIRA_ERR_SHAPE, HIRA_ERR_DTYPE, HIRA_ERR_CAPACITY, HIRA_ERR_CUDA = -1, -2, -3, -4, -5
HIRA_F32, HIRA_BF16 = 0, 1
HIRA_STATUS_PARENTS_FULL, HIRA_STATUS_GP_FULL, HIRA_STATUS_ASSIGN_FAILED = 1, 2, 4
HIRA_GATE_GT, HIRA_GATE_GE = 0x0, 0x1
HIRA_LEAF_CANDIDATES, HIRA_LEAF_GE, HIRA_LEAF_GT = 0x0, 0x2, 0x4
HIRA_TAU_SAMPLE_MAX, HIRA_TAU_SAMPLE_MEAN_TOPK, HIRA_TAU_SAMPLE_KTH = 0, 1, 2

EXPORTED_SYMBOLS = [
    "hira_last_error", "hira_version", "hira_search_tile_parents", "hira_search",
    "hira_attn_default_splits", "hira_sparse_attn", "hira_merge_partials", "hira_append",
    "hira_append_workspace_bytes",
    "hira_threshold", "hira_kth_score", "hira_prepare_query", "hira_build_workspace_bytes", "hira_build",
    "hira_recompute_radii", "hira_export", "hira_assign", "hira_sparse_attn_noalloc", "hira_decode_attention",
    "hira_search_scan", "hira_append_scanned", "hira_step_events_create", "hira_step_events_destroy",
    "hira_decode_step", "hira_q8_refresh", "hira_q8_fallback_count",
    "hira_exchange_bytes", "hira_peer_alloc", "hira_peer_open", "hira_peer_close", "hira_peer_free", "hira_exchange_merge",
]
MAX_PEERS = 16            # HIRA_MAX_PEERS
PEER_HANDLE_BYTES = 64    # HIRA_PEER_HANDLE_BYTES
NOALLOC_SCRATCH_FLOATS = 1 << 20
SEARCH_STATS = 10     # uint32 counters per query head (HIRA_SEARCH_STATS)
Q8_CHAN = 136         # floats per head in q8_chan_scale (HIRA_Q8_CHAN)
Q8_QUERY_BYTES = 4 * 2112   # bytes per head in q8_query_scratch (HIRA_Q8_QUERY_CHUNKS * HIRA_Q8_QUERY_BYTES)


class HiraIndexStruct(C.Structure):
    """Mirror of hira_index_t."""
    _fields_ = [
        ("dtype", C.c_int32), ("vdtype", C.c_int32), ("depth", C.c_int32), ("bf", C.c_int32),
        ("dim", C.c_int32), ("vdim", C.c_int32), ("n_heads", C.c_int32), ("cap_parents", C.c_int32),
        ("cap_gp", C.c_int32), ("active_parents", C.c_int32),
        ("children", C.c_void_p), ("values", C.c_void_p), ("slot2token", C.c_void_p),
        ("parents", C.c_void_p), ("parent_radii", C.c_void_p), ("parent_sqnorm", C.c_void_p),
        ("child_counts", C.c_void_p), ("grand_parents", C.c_void_p), ("gp_radii", C.c_void_p),
        ("gp_sqnorm", C.c_void_p), ("gp_counts", C.c_void_p), ("used", C.c_void_p),
        ("children_q8", C.c_void_p), ("children_q8_meta", C.c_void_p), ("q8_chan_scale", C.c_void_p),
        ("q8_query_scratch", C.c_void_p),
    ]


class HiraStepStruct(C.Structure):
    """Mirror of hira_step_t."""
    _fields_ = [
        ("q_dev", C.c_void_p), ("k_dev", C.c_void_p), ("v_dev", C.c_void_p), ("q_hat", C.c_void_p),
        ("logit_scale", C.c_void_p), ("tau", C.c_void_p), ("idx", C.c_void_p), ("score", C.c_void_p),
        ("count", C.c_void_p), ("workspace", C.c_void_p), ("out_dev", C.c_void_p), ("scan", C.c_void_p),
        ("status", C.c_void_p), ("append_ws", C.c_void_p), ("append_ws_bytes", C.c_size_t),
        ("tau_samples", C.c_void_p), ("samples_head_stride", C.c_int64),
        ("n_samples", C.c_int32), ("tau_method", C.c_int32), ("tau_k", C.c_int32),
        ("n_splits", C.c_int32), ("tile_parents", C.c_int32), ("flags", C.c_int32),
        ("ev_copied", C.c_void_p), ("ev_searched", C.c_void_p), ("ev_appended", C.c_void_p),
    ]


_lib = None


def _declare(lib):
    P, I32, I64, SZ = C.c_void_p, C.c_int32, C.c_int64, C.c_size_t
    IX = C.POINTER(HiraIndexStruct)
    lib.hira_last_error.restype = C.c_char_p
    lib.hira_last_error.argtypes = []
    lib.hira_version.restype = C.c_char_p
    lib.hira_version.argtypes = []
    lib.hira_search_tile_parents.restype = C.c_int
    lib.hira_search_tile_parents.argtypes = [IX]
    lib.hira_search.restype = C.c_int
    lib.hira_search.argtypes = [IX, P, P, P, P, P, I32, I32, I32, I32, P, P, P, P, P, P]
    lib.hira_attn_default_splits.restype = C.c_int
    lib.hira_attn_default_splits.argtypes = [I32, I32]
    lib.hira_sparse_attn.restype = C.c_int
    lib.hira_sparse_attn.argtypes = [IX, P, P, P, I32, I32, P, P, P, P, P, I32, I64, I32, P, P, P, I64, I64, P]
    lib.hira_decode_attention.restype = C.c_int
    lib.hira_decode_attention.argtypes = [IX, P, I32, C.c_float, P, P, I32, I32, I32, I32, P, P, P, P, P, P, P, I32, I64,
                                          I32, P, P, P, I64, I64, P, I64, P, P, P]
    ST = C.POINTER(HiraStepStruct)
    lib.hira_step_events_create.restype = C.c_int
    lib.hira_step_events_create.argtypes = [ST]
    lib.hira_step_events_destroy.restype = C.c_int
    lib.hira_step_events_destroy.argtypes = [ST]
    lib.hira_decode_step.restype = C.c_int
    lib.hira_decode_step.argtypes = [IX, ST, P, I32, C.c_float, I32, P, P, P, P, P, P]
    lib.hira_search_scan.restype = C.c_int
    lib.hira_search_scan.argtypes = [IX, P, P, P, P, I32, I32, I32, P, P, P, P, P, P, I64, P, P]
    lib.hira_append_scanned.restype = C.c_int
    lib.hira_append_scanned.argtypes = [IX, P, P, I64, I64, I32, P, P, P]
    lib.hira_sparse_attn_noalloc.restype = C.c_int
    lib.hira_sparse_attn_noalloc.argtypes = [IX, P, P, P, I32, I32, P, P, P, P, P, I32, I64, I32, P, P, I64, I64, P]
    lib.hira_merge_partials.restype = C.c_int
    lib.hira_merge_partials.argtypes = [P, P, I32, I32, I32, I64, I64, I64, I64, P, P, P]
    lib.hira_q8_fallback_count.restype = C.c_int
    lib.hira_q8_fallback_count.argtypes = [C.POINTER(C.c_uint32)]
    lib.hira_exchange_bytes.restype = I64
    lib.hira_exchange_bytes.argtypes = [I32, I32, I32]
    lib.hira_peer_alloc.restype = C.c_int
    lib.hira_peer_alloc.argtypes = [I64, C.POINTER(C.c_void_p), C.c_char_p]
    lib.hira_peer_open.restype = C.c_int
    lib.hira_peer_open.argtypes = [C.c_char_p, C.POINTER(C.c_void_p)]
    lib.hira_peer_close.restype = C.c_int
    lib.hira_peer_close.argtypes = [P]
    lib.hira_peer_free.restype = C.c_int
    lib.hira_peer_free.argtypes = [P]
    lib.hira_exchange_merge.restype = C.c_int
    lib.hira_exchange_merge.argtypes = [P, C.POINTER(C.c_void_p), I32, I32, I32, I32, C.c_uint32, I32, C.c_float, P, P, P, P]
    lib.hira_append.restype = C.c_int
    lib.hira_append.argtypes = [IX, P, P, I32, I64, I64, I32, P, P, SZ, P]
    lib.hira_append_workspace_bytes.restype = SZ
    lib.hira_append_workspace_bytes.argtypes = [IX, I32]
    lib.hira_threshold.restype = C.c_int
    lib.hira_threshold.argtypes = [P, I32, I32, I32, I32, I64, P, P, I32, I32, I32, P, P]
    lib.hira_prepare_query.restype = C.c_int
    lib.hira_prepare_query.argtypes = [P, I32, I32, I32, C.c_float, P, P, P]
    lib.hira_kth_score.restype = C.c_int
    lib.hira_kth_score.argtypes = [IX, I32, I32, P, P, P, P, P]
    lib.hira_build_workspace_bytes.restype = SZ
    lib.hira_build_workspace_bytes.argtypes = [IX, I32]
    lib.hira_build.restype = C.c_int
    lib.hira_build.argtypes = [IX, P, P, I32, I64, I64, I32, P, P, I32, I32, I32, P, P, SZ, P]
    lib.hira_q8_refresh.restype = C.c_int
    lib.hira_q8_refresh.argtypes = [IX, P]
    lib.hira_recompute_radii.restype = C.c_int
    lib.hira_recompute_radii.argtypes = [IX, P]
    lib.hira_export.restype = C.c_int
    lib.hira_export.argtypes = [IX, I32, I32, P, P, P]
    lib.hira_assign.restype = C.c_int
    lib.hira_assign.argtypes = [P, P, I32, I32, I32, I32, I32, I32, P, P, P, P]


def load():
    """Returns the loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build the CUDA library first with `python -m hira_b200.build` "
                "(there is no CPU or PyTorch fallback)"
            )
        lib = C.CDLL(str(LIB_PATH))
        _declare(lib)
        _lib = lib
    return _lib


class HiraError(RuntimeError):
    pass


def check(rc: int, what: str = ""):
    """Raises for a negative status: ValueError for argument/shape/dtype errors (the
    reference's wrappers raise ValueError, kernels/triton_search_wrappers.py:136-180),
    RuntimeError for CUDA failures."""
    if rc == HIRA_OK:
        return
    msg = load().hira_last_error().decode("utf-8", "replace")
    if rc in (HIRA_ERR_ARG, HIRA_ERR_SHAPE, HIRA_ERR_DTYPE):
        raise ValueError(f"{what}: {msg}" if what else msg)
    raise HiraError(f"{what}: {msg} (status {rc})" if what else f"{msg} (status {rc})")


def ptr(t) -> int | None:
    """Device pointer of a tensor (None stays NULL)."""
    if t is None:
        return None
    return t.data_ptr()


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return HIRA_F32
    if dt == torch.bfloat16:
        return HIRA_BF16
    raise ValueError(f"unsupported dtype {dt}: the index stores float32 or bfloat16")


def current_stream(device=None) -> int:
    return torch.cuda.current_stream(device).cuda_stream
