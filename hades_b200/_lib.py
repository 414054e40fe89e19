"""ctypes binding of ``libhades_b200.so`` (see ``include/hades_b200.h``).

There is no CPU or PyTorch fallback: if the library is missing, or a call fails, an
exception is raised.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libhades_b200.so"

HB_OK = 0
LOOKUP_SETASSOC = 0
LOOKUP_SORTED = 1
MOVER_AUTO = 0
MOVER_LSU = 1
MOVER_BULK = 2

_p = C.c_void_p
_i64 = C.c_int64
_int = C.c_int
_sz = C.c_size_t
_f32 = C.c_float

# name -> (restype, argtypes); every symbol that include/hades_b200.h declares
PROTOTYPES: dict[str, tuple] = {
    "hb_last_error": (C.c_char_p, []),
    "hb_version": (_int, []),
    "hb_launch_count": (_i64, []),
    "hb_device_status": (_int, [_p, _p]),
    "hb_index_create": (_int, [_i64, _p]),
    "hb_index_destroy": (_int, [_p]),
    "hb_index_handle_bytes": (_sz, []),
    "hb_index_export_handle": (_int, [_p, _p]),
    "hb_index_open": (_int, [_p, _p]),
    "hb_index_size": (_i64, [_p]),
    "hb_index_capacity": (_i64, [_p]),
    "hb_index_space": (_i64, [_p]),
    "hb_index_lines": (_i64, [_p]),
    "hb_index_valid_entries": (_int, [_p, _p, _p]),
    "hb_index_add_workspace_bytes": (_sz, [_i64]),
    "hb_index_add": (_int, [_p, _p, _i64, _p, _p, _p, _sz, _p]),
    "hb_index_lookup": (_int, [_p, _p, _i64, _p, _p, _int, _p]),
    "hb_index_touch_lru_workspace_bytes": (_sz, [_i64]),
    "hb_index_touch_lru": (_int, [_p, _p, _i64, _p, _sz, _p]),
    "hb_index_touch_lru_runs": (_int, [_p, _p, _p, _p, _i64, _p, _i64, _p, _int, _p]),
    "hb_index_reset": (_int, [_p, _p, _i64, _p]),
    "hb_index_getall": (_int, [_p, _p, _p, _i64, _p, _p]),
    "hb_index_build_sorted": (_int, [_p, _p]),
    "hb_index_export": (_int, [_p, _p, _p, _p]),
    "hb_index_import": (_int, [_p, _p, _p, _p]),
    "hb_rows_gather": (_int, [_p, _p, _p, _p, _i64, _i64, _int, _int, _p]),
    "hb_rows_scatter": (_int, [_p, _p, _p, _i64, _i64, _int, _int, _p]),
    "hb_rows_gather_cached": (_int, [_p, _p, _p, _p, _p, _p, _i64, _i64, _int, _p]),
    "hb_rows_scatter_cached": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _int, _p]),
    "hb_rows_accumulate_f32": (_int, [_p, _p, _p, _p, _i64, _i64, _int, _p]),
    "hb_lookup_fetch": (_int, [_p, _p, _i64, _p, _p, _i64, _p, _p, _p, _int, _int, _p]),
    "hb_partition_workspace_bytes": (_sz, [_i64, _int]),
    "hb_split_masks": (_int, [_p, _i64, _p, _p, _p, _p, _p]),
    "hb_split_compact": (_int, [_p, _i64, _p, _p, _p, _p, _p, _p, _p, _sz, _p]),
    "hb_owner_mod": (_int, [_p, _i64, _int, _i64, _p, _p]),
    "hb_owner_range": (_int, [_p, _i64, _int, _p, _i64, _i64, _p, _p]),
    "hb_upper_bound": (_int, [_p, _i64, _int, _p, _i64, _p, _p]),
    "hb_bucket_pack": (_int, [_p, _p, _p, _i64, _p, _i64, _int, _p, _i64, _i64, _p, _p, _p, _p, _p, _sz, _p]),
    "hb_bucket_pack_noalloc_max_items": (_i64, []),
    "hb_bucket_pack_noalloc_max_buckets": (_int, []),
    "hb_bucket_pack_noalloc": (_int, [_p, _p, _p, _i64, _p, _i64, _int, _p, _i64, _i64, _p, _p, _p, _p, _p]),
    "hb_table_split3": (_int, [_p, _p, _p, _i64, _p, _i64, _p, _p, _p, _p, _p, _p, _sz, _p]),
    "hb_grad_split3": (_int, [_p, _p, _p, _p, _i64, _i64, _p, _p, _p, _p, _sz, _p]),
    "hb_unique_segsum_workspace_bytes": (_sz, [_i64, _i64]),
    "hb_unique_segsum_f32": (_int, [_p, _p, _p, _i64, _p, _p, _i64, _i64, _int, _int, _p, _p, _p, _p, _p, _p, _p, _sz, _p]),
    "hb_runs_workspace_bytes": (_sz, [_i64]),
    "hb_runs_build": (_int, [_p, _i64, _p, _p, _i64, _int, _p, _i64, _p, _p, _p, _p, _p, _sz, _p, _p]),
    "hb_segsum_runs_workspace_bytes": (_sz, [_i64, _i64]),
    "hb_segsum_runs_f32": (_int, [_p, _p, _p, _i64, _int, _p, _p, _p, _p, _sz, _p]),
    "hb_lookup_fetch_runs_workspace_bytes": (_sz, [_i64, _i64, _int]),
    "hb_lookup_fetch_runs": (_int, [_p, _p, _p, _p, _i64, _p, _i64, _p, _p, _p, _p, _int, _p, _sz, _p]),
    "hb_runs_resolve_requests": (_int, [_p, _p, _p, _p, _i64, _p, _i64, _p, _p, _p, _int, _p, _sz, _p]),
    "hb_runs_expand": (_int, [_p, _p, _p, _i64, _int, _p, _p, _p, _p, _p, _sz, _p]),
    "hb_runs_miss_list_workspace_bytes": (_sz, [_i64]),
    "hb_runs_miss_list": (_int, [_p, _p, _int, _int, _i64, _p, _p, _p, _p, _sz, _p]),
    "hb_staging_accumulate_cached": (_int, [_p, _p, _p, _p, _i64, _p, _p, C.c_int32, _int, _p, _p, _p]),
    "hb_staging_accumulate_direct": (_int, [_p, _p, _p, _i64, _p, _i64, _i64, _p]),
    "hb_staging_flush_workspace_bytes": (_sz, [_i64, _int]),
    "hb_staging_flush": (_int, [_p, _p, C.c_int32, _int, _i64, _p, _p, _p, _p, _p, _sz, _p]),
    "hb_staging_insert_workspace_bytes": (_sz, [_i64]),
    "hb_staging_insert_rows": (_int, [_p, _p, _p, _i64, _p, _i64, _p, _p, _p]),
    "hb_staging_insert": (_int, [_p, _p, _p, _p, _i64, _p, _i64, _p, _p, _sz, _p]),
    "hb_staging_insert_gather": (_int, [_p, _p, _p, _p, _p, _i64, _p, _i64, _p, _p, _sz, _p]),
    "hb_sparse_adam": (_int, [_p, _p, _p, _i64, _p, _i64, _i64, _i64, _i64, _p, _p, _p, _p, _int,
                              C.c_double, C.c_double, C.c_double, C.c_double, _p]),
    "hb_sparse_adagrad": (_int, [_p, _p, _p, _i64, _p, _i64, _i64, _i64, _i64, _p, _p, _int,
                                 C.c_double, C.c_double, _p]),
    "hb_a2a_create": (_int, [_int, _int, _i64, _i64, _p]),
    "hb_a2a_handle_bytes": (_sz, []),
    "hb_a2a_export_handle": (_int, [_p, _p]),
    "hb_a2a_connect": (_int, [_p, _p]),
    "hb_a2a_disconnect": (_int, [_p]),
    "hb_a2a_destroy": (_int, [_p]),
    "hb_a2a_push_workspace_bytes": (_sz, [_i64, _int]),
    "hb_a2a_push": (_int, [_p, _p, _p, _p, _i64, _p, _p, _p, _p, _sz, _p]),
    "hb_a2a_fence": (_int, [_p, _p]),
    "hb_a2a_reset": (_int, [_p, _p]),
    "hb_wait_flag": (_int, [_p, C.c_uint64, _p]),
    "hb_a2a_recv_view": (_int, [_p, _int, _p, _p, _p, _p, _p]),
    "hb_merge_sorted_slabs_workspace_bytes": (_sz, [_i64, _i64]),
    "hb_merge_sorted_slabs_f32": (_int, [_p, _p, _p, _p, _i64, _i64, _i64, _int, _p, _p, _p, _p, _p, _sz, _p]),
    "hb_peer_table_create": (_int, [_int, _int, _i64, _i64, _p]),
    "hb_peer_table_handle_bytes": (_sz, []),
    "hb_peer_table_export_handle": (_int, [_p, _p]),
    "hb_peer_table_connect": (_int, [_p, _p]),
    "hb_peer_table_set_peer": (_int, [_p, _int, _p]),
    "hb_peer_table_local": (_int, [_p, _p, _p]),
    "hb_peer_table_disconnect": (_int, [_p]),
    "hb_peer_table_destroy": (_int, [_p]),
    "hb_peer_table_gather": (_int, [_p, _p, _i64, _p, _p, _p]),
    "hb_lookup_fetch_sharded": (_int, [_p, _p, _i64, _p, _p, _p, _p, _p, _int, _p]),
    "hb_fetch_serve": (_int, [_p, _p, _p, _p, _p, _i64, _p]),
}


class RunsDesc(C.Structure):
    """hb_runs_t"""
    _fields_ = [("perm", _p), ("run_start", _p), ("num_runs", _p), ("n", _i64), ("keys", _p),
                ("key_bytes", _int), ("head", _p), ("uniq_ids", _p), ("dclass", _p), ("dpos", _p),
                ("class_counts", _p), ("n_dev", _p), ("base8", _p)]


class ClassSplitDesc(C.Structure):
    """hb_class_split_t"""
    _fields_ = [("table", _p), ("table_len", _i64), ("out_ids", _p * 3), ("out_rows", _p * 3),
                ("out_cnt", _p * 3), ("class_counts", _p)]


class StagingDesc(C.Structure):
    """hb_staging_t"""
    _fields_ = [("grad", _p), ("cnt", _p), ("idx", _p), ("iter_count", _p),
                ("iter_threshold", _p), ("slots", _i64), ("dim", _i64)]

_LIB: C.CDLL | None = None


class HadesError(RuntimeError):
    """A libhades_b200 call returned a non-zero status."""


def load() -> C.CDLL:
    """Load the C-ABI library; fails loudly when it has not been built."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m hades_b200._build` "
            "(nvcc, sm_100a). hades_b200 has no CPU fallback.")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError here = header and library out of sync
        fn.restype = res
        fn.argtypes = args
    _LIB = lib
    return lib


def check(rc: int) -> None:
    if rc != HB_OK:
        msg = load().hb_last_error().decode(errors="replace")
        raise HadesError(f"libhades_b200 status {rc}: {msg}")


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


_WORKSPACES: dict[int, torch.Tensor] = {}
_RETIRED: list = []  # outgrown scratch buffers: captured CUDA graphs may still hold their addresses


def workspace(nbytes: int) -> torch.Tensor:
    """A per-device scratch buffer of at least nbytes, reused across calls on the
    current stream."""
    dev = torch.cuda.current_device()
    ws = _WORKSPACES.get(dev)
    if ws is None or ws.numel() < nbytes:
        if ws is not None:
            _RETIRED.append(ws)
        ws = torch.empty(max(int(nbytes * 1.25), 1 << 20), dtype=torch.uint8, device=f"cuda:{dev}")
        _WORKSPACES[dev] = ws
    return ws


def device_status() -> int:
    out = C.c_int(0)
    check(load().hb_device_status(C.byref(out), stream_ptr()))
    return out.value


def launch_count() -> int:
    return load().hb_launch_count()
