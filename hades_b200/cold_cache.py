"""Per-GPU cold data cache: the arithmetic of the reference's cache-server process
(python/EmbCache/server.py) with every buffer in HBM and no sockets or shared memory.

``ColdCache`` owns the cache index, the cached embedding rows and the gradient staging table
that the server keeps per machine (``_create_cache``, server.py:76-175) and offers the steps
of the server loop (server.py:259-298) as methods on the current CUDA stream:

* ``insert``            = ``_update_cache``                      (server.py:499-544)
* ``accumulate_remote`` = ``_accumulate_gradients_cold_remote``  (server.py:546-562)
* ``accumulate_local``  = ``_accumulate_gradients_cold_local``   (server.py:564-574)
* ``flush_remote`` / ``flush_local`` = ``_send_staled_gradients`` (server.py:346-497)

Flushed rows are read and zeroed.  (The reference zeroes a temporary copy,
``self._grad_cache_buff[idx][:] = 0`` at server.py:414,489,537, so its buffers keep growing;
this is the intended behaviour, not that one.)
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from .EmbCacheLib import IndexCache, LOOKUP_SETASSOC, _check


def flush_thresholds(hotness: torch.Tensor) -> torch.Tensor:
    """Per-node flush period, server.py:87-88: ceil(1 / (0.001 + hotness)) capped at 100."""
    return (1 / (0.001 + hotness)).ceil().int().clamp(max=100)


class StagingTable:
    """Gradient staging buffers (one row per slot) and their C descriptor."""

    def __init__(self, slots: int, dim: int, device, iter_threshold: torch.Tensor | None = None):
        self.slots, self.dim = int(slots), int(dim)
        self.grad = torch.zeros((slots, dim), dtype=torch.float32, device=device)
        self.cnt = torch.zeros(slots, dtype=torch.int32, device=device)
        self.idx = torch.full((slots,), -1, dtype=torch.int64, device=device)
        self.iter_count = torch.zeros(slots, dtype=torch.int32, device=device)
        if iter_threshold is None:
            self.iter_threshold = torch.zeros(slots, dtype=torch.int32, device=device)
        else:
            self.iter_threshold = iter_threshold.to(device=device, dtype=torch.int32).contiguous()
        self.desc = _lib.StagingDesc(self.grad.data_ptr(), self.cnt.data_ptr(), self.idx.data_ptr(),
                                     self.iter_count.data_ptr(), self.iter_threshold.data_ptr(),
                                     self.slots, self.dim)

    def flush(self, index: IndexCache | None, cnt_threshold: int, num_clients: int, sync: bool = True,
              out_cap: int = 0):
        """sync=True: one host read of the counts, outputs sliced to the rows that left.
        sync=False: no host read; the outputs hold out_cap entries (0: one per slot) of which
        the first min(counts.sum(), out_cap) are valid.  out_cap < slots needs num_clients == 1:
        stale rows beyond it stay staged until the next flush."""
        lib = _lib.load()
        dev = self.grad.device
        cap = self.slots if out_cap <= 0 else min(int(out_cap), self.slots)
        out_ids = torch.empty(cap, dtype=torch.int64, device=dev)
        out_rows = torch.empty((cap, self.dim), dtype=torch.float32, device=dev)
        out_cnt = torch.empty(cap, dtype=torch.int64, device=dev)
        counts = torch.empty(num_clients, dtype=torch.int64, device=dev)
        ws = _lib.workspace(lib.hb_staging_flush_workspace_bytes(self.slots, num_clients))
        _lib.check(lib.hb_staging_flush(index.handle if index is not None else None, C.byref(self.desc),
                                        int(cnt_threshold), int(num_clients), cap, out_ids.data_ptr(),
                                        out_rows.data_ptr(), out_cnt.data_ptr(), counts.data_ptr(),
                                        ws.data_ptr(), ws.numel(), _lib.stream_ptr()))
        if not sync:
            return out_ids, out_rows, out_cnt, counts
        self.last_counts_host = counts.tolist()  # the one host read of a flush
        total = min(sum(self.last_counts_host), cap)
        return out_ids[:total], out_rows[:total], out_cnt[:total], counts


class ColdCache:
    def __init__(self, name: str, cache_entries: int, dim: int, threshold: torch.Tensor | None = None,
                 cnt_threshold: int = 16, default_threshold: int = 1, num_clients: int = 1,
                 local_nodes: int = 0, local_start: int = 0, emb_dtype=torch.float32,
                 lookup_mode: int = LOOKUP_SETASSOC, device=None):
        """threshold: int32 per-node flush period (``flush_thresholds``) or None for a fixed
        period ``default_threshold``; cnt_threshold: server.py:85 (16 in dist_emb.py:139)."""
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        self.device = device
        self.dim = dim
        self.cnt_threshold = int(cnt_threshold)
        self.default_threshold = int(default_threshold)
        self.num_clients = int(num_clients)
        self.lookup_mode = lookup_mode
        self.threshold = None if threshold is None else threshold.to(device=device, dtype=torch.int32).contiguous()
        self.index = IndexCache(cache_entries, name, True, False, lookup_mode=lookup_mode)
        slots = self.index.get_capacity()
        self.emb = torch.zeros((slots, dim), dtype=emb_dtype, device=device)
        self.remote = StagingTable(slots, dim, device)
        self.local = None
        self.local_start = int(local_start)
        if local_nodes > 0:
            thr = None
            if self.threshold is not None:
                thr = self.threshold[local_start:local_start + local_nodes]
            else:
                thr = torch.full((local_nodes,), self.default_threshold, dtype=torch.int32, device=device)
            self.local = StagingTable(local_nodes, dim, device, thr)
        self.dropped = torch.zeros(1, dtype=torch.int64, device=device)

    # -- server step 2 -------------------------------------------------------------------
    def insert(self, ids: torch.Tensor, embs: torch.Tensor) -> torch.Tensor:
        _check(ids.is_cuda and ids.dtype == torch.int64, "ids is a CUDA int64 tensor")
        _check(embs.size(0) == ids.numel() and embs.size(1) == self.dim, "embs matches ids and dim")
        lib = _lib.load()
        n = ids.numel()
        locs = torch.empty(n, dtype=torch.int64, device=ids.device)
        ws = _lib.workspace(lib.hb_staging_insert_workspace_bytes(n))
        _lib.check(lib.hb_staging_insert(self.index.handle, C.byref(self.remote.desc), ids.contiguous().data_ptr(),
                                         embs.contiguous().data_ptr(), n, self.emb.data_ptr(),
                                         self.dim * self.emb.element_size(), locs.data_ptr(),
                                         ws.data_ptr(), ws.numel(), _lib.stream_ptr()))
        return locs

    def insert_gather(self, ids: torch.Tensor, rows: torch.Tensor, row_index: torch.Tensor,
                      ws: torch.Tensor | None = None) -> torch.Tensor:
        """``insert`` with the embedding of ids[i] at rows[row_index[i]]; negative ids (padding
        of a fixed-size miss list) are ignored.  ws: scratch of at least
        hb_staging_insert_workspace_bytes(len(ids)) bytes (the shared one when None)."""
        _check(ids.is_cuda and ids.dtype == torch.int64 and row_index.dtype == torch.int64, "int64 CUDA tensors")
        _check(rows.size(1) == self.dim, "rows matches dim")
        lib = _lib.load()
        n = ids.numel()
        locs = torch.empty(n, dtype=torch.int64, device=ids.device)
        need = lib.hb_staging_insert_workspace_bytes(n)
        if ws is None:
            ws = _lib.workspace(need)
        _check(ws.numel() >= need, "workspace holds hb_staging_insert_workspace_bytes")
        _lib.check(lib.hb_staging_insert_gather(self.index.handle, C.byref(self.remote.desc), ids.data_ptr(),
                                                rows.data_ptr(), row_index.data_ptr(), n, self.emb.data_ptr(),
                                                self.dim * self.emb.element_size(), locs.data_ptr(),
                                                ws.data_ptr(), ws.numel(), _lib.stream_ptr()))
        return locs

    def insert_index(self, ids: torch.Tensor, ws: torch.Tensor):
        """First half of ``insert_gather``: ``add`` of the ids (negative ones ignored) to the index.
        Returns (locs, last_writer) for ``insert_rows``; ws as for ``insert_gather``, untouched
        until then."""
        lib = _lib.load()
        n = ids.numel()
        locs = torch.empty(n, dtype=torch.int64, device=ids.device)
        need = lib.hb_staging_insert_workspace_bytes(n)
        _check(ws.numel() >= need, "workspace holds hb_staging_insert_workspace_bytes")
        flag_bytes = -(-max(n, 1) // 256) * 256
        _lib.check(lib.hb_index_add(self.index.handle, ids.data_ptr(), n, locs.data_ptr(), ws.data_ptr(),
                                    ws.data_ptr() + flag_bytes, ws.numel() - flag_bytes, _lib.stream_ptr()))
        return locs, ws[:max(n, 1)]

    def insert_rows(self, rows: torch.Tensor, row_index: torch.Tensor, locs: torch.Tensor,
                    last_writer: torch.Tensor) -> None:
        """Second half: the embeddings rows[row_index[i]] into the cache rows at the slots the index
        gave, staging slots of the inserted entries reset."""
        _check(rows.size(1) == self.dim, "rows matches dim")
        lib = _lib.load()
        _lib.check(lib.hb_staging_insert_rows(C.byref(self.remote.desc), rows.data_ptr(), row_index.data_ptr(),
                                              locs.numel(), self.emb.data_ptr(), self.dim * self.emb.element_size(),
                                              locs.data_ptr(), last_writer.data_ptr(), _lib.stream_ptr()))

    # -- server step 3 -------------------------------------------------------------------
    def accumulate_remote(self, ids: torch.Tensor, grads: torch.Tensor, n_dev: torch.Tensor | None = None,
                          touch_lru: bool = True) -> None:
        """touch_lru=True also applies the LRU ageing of the server's CPU lookup
        (server.py:550 -> src/cache/cache.h:101).  n_dev: device int64 that caps the number
        of ids taken."""
        lib = _lib.load()
        locs = torch.empty_like(ids) if touch_lru else None  # written for every id the call takes (n_dev)
        _lib.check(lib.hb_staging_accumulate_cached(
            self.index.handle, C.byref(self.remote.desc), ids.data_ptr(), grads.data_ptr(), ids.numel(),
            _lib.ptr(n_dev), _lib.ptr(self.threshold), self.default_threshold, self.lookup_mode,
            self.dropped.data_ptr(), _lib.ptr(locs), _lib.stream_ptr()))
        if touch_lru:
            # ids are unique, so every position is its own run: no sort needed
            self.index.cuda_touch_lru_runs(locs, None, n_dev)

    def accumulate_local(self, ids: torch.Tensor, grads: torch.Tensor, n_dev: torch.Tensor | None = None) -> None:
        _check(self.local is not None, "a local staging table was configured")
        lib = _lib.load()
        _lib.check(lib.hb_staging_accumulate_direct(C.byref(self.local.desc), ids.data_ptr(), grads.data_ptr(),
                                                    ids.numel(), _lib.ptr(n_dev), self.local_start, 1,
                                                    _lib.stream_ptr()))

    # -- server step 0 -------------------------------------------------------------------
    def flush_remote(self, sync: bool = True, out_cap: int = 0):
        return self.remote.flush(self.index, self.cnt_threshold, self.num_clients, sync, out_cap)

    def flush_local(self, sync: bool = True, out_cap: int = 0):
        _check(self.local is not None, "a local staging table was configured")
        return self.local.flush(None, self.cnt_threshold, self.num_clients, sync, out_cap)
