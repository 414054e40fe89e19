"""Host side of ``hb_peer_table_*``: an embedding table sharded by owner (``id % world``) whose
shards every GPU of the box can read.  ``PeerTable.weight`` is this rank's shard as a tensor (the
optimiser updates it in place); ``lookup_fetch`` is the fused cache lookup + fetch whose misses
read the authoritative row from the owner's HBM over NVLink; ``gather`` fetches authoritative rows
without the cache (the reference's ``DistTensor.__getitem__``, python/EmbCache/dist_emb.py:168-169,
241-243).  Between an optimiser update and the next read all ranks pass a fence
(``EmbeddingPath`` does this)."""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import _lib
from .exchange import _as_tensor

_TYPESTR = {torch.float32: "<f4", torch.float16: "<f2", torch.float64: "<f8"}


class PeerTable:
    def __init__(self, num_rows: int, dim: int, rank: int = 0, world: int = 1, dtype=torch.float32,
                 device=None, group=None, connect: bool = True):
        """connect=False leaves the peers unmapped (``set_peer`` supplies their pointers: one
        process driving several GPUs, or tests)."""
        self.lib = _lib.load()
        self.rank, self.world, self.num_rows, self.dim, self.dtype = rank, world, int(num_rows), int(dim), dtype
        self.group = group
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        elem = torch.empty(0, dtype=dtype).element_size()
        self.row_bytes = dim * elem
        h = C.c_void_p()
        nbytes = self.lib.hb_peer_table_handle_bytes()
        mine = C.create_string_buffer(nbytes)
        err = None
        try:
            _lib.check(self.lib.hb_peer_table_create(rank, world, self.num_rows, self.row_bytes, C.byref(h)))
            self._h = h
            if world > 1 and connect:
                _lib.check(self.lib.hb_peer_table_export_handle(self._h, mine))
        except Exception as e:  # noqa: BLE001
            err = str(e)
        if world > 1 and connect:
            # collectives are entered by every rank, whether or not its local set-up worked
            gathered = [None] * world
            dist.all_gather_object(gathered, (err, bytes(mine.raw)), group=group)
            errs = [g[0] for g in gathered if g[0]]
            if errs:
                raise RuntimeError("peer table set-up failed on a rank: " + errs[0])
            try:
                _lib.check(self.lib.hb_peer_table_connect(self._h, b"".join(g[1] for g in gathered)))
                err = None
            except Exception as e:  # noqa: BLE001
                err = str(e)
            gathered = [None] * world
            dist.all_gather_object(gathered, err, group=group)
            errs = [g for g in gathered if g]
            if errs:
                raise RuntimeError("peer table could not map a peer's shard: " + errs[0])
        elif err:
            raise RuntimeError(err)
        ptr, rows = C.c_void_p(), C.c_int64()
        _lib.check(self.lib.hb_peer_table_local(self._h, C.byref(ptr), C.byref(rows)))
        self.rows_local = rows.value
        self.weight = _as_tensor(ptr.value, (max(self.rows_local, 1), dim), _TYPESTR[dtype], self.device)[: self.rows_local]

    def close(self) -> None:
        """Release the shared memory.  A collective when world > 1: every rank calls it, at a
        point where no kernel of any rank touches a peer's memory any more.  (Mappings are closed
        on all ranks before any rank frees: freeing memory a peer still has mapped is undefined
        behaviour of the CUDA IPC interface.  Dropping the last reference without close() only
        frees this rank's side, which is safe at process exit.)"""
        if not getattr(self, "_h", None):
            return
        if self.world > 1:
            torch.cuda.synchronize()
            dist.barrier(group=self.group)
        self.lib.hb_peer_table_disconnect(self._h)
        if self.world > 1:
            dist.barrier(group=self.group)
        self.lib.hb_peer_table_destroy(self._h)
        self._h = None

    def __del__(self):
        if getattr(self, "_h", None):
            try:
                self.lib.hb_peer_table_destroy(self._h)
            except Exception:
                pass
            self._h = None

    @property
    def handle(self):
        return self._h

    def set_peer(self, rank: int, shard: torch.Tensor) -> None:
        _lib.check(self.lib.hb_peer_table_set_peer(self._h, rank, shard.data_ptr()))

    def gather(self, ids: torch.Tensor, n_dev: torch.Tensor | None = None, out: torch.Tensor | None = None):
        n = ids.numel()
        if out is None:
            out = torch.empty((n, self.dim), dtype=self.dtype, device=ids.device)
        _lib.check(self.lib.hb_peer_table_gather(self._h, ids.contiguous().data_ptr(), n, _lib.ptr(n_dev),
                                                 out.data_ptr(), _lib.stream_ptr()))
        return out

    def serve(self, stages: "PeerTable", req_ids: torch.Tensor, req_rows: torch.Tensor, req_counts: torch.Tensor,
              seg_cap: int) -> None:
        """The owner's half of a forward fetch in which the owners deliver (``hb_fetch_serve``):
        requests as they arrived through a ``PeerExchange`` (segment s from rank s, req_counts[s]
        valid): the row of req_ids[k] in this rank's shard goes into row req_rows[k] of rank s's
        stage.  stages: a PeerTable whose local shard on every rank is that rank's stage."""
        _lib.check(self.lib.hb_fetch_serve(self._h, stages.handle, req_ids.data_ptr(), req_rows.data_ptr(),
                                           req_counts.data_ptr(), int(seg_cap), _lib.stream_ptr()))

    def lookup_fetch(self, index, ids: torch.Tensor, cache_rows: torch.Tensor, out_rows: torch.Tensor | None = None,
                     mode: int | None = None):
        """(rows, locs, found) as ``EmbCacheLib.cudaLookupFetch``, misses from the owners' shards."""
        n = ids.numel()
        if out_rows is None:
            out_rows = torch.empty((n, self.dim), dtype=self.dtype, device=ids.device)
        locs = torch.empty(n, dtype=torch.int64, device=ids.device)
        found = torch.empty(n, dtype=torch.bool, device=ids.device)
        _lib.check(self.lib.hb_lookup_fetch_sharded(index.handle, ids.contiguous().data_ptr(), n, cache_rows.data_ptr(),
                                                    self._h, out_rows.data_ptr(), locs.data_ptr(), found.data_ptr(),
                                                    index.lookup_mode if mode is None else mode, _lib.stream_ptr()))
        return out_rows, locs, found
