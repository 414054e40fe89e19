"""Owner-partitioned exchange of (id, cnt, row) over peer memory: the host side of
``hb_a2a_*``.  One fused pack+push kernel per rank stores every bucket into its owner's receive
slab over NVLink; one small collective orders the push before the use of what was received.
No sizes travel through the host, so a step that uses it has no host synchronisation at all
(the reference reads the split sizes on the host twice per exchange,
python/EmbCache/sparse_optim.py:55,77).
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import _lib


class _RawCuda:
    """A device buffer owned by the library, exposed through __cuda_array_interface__."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False),
                                         "version": 3, "strides": None}


def _as_tensor(ptr: int, shape, typestr: str, device) -> torch.Tensor:
    return torch.as_tensor(_RawCuda(ptr, shape, typestr), device=device)


class PeerExchange:
    def __init__(self, rank: int, world: int, cap_rows: int, dim: int, row_dtype=torch.float32,
                 device=None, group=None, fence: str = "device"):
        """fence: "device" = hb_a2a_fence (flags in peer memory, bounded wait, no collective
        library); "nccl" = a 4-byte all-reduce."""
        self.fence_kind = fence
        self.next_parity = 0  # receive area the next push fills
        self.lib = _lib.load()
        self.rank, self.world, self.cap, self.dim, self.group = rank, world, int(cap_rows), dim, group
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        self.row_dtype = row_dtype
        elem = torch.empty(0, dtype=row_dtype).element_size()
        h = C.c_void_p()
        nbytes = self.lib.hb_a2a_handle_bytes()
        mine = C.create_string_buffer(nbytes)
        err = None
        try:
            _lib.check(self.lib.hb_a2a_create(rank, world, self.cap, dim * elem, C.byref(h)))
            self._h = h
            _lib.check(self.lib.hb_a2a_export_handle(self._h, mine))
        except Exception as e:  # noqa: BLE001
            err = str(e)
        if world > 1:
            # collectives are entered by every rank, whether or not its local set-up worked
            gathered = [None] * world
            dist.all_gather_object(gathered, (err, bytes(mine.raw), (self.cap, dim * elem)), group=group)
            errs = [g[0] for g in gathered if g[0]]
            if errs:
                raise RuntimeError("peer exchange set-up failed on a rank: " + errs[0])
            shapes = {g[2] for g in gathered}
            if len(shapes) != 1:
                # every rank computes the offsets inside a peer's area from its own numbers
                raise RuntimeError(f"peer exchange: (slab rows, row bytes) differ between the ranks: {sorted(shapes)}")
            blob = b"".join(g[1] for g in gathered)
        else:
            if err:
                raise RuntimeError(err)
            blob = bytes(mine.raw)
        try:
            _lib.check(self.lib.hb_a2a_connect(self._h, blob))
            err = None
        except Exception as e:  # noqa: BLE001
            err = str(e)
        if world > 1:
            gathered = [None] * world
            dist.all_gather_object(gathered, err, group=group)
            errs = [g for g in gathered if g]
            if errs:
                raise RuntimeError("peer exchange could not map a peer's memory: " + errs[0])
        elif err:
            raise RuntimeError(err)
        self._token = torch.zeros(1, dtype=torch.int32, device=self.device)
        typestr = {torch.float32: "<f4", torch.float16: "<f2", torch.float64: "<f8"}[row_dtype]
        self._views = []
        for parity in (0, 1):
            ids, rows, cnt, counts = C.c_void_p(), C.c_void_p(), C.c_void_p(), C.c_void_p()
            cap = C.c_int64()
            _lib.check(self.lib.hb_a2a_recv_view(self._h, parity, C.byref(ids), C.byref(rows), C.byref(cnt),
                                                 C.byref(counts), C.byref(cap)))
            n = world * self.cap
            self._views.append((_as_tensor(ids.value, (n,), "<i8", self.device),
                                _as_tensor(rows.value, (n, dim), typestr, self.device),
                                _as_tensor(cnt.value, (n,), "<i8", self.device),
                                _as_tensor(counts.value, (world,), "<i8", self.device)))
        if world > 1:
            dist.barrier(group=group)  # every rank has mapped every area before anyone pushes

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
        self.lib.hb_a2a_disconnect(self._h)
        if self.world > 1:
            dist.barrier(group=self.group)
        self.lib.hb_a2a_destroy(self._h)
        self._h = None

    def __del__(self):
        if getattr(self, "_h", None):
            try:
                self.lib.hb_a2a_destroy(self._h)
            except Exception:
                pass
            self._h = None

    @property
    def handle(self):
        return self._h

    def push_workspace_bytes(self, n: int) -> int:
        return self.lib.hb_a2a_push_workspace_bytes(int(n), self.world)

    def push(self, ids, rows, cnt=None, n_dev=None, sent_counts=None, ws=None) -> int:
        """Bucket by owner and store into the owners' slabs; returns the parity to read.  ws: scratch
        of ``push_workspace_bytes(n)`` bytes (default: the library-wide scratch of the device, which
        is only safe on the stream that everything else using it runs on)."""
        n = ids.numel()
        need = self.lib.hb_a2a_push_workspace_bytes(n, self.world)
        if ws is None or ws.numel() < need:
            ws = _lib.workspace(need)
        parity = C.c_int(0)
        _lib.check(self.lib.hb_a2a_push(self._h, ids.data_ptr(), rows.data_ptr(), _lib.ptr(cnt), n,
                                        _lib.ptr(n_dev), _lib.ptr(sent_counts), C.byref(parity),
                                        ws.data_ptr(), ws.numel(), _lib.stream_ptr()))
        self.next_parity = parity.value ^ 1
        return parity.value

    def fence(self) -> None:
        """Order every rank's push before every rank's reads: one tiny collective on the
        current stream (no host synchronisation)."""
        if self.world > 1:
            if self.fence_kind == "device":
                _lib.check(self.lib.hb_a2a_fence(self._h, _lib.stream_ptr()))
            else:
                dist.all_reduce(self._token, group=self.group)

    def reset(self) -> None:
        """Back to the state after set-up (``hb_a2a_reset``): every rank calls it, after the host
        side has agreed that all ranks are alive, and nobody pushes until all have returned."""
        if self.world > 1:
            torch.cuda.synchronize()
            dist.barrier(group=self.group)  # nobody still pushes or polls
        _lib.check(self.lib.hb_a2a_reset(self._h, _lib.stream_ptr()))
        self.next_parity = 0
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier(group=self.group)  # every area is clean before the next push

    def received(self, parity: int):
        """(ids [world*cap], rows [world*cap, dim], cnt [world*cap], counts [world]) of this
        rank's receive area: segment s holds counts[s] valid rows from rank s."""
        return self._views[parity]
