"""Drop-in for the reference's pybind module ``EmbCacheLib`` (src/pybind.cc:16-71).

Same names, argument order and error behaviour (shape mismatches raise ``RuntimeError`` as
the reference's ``CHECK`` does); every operation runs in ``libhades_b200.so`` on the
current CUDA stream.  New capabilities have new names (``cudaLookupFetch``,
``cudaUniqueSegSum``, ...); no reference name changes meaning.

Differences that a caller can observe:

* kernels run on torch's current stream, not on the legacy default stream
  (the reference launches ``<<<grid, block>>>`` with no stream, e.g. src/cuda/uva_fetch.cu:39);
* a CUDA error raises instead of ending the process (src/utils.h:12-24 calls ``exit``);
* ``IndexCache`` keeps its state in HBM.  ``create=True`` also leaves a small file
  ``/dev/shm/hades_b200_index_<name>`` with a CUDA IPC handle, through which
  ``IndexCache(size, name, create=False)`` in ANOTHER process of the box opens the same lines
  (the reference opens the creator's POSIX segment, src/cache/cache.h:145-167); inside one
  process the name resolves in a registry.  ``pin_memory`` is accepted and ignored (there is
  no host copy to pin);
* ``IndexCache.add`` applies ids in input order per set, which is the reference's result at
  ``OMP_NUM_THREADS=1`` (its multi-threaded result depends on thread timing).
"""
from __future__ import annotations

import atexit
import ctypes as C

import torch

from . import _lib
from ._lib import LOOKUP_SETASSOC, LOOKUP_SORTED, MOVER_AUTO, MOVER_BULK, MOVER_LSU  # noqa: F401

_REGISTRY: dict[str, "IndexCache"] = {}


def _index_handle_path(name: str) -> str:
    return "/dev/shm/hades_b200_index_" + name.replace("/", "_")


_PUBLISHED: set = set()  # handle files this process left in /dev/shm


def _withdraw_published() -> None:
    import os

    for path in list(_PUBLISHED):
        try:
            os.unlink(path)
        except OSError:
            pass
    _PUBLISHED.clear()


atexit.register(_withdraw_published)


def _check(cond: bool, what: str) -> None:
    if not cond:
        raise RuntimeError(f"Check failed: {what}")


def _idx_bytes(t: torch.Tensor) -> int:
    if t.dtype == torch.int64:
        return 8
    if t.dtype == torch.int32:
        return 4
    raise RuntimeError("ID can only be int32 or int64")  # src/utils.h:48


def _check_float(t: torch.Tensor) -> None:
    if t.dtype not in (torch.float32, torch.float64):
        raise RuntimeError("Type can only be float or double")  # src/utils.h:35


def _row_bytes(t: torch.Tensor) -> int:
    dim = 1 if t.dim() == 1 else t.size(1)
    return dim * t.element_size()


def _dev_ptr(t: torch.Tensor, what: str) -> int:
    """Device-usable address of a tensor: CUDA memory, or pinned host memory (the
    reference's UVA arguments, registered with cudaPin)."""
    if t.is_cuda or t.is_pinned() or t.data_ptr() in _PINNED:
        if not t.is_contiguous():
            raise RuntimeError(f"{what} must be contiguous")
        return t.data_ptr()
    raise RuntimeError(f"{what} must be a CUDA tensor or pinned host memory (cudaPin)")


class IndexCache:
    """IndexCache(cache_size, name, create, pin_memory=True), src/pybind.cc:17-33."""

    def __init__(self, cache_size: int, name: str, create: bool, pin_memory: bool = True,
                 lookup_mode: int = LOOKUP_SETASSOC):
        self._lib = _lib.load()
        self._name = name
        self.lookup_mode = lookup_mode
        self._shm_file = None
        if create:
            h = C.c_void_p()
            _lib.check(self._lib.hb_index_create(int(cache_size), C.byref(h)))
            self._h = h
            self._owner = True
            self._device = torch.cuda.current_device()
            _REGISTRY[name] = self
            self._publish()
        elif name in _REGISTRY:
            other = _REGISTRY[name]
            self._h = other._h
            self._owner = False
            self._device = other._device
        else:
            # another process of this box created it: map its lines (src/cache/cache.h:155-158)
            path = _index_handle_path(name)
            try:
                with open(path, "rb") as f:
                    blob = f.read()
            except OSError as e:
                raise RuntimeError(f"fail to open {name}: no such index on this box ({e.strerror})") from e
            _check(len(blob) == self._lib.hb_index_handle_bytes(), "index handle file has the expected size")
            h = C.c_void_p()
            _lib.check(self._lib.hb_index_open(blob, C.byref(h)))
            self._h = h
            self._owner = True  # of the mapping: destroyed (closed) with this object
            self._device = torch.cuda.current_device()

    def _publish(self) -> None:
        """Leave the IPC handle where other processes of the box find it by name."""
        import os

        buf = C.create_string_buffer(self._lib.hb_index_handle_bytes())
        try:
            _lib.check(self._lib.hb_index_export_handle(self._h, buf))
            path = _index_handle_path(self._name)
            with open(path + ".tmp", "wb") as f:
                f.write(buf.raw)
            os.replace(path + ".tmp", path)
            self._shm_file = path
            _PUBLISHED.add(path)
        except (OSError, _lib.HadesError):
            self._shm_file = None  # no IPC here (or no /dev/shm): the index stays private to this process

    def close(self) -> None:
        """Withdraw the published handle and free the index (the creator) or unmap it (an opener).
        Openers close before the creator does.  The object cannot be used afterwards."""
        if getattr(self, "_shm_file", None):
            _PUBLISHED.discard(self._shm_file)
            try:
                import os

                os.unlink(self._shm_file)
            except Exception:
                pass
            self._shm_file = None
        if getattr(self, "_owner", False) and getattr(self, "_h", None):
            try:
                self._lib.hb_index_destroy(self._h)
                if _REGISTRY is not None and _REGISTRY.get(self._name) is self:
                    _REGISTRY.pop(self._name, None)
            except Exception:  # interpreter shutdown: modules may already be gone
                pass
        self._h = None

    def __del__(self):
        self.close()

    # --- sizes -------------------------------------------------------------------------
    def get_size(self) -> int:
        return self._lib.hb_index_size(self._h)

    def get_capacity(self) -> int:
        return self._lib.hb_index_capacity(self._h)

    def get_space(self) -> int:
        return self._lib.hb_index_space(self._h)

    def get_valid_entries_num(self) -> int:
        out = C.c_int64(0)
        _lib.check(self._lib.hb_index_valid_entries(self._h, C.byref(out), _lib.stream_ptr()))
        return out.value

    # --- reference surface: CPU tensors in and out --------------------------------------
    def _to_dev(self, ids: torch.Tensor) -> torch.Tensor:
        _check(ids.dtype == torch.int64, "ids.dtype == int64")
        return ids.contiguous().to(f"cuda:{self._device}", non_blocking=False)

    def add(self, ids: torch.Tensor) -> torch.Tensor:
        out = self.cuda_add(self._to_dev(ids))
        return out if ids.is_cuda else out.cpu()

    def lookup(self, ids: torch.Tensor) -> torch.Tensor:
        """CPU lookup of the reference (src/cache/cache.h:213-222): returns the slots and
        applies the LRU side effect of every hit, in batch order."""
        dev = self._to_dev(ids)
        locs = self.cudalookup(dev)
        self.cuda_touch_lru(locs)
        return locs if ids.is_cuda else locs.cpu()

    def reset(self, ids: torch.Tensor) -> None:
        dev = self._to_dev(ids)
        _lib.check(self._lib.hb_index_reset(self._h, dev.data_ptr(), dev.numel(), _lib.stream_ptr()))

    def getall(self, length: int):
        dev = f"cuda:{self._device}"
        ids = torch.zeros(length, dtype=torch.int64, device=dev)
        locs = torch.full((length,), -1, dtype=torch.int64, device=dev)
        n = C.c_int64(0)
        _lib.check(self._lib.hb_index_getall(self._h, ids.data_ptr(), locs.data_ptr(), int(length),
                                             C.byref(n), _lib.stream_ptr()))
        return ids.cpu(), locs.cpu()

    def cudalookup(self, ids: torch.Tensor, mode: int | None = None) -> torch.Tensor:
        """GPU lookup (src/cache/lookup.cu:64-85): CUDA ids in, CUDA slots out, LRU
        counters untouched."""
        _check(ids.is_cuda and ids.dtype == torch.int64, "ids is a CUDA int64 tensor")
        ids = ids.contiguous()
        locs = torch.empty_like(ids)
        _lib.check(self._lib.hb_index_lookup(self._h, ids.data_ptr(), ids.numel(), locs.data_ptr(),
                                             None, self.lookup_mode if mode is None else mode,
                                             _lib.stream_ptr()))
        return locs

    # --- device-side extensions ------------------------------------------------------------
    def cuda_add(self, ids: torch.Tensor) -> torch.Tensor:
        _check(ids.is_cuda and ids.dtype == torch.int64, "ids is a CUDA int64 tensor")
        ids = ids.contiguous()
        locs = torch.empty_like(ids)
        need = self._lib.hb_index_add_workspace_bytes(ids.numel())
        ws = _lib.workspace(need)
        _lib.check(self._lib.hb_index_add(self._h, ids.data_ptr(), ids.numel(), locs.data_ptr(), None,
                                          ws.data_ptr(), ws.numel(), _lib.stream_ptr()))
        return locs

    def cuda_touch_lru(self, locs: torch.Tensor) -> None:
        need = self._lib.hb_index_touch_lru_workspace_bytes(locs.numel())
        ws = _lib.workspace(need)
        _lib.check(self._lib.hb_index_touch_lru(self._h, locs.data_ptr(), locs.numel(),
                                                ws.data_ptr(), ws.numel(), _lib.stream_ptr()))

    def cuda_touch_lru_runs(self, locs: torch.Tensor, runs=None, n_dev: torch.Tensor | None = None,
                            locs_kind: int = 0) -> None:
        """LRU ageing for a batch grouped in runs of equal ids (no sort).  runs: the
        ``BatchRuns`` of ``cudaRunsBuild`` (or the ``RunsDesc`` returned by
        ``cudaUniqueSegSum(..., want_runs=True)``, valid until another call uses the shared
        workspace) for the ids that were looked up; None: the batch holds each id once (every
        position is its own run).  locs_kind: locs holds a slot per batch position (0), per
        sorted entry (1) or per run (2: ``BatchRuns.slots`` after ``cudaLookupFetchRuns``)."""
        n = locs.numel()
        if runs is None:
            _lib.check(self._lib.hb_index_touch_lru_runs(self._h, locs.data_ptr(), None, None, n, None, n,
                                                         _lib.ptr(n_dev), 0, _lib.stream_ptr()))
        else:
            runs = getattr(runs, "desc", runs)  # a BatchRuns or its RunsDesc
            cap = _lib.ptr(n_dev) if n_dev is not None else runs.n_dev
            _lib.check(self._lib.hb_index_touch_lru_runs(self._h, locs.data_ptr(), runs.perm, runs.run_start,
                                                         n, runs.num_runs, n, cap, int(locs_kind),
                                                         _lib.stream_ptr()))

    def cuda_lookup_found(self, ids: torch.Tensor, mode: int | None = None):
        """(slots, found mask) in one launch."""
        ids = ids.contiguous()
        locs = torch.empty_like(ids)
        found = torch.empty(ids.shape, dtype=torch.bool, device=ids.device)
        _lib.check(self._lib.hb_index_lookup(self._h, ids.data_ptr(), ids.numel(), locs.data_ptr(),
                                             found.data_ptr(),
                                             self.lookup_mode if mode is None else mode,
                                             _lib.stream_ptr()))
        return locs, found

    def build_sorted(self) -> None:
        _lib.check(self._lib.hb_index_build_sorted(self._h, _lib.stream_ptr()))

    def export_state(self):
        cap = self.get_capacity()
        dev = f"cuda:{self._device}"
        ids = torch.empty(cap, dtype=torch.int64, device=dev)
        lru = torch.empty(cap, dtype=torch.int32, device=dev)
        _lib.check(self._lib.hb_index_export(self._h, ids.data_ptr(), lru.data_ptr(), _lib.stream_ptr()))
        return ids, lru

    def import_state(self, line_ids: torch.Tensor, lru: torch.Tensor) -> None:
        cap = self.get_capacity()
        _check(line_ids.numel() == cap and lru.numel() == cap, "state tensors have capacity entries")
        dev = f"cuda:{self._device}"
        line_ids = line_ids.to(dev, torch.int64).contiguous()
        lru = lru.to(dev, torch.int32).contiguous()
        _lib.check(self._lib.hb_index_import(self._h, line_ids.data_ptr(), lru.data_ptr(),
                                             _lib.stream_ptr()))

    @property
    def handle(self) -> C.c_void_p:
        return self._h


# ---------------------------------------------------------------------------------------
# host pinning: src/cuda/pin_memory.cu:9-26
# ---------------------------------------------------------------------------------------
_PINNED: dict[int, int] = {}


def _cudart():
    return torch.cuda.cudart()


def cudaPin(tensor: torch.Tensor) -> None:
    ptr_, size = tensor.data_ptr(), tensor.numel() * tensor.element_size()
    cudaPinPtr(ptr_, size)


def cudaUnpin(tensor: torch.Tensor) -> None:
    cudaUnpinPtr(tensor.data_ptr())


def cudaPinPtr(ptr: int, size: int) -> None:
    err = _cudart().cudaHostRegister(ptr, size, 0)
    if int(err) != 0:
        raise RuntimeError(f"cudaHostRegister failed with error {int(err)}")
    _PINNED[ptr] = size


def cudaUnpinPtr(ptr: int) -> None:
    err = _cudart().cudaHostUnregister(ptr)
    if int(err) != 0:
        raise RuntimeError(f"cudaHostUnregister failed with error {int(err)}")
    _PINNED.pop(ptr, None)


# ---------------------------------------------------------------------------------------
# named host shared memory: src/shm/shared_memory.h:14-64 (bound in src/pybind.cc:37-45)
# Host plumbing of the reference's socket/shm control plane; kept so that code which creates
# shared tensors through this module still runs.  No GPU work happens here.
# ---------------------------------------------------------------------------------------
_SHM: dict[int, tuple] = {}


def _shm_path(name: str) -> str:
    return "/dev/shm/" + name.lstrip("/")


def _map_shared(name: str, size: int, create: bool, pin_memory: bool):
    import mmap
    import os

    flags = os.O_RDWR | (os.O_CREAT if create else 0)
    try:
        fd = os.open(_shm_path(name), flags, 0o600)
    except OSError as e:
        raise RuntimeError(f"fail to open {name}: {e.strerror}") from e
    if create:
        os.ftruncate(fd, int(size))
    mm = mmap.mmap(fd, int(size), mmap.MAP_SHARED, mmap.PROT_READ | mmap.PROT_WRITE)
    buf = (C.c_char * int(size)).from_buffer(mm)
    ptr_ = C.addressof(buf)
    _SHM[ptr_] = (mm, buf, fd, name)
    if pin_memory:
        cudaPinPtr(ptr_, int(size))
    return ptr_, fd


def create_shared_mem(name: str, size: int, pin_memory: bool = True):
    """(ptr, fd) of a new named segment; src/shm/shared_memory.h:14-32."""
    return _map_shared(name, size, True, pin_memory)


def open_shared_mem(name: str, size: int, pin_memory: bool = True):
    """(ptr, fd) of an existing named segment; src/shm/shared_memory.h:34-48."""
    return _map_shared(name, size, False, pin_memory)


def release_shared_mem(name: str, size: int, ptr: int, fd: int, pin_memory: bool = True) -> None:
    """Unpin, unmap, close and unlink; src/shm/shared_memory.h:50-57."""
    import os

    if pin_memory:
        cudaUnpinPtr(ptr)
    ent = _SHM.pop(ptr, None)
    if ent is not None:
        mm, buf, _, _ = ent
        del buf
        try:
            mm.close()
        except BufferError:
            pass  # a tensor still views the mapping; it is released with that tensor
    try:
        os.close(fd)
    except OSError:
        pass
    try:
        os.unlink(_shm_path(name))
    except FileNotFoundError:
        pass


def open_shared_tensor(ptr: int, dtype, shape):
    """A tensor over shared memory (torch::from_blob); src/shm/shared_memory.h:59-64."""
    numel = 1
    for d in shape:
        numel *= int(d)
    nbytes = numel * torch.empty(0, dtype=dtype).element_size()
    raw = (C.c_char * nbytes).from_address(ptr)
    return torch.frombuffer(raw, dtype=dtype, count=numel).view(*shape) if numel else torch.empty(shape, dtype=dtype)


# ---------------------------------------------------------------------------------------
# row movers: src/cuda/ops.h:15-31
# ---------------------------------------------------------------------------------------
def cudaFetch(src, src_index, dst, dst_index, mover: int = MOVER_AUTO) -> None:
    """dst[dst_index] = src[src_index] (src/cuda/uva_fetch.cu:28-45)."""
    _check(src.size(1) == dst.size(1), "src.size(1) == dst.size(1)")
    _check(dst_index.numel() == src_index.numel(), "dst_index.numel() == src_index.numel()")
    _check_float(src)
    _check(dst_index.dtype == src_index.dtype, "index dtypes match")
    lib = _lib.load()
    _lib.check(lib.hb_rows_gather(_dev_ptr(src, "src"), _dev_ptr(src_index, "src_index"),
                                  _dev_ptr(dst, "dst"), _dev_ptr(dst_index, "dst_index"),
                                  src_index.numel(), _row_bytes(src), _idx_bytes(src_index), mover,
                                  _lib.stream_ptr()))


def cudaFetch2(src, src_index, dst, mover: int = MOVER_AUTO) -> None:
    """dst[i] = src[src_index[i]], 1-D or 2-D (src/cuda/uva_fetch.cu:72-106)."""
    _check(src.dim() in (1, 2), "src.sizes().size() == 1 || src.sizes().size() == 2")
    _check(src.dim() == dst.dim(), "src.sizes().size() == dst.sizes().size()")
    if src.dim() == 2:
        _check(src.size(1) == dst.size(1), "src.size(1) == dst.size(1)")
    _check_float(src)
    lib = _lib.load()
    _lib.check(lib.hb_rows_gather(_dev_ptr(src, "src"), _dev_ptr(src_index, "src_index"),
                                  _dev_ptr(dst, "dst"), None, src_index.numel(), _row_bytes(src),
                                  _idx_bytes(src_index), mover, _lib.stream_ptr()))


def cudaFetchWithCache2(cpu_src, gpu_src, src_index, index_map, dst, found=None) -> None:
    """Cached fetch through a dense index map (src/cuda/uva_fetch.cu:149-192)."""
    _check(gpu_src.dim() in (1, 2), "gpu_src.sizes().size() == 1 || gpu_src.sizes().size() == 2")
    _check(gpu_src.dim() == cpu_src.dim(), "gpu_src.sizes().size() == cpu_src.sizes().size()")
    _check(gpu_src.dim() == dst.dim(), "gpu_src.sizes().size() == dst.sizes().size()")
    if gpu_src.dim() == 2:
        _check(gpu_src.size(1) == cpu_src.size(1), "gpu_src.size(1) == cpu_src.size(1)")
        _check(gpu_src.size(1) == dst.size(1), "gpu_src.size(1) == dst.size(1)")
    _check_float(gpu_src)
    _check(src_index.dtype == index_map.dtype, "index dtypes match")
    lib = _lib.load()
    _lib.check(lib.hb_rows_gather_cached(_dev_ptr(cpu_src, "cpu_src"), _dev_ptr(gpu_src, "gpu_src"),
                                         _dev_ptr(src_index, "src_index"),
                                         _dev_ptr(index_map, "index_map"), _dev_ptr(dst, "dst"),
                                         _lib.ptr(found), src_index.numel(), _row_bytes(gpu_src),
                                         _idx_bytes(src_index), _lib.stream_ptr()))


def cudaSet(src, dst, dst_index, mover: int = MOVER_AUTO) -> None:
    """dst[dst_index[i]] = src[i] (src/cuda/uva_set.cu:35-69)."""
    _check(src.dim() in (1, 2), "src.sizes().size() == 1 || src.sizes().size() == 2")
    _check(src.dim() == dst.dim(), "src.sizes().size() == dst.sizes().size()")
    if src.dim() == 2:
        _check(src.size(1) == dst.size(1), "src.size(1) == dst.size(1)")
    _check_float(src)
    lib = _lib.load()
    _lib.check(lib.hb_rows_scatter(_dev_ptr(src, "src"), _dev_ptr(dst, "dst"),
                                   _dev_ptr(dst_index, "dst_index"), dst_index.numel(),
                                   _row_bytes(src), _idx_bytes(dst_index), mover, _lib.stream_ptr()))


def cudaSetWithCache(src, cpu_dst, gpu_dst, dst_index, index_map) -> None:
    """Cached set through a dense index map (src/cuda/uva_set.cu:112-154)."""
    _check(gpu_dst.dim() in (1, 2), "gpu_dst.sizes().size() == 1 || gpu_dst.sizes().size() == 2")
    _check(gpu_dst.dim() == cpu_dst.dim(), "gpu_dst.sizes().size() == cpu_dst.sizes().size()")
    _check(gpu_dst.dim() == src.dim(), "gpu_dst.sizes().size() == src.sizes().size()")
    if gpu_dst.dim() == 2:
        _check(gpu_dst.size(1) == cpu_dst.size(1), "gpu_dst.size(1) == cpu_dst.size(1)")
        _check(gpu_dst.size(1) == src.size(1), "gpu_dst.size(1) == src.size(1)")
    _check_float(gpu_dst)
    _check(dst_index.dtype == index_map.dtype, "index dtypes match")
    lib = _lib.load()
    _lib.check(lib.hb_rows_scatter_cached(_dev_ptr(src, "src"), _dev_ptr(cpu_dst, "cpu_dst"),
                                          _dev_ptr(gpu_dst, "gpu_dst"),
                                          _dev_ptr(dst_index, "dst_index"),
                                          _dev_ptr(index_map, "index_map"), dst_index.numel(),
                                          _row_bytes(gpu_dst), _idx_bytes(dst_index),
                                          _lib.stream_ptr()))


def cudaCombine(src, dst, dst_index, mover: int = MOVER_AUTO) -> None:
    """dst[dst_index[i]] = src[i] (src/cuda/uva_fetch.cu:212-228)."""
    _check(src.size(1) == dst.size(1), "src.size(1) == dst.size(1)")
    _check_float(src)
    lib = _lib.load()
    _lib.check(lib.hb_rows_scatter(_dev_ptr(src, "src"), _dev_ptr(dst, "dst"),
                                   _dev_ptr(dst_index, "dst_index"), dst_index.numel(),
                                   _row_bytes(src), _idx_bytes(dst_index), mover, _lib.stream_ptr()))


# ---------------------------------------------------------------------------------------
# split and owner search: src/cuda/ops.h:11,35-41
# ---------------------------------------------------------------------------------------
def cudaSplit(ids: torch.Tensor, mask: torch.Tensor):
    """[local_mask, remote_hot_mask, remote_cold_mask] (src/cuda/split.cu:12-56)."""
    _check(ids.is_cuda and mask.is_cuda, "ids and mask are CUDA tensors")
    _check(ids.dtype == torch.int64, "ids.dtype == int64")
    _check(mask.dtype == torch.int8, "mask.dtype == int8")
    n = ids.numel()
    out = [torch.zeros(n, dtype=torch.bool, device=ids.device) for _ in range(3)]
    lib = _lib.load()
    _lib.check(lib.hb_split_masks(ids.contiguous().data_ptr(), n, mask.data_ptr(),
                                  out[0].data_ptr(), out[1].data_ptr(), out[2].data_ptr(),
                                  _lib.stream_ptr()))
    return out


def cudaReminder(input: torch.Tensor, local_num_gpus: int) -> torch.Tensor:
    """in % local_num_gpus (src/cuda/binary_search.cu:76-89)."""
    out = torch.empty_like(input)
    lib = _lib.load()
    _lib.check(lib.hb_owner_mod(_dev_ptr(input, "in"), input.size(0), _idx_bytes(input),
                                int(local_num_gpus), out.data_ptr(), _lib.stream_ptr()))
    return out


def cudaBinarySearch(input: torch.Tensor, range_partition: torch.Tensor,
                     local_num_gpus: int) -> torch.Tensor:
    """(upper_bound(range_partition, in) - 1) * g + in % g (src/cuda/binary_search.cu:45-59)."""
    _check(input.dtype == range_partition.dtype, "in and range_partition dtypes match")
    out = torch.empty_like(input)
    lib = _lib.load()
    _lib.check(lib.hb_owner_range(_dev_ptr(input, "in"), input.size(0), _idx_bytes(input),
                                  _dev_ptr(range_partition, "range_partition"),
                                  range_partition.size(0), int(local_num_gpus), out.data_ptr(),
                                  _lib.stream_ptr()))
    return out


def cudaBinarySearch2(input: torch.Tensor, range: torch.Tensor) -> torch.Tensor:
    """upper_bound(range, in) (src/cuda/binary_search.cu:61-74)."""
    _check(input.dtype == range.dtype, "in and range dtypes match")
    out = torch.empty_like(input)
    lib = _lib.load()
    _lib.check(lib.hb_upper_bound(_dev_ptr(input, "in"), input.size(0), _idx_bytes(input),
                                  _dev_ptr(range, "range"), range.size(0), out.data_ptr(),
                                  _lib.stream_ptr()))
    return out


# ---------------------------------------------------------------------------------------
# new entry points (no counterpart name in the reference module)
# ---------------------------------------------------------------------------------------
def cudaLookupFetch(index: IndexCache, ids, cache_rows, backing_rows, out_rows=None,
                    mode: int | None = None, mover: int = MOVER_AUTO, want_locs: bool = True):
    """Fused IndexCache lookup + cached fetch: returns (out_rows, locs, found)."""
    _check(ids.is_cuda and ids.dtype == torch.int64, "ids is a CUDA int64 tensor")
    ids = ids.contiguous()
    n = ids.numel()
    if out_rows is None:
        out_rows = torch.empty((n, cache_rows.size(1)), dtype=cache_rows.dtype, device=ids.device)
    _check(out_rows.size(1) == cache_rows.size(1), "out_rows.size(1) == cache_rows.size(1)")
    if backing_rows is not None:
        _check(backing_rows.size(1) == cache_rows.size(1), "backing_rows.size(1) == cache_rows.size(1)")
    locs = torch.empty(n, dtype=torch.int64, device=ids.device) if want_locs else None
    found = torch.empty(n, dtype=torch.bool, device=ids.device)
    lib = _lib.load()
    _lib.check(lib.hb_lookup_fetch(index.handle, ids.data_ptr(), n, _dev_ptr(cache_rows, "cache_rows"),
                                   None if backing_rows is None else _dev_ptr(backing_rows, "backing_rows"),
                                   _row_bytes(cache_rows), out_rows.data_ptr(), _lib.ptr(locs),
                                   found.data_ptr(), index.lookup_mode if mode is None else mode,
                                   mover, _lib.stream_ptr()))
    return out_rows, locs, found


def cudaAccumulate(src, dst, dst_index, cnt=None) -> None:
    """dst[dst_index[i]] += src[i]; cnt[dst_index[i]] += 1 (unique indices, fp32)."""
    _check(src.dtype == torch.float32 and dst.dtype == torch.float32, "fp32 rows")
    _check(src.dim() == 2 and dst.dim() == 2 and src.size(1) == dst.size(1), "src.size(1) == dst.size(1)")
    if cnt is not None:
        _check(cnt.dtype == torch.int32, "cnt.dtype == int32")
    lib = _lib.load()
    _lib.check(lib.hb_rows_accumulate_f32(src.data_ptr(), dst.data_ptr(), dst_index.data_ptr(),
                                          _lib.ptr(cnt), dst_index.numel(), src.size(1),
                                          _idx_bytes(dst_index), _lib.stream_ptr()))


def cudaSplitCompact(ids: torch.Tensor, mask: torch.Tensor, want_masks: bool = True):
    """cudaSplit fused with the nonzero() calls that follow it: returns
    (masks or None, index tensor, counts[3] on the device).  index holds the positions of the
    local ids, then the remote-hot ones, then the remote-cold ones."""
    _check(ids.is_cuda and ids.dtype == torch.int64, "ids is a CUDA int64 tensor")
    _check(mask.dtype == torch.int8, "mask.dtype == int8")
    n = ids.numel()
    masks = [torch.zeros(n, dtype=torch.bool, device=ids.device) for _ in range(3)] if want_masks else None
    index = torch.empty(n, dtype=torch.int64, device=ids.device)
    counts = torch.empty(3, dtype=torch.int64, device=ids.device)
    lib = _lib.load()
    ws = _lib.workspace(lib.hb_partition_workspace_bytes(n, 3))
    mp = [m.data_ptr() for m in masks] if masks else [None, None, None]
    _lib.check(lib.hb_split_compact(ids.contiguous().data_ptr(), n, mask.data_ptr(), mp[0], mp[1], mp[2],
                                    index.data_ptr(), counts.data_ptr(), ws.data_ptr(), ws.numel(),
                                    _lib.stream_ptr()))
    return masks, index, counts


def cudaBucketPack(ids, rows, cnt, num_buckets: int, range_partition=None, local_num_gpus: int | None = None,
                   n_dev: torch.Tensor | None = None):
    """Bucket (ids, rows, cnt) by owner, stable inside a bucket.  Returns
    (ids, rows, cnt, counts[num_buckets] on the device).  owner = id % num_buckets, or the
    cudaBinarySearch rule when range_partition is given."""
    _check(ids.is_cuda and ids.dtype == torch.int64, "ids is a CUDA int64 tensor")
    n = ids.numel()
    g = int(local_num_gpus) if local_num_gpus is not None else int(num_buckets)
    out_ids = torch.empty_like(ids)
    out_rows = torch.empty_like(rows) if rows is not None else None
    out_cnt = torch.empty_like(cnt) if cnt is not None else None
    counts = torch.empty(num_buckets, dtype=torch.int64, device=ids.device)
    lib = _lib.load()
    ws = _lib.workspace(lib.hb_partition_workspace_bytes(n, num_buckets))
    _lib.check(lib.hb_bucket_pack(ids.contiguous().data_ptr(), _lib.ptr(rows), _lib.ptr(cnt), n,
                                  _lib.ptr(n_dev),
                                  _row_bytes(rows) if rows is not None else 0, int(num_buckets),
                                  _lib.ptr(range_partition),
                                  range_partition.numel() if range_partition is not None else 0, g,
                                  out_ids.data_ptr(), _lib.ptr(out_rows), _lib.ptr(out_cnt),
                                  counts.data_ptr(), ws.data_ptr(), ws.numel(), _lib.stream_ptr()))
    return out_ids, out_rows, out_cnt, counts


def cudaTableSplit3(ids, rows, cnt, table, n_dev: torch.Tensor | None = None, keep=(True, True, True),
                    caps=(None, None, None)):
    """(ids, rows, cnt) split by class table[id] in {0, 1, 2} into one buffer set per class
    (each compacted from entry 0, input order kept).  Returns ([ (ids, rows, cnt) | None ] * 3,
    counts[3] on the device); keep[c] = False only counts class c.  caps[c]: an upper bound
    the caller can prove on the size of class c (e.g. unique ids of a class with that many
    members), to allocate less than n entries for it."""
    _check(ids.is_cuda and ids.dtype == torch.int64, "ids is a CUDA int64 tensor")
    _check(table.dtype == torch.int8, "table.dtype == int8")
    n = ids.numel()
    outs = []
    for c in range(3):
        if keep[c]:
            m = n if caps[c] is None else min(n, int(caps[c]))
            outs.append((torch.empty(m, dtype=ids.dtype, device=ids.device),
                         torch.empty((m, rows.size(1)), dtype=rows.dtype, device=ids.device),
                         torch.empty(m, dtype=cnt.dtype, device=ids.device) if cnt is not None else None))
        else:
            outs.append(None)
    counts = torch.empty(3, dtype=torch.int64, device=ids.device)
    arr = C.c_void_p * 3
    p_ids = arr(*[(o[0].data_ptr() if o else None) for o in outs])
    p_rows = arr(*[(o[1].data_ptr() if o else None) for o in outs])
    p_cnt = arr(*[(o[2].data_ptr() if (o and o[2] is not None) else None) for o in outs])
    lib = _lib.load()
    ws = _lib.workspace(lib.hb_partition_workspace_bytes(n, 3))
    _lib.check(lib.hb_table_split3(ids.contiguous().data_ptr(), rows.data_ptr(), _lib.ptr(cnt), n,
                                   _lib.ptr(n_dev), _row_bytes(rows), table.data_ptr(), p_ids, p_rows,
                                   p_cnt, counts.data_ptr(), ws.data_ptr(), ws.numel(),
                                   _lib.stream_ptr()))
    return outs, counts


def cudaGradSplit3(ids, rows, hot_mask, local_mask):
    """(ids, rows) reordered as hot | cold-local | cold-remote; counts[3] on the device."""
    _check(ids.is_cuda and ids.dtype == torch.int64, "ids is a CUDA int64 tensor")
    _check(hot_mask.dtype == torch.bool and local_mask.dtype == torch.bool, "bool masks")
    n = ids.numel()
    out_ids = torch.empty_like(ids)
    out_rows = torch.empty_like(rows)
    counts = torch.empty(3, dtype=torch.int64, device=ids.device)
    lib = _lib.load()
    ws = _lib.workspace(lib.hb_partition_workspace_bytes(n, 3))
    _lib.check(lib.hb_grad_split3(ids.contiguous().data_ptr(), rows.data_ptr(), hot_mask.data_ptr(),
                                  local_mask.data_ptr(), n, _row_bytes(rows), out_ids.data_ptr(),
                                  out_rows.data_ptr(), counts.data_ptr(), ws.data_ptr(), ws.numel(),
                                  _lib.stream_ptr()))
    return out_ids, out_rows, counts


def cudaUniqueSegSumSplit(ids, grads, table, keep=(True, True, True), caps=(None, None, None),
                          id_bits: int = 64, want_runs: bool = False):
    """only_unique_grads fused with the hot/cold selects that follow it: the per-id sums,
    ids and counts of class table[id] go straight into that class's buffers.  Returns
    ([(ids, rows, cnt) | None] * 3, class_counts[3] on the device, num_unique on the device
    [, runs]).  caps[c]: a proven upper bound on the unique ids of class c (allocation)."""
    _check(ids.is_cuda and ids.dtype == torch.int64, "ids is a CUDA int64 tensor")
    _check(grads.dtype == torch.float32 and grads.dim() == 2, "grads is a 2-D fp32 tensor")
    _check(table.dtype == torch.int8, "table.dtype == int8")
    n, dim = ids.numel(), grads.size(1)
    dev = ids.device
    outs = []
    for c in range(3):
        if keep[c]:
            m = n if caps[c] is None else min(n, int(caps[c]))
            outs.append((torch.empty(m, dtype=torch.int64, device=dev),
                         torch.empty((m, dim), dtype=torch.float32, device=dev),
                         torch.empty(m, dtype=torch.int64, device=dev)))
        else:
            outs.append(None)
    class_counts = torch.empty(3, dtype=torch.int64, device=dev)
    num = torch.zeros(1, dtype=torch.int64, device=dev)
    desc = _lib.ClassSplitDesc()
    desc.table = table.data_ptr()
    desc.table_len = table.numel()
    for c in range(3):
        desc.out_ids[c] = outs[c][0].data_ptr() if outs[c] else None
        desc.out_rows[c] = outs[c][1].data_ptr() if outs[c] else None
        desc.out_cnt[c] = outs[c][2].data_ptr() if outs[c] else None
    desc.class_counts = class_counts.data_ptr()
    lib = _lib.load()
    ws = _lib.workspace(lib.hb_unique_segsum_workspace_bytes(n, dim))
    runs = _lib.RunsDesc() if want_runs else None
    _lib.check(lib.hb_unique_segsum_f32(ids.contiguous().data_ptr(), grads.contiguous().data_ptr(), None, n,
                                        None, None, 0, dim, int(id_bits), 0, None, None, None,
                                        num.data_ptr(), C.byref(runs) if want_runs else None,
                                        C.byref(desc), ws.data_ptr(), ws.numel(), _lib.stream_ptr()))
    if want_runs:
        return outs, class_counts, num, runs
    return outs, class_counts, num


class BatchRuns:
    """A batch of ids grouped into runs of equal ids (``hb_runs_t``): the sort of a step, done
    once and used by the forward fetch, the LRU ageing, the miss list and the backward
    aggregation.  Keeps its own workspace (the grouping must outlive other library calls).

    desc: the ``RunsDesc`` for C calls; num_unique: device int64[1]; class_counts: device
    int64[3] and class_ids[c]: the distinct ids of class c, ascending (None when that class is
    not kept or no class table was given)."""

    def __init__(self, ids, desc, ws, num_unique, class_counts, class_ids, uniq_ids):
        self.ids, self.desc, self.ws = ids, desc, ws
        self.num_unique, self.class_counts, self.class_ids, self.uniq_ids = num_unique, class_counts, class_ids, uniq_ids
        self.n = ids.numel()
        self._version = ids._version
        self.slots = None  # slot of every RUN (distinct id), written by cudaLookupFetchRuns
        self.fetch_ws = None

    def matches(self, ids: torch.Tensor) -> bool:
        """True when `ids` is the tensor these runs were built from, unchanged since."""
        return (ids.data_ptr() == self.ids.data_ptr() and ids.numel() == self.n
                and ids._version == self._version)


def cudaRunsBuild(ids, id_bits: int = 64, table=None, keep=(True, True, True), caps=(None, None, None),
                  n_dev: torch.Tensor | None = None, seg_counts: torch.Tensor | None = None, seg_cap: int = 0,
                  ws: torch.Tensor | None = None, want_uniq: bool = False) -> BatchRuns:
    """Sort (id, position) once and number the runs of equal ids (torch.unique of
    python/EmbCache/sparse_optim.py:133).  table: int8 class per node; then the distinct ids of
    every kept class are compacted into ``class_ids[c]`` (caps[c]: a proven bound on their
    number).  ws: a uint8 CUDA tensor to hold the grouping (allocated when None or too small)."""
    _check(ids.is_cuda and ids.dtype == torch.int64, "ids is a CUDA int64 tensor")
    ids = ids.contiguous()
    n, dev = ids.numel(), ids.device
    lib = _lib.load()
    need = lib.hb_runs_workspace_bytes(n)
    if ws is None or ws.numel() < need:
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
    class_ids, class_counts = [None, None, None], None
    arr = None
    if table is not None:
        _check(table.dtype == torch.int8, "table.dtype == int8")
        for c in range(3):
            if keep[c]:
                m = n if caps[c] is None else min(n, int(caps[c]))
                class_ids[c] = torch.empty(max(m, 1), dtype=torch.int64, device=dev)
        class_counts = torch.empty(3, dtype=torch.int64, device=dev)  # written by the call (zeros for n == 0)
        arr = (C.c_void_p * 3)(*[(t.data_ptr() if t is not None else None) for t in class_ids])
    num = torch.empty(1, dtype=torch.int64, device=dev)
    uniq = torch.empty(max(n, 1), dtype=torch.int64, device=dev) if want_uniq else None
    desc = _lib.RunsDesc()
    _lib.check(lib.hb_runs_build(ids.data_ptr(), n, _lib.ptr(n_dev), _lib.ptr(seg_counts), int(seg_cap),
                                 int(id_bits), _lib.ptr(table), table.numel() if table is not None else 0,
                                 arr, _lib.ptr(class_counts), _lib.ptr(uniq), num.data_ptr(), ws.data_ptr(),
                                 ws.numel(), C.byref(desc), _lib.stream_ptr()))
    return BatchRuns(ids, desc, ws, num, class_counts, class_ids, uniq)


def cudaLookupFetchRuns(index: IndexCache, runs: BatchRuns, cache_rows, backing_rows=None, peer_table=None,
                        out_rows=None, mode: int | None = None, want_locs: bool = True,
                        ws: torch.Tensor | None = None, resolve_only: bool = False):
    """``cudaLookupFetch`` over a batch that ``cudaRunsBuild`` sorted: (out_rows, locs, found) at
    the batch positions, every distinct id read once per warp that meets it.  Misses read
    backing_rows on this GPU, or the owners' shards of peer_table (``peer_table.PeerTable``).
    The slot of every RUN (distinct id, in the order of ``runs.uniq_ids``) is left in
    ``runs.slots``; want_locs=False skips the per-position ``locs`` (8-byte writes scattered over
    the batch, about 15 % of the time) and returns None for them.  Rows of other GPUs' shards are
    first copied, once per distinct id, into a staging buffer on this GPU.  resolve_only=True runs
    that first, per-distinct-id launch alone (``runs.slots`` filled, nothing written per position)
    and returns (None, None, None)."""
    n = runs.n
    dev = runs.ids.device
    if resolve_only:
        want_locs = False
    elif out_rows is None:
        out_rows = torch.empty((n, cache_rows.size(1)), dtype=cache_rows.dtype, device=dev)
    if not resolve_only:
        _check(out_rows.size(1) == cache_rows.size(1), "out_rows.size(1) == cache_rows.size(1)")
    if backing_rows is not None:
        _check(backing_rows.size(1) == cache_rows.size(1), "backing_rows.size(1) == cache_rows.size(1)")
    locs = torch.empty(n, dtype=torch.int64, device=dev) if want_locs else None
    found = None if resolve_only else torch.empty(n, dtype=torch.bool, device=dev)
    if runs.slots is None:
        runs.slots = torch.empty(max(n, 1), dtype=torch.int64, device=dev)
    lib = _lib.load()
    sharded = peer_table is not None and peer_table.world > 1
    need = lib.hb_lookup_fetch_runs_workspace_bytes(n, _row_bytes(cache_rows), int(sharded))
    if ws is not None and ws.numel() >= need:
        runs.fetch_ws = ws  # the caller's scratch (hb_lookup_fetch_runs_workspace_bytes)
    elif runs.fetch_ws is None or runs.fetch_ws.numel() < need:
        runs.fetch_ws = torch.empty(need, dtype=torch.uint8, device=dev)
    _lib.check(lib.hb_lookup_fetch_runs(index.handle, C.byref(runs.desc), _dev_ptr(cache_rows, "cache_rows"),
                                        None if backing_rows is None else _dev_ptr(backing_rows, "backing_rows"),
                                        0 if backing_rows is None else backing_rows.size(0),
                                        None if peer_table is None else peer_table.handle,
                                        _row_bytes(cache_rows), None if resolve_only else out_rows.data_ptr(),
                                        _lib.ptr(locs), _lib.ptr(found), runs.slots.data_ptr(),
                                        index.lookup_mode if mode is None else mode, runs.fetch_ws.data_ptr(),
                                        runs.fetch_ws.numel(), _lib.stream_ptr()))
    if resolve_only:
        return None, None, None
    return out_rows, locs, found


def cudaRunsResolveRequests(index: IndexCache, runs: BatchRuns, cache_rows, peer_table, stage_rows: torch.Tensor,
                            requests, mode: int | None = None, ws: torch.Tensor | None = None) -> int:
    """First third of the forward fetch whose remote rows the OWNERS deliver
    (``hb_runs_resolve_requests``): index probe per distinct id, slots into ``runs.slots``, and for
    every run whose row lives on another GPU the request (id, run) stored straight into the owner's
    receive area of ``requests`` (an ``exchange.PeerExchange``); the run is also the row of
    ``stage_rows`` (this GPU's stage, mapped by the peers) that the owner fills.  Returns the
    receive area (parity) filled.  Then: ``requests.fence()``, every rank serves what it was asked
    for (``PeerTable.serve`` on ``requests.received(parity)``), ``requests.fence()``,
    ``cudaRunsExpand``."""
    n = runs.n
    dev = runs.ids.device
    if runs.slots is None:
        runs.slots = torch.empty(max(n, 1), dtype=torch.int64, device=dev)
    lib = _lib.load()
    need = lib.hb_lookup_fetch_runs_workspace_bytes(n, _row_bytes(cache_rows), 0)
    if ws is not None and ws.numel() >= need:
        runs.fetch_ws = ws
    elif runs.fetch_ws is None or runs.fetch_ws.numel() < need:
        runs.fetch_ws = torch.empty(need, dtype=torch.uint8, device=dev)
    parity = C.c_int(0)
    _lib.check(lib.hb_runs_resolve_requests(index.handle, C.byref(runs.desc), _dev_ptr(cache_rows, "cache_rows"),
                                            peer_table.handle, _row_bytes(cache_rows), stage_rows.data_ptr(),
                                            stage_rows.size(0), runs.slots.data_ptr(), requests.handle,
                                            C.byref(parity), index.lookup_mode if mode is None else mode,
                                            runs.fetch_ws.data_ptr(), runs.fetch_ws.numel(), _lib.stream_ptr()))
    requests.next_parity = parity.value ^ 1
    return parity.value


def cudaRunsExpand(runs: BatchRuns, cache_rows, other_rows=None, out_rows=None, want_locs: bool = True,
                   peer_sources: bool = True):
    """The last launch of the forward fetch (``hb_runs_expand``): (out_rows, locs, found) at the
    batch positions from what the per-distinct-id launch left in ``runs`` -- after
    ``cudaRunsResolveRequests`` and the owners' delivery, or after
    ``cudaLookupFetchRuns(resolve_only=True)``, so that work which needs only the slots (LRU ageing,
    insertion of the misses into the index) can run beside it.  other_rows: the backing table or
    the stage the first call was given; peer_sources: it had a table sharded over several GPUs."""
    n = runs.n
    dev = runs.ids.device
    if out_rows is None:
        out_rows = torch.empty((n, cache_rows.size(1)), dtype=cache_rows.dtype, device=dev)
    locs = torch.empty(n, dtype=torch.int64, device=dev) if want_locs else None
    found = torch.empty(n, dtype=torch.bool, device=dev)
    lib = _lib.load()
    _lib.check(lib.hb_runs_expand(C.byref(runs.desc), _dev_ptr(cache_rows, "cache_rows"),
                                  None if other_rows is None else other_rows.data_ptr(), _row_bytes(cache_rows),
                                  int(bool(peer_sources)), out_rows.data_ptr(), _lib.ptr(locs), found.data_ptr(),
                                  runs.slots.data_ptr(), runs.fetch_ws.data_ptr(), runs.fetch_ws.numel(),
                                  _lib.stream_ptr()))
    return out_rows, locs, found


def cudaSegSumRuns(runs: BatchRuns, grads, cnt=None, mean: bool = False, split_keep=None, caps=(None, None, None),
                   ws: torch.Tensor | None = None):
    """The aggregation of ``cudaUniqueSegSum`` over existing runs (the ids of ``grads`` are the ids
    the runs were built from).  split_keep=None: returns (sums [n, dim], counts [n]) in the order
    of ``runs.uniq_ids``.  split_keep=(k0, k1, k2) (runs built with a class table): returns
    [(rows, cnt) | None] * 3, the per-id sums and counts of class c at the positions of
    ``runs.class_ids[c]``."""
    _check(grads.dtype == torch.float32 and grads.dim() == 2 and grads.size(0) == runs.n,
           "grads is fp32 [len(ids), dim]")
    n, dim, dev = runs.n, grads.size(1), grads.device
    lib = _lib.load()
    need = lib.hb_segsum_runs_workspace_bytes(n, dim)
    if ws is None:
        ws = _lib.workspace(need)
    _check(ws.numel() >= need, "workspace holds hb_segsum_runs_workspace_bytes")
    grads = grads.contiguous()
    if split_keep is None:
        sums = torch.empty((max(n, 1), dim), dtype=torch.float32, device=dev)
        counts = torch.empty(max(n, 1), dtype=torch.int64, device=dev)
        _lib.check(lib.hb_segsum_runs_f32(C.byref(runs.desc), grads.data_ptr(), _lib.ptr(cnt), dim, int(mean),
                                          sums.data_ptr(), counts.data_ptr(), None, ws.data_ptr(), ws.numel(),
                                          _lib.stream_ptr()))
        return sums, counts
    outs = []
    desc = _lib.ClassSplitDesc()
    for c in range(3):
        if split_keep[c]:
            m = runs.class_ids[c].numel() if runs.class_ids[c] is not None else (
                n if caps[c] is None else min(n, int(caps[c])))
            outs.append((torch.empty((max(m, 1), dim), dtype=torch.float32, device=dev),
                         torch.empty(max(m, 1), dtype=torch.int64, device=dev)))
            desc.out_rows[c], desc.out_cnt[c] = outs[c][0].data_ptr(), outs[c][1].data_ptr()
        else:
            outs.append(None)
    _lib.check(lib.hb_segsum_runs_f32(C.byref(runs.desc), grads.data_ptr(), _lib.ptr(cnt), dim, int(mean), None,
                                      None, C.byref(desc), ws.data_ptr(), ws.numel(), _lib.stream_ptr()))
    return outs


def cudaRunsMissList(runs: BatchRuns, locs, want_class: int, cap: int, ws: torch.Tensor | None = None,
                     locs_kind: int = 0):
    """The distinct ids of class want_class (< 0: any) whose lookup missed, ascending, at most
    cap: (miss_ids [cap] padded with -1, miss_src [cap] = a batch position of the id,
    miss_count on the device).  locs: the slots by batch position (locs_kind 0), by sorted entry
    (1) or by run (2: ``runs.slots``).  What DistEmbeddingTensor.__call__ ships to the cache server,
    python/EmbCache/dist_emb.py:218-259."""
    dev = locs.device
    lib = _lib.load()
    need = lib.hb_runs_miss_list_workspace_bytes(runs.n)
    if ws is None:
        ws = _lib.workspace(need)
    _check(ws.numel() >= need, "workspace holds hb_runs_miss_list_workspace_bytes")
    miss_ids = torch.empty(cap, dtype=torch.int64, device=dev)
    miss_src = torch.empty(cap, dtype=torch.int64, device=dev)  # defined for the first `count` entries
    count = torch.empty(1, dtype=torch.int64, device=dev)
    _lib.check(lib.hb_runs_miss_list(C.byref(runs.desc), locs.data_ptr(), int(locs_kind), int(want_class), int(cap),
                                     miss_ids.data_ptr(), miss_src.data_ptr(), count.data_ptr(), ws.data_ptr(),
                                     ws.numel(), _lib.stream_ptr()))
    return miss_ids, miss_src, count


def cudaUniqueSegSum(ids, grads, cnt=None, mean: bool = False, id_bits: int = 64, sync: bool = True,
                     n_dev: torch.Tensor | None = None, want_runs: bool = False,
                     seg_counts: torch.Tensor | None = None, seg_cap: int = 0):
    """Sorted unique ids, per-id fp32 sum (or mean) of the rows, per-id counts;
    deterministic.  With sync=True the outputs are sliced to the number of unique ids
    (one device-to-host read, as torch.unique does); with sync=False the full-size
    buffers and the device count are returned."""
    _check(ids.is_cuda and ids.dtype == torch.int64, "ids is a CUDA int64 tensor")
    _check(grads.dtype == torch.float32 and grads.dim() == 2, "grads is a 2-D fp32 tensor")
    _check(grads.size(0) == ids.numel(), "grads.size(0) == ids.numel()")
    n, dim = ids.numel(), grads.size(1)
    dev = ids.device
    uniq = torch.empty(n, dtype=torch.int64, device=dev)
    sums = torch.empty((n, dim), dtype=torch.float32, device=dev)
    counts = torch.empty(n, dtype=torch.int64, device=dev)
    num = torch.zeros(1, dtype=torch.int64, device=dev)
    lib = _lib.load()
    ws = _lib.workspace(lib.hb_unique_segsum_workspace_bytes(n, dim))
    runs = _lib.RunsDesc() if want_runs else None
    _lib.check(lib.hb_unique_segsum_f32(ids.contiguous().data_ptr(), grads.contiguous().data_ptr(),
                                        _lib.ptr(cnt), n, _lib.ptr(n_dev), _lib.ptr(seg_counts),
                                        int(seg_cap), dim, int(id_bits), int(mean),
                                        uniq.data_ptr(), sums.data_ptr(), counts.data_ptr(),
                                        num.data_ptr(), C.byref(runs) if want_runs else None, None,
                                        ws.data_ptr(), ws.numel(), _lib.stream_ptr()))
    if want_runs:
        # the runs point into the shared workspace: use them before the next library call
        return uniq, sums, counts, num, runs
    if not sync:
        return uniq, sums, counts, num
    u = int(num.item())
    return uniq[:u], sums[:u], counts[:u]


def cudaMergeSortedSlabs(ids, rows, cnt, seg_counts, seg_cap: int, mean: bool = True):
    """unique_grads over receive slabs whose segments each hold strictly ascending ids (what the
    peer-memory push delivers): (unique ids, rows, counts, num_unique on the device), full-size
    buffers, no host read.  Same results as ``cudaUniqueSegSum(..., seg_counts=...)`` without
    its sort."""
    _check(ids.is_cuda and ids.dtype == torch.int64, "ids is a CUDA int64 tensor")
    _check(rows.dtype == torch.float32 and rows.dim() == 2 and rows.size(0) == ids.numel(),
           "rows is fp32 [len(ids), dim]")
    _check(seg_cap > 0 and ids.numel() % seg_cap == 0, "ids holds whole segments of seg_cap entries")
    n, dim = ids.numel(), rows.size(1)
    num_seg = n // seg_cap
    dev = ids.device
    uniq = torch.empty(n, dtype=torch.int64, device=dev)
    out = torch.empty((n, dim), dtype=torch.float32, device=dev)
    counts = torch.empty(n, dtype=torch.int64, device=dev)
    num = torch.zeros(1, dtype=torch.int64, device=dev)
    lib = _lib.load()
    ws = _lib.workspace(lib.hb_merge_sorted_slabs_workspace_bytes(num_seg, seg_cap))
    _lib.check(lib.hb_merge_sorted_slabs_f32(ids.contiguous().data_ptr(), rows.contiguous().data_ptr(),
                                             _lib.ptr(cnt), seg_counts.data_ptr(), num_seg, int(seg_cap), dim,
                                             int(mean), uniq.data_ptr(), out.data_ptr(), counts.data_ptr(),
                                             num.data_ptr(), ws.data_ptr(), ws.numel(), _lib.stream_ptr()))
    return uniq, out, counts, num
