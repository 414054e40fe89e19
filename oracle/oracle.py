"""TEST INFRASTRUCTURE -- not part of the product.

CPU checker for the CUDA library: ctypes front ends of ``oracle/_oracle.so`` (the plain-C
restatement, ``hades_oracle.c``) and of ``oracle/_ref/libhades_ref.so`` (the reference's own
CPU index compiled through ``ref_shim.cpp``), plus numpy restatements of the hot-path
arithmetic that the reference does with torch expressions.  Only ``tests/``,
``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline legs may import this module.

Each function cites the reference file:line (paths inside the HADES project) it follows.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
_i64p = C.c_void_p


def _ptr(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _ids(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a), dtype=np.int64)


def _load_oracle() -> C.CDLL:
    so = HERE / "_oracle.so"
    if not so.exists():
        from . import build_oracle  # type: ignore

        build_oracle.build_oracle()
    lib = C.CDLL(str(so))
    lib.oracle_index_create.restype = C.c_void_p
    lib.oracle_index_create.argtypes = [C.c_int64]
    for name in ("lines", "capacity", "space", "valid"):
        f = getattr(lib, f"oracle_index_{name}")
        f.restype = C.c_int64
        f.argtypes = [C.c_void_p]
    lib.oracle_index_destroy.argtypes = [C.c_void_p]
    lib.oracle_index_add.argtypes = [C.c_void_p, _i64p, C.c_int64, _i64p]
    lib.oracle_index_lookup.argtypes = [C.c_void_p, _i64p, C.c_int64, _i64p, C.c_int]
    lib.oracle_index_touch.argtypes = [C.c_void_p, _i64p, C.c_int64]
    lib.oracle_index_reset.argtypes = [C.c_void_p, _i64p, C.c_int64]
    lib.oracle_index_getall.restype = C.c_int64
    lib.oracle_index_getall.argtypes = [C.c_void_p, _i64p, _i64p, C.c_int64]
    lib.oracle_index_export.argtypes = [C.c_void_p, _i64p, C.c_void_p]
    return lib


_LIB: C.CDLL | None = None


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        _LIB = _load_oracle()
    return _LIB


class OracleIndex:
    """C restatement of SACacheIndex (src/cache/cache.h:11-257), single-threaded."""

    def __init__(self, cache_size: int):
        self._h = C.c_void_p(lib().oracle_index_create(int(cache_size)))

    def __del__(self):
        if getattr(self, "_h", None):
            lib().oracle_index_destroy(self._h)
            self._h = None

    def get_size(self) -> int:
        return lib().oracle_index_capacity(self._h)

    get_capacity = get_size

    def get_space(self) -> int:
        return lib().oracle_index_space(self._h)

    def get_valid_entries_num(self) -> int:
        return lib().oracle_index_valid(self._h)

    def lines(self) -> int:
        return lib().oracle_index_lines(self._h)

    def add(self, ids) -> np.ndarray:
        ids = _ids(ids)
        locs = np.empty_like(ids)
        lib().oracle_index_add(self._h, _ptr(ids), ids.size, _ptr(locs))
        return locs

    def lookup(self, ids, touch: bool = True) -> np.ndarray:
        ids = _ids(ids)
        locs = np.empty_like(ids)
        lib().oracle_index_lookup(self._h, _ptr(ids), ids.size, _ptr(locs), int(touch))
        return locs

    def touch(self, locs) -> None:
        locs = _ids(locs)
        lib().oracle_index_touch(self._h, _ptr(locs), locs.size)

    def reset(self, ids) -> None:
        ids = _ids(ids)
        lib().oracle_index_reset(self._h, _ptr(ids), ids.size)

    def getall(self, length: int):
        ids = np.zeros(length, dtype=np.int64)      # torch::zeros, cache.h:244-247
        locs = np.full(length, -1, dtype=np.int64)  # torch::full(-1), cache.h:248-252
        lib().oracle_index_getall(self._h, _ptr(ids), _ptr(locs), length)
        return ids, locs

    def export(self):
        cap = self.get_capacity()
        ids = np.empty(cap, dtype=np.int64)
        lru = np.empty(cap, dtype=np.int32)
        lib().oracle_index_export(self._h, _ptr(ids), _ptr(lru))
        return ids, lru


class RefIndex:
    """The reference's own SACacheIndex<int64,int64>, compiled from its sources
    (oracle/_ref/libhades_ref.so).  ``available()`` is False when that library could not
    be built or did not travel."""

    _lib: C.CDLL | None = None

    @classmethod
    def _load(cls) -> C.CDLL | None:
        if cls._lib is None:
            so = HERE / "_ref" / "libhades_ref.so"
            if not so.exists():
                return None
            import torch  # noqa: F401  (libtorch must be loaded before the shim)

            r = C.CDLL(str(so))
            r.ref_index_create.restype = C.c_void_p
            r.ref_index_create.argtypes = [C.c_int64]
            r.ref_index_destroy.argtypes = [C.c_void_p]
            for name in ("size", "capacity", "space", "valid"):
                f = getattr(r, f"ref_index_{name}")
                f.restype = C.c_int64
                f.argtypes = [C.c_void_p]
            r.ref_index_add.argtypes = [C.c_void_p, _i64p, C.c_int64, _i64p]
            r.ref_index_lookup.argtypes = [C.c_void_p, _i64p, C.c_int64, _i64p]
            r.ref_index_reset.argtypes = [C.c_void_p, _i64p, C.c_int64]
            r.ref_index_getall.argtypes = [C.c_void_p, _i64p, _i64p, C.c_int64]
            r.ref_set_threads.argtypes = [C.c_int]
            r.ref_max_threads.restype = C.c_int
            cls._lib = r
        return cls._lib

    @classmethod
    def available(cls) -> bool:
        return cls._load() is not None

    @classmethod
    def set_threads(cls, n: int) -> None:
        cls._load().ref_set_threads(int(n))

    @classmethod
    def max_threads(cls) -> int:
        return cls._load().ref_max_threads()

    def __init__(self, cache_size: int):
        r = self._load()
        if r is None:
            raise RuntimeError("oracle/_ref/libhades_ref.so is missing; run oracle/build_oracle.py")
        self._h = C.c_void_p(r.ref_index_create(int(cache_size)))

    def __del__(self):
        if getattr(self, "_h", None) and self._lib is not None:
            self._lib.ref_index_destroy(self._h)
            self._h = None

    def get_size(self) -> int:
        return self._lib.ref_index_size(self._h)

    def get_capacity(self) -> int:
        return self._lib.ref_index_capacity(self._h)

    def get_space(self) -> int:
        return self._lib.ref_index_space(self._h)

    def get_valid_entries_num(self) -> int:
        return self._lib.ref_index_valid(self._h)

    def add(self, ids) -> np.ndarray:
        ids = _ids(ids)
        locs = np.empty_like(ids)
        self._lib.ref_index_add(self._h, _ptr(ids), ids.size, _ptr(locs))
        return locs

    def lookup(self, ids) -> np.ndarray:
        ids = _ids(ids)
        locs = np.empty_like(ids)
        self._lib.ref_index_lookup(self._h, _ptr(ids), ids.size, _ptr(locs))
        return locs

    def reset(self, ids) -> None:
        ids = _ids(ids)
        self._lib.ref_index_reset(self._h, _ptr(ids), ids.size)

    def getall(self, length: int):
        ids = np.empty(length, dtype=np.int64)
        locs = np.empty(length, dtype=np.int64)
        self._lib.ref_index_getall(self._h, _ptr(ids), _ptr(locs), length)
        return ids, locs


# ---------------------------------------------------------------------------------------
# Row movers (numpy form of the torch expressions the reference tests compare against)
# ---------------------------------------------------------------------------------------
def rows_gather(src, src_index, dst, dst_index=None):
    """test/test_fetch.py:16 ``dst[dst_index] = src[src_index]`` (CUDAFetch,
    src/cuda/uva_fetch.cu:28-45); dst_index None: CUDAFetch2 (:72-106)."""
    if dst_index is None:
        dst[: len(src_index)] = src[src_index]
    else:
        dst[dst_index] = src[src_index]
    return dst


def rows_scatter(src, dst, dst_index):
    """test/test_combine.py:16 / test_cached_set.py ``dst[index] = src`` (CUDASet,
    src/cuda/uva_set.cu:35-69; CUDACombine, src/cuda/uva_fetch.cu:212-228)."""
    dst[dst_index] = src
    return dst


def rows_gather_cached(backing, cached, index, index_map, dst):
    """test/test_cached_fetch.py:33-36 (CUDAFetchWithCache2, src/cuda/uva_fetch.cu:149-192)."""
    g = index_map[index]
    hit = g != -1
    dst[hit] = cached[g[hit]]
    dst[~hit] = backing[index[~hit]]
    return dst, hit


def rows_scatter_cached(src, backing, cached, index, index_map):
    """test/test_cached_set.py:33-36 (CUDASetWithCache, src/cuda/uva_set.cu:112-154)."""
    g = index_map[index]
    hit = g != -1
    cached[g[hit]] = src[hit]
    backing[index[~hit]] = src[~hit]
    return backing, cached


def rows_accumulate(src, dst, dst_index, cnt=None):
    """python/EmbCache/server.py:564-574 ``buf[local_id] += grad; cnt[local_id] += 1``
    (unique ids)."""
    dst[dst_index] += src
    if cnt is not None:
        cnt[dst_index] += 1
    return dst


def lookup_fetch(index: OracleIndex, ids, cache_rows, backing_rows, out_rows):
    """python/EmbCache/dist_emb.py:184-243: locs = lookup(ids); rows found in the cache come
    from the cache buffer at locs, the others from the backing table at ids."""
    locs = index.lookup(ids, touch=False)
    hit = locs >= 0
    out_rows[hit] = cache_rows[locs[hit]]
    if backing_rows is not None:
        out_rows[~hit] = backing_rows[np.asarray(ids)[~hit]]
    return locs, hit


# ---------------------------------------------------------------------------------------
# split, owner search, owner bucketing
# ---------------------------------------------------------------------------------------
def split_masks(ids, mask_table):
    """_split, src/cuda/split.cu:34-44: 0 local, 1 remote hot, 2 remote cold."""
    v = mask_table[ids]
    return v == 0, v == 1, v == 2


def split_compact(ids, mask_table):
    """split + torch.nonzero of each mask (python/EmbCache/dist_emb.py:174-191)."""
    masks = split_masks(ids, mask_table)
    idx = [np.nonzero(m)[0].astype(np.int64) for m in masks]
    return masks, np.concatenate(idx), np.array([i.size for i in idx], dtype=np.int64)


def owner_mod(ids, g):
    """ReminderKernel, src/cuda/binary_search.cu:35-43."""
    return ids % g


def owner_range(ids, range_partition, g):
    """BinarySearchKernel, src/cuda/binary_search.cu:10-21 (cub::UpperBound)."""
    return (np.searchsorted(range_partition, ids, side="right") - 1) * g + ids % g


def upper_bound(values, sorted_range):
    """BinarySearchKernel2, src/cuda/binary_search.cu:23-33."""
    return np.searchsorted(sorted_range, values, side="right").astype(values.dtype)


def bucket_pack(ids, rows, cnt, num_buckets, range_partition=None, g=None):
    """swap_gradients' local part, python/EmbCache/sparse_optim.py:36-55: owner, sort by
    owner, gather ids/grads/cnt, per-destination counts.  torch.sort there is not stable;
    the restatement (and the CUDA kernel) keep input order inside a bucket, which is one of
    the orders the reference may produce."""
    g = num_buckets if g is None else g
    own = owner_mod(ids, g) if range_partition is None else owner_range(ids, range_partition, g)
    order = np.argsort(own, kind="stable")
    counts = np.bincount(own, minlength=num_buckets).astype(np.int64)
    return (ids[order], None if rows is None else rows[order],
            None if cnt is None else cnt[order], counts)


def grad_split3(ids, rows, hot_mask, local_mask):
    """DistembSparseGradOptimizer.step, python/EmbCache/sparse_optim.py:243-259."""
    sel = [hot_mask, ~hot_mask & local_mask, ~hot_mask & ~local_mask]
    return (np.concatenate([ids[s] for s in sel]), np.concatenate([rows[s] for s in sel]),
            np.array([int(s.sum()) for s in sel], dtype=np.int64))


# ---------------------------------------------------------------------------------------
# hot-node local aggregation
# ---------------------------------------------------------------------------------------
def only_unique_grads(idx, grad):
    """python/EmbCache/sparse_optim.py:132-139: torch.unique(return_inverse, return_counts)
    + index_add_ in fp32, rows added in input order."""
    uniq, inverse, counts = np.unique(idx, return_inverse=True, return_counts=True)
    values = np.zeros((uniq.size, grad.shape[1]), dtype=np.float32)
    np.add.at(values, inverse, grad)
    return uniq, values, counts.astype(np.int64)


def unique_grads(idx, grad, cnt=None):
    """python/EmbCache/sparse_optim.py:142-157.  With cnt the counts start from ONES and
    cnt is added (:145-148), so the divisor is 1 + sum(cnt): the reference's result."""
    if cnt is not None:
        uniq, inverse = np.unique(idx, return_inverse=True)
        counts = np.ones(uniq.size, dtype=cnt.dtype)
        np.add.at(counts, inverse, cnt)
    else:
        uniq, inverse, counts = np.unique(idx, return_inverse=True, return_counts=True)
    values = np.zeros((uniq.size, grad.shape[1]), dtype=np.float32)
    np.add.at(values, inverse, grad)
    values = values / counts[:, None].astype(np.float32)
    return uniq, values.astype(np.float32), counts.astype(np.int64)
