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


# ---------------------------------------------------------------------------------------
# the reference's own CUDA operators (GPU box only)
# ---------------------------------------------------------------------------------------
class RefCuda:
    """The reference's CUDA operators (src/cuda/ops.h:9-41), compiled from its own .cu files into
    oracle/_ref/libhades_ref_cuda.so by oracle/build_oracle.py.  Arguments are torch CUDA tensors;
    the kernels run on the legacy default stream like in the reference, so every call here
    synchronises the device before and after.  ``available()`` is False when the library did not
    build or did not travel, or when there is no CUDA device."""

    _lib = None

    @classmethod
    def _load(cls):
        if cls._lib is None:
            so = HERE / "_ref" / "libhades_ref_cuda.so"
            if not so.exists():
                return None
            import torch

            if not torch.cuda.is_available():
                return None
            cls._lib = C.CDLL(str(so))
            for name in ("fetch", "fetch2", "fetch_with_cache2", "set", "set_with_cache", "combine", "split",
                         "reminder", "binary_search", "binary_search2"):
                getattr(cls._lib, f"ref_cuda_{name}").restype = None
        return cls._lib

    @classmethod
    def available(cls) -> bool:
        try:
            return cls._load() is not None
        except OSError:
            return False

    @staticmethod
    def _p(t):
        return C.c_void_p(t.data_ptr())

    @staticmethod
    def _dim(t):
        return C.c_int64(t.size(1) if t.dim() == 2 else 0)

    @classmethod
    def _call(cls, name, *args):
        import torch

        torch.cuda.synchronize()
        getattr(cls._load(), f"ref_cuda_{name}")(*args)
        torch.cuda.synchronize()

    @classmethod
    def fetch(cls, src, src_index, dst, dst_index):
        cls._call("fetch", cls._p(src), C.c_int64(src.size(0)), cls._p(src_index), cls._p(dst),
                  C.c_int64(dst.size(0)), cls._p(dst_index), C.c_int64(src_index.numel()), cls._dim(src),
                  C.c_int(src.element_size()), C.c_int(src_index.element_size()))

    @classmethod
    def fetch2(cls, src, src_index, dst):
        cls._call("fetch2", cls._p(src), C.c_int64(src.size(0)), cls._p(src_index), cls._p(dst),
                  C.c_int64(src_index.numel()), cls._dim(src), C.c_int(src.element_size()),
                  C.c_int(src_index.element_size()))

    @classmethod
    def fetch_with_cache2(cls, backing, cached, src_index, index_map, dst):
        cls._call("fetch_with_cache2", cls._p(backing), C.c_int64(backing.size(0)), cls._p(cached),
                  C.c_int64(cached.size(0)), cls._p(src_index), cls._p(index_map), cls._p(dst),
                  C.c_int64(src_index.numel()), cls._dim(backing), C.c_int(backing.element_size()),
                  C.c_int(src_index.element_size()))

    @classmethod
    def set(cls, src, dst, dst_index):
        cls._call("set", cls._p(src), cls._p(dst), C.c_int64(dst.size(0)), cls._p(dst_index),
                  C.c_int64(dst_index.numel()), cls._dim(src), C.c_int(src.element_size()),
                  C.c_int(dst_index.element_size()))

    @classmethod
    def set_with_cache(cls, src, backing, cached, dst_index, index_map):
        cls._call("set_with_cache", cls._p(src), cls._p(backing), C.c_int64(backing.size(0)), cls._p(cached),
                  C.c_int64(cached.size(0)), cls._p(dst_index), cls._p(index_map), C.c_int64(dst_index.numel()),
                  cls._dim(src), C.c_int(src.element_size()), C.c_int(dst_index.element_size()))

    @classmethod
    def combine(cls, src, dst, dst_index):
        cls._call("combine", cls._p(src), cls._p(dst), C.c_int64(dst.size(0)), cls._p(dst_index),
                  C.c_int64(dst_index.numel()), cls._dim(src), C.c_int(src.element_size()),
                  C.c_int(dst_index.element_size()))

    @classmethod
    def split(cls, ids, mask):
        import torch

        outs = [torch.zeros(ids.numel(), dtype=torch.bool, device=ids.device) for _ in range(3)]
        cls._call("split", cls._p(ids), C.c_int64(ids.numel()), cls._p(mask), C.c_int64(mask.numel()),
                  cls._p(outs[0]), cls._p(outs[1]), cls._p(outs[2]))
        return outs

    @classmethod
    def reminder(cls, ids, g):
        import torch

        out = torch.empty_like(ids)
        cls._call("reminder", cls._p(ids), C.c_int64(ids.numel()), C.c_int64(g), cls._p(out),
                  C.c_int(ids.element_size()))
        return out

    @classmethod
    def binary_search(cls, ids, range_partition, g):
        import torch

        out = torch.empty_like(ids)
        cls._call("binary_search", cls._p(ids), C.c_int64(ids.numel()), cls._p(range_partition),
                  C.c_int64(range_partition.numel()), C.c_int64(g), cls._p(out), C.c_int(ids.element_size()))
        return out

    @classmethod
    def binary_search2(cls, values, sorted_range):
        import torch

        out = torch.empty_like(values)
        cls._call("binary_search2", cls._p(values), C.c_int64(values.numel()), cls._p(sorted_range),
                  C.c_int64(sorted_range.numel()), cls._p(out), C.c_int(values.element_size()))
        return out


# ---------------------------------------------------------------------------------------
# cold-gradient staging table: python/EmbCache/server.py
# ---------------------------------------------------------------------------------------
def flush_thresholds(hotness):
    """server.py:87-88: (1 / (0.001 + hotness)).ceil().int().clamp(max=100)."""
    return np.minimum(np.ceil(1.0 / (np.float32(0.001) + hotness.astype(np.float32))), 100).astype(np.int32)


class OracleStaging:
    """The server's gradient buffers (server.py:76-175) and the loop steps that touch them.
    compat_no_clear=True reproduces the reference's behaviour of never zeroing the gradient
    rows after a flush (server.py:414,489,537 zero a temporary copy); the default is the
    intended read-and-zero, which is what the CUDA library implements."""

    def __init__(self, slots, dim, cnt_threshold=16, iter_threshold=None, compat_no_clear=False):
        self.grad = np.zeros((slots, dim), np.float32)
        self.cnt = np.zeros(slots, np.int32)
        self.idx = np.full(slots, -1, np.int64)
        self.iter_count = np.zeros(slots, np.int32)
        self.iter_threshold = (np.zeros(slots, np.int32) if iter_threshold is None
                               else np.asarray(iter_threshold, np.int32).copy())
        self.cnt_threshold = cnt_threshold
        self.compat_no_clear = compat_no_clear

    def accumulate_cached(self, index: OracleIndex, ids, grads, threshold_table, default_threshold):
        """_accumulate_gradients_cold_remote, server.py:546-562 (ids unique)."""
        locs = index.lookup(ids, touch=True)   # the server's lookup is the CPU one (server.py:550)
        hit = np.nonzero(locs >= 0)[0]
        if hit.size:
            s = locs[hit]
            self.idx[s] = ids[hit]
            self.iter_threshold[s] = (threshold_table[ids[hit]] if threshold_table is not None
                                      else default_threshold)
            self.grad[s] += grads[hit]
            self.cnt[s] += 1
        return int((locs < 0).sum())

    def accumulate_direct(self, ids, grads, id_offset=0, id_stride=1):
        """_accumulate_gradients_cold_local, server.py:564-574 (ids unique)."""
        if len(ids):
            s = (ids - id_offset) // id_stride
            self.grad[s] += grads
            self.cnt[s] += 1
            self.idx[s] = ids

    def flush(self, index: OracleIndex | None, num_clients, out_cap=0):
        """_send_staled_gradients, server.py:346-425: returns (ids, rows, cnt, counts) with
        rows bucketed by id % num_clients, slot order inside a bucket.  out_cap > 0 (one client
        only; no counterpart in the reference): at most that many rows leave, in slot order; the
        other stale slots stay staged and age like live ones."""
        live = np.nonzero(self.cnt > 0)[0]
        stale_mask = (self.iter_count[live] >= self.iter_threshold[live]) | (self.cnt[live] >= self.cnt_threshold)
        stale = live[stale_mask]
        if out_cap and stale.size > out_cap:
            assert num_clients == 1
            stale = stale[:out_cap]
        ids = self.idx[stale]
        rows = self.grad[stale].copy()
        cnts = self.cnt[stale].astype(np.int64)
        split = ids % num_clients
        order = np.concatenate([np.nonzero(split == r)[0] for r in range(num_clients)]) if stale.size else np.empty(0, np.int64)
        counts = np.bincount(split, minlength=num_clients).astype(np.int64) if stale.size else np.zeros(num_clients, np.int64)
        if index is not None:
            index.reset(ids)                      # server.py:413
        if not self.compat_no_clear:
            self.grad[stale] = 0                  # intended meaning of server.py:414
        self.cnt[stale] = 0                       # server.py:415
        self.iter_count[live] += 1                # server.py:418
        self.iter_count[stale] = 0                # server.py:419
        order = order.astype(np.int64)
        return ids[order], rows[order], cnts[order], counts

    def insert(self, index: OracleIndex, ids, embs, cache_rows):
        """_update_cache, server.py:499-544."""
        locs = index.add(ids)
        ok = np.nonzero(locs >= 0)[0]
        s = locs[ok]
        cache_rows[s] = embs[ok]
        if not self.compat_no_clear:
            self.grad[s] = 0                      # intended meaning of server.py:537
        self.cnt[s] = 0
        self.idx[s] = -1
        return locs


# ---------------------------------------------------------------------------------------
# sparse optimisers
# ---------------------------------------------------------------------------------------
def sparse_adam_update(idx, grad, step, mem, power, emb, lr, beta1=0.9, beta2=0.999, eps=1e-8,
                       cnt=None, id_offset=0, id_stride=1):
    """SparseAdam.update with is_unique=True, python/EmbCache/sparse_optim.py:606-681, in
    float32 like the torch expressions there.  Updates step/mem/power/emb in place."""
    f = np.float32
    g = grad.astype(f)
    if cnt is not None:
        g = g / cnt.astype(f)[:, None]                                   # :609
    rows = (idx - id_offset) // id_stride
    t = step[rows] + f(1)                                                # :624
    m = f(beta1) * mem[rows] + f(1.0 - beta1) * g                        # :631
    v = f(beta2) * power[rows] + f(1.0 - beta2) * (g * g)                # :632
    mc = m / (f(1) - np.power(f(beta1), t, dtype=f))[:, None]            # :642-643
    vc = v / (f(1) - np.power(f(beta2), t, dtype=f))[:, None]            # :644-645
    std = f(lr) * mc / (np.sqrt(vc) + f(eps))                            # :646-647
    step[rows] = t
    mem[rows] = m
    power[rows] = v
    emb[rows] = (emb[rows].astype(f) - std).astype(emb.dtype)            # :681
    return std


def sparse_adagrad_update(idx, grad, state_sum, emb, lr, eps=1e-10, cnt=None, id_offset=0, id_stride=1):
    """Sparse Adagrad (no reference counterpart: parity unpinned by the reference)."""
    f = np.float32
    g = grad.astype(f)
    if cnt is not None:
        g = g / cnt.astype(f)[:, None]
    rows = (idx - id_offset) // id_stride
    s = state_sum[rows] + g * g
    state_sum[rows] = s
    emb[rows] = (emb[rows].astype(f) - f(lr) * g / (np.sqrt(s) + f(eps))).astype(emb.dtype)
