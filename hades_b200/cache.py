"""Mirror of python/EmbCache/cache.py of the reference on top of ``hades_b200.EmbCacheLib``.

* ``LocalCache``                      cache.py:6-31    thin wrapper over ``IndexCache``
* ``LocalSparseAdamStateCache``       cache.py:34-199  optimiser state behind a hotness-ranked GPU
  cache with a dense index map: cached fetch (``__getitem__``), cached set (``__setitem__``),
  ``create_cache`` (top-``cached_num`` ids by hotness among ``id % world == rank``).

The backing state tensors may live in pinned host memory (the reference's layout, reached
through UVA) or in HBM; the cached copies and the index map are always in HBM.
"""
from __future__ import annotations

import torch

from . import EmbCacheLib


class LocalCache:
    def __init__(self, name: str, cache_size: int, create: bool, pin_memory: bool = False):
        self._cache_size = cache_size
        self._idx_cache = EmbCacheLib.IndexCache(cache_size, name, create, pin_memory)

    def lookup(self, ids):
        return self._idx_cache.lookup(ids)

    def cudalookup(self, ids):
        return self._idx_cache.cudalookup(ids)

    def add(self, ids):
        return self._idx_cache.add(ids)

    def get_num_entries(self):
        return self._idx_cache.get_size()

    def reset(self, ids):
        self._idx_cache.reset(ids)


class LocalSparseAdamStateCache:
    """state = (step [n], mem [n, d], power [n, d]) of one partition, fp32.  ``hotness`` is a
    per-node score; ``partition_start`` the first global id of the partition."""

    def __init__(self, state_step, state_mem, state_power, hotness, partition_start: int = 0,
                 rank: int = 0, world_size: int = 1, count_hit: bool = False, idx_dtype=torch.int64):
        self.local_state = (state_step, state_mem, state_power)
        self._pinned = []
        for t in self.local_state:
            if not t.is_cuda and not t.is_pinned():
                EmbCacheLib.cudaPin(t)  # cache.py:44-45
                self._pinned.append(t)
        self._partition_start = int(partition_start)
        self._hotness = hotness
        self._local_num = state_step.numel()
        self._rank, self._world_size, self._idx_dtype = rank, world_size, idx_dtype
        self.cached_state = None
        self.idx_map = None
        self.has_cached = False
        self._hit_num = 0
        self._lookup_num = 0
        self._count_hit = count_hit

    def __del__(self):
        for t in getattr(self, "_pinned", []):
            try:
                EmbCacheLib.cudaUnpin(t)
            except Exception:
                pass

    def __getitem__(self, index):
        """index: CUDA tensor of global ids -> CUDA tensors (step, mem, power); cache.py:66-104."""
        n = index.numel()
        dim = self.local_state[1].shape[1]
        step = torch.empty((n,), device="cuda", dtype=torch.float32)
        mem = torch.empty((n, dim), device="cuda", dtype=torch.float32)
        power = torch.empty((n, dim), device="cuda", dtype=torch.float32)
        local_index = index - self._partition_start
        outs = (step, mem, power)
        if self.has_cached:
            for backing, cached, out in zip(self.local_state, self.cached_state, outs):
                EmbCacheLib.cudaFetchWithCache2(backing, cached, local_index, self.idx_map, out)
            if self._count_hit:
                self._hit_num += int((self.idx_map[local_index] != -1).sum().item())
                self._lookup_num += n
        else:
            for backing, out in zip(self.local_state, outs):
                EmbCacheLib.cudaFetch2(backing, local_index, out)
        return outs

    def __setitem__(self, index, value):
        """value: CUDA tensors (step, mem, power); cache.py:106-131."""
        local_index = index - self._partition_start
        if self.has_cached:
            for v, backing, cached in zip(value, self.local_state, self.cached_state):
                EmbCacheLib.cudaSetWithCache(v, backing, cached, local_index, self.idx_map)
            if self._count_hit:
                self._hit_num += int((self.idx_map[local_index] != -1).sum().item())
                self._lookup_num += local_index.numel()
        else:
            for v, backing in zip(value, self.local_state):
                EmbCacheLib.cudaSet(v, backing, local_index)

    def create_cache(self, alloca_mem_size: int) -> int:
        """Choose the hottest ids this rank owns and copy their state to HBM; cache.py:133-194.
        Returns the bytes used."""
        elem = torch.empty(0, dtype=self._idx_dtype).element_size()
        idx_map_size = elem * self._local_num
        alloca_mem_size -= idx_map_size
        dev = torch.device("cuda", torch.cuda.current_device())
        local_ids = torch.arange(self._local_num, dtype=self._idx_dtype, device=dev) + self._partition_start
        part_local_ids = local_ids[local_ids % self._world_size == self._rank]
        dim = self.local_state[1].shape[1]
        item_size = 4 + 4 * dim + 4 * dim
        cached_num = int(min(max(alloca_mem_size, 0) // item_size, part_local_ids.numel()))
        if cached_num > 0:
            hot = self._hotness.to(dev)[part_local_ids]
            order = torch.argsort(hot, descending=True, stable=True)
            cached_index = part_local_ids[order][:cached_num] - self._partition_start
            idx_map = torch.full((self._local_num,), -1, dtype=self._idx_dtype, device=dev)
            idx_map[cached_index] = torch.arange(cached_num, dtype=self._idx_dtype, device=dev)
            self.idx_map = idx_map
            cached = []
            for v in self.local_state:
                shape = (cached_num,) if v.dim() == 1 else (cached_num, v.shape[1])
                out = torch.empty(shape, dtype=v.dtype, device=dev)
                EmbCacheLib.cudaFetch2(v, cached_index, out)
                cached.append(out)
            self.cached_state = tuple(cached)
            self.has_cached = True
            mem_used = cached_num * item_size + idx_map_size
        else:
            self.has_cached = False
            mem_used = 0
        self._hit_num = 0
        self._lookup_num = 0
        return mem_used

    def get_hit_rate(self) -> float:
        return 0 if self._lookup_num == 0 else self._hit_num / self._lookup_num
