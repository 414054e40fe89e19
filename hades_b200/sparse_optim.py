"""Sparse-gradient aggregation, owner-partitioned exchange and sparse optimisers, mirroring
python/EmbCache/sparse_optim.py of the reference with the arithmetic in libhades_b200.

* ``only_unique_grads`` / ``unique_grads``   sparse_optim.py:132-157
* ``swap_gradients``                         sparse_optim.py:19-129 (owner bucketing + all-to-all)
* ``SparseAdam.update``                      sparse_optim.py:590-685
* ``SparseAdagrad.update``                   no counterpart in the reference (it ships only
  SparseAdam); the usual sparse Adagrad rule.

The embedding table and the optimiser state live in HBM, sharded ``owner = id % world``,
``local row = id // world`` (the reference keeps them in DGL DistTensors on the host and
ships rows over PCIe and RPC).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import _lib
from .EmbCacheLib import _check, cudaBucketPack, cudaMergeSortedSlabs, cudaUniqueSegSum


def only_unique_grads(idx: torch.Tensor, grad: torch.Tensor, id_bits: int = 64):
    """(unique ids sorted, per-id fp32 sums, per-id counts); sparse_optim.py:132-139."""
    return cudaUniqueSegSum(idx, grad, None, mean=False, id_bits=id_bits)


def unique_grads(idx: torch.Tensor, grad: torch.Tensor, cnt: torch.Tensor | None = None, id_bits: int = 64):
    """(unique ids sorted, per-id mean); with cnt the divisor is 1 + sum(cnt), as in the
    reference (sparse_optim.py:142-157, counts start from ones at :145)."""
    ids, vals, _ = cudaUniqueSegSum(idx, grad, cnt, mean=True, id_bits=id_bits)
    return ids, vals


def exchange_packed(ids, rows, cnt, counts, group=None, return_splits: bool = False,
                    counts_host: list | None = None):
    """Deliver owner-bucketed rows to their owners.  ids/rows/cnt hold the buckets back to back
    (bucket b = rows for rank b), counts[b] their sizes (int64, on the same device).  Returns
    (ids, rows, cnt) received by this rank, source ranks in order.  Ragged
    ``all_to_all_single`` calls as the reference's swap_gradients makes them
    (sparse_optim.py:73-118); the split sizes are read on the host, as there (:55,:77).
    Works on CUDA tensors over NCCL and on CPU tensors over gloo.  return_splits: also return
    (rows sent to each rank, rows received from each rank), for an exchange in reverse."""
    out_counts = torch.empty_like(counts)
    dist.all_to_all_single(out_counts, counts, group=group)
    in_splits = counts.tolist() if counts_host is None else list(counts_host)  # sizes the caller already read
    out_splits = out_counts.tolist()
    total, sent = sum(out_splits), sum(in_splits)
    r_ids = torch.empty(total, dtype=ids.dtype, device=ids.device)
    dist.all_to_all_single(r_ids, ids[:sent], out_splits, in_splits, group=group)
    r_rows = None
    if rows is not None:
        r_rows = torch.empty((total, rows.shape[1]), dtype=rows.dtype, device=ids.device)
        dist.all_to_all_single(r_rows, rows[:sent], out_splits, in_splits, group=group)
    r_cnt = None
    if cnt is not None:
        r_cnt = torch.empty(total, dtype=cnt.dtype, device=ids.device)
        dist.all_to_all_single(r_cnt, cnt[:sent], out_splits, in_splits, group=group)
    if return_splits:
        return r_ids, r_rows, r_cnt, (in_splits, out_splits)
    return r_ids, r_rows, r_cnt


def swap_gradients(idics, grads, partition_range, num_parts, num_trainers_per_part, device,
                   grads_cnt=None, group=None):
    """Bucket rows by owner and exchange them: every rank receives the rows it owns.
    owner = id % num_trainers_per_part when partition_range is None, else the range rule of
    cudaBinarySearch.  Returns (ids, grads, cnt or None).  One fused pack kernel replaces
    the reference's owner kernel + torch.sort + three gathers + cudaBinarySearch2
    (sparse_optim.py:36-52); the exchange itself is NCCL all_to_all_single as there."""
    world = int(num_parts * num_trainers_per_part)
    ids_p, rows_p, cnt_p, counts = cudaBucketPack(idics, grads, grads_cnt, world, partition_range,
                                                  num_trainers_per_part)
    if world == 1 or not dist.is_initialized():
        return ids_p, rows_p, cnt_p
    return exchange_packed(ids_p, rows_p, cnt_p, counts, group)


def _merge_duplicates(idx, grad, cnt, n_dev, id_bits, seg_counts, seg_cap, sorted_segments):
    """unique_grads (sparse_optim.py:611) without reading the unique count on the host."""
    if sorted_segments and seg_counts is not None:
        idx, grad, _, n_dev = cudaMergeSortedSlabs(idx, grad, cnt, seg_counts, seg_cap, mean=True)
    else:
        idx, grad, _, n_dev = cudaUniqueSegSum(idx, grad, cnt, mean=True, id_bits=id_bits, sync=False,
                                               n_dev=n_dev, seg_counts=seg_counts, seg_cap=seg_cap)
    return idx, grad, n_dev


class ShardedEmbedding:
    """The rows of a [num_embeddings, dim] table owned by this rank (owner = id % world)."""

    def __init__(self, num_embeddings: int, dim: int, rank: int = 0, world: int = 1,
                 dtype=torch.float32, device=None, init_sigma: float | None = None, seed: int = 0,
                 shared: bool = False, group=None):
        """shared: keep the shard in memory that every GPU of the box can read
        (``peer_table.PeerTable``), so that forward passes on other ranks fetch the authoritative
        rows; a collective call (every rank constructs it)."""
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        self.num_embeddings, self.embedding_dim = int(num_embeddings), int(dim)
        self.rank, self.world = int(rank), int(world)
        self.rows = (self.num_embeddings - self.rank + self.world - 1) // self.world
        self.peer_table = None
        if shared:
            from .peer_table import PeerTable

            self.peer_table = PeerTable(num_embeddings, dim, rank, world, dtype, device, group)
            self.weight = self.peer_table.weight
            self.weight.zero_()
        else:
            self.weight = torch.zeros((self.rows, dim), dtype=dtype, device=device)
        if init_sigma is not None:
            g = torch.Generator(device=device)
            g.manual_seed(seed * 1000 + rank)
            self.weight.normal_(0.0, init_sigma, generator=g)


class _SparseOptimizer:
    def __init__(self, emb: ShardedEmbedding, lr: float):
        self.emb = emb
        self._lr = float(lr)

    def _args(self, idx, grad, cnt):
        _check(idx.is_cuda and idx.dtype == torch.int64, "idx is a CUDA int64 tensor")
        _check(grad.dtype == torch.float32 and grad.size(1) == self.emb.embedding_dim, "grad is fp32 [n, dim]")
        if cnt is not None:
            _check(cnt.dtype == torch.int64, "cnt.dtype == int64")
        return idx.contiguous(), grad.contiguous(), None if cnt is None else cnt.contiguous()


class SparseAdam(_SparseOptimizer):
    """SparseAdam of the reference (sparse_optim.py:531-702) on this rank's shard.

    state_budget_bytes: HBM the optimiser state may take.  When step + mem + power of the whole
    shard fit (or no budget is given) they live in HBM and one kernel updates state and weights
    in place.  Otherwise they live in pinned host memory behind a
    ``cache.LocalSparseAdamStateCache`` whose HBM copy holds the rows of the hottest ids (`hotness`:
    per row of this shard; None = the first rows), as the reference keeps its state
    (sparse_optim.py:556-586, cache.py:133-194): an update then gathers the state rows of its
    ids (cached fetch), runs the same kernel on the gathered rows and scatters them back (cached
    set), sparse_optim.py:621-681.  That path reads the number of ids on the host."""

    def __init__(self, emb: ShardedEmbedding, lr: float, betas=(0.9, 0.999), eps: float = 1e-8,
                 state_budget_bytes: int | None = None, hotness: torch.Tensor | None = None):
        super().__init__(emb, lr)
        self._beta1, self._beta2, self._eps = float(betas[0]), float(betas[1]), float(eps)
        dev = emb.weight.device
        dim = emb.embedding_dim
        self.state_cache = None
        full = emb.rows * (4 + 8 * dim)
        if state_budget_bytes is not None and full > state_budget_bytes:
            from .cache import LocalSparseAdamStateCache

            step = torch.zeros(emb.rows, dtype=torch.float32).pin_memory()
            mem = torch.zeros((emb.rows, dim), dtype=torch.float32).pin_memory()
            power = torch.zeros((emb.rows, dim), dtype=torch.float32).pin_memory()
            if hotness is None:
                hotness = torch.zeros(emb.rows, dtype=torch.float32)
            _check(hotness.numel() == emb.rows, "hotness has one score per row of this shard")
            # the cache is addressed by the LOCAL row (id // world): one partition, one owner
            self.state_cache = LocalSparseAdamStateCache(step, mem, power, hotness, 0, 0, 1)
            self.state_cache_budget = int(state_budget_bytes)
            self.state_cache_bytes = self.state_cache.create_cache(self.state_cache_budget)
            self.state_step, self.state_mem, self.state_power = step, mem, power  # the backing tensors
            return
        self.state_step = torch.zeros(emb.rows, dtype=torch.float32, device=dev)
        self.state_mem = torch.zeros((emb.rows, dim), dtype=torch.float32, device=dev)
        self.state_power = torch.zeros((emb.rows, dim), dtype=torch.float32, device=dev)

    def full_state(self):
        """(step, mem, power) of the whole shard as CUDA tensors, whichever tier the rows are in."""
        if self.state_cache is None:
            return self.state_step, self.state_mem, self.state_power
        rows = torch.arange(self.emb.rows, dtype=torch.int64, device=self.emb.weight.device)
        return self.state_cache[rows]

    def sync_state_to_backing(self) -> None:
        """Tiered state only: write the rows held in the HBM copy back to the pinned backing
        tensors (before saving them)."""
        if self.state_cache is None or not self.state_cache.has_cached:
            return
        cached_rows = torch.nonzero(self.state_cache.idx_map != -1).flatten()
        slots = self.state_cache.idx_map[cached_rows]
        for backing, cached in zip(self.state_cache.local_state, self.state_cache.cached_state):
            backing[cached_rows.cpu()] = cached[slots].cpu()

    def reload_state_cache(self) -> None:
        """Tiered state only: fill the HBM copy from the backing tensors again (after loading them)."""
        if self.state_cache is not None:
            self.state_cache.create_cache(int(self.state_cache_budget))

    def _update_tiered(self, idx, grad, cnt, n_dev) -> None:
        n = idx.numel() if n_dev is None else min(int(n_dev.item()), idx.numel())
        if n == 0:
            return
        idx, grad = idx[:n], grad[:n].contiguous()
        cnt = None if cnt is None else cnt[:n].contiguous()
        e = self.emb
        rows = torch.div(idx - e.rank, e.world, rounding_mode="floor")
        step, mem, power = self.state_cache[rows]                  # cached fetch, cache.py:66-104
        w = e.weight[rows].contiguous()
        ar = torch.arange(n, dtype=torch.int64, device=idx.device)
        lib = _lib.load()
        _lib.check(lib.hb_sparse_adam(ar.data_ptr(), grad.data_ptr(), _lib.ptr(cnt), n, None, e.embedding_dim, 0, 1, n,
                                      step.data_ptr(), mem.data_ptr(), power.data_ptr(), w.data_ptr(),
                                      w.element_size(), self._lr, self._beta1, self._beta2, self._eps,
                                      _lib.stream_ptr()))
        self.state_cache[rows] = (step, mem, power)                # cached set, cache.py:106-131
        e.weight[rows] = w                                         # emb.tensor[state_idx] -= std, :681

    def update(self, idx, grad, cnt=None, is_unique: bool = False, n_dev: torch.Tensor | None = None,
               id_bits: int = 64, seg_counts: torch.Tensor | None = None, seg_cap: int = 0,
               sorted_segments: bool = False) -> None:
        """seg_counts / seg_cap: idx, grad, cnt are the receive slabs of a peer-memory exchange
        (segment s holds seg_counts[s] valid rows); only with is_unique=False.  sorted_segments:
        every segment holds strictly ascending ids (merge instead of sort)."""
        idx, grad, cnt = self._args(idx, grad, cnt)
        if not is_unique:
            idx, grad, n_dev = _merge_duplicates(idx, grad, cnt, n_dev, id_bits, seg_counts, seg_cap, sorted_segments)
            cnt = None
        if self.state_cache is not None:
            return self._update_tiered(idx, grad, cnt, n_dev)
        lib = _lib.load()
        w = self.emb.weight
        _lib.check(lib.hb_sparse_adam(idx.data_ptr(), grad.data_ptr(), _lib.ptr(cnt), idx.numel(),
                                      _lib.ptr(n_dev), self.emb.embedding_dim, self.emb.rank,
                                      self.emb.world, self.emb.rows, self.state_step.data_ptr(),
                                      self.state_mem.data_ptr(), self.state_power.data_ptr(),
                                      w.data_ptr(), w.element_size(), self._lr, self._beta1,
                                      self._beta2, self._eps, _lib.stream_ptr()))


class SparseAdagrad(_SparseOptimizer):
    """Sparse Adagrad: sum += g*g; emb -= lr * g / (sqrt(sum) + eps)."""

    def __init__(self, emb: ShardedEmbedding, lr: float, eps: float = 1e-10):
        super().__init__(emb, lr)
        self._eps = float(eps)
        self.state_sum = torch.zeros((emb.rows, emb.embedding_dim), dtype=torch.float32,
                                     device=emb.weight.device)

    def update(self, idx, grad, cnt=None, is_unique: bool = False, n_dev: torch.Tensor | None = None,
               id_bits: int = 64, seg_counts: torch.Tensor | None = None, seg_cap: int = 0,
               sorted_segments: bool = False) -> None:
        """seg_counts / seg_cap: idx, grad, cnt are the receive slabs of a peer-memory exchange
        (segment s holds seg_counts[s] valid rows); only with is_unique=False.  sorted_segments:
        every segment holds strictly ascending ids (merge instead of sort)."""
        idx, grad, cnt = self._args(idx, grad, cnt)
        if not is_unique:
            idx, grad, n_dev = _merge_duplicates(idx, grad, cnt, n_dev, id_bits, seg_counts, seg_cap, sorted_segments)
            cnt = None
        lib = _lib.load()
        w = self.emb.weight
        _lib.check(lib.hb_sparse_adagrad(idx.data_ptr(), grad.data_ptr(), _lib.ptr(cnt), idx.numel(),
                                         _lib.ptr(n_dev), self.emb.embedding_dim, self.emb.rank,
                                         self.emb.world, self.emb.rows, self.state_sum.data_ptr(),
                                         w.data_ptr(), w.element_size(), self._lr, self._eps,
                                         _lib.stream_ptr()))
