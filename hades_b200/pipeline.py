"""One trainer's embedding hot path on one GPU, end to end:

    forward   lookup + cached fetch (+ the LRU ageing of the reference's CPU lookup)
    backward  local aggregation -> hot/cold split -> cold-cache accumulate ->
              owner-partitioned exchange of the hot rows -> optimiser update on the owner;
              every ``flush_every`` steps the cold cache is flushed through the same exchange
              and refilled

It strings together what ``DistEmb.__call__`` (python/EmbCache/dist_emb.py:167-292),
``DistembSparseGradOptimizer.step`` (python/EmbCache/sparse_optim.py:212-448) and the cache
server loop (python/EmbCache/server.py:259-298) do across three processes in the reference.
Everything is ordered on the current CUDA stream (the cold accumulate forks to a side stream and
joins before the step ends); the only host reads are the exchange sizes when NCCL carries the
exchange (world > 1) and the flushed-row counts on flush steps.  With several GPUs the table
exists once, sharded by owner and readable from every GPU (``peer_table.PeerTable``): cache misses
read the owner's current row.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from . import EmbCacheLib as E
from .cold_cache import ColdCache
from .sparse_optim import ShardedEmbedding, SparseAdam, SparseAdagrad, exchange_packed

HOT, COLD = 1, 2  # classes of the per-node table (remote hot / remote cold, src/cuda/split.cu:39-43)


@dataclass
class StepStats:
    """Device-side counters of one step (read them only when needed: each is a host sync)."""
    num_unique: torch.Tensor | None = None
    split_counts: torch.Tensor | None = None
    sent_counts: torch.Tensor | None = None
    flushed: int = 0
    extra: dict = field(default_factory=dict)


class EmbeddingPath:
    def __init__(self, table: torch.Tensor, class_table: torch.Tensor, cold: ColdCache,
                 optimizer, rank: int = 0, world: int = 1, flush_every: int = 8, id_bits: int = 64,
                 lookup_mode: int = E.LOOKUP_SETASSOC, mover: int = E.MOVER_AUTO,
                 touch_lru: bool = True, group=None, peer_exchange=None):
        """table: backing rows for cache misses, [num_nodes, dim] fp32 on this GPU; None when the
        optimiser's shard is a ``PeerTable`` (misses then read the owners' shards).
        class_table: int8 per node, HOT or COLD.  optimizer: SparseAdam / SparseAdagrad on this
        rank's shard (owner = id % world)."""
        self.table, self.class_table, self.cold, self.opt = table, class_table, cold, optimizer
        self.rank, self.world = rank, world
        self.flush_every, self.id_bits = flush_every, id_bits
        self.lookup_mode, self.mover, self.touch_lru = lookup_mode, mover, touch_lru
        self.group = group
        self.px = peer_exchange  # PeerExchange for the per-step hot rows (None: NCCL all-to-all)
        self.step_no = 0
        self._graphs, self._g_ids, self._g_grads, self._g_out, self._g_next = [], None, None, None, 0
        self._whole_step_graphs = True
        # unique hot ids of a batch cannot outnumber the hot ids of the table
        self.num_hot_ids = int((class_table == HOT).sum().item())
        self.num_nodes, self.dim, self.row_dtype = class_table.numel(), cold.dim, cold.emb.dtype
        self.device = class_table.device
        # owner shards that every GPU can read: cache misses fetch the authoritative row from the
        # owner (table is then None); otherwise misses read `table` on this GPU
        self.shared = getattr(optimizer.emb, "peer_table", None)
        self._token = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._side, self._cold_done, self._cold_refs = None, None, None

    # ---- forward -------------------------------------------------------------------------
    def forward(self, ids: torch.Tensor, out_rows: torch.Tensor | None = None, defer_touch: bool = False):
        """defer_touch: leave the LRU ageing of this lookup to ``backward(..., locs=locs)``,
        which sorts the same ids anyway and can age the counters without a sort of its own."""
        if self.shared is not None:
            rows, locs, found = self.shared.lookup_fetch(self.cold.index, ids, self.cold.emb, out_rows,
                                                         self.lookup_mode)
        else:
            rows, locs, found = E.cudaLookupFetch(self.cold.index, ids, self.cold.emb, self.table,
                                                  out_rows=out_rows, mode=self.lookup_mode, mover=self.mover)
        if self.touch_lru and not defer_touch:
            self.cold.index.cuda_touch_lru(locs)
        return rows, locs, found

    def _fence_shards(self) -> None:
        """All ranks' optimiser updates before anyone's next read of a shard (and the other way
        round at the next exchange): the exchange's device-side fence, else a 4-byte all-reduce."""
        if self.shared is None or self.world == 1:
            return
        if self.px is not None and self.px.fence_kind == "device":
            self.px.fence()
        else:
            import torch.distributed as dist

            dist.all_reduce(self._token, group=self.group)

    # ---- exchange ------------------------------------------------------------------------
    def _exchange(self, ids, rows, cnt, n_dev):
        """Bucket by owner and deliver to the owners.  Returns (ids, rows, cnt, n_dev)."""
        p_ids, p_rows, p_cnt, counts = E.cudaBucketPack(ids, rows, cnt, self.world, n_dev=n_dev)
        if self.world == 1:
            return p_ids, p_rows, p_cnt, counts, counts
        r_ids, r_rows, r_cnt = exchange_packed(p_ids, p_rows, p_cnt, counts, self.group)
        return r_ids, r_rows, r_cnt, None, counts

    # ---- backward ------------------------------------------------------------------------
    def backward(self, ids: torch.Tensor, grads: torch.Tensor, locs: torch.Tensor | None = None) -> StepStats:
        """locs: the slots the forward pass found for `ids`, when its LRU ageing was deferred."""
        st = self._backward_core(ids, grads, locs)
        self._after_step(st)
        return st

    def _after_step(self, st: StepStats) -> None:
        self.step_no += 1
        if self.flush_every > 0 and self.step_no % self.flush_every == 0:
            st.flushed = self.flush()

    def _backward_local(self, ids, grads, locs, join: bool = True):
        """Backward up to the exchange: aggregation, LRU ageing, hot/cold split, cold
        accumulate.  No host read and no collective.  Returns (stats, hot ids, rows, cnt).

        The cold accumulate touches only the staging table and the index, the hot rows' way to
        their owners only the exchange buffers and the optimiser state, so the former runs on a
        side stream; join=False leaves the join to the caller (``_join_cold``)."""
        st = StepStats()
        # hot-node local aggregation (only_unique_grads, sparse_optim.py:132-139) with the hot /
        # cold selects (sparse_optim.py:243-259) fused into its output
        outs, split_counts, num, runs = E.cudaUniqueSegSumSplit(
            ids, grads, self.class_table, keep=(False, True, True), caps=(None, self.num_hot_ids, None),
            id_bits=self.id_bits, want_runs=True)
        if locs is not None and self.touch_lru:
            self.cold.index.cuda_touch_lru_runs(locs, runs)
        st.num_unique = num
        st.split_counts = split_counts
        hot_ids, hot_rows, hot_cnt = outs[HOT]
        cold_ids, cold_rows, _ = outs[COLD]
        # cold rows wait in the staging table
        main = torch.cuda.current_stream()
        if self._side is None:
            self._side = torch.cuda.Stream(device=self.device)
        forked = torch.cuda.Event()
        forked.record(main)
        with torch.cuda.stream(self._side):
            self._side.wait_event(forked)
            self.cold.accumulate_remote(cold_ids, cold_rows, n_dev=split_counts[COLD:COLD + 1],
                                        touch_lru=self.touch_lru)
            self._cold_done = torch.cuda.Event()
            self._cold_done.record(self._side)
        # the side stream reads buffers that belong to this stream's allocator: keep them
        # until the join is enqueued, so that nothing allocated in between can reuse them
        self._cold_refs = (outs, split_counts)
        if join:
            self._join_cold()
        return st, hot_ids, hot_rows, hot_cnt

    def _join_cold(self) -> None:
        if self._cold_done is not None:
            torch.cuda.current_stream().wait_event(self._cold_done)
            self._cold_done, self._cold_refs = None, None

    def _owner_update_from_slabs(self, parity: int) -> None:
        """Owner side after a peer-memory push: merge the senders' slabs and update."""
        r_ids, r_rows, r_cnt, seg_counts = self.px.received(parity)
        # every slab holds the sorted unique hot ids of its sender (stable bucketing): a merge
        self.opt.update(r_ids, r_rows, r_cnt, is_unique=False, id_bits=self.id_bits,
                        seg_counts=seg_counts, seg_cap=self.px.cap, sorted_segments=True)

    def _backward_core(self, ids, grads, locs) -> StepStats:
        """Everything of the backward path that runs every step (no host read unless NCCL
        carries the exchange)."""
        st, hot_ids, hot_rows, hot_cnt = self._backward_local(ids, grads, locs, join=False)
        n_hot = st.split_counts[HOT:HOT + 1]
        # hot rows go to their owners now
        if self.world == 1:
            # One trainer: bucketing by owner is the identity (the reference skips the exchange
            # too, sparse_optim.py:263,320), and the hot ids are already unique and ascending, so
            # unique_grads (sparse_optim.py:142-157) reduces to its division by 1 + cnt.
            st.sent_counts = n_hot
            self.opt.update(hot_ids, hot_rows, hot_cnt + 1, is_unique=True, n_dev=n_hot)
        elif self.px is not None:
            parity = self.px.push(hot_ids, hot_rows, hot_cnt, n_hot)
            self.px.fence()
            self._owner_update_from_slabs(parity)
        else:
            r_ids, r_rows, r_cnt, r_n, sent = self._exchange(hot_ids, hot_rows, hot_cnt, n_hot)
            st.sent_counts = sent
            if r_n is not None:
                r_n = r_n[:1]
            # owner: merge the senders' rows (unique_grads with counts) and update
            self.opt.update(r_ids, r_rows, r_cnt, is_unique=False, n_dev=r_n, id_bits=self.id_bits)
        self._join_cold()
        self._fence_shards()
        return st

    def flush(self) -> int:
        """Stale cold rows leave through the same exchange; their cache entries are evicted by
        the flush (server.py:413) and come back with the current table rows, as the next
        forward pass of the reference would re-insert them (server.py:499-544)."""
        f_ids, f_rows, f_cnt, counts = self.cold.flush_remote(sync=True)
        n = f_ids.numel()
        if n == 0 and self.world == 1:
            return 0
        if self.world == 1:
            # one trainer: every flushed row is its own (is_unique=True, sparse_optim.py:405-421)
            self.opt.update(f_ids, f_rows, f_cnt, is_unique=True)
            if n:
                fresh = torch.empty((n, self.dim), dtype=self.table.dtype, device=f_ids.device)
                E.cudaFetch2(self.table, f_ids, fresh)
                self.cold.insert(f_ids, fresh)
            return n
        import torch.distributed as dist

        # the flush already leaves its rows bucketed by owner (num_clients = world)
        r_ids, r_rows, r_cnt, (sent, received) = exchange_packed(
            f_ids, f_rows, f_cnt, counts, self.group, return_splits=True,
            counts_host=self.cold.remote.last_counts_host)
        self.opt.update(r_ids, r_rows, r_cnt, is_unique=False, id_bits=self.id_bits)
        if self.shared is not None:
            # The exchange in reverse: every owner returns the rows it now holds, in the order
            # the ids arrived, so the refill costs one local gather and one all-to-all instead of
            # row-by-row reads over NVLink.  A rank has all its rows back only after every
            # owner's update, so this is also the fence before the next read of a shard.
            w = self.opt.emb.weight
            back = torch.empty((r_ids.numel(), self.dim), dtype=w.dtype, device=w.device)
            E.cudaFetch2(w, r_ids // self.world, back)
            fresh = torch.empty((sum(sent), self.dim), dtype=w.dtype, device=w.device)
            dist.all_to_all_single(fresh, back, sent, received, group=self.group)
            if n:
                self.cold.insert(f_ids, fresh)
        elif n:
            fresh = torch.empty((n, self.dim), dtype=self.table.dtype, device=f_ids.device)
            E.cudaFetch2(self.table, f_ids, fresh)
            self.cold.insert(f_ids, fresh)
        return n

    def step(self, ids: torch.Tensor, grads: torch.Tensor, out_rows: torch.Tensor | None = None):
        if self._graphs and grads is self._g_grads and out_rows is self._g_out:
            if ids is not self._g_ids:
                self._g_ids.copy_(ids, non_blocking=True)
            if self._whole_step_graphs:
                # one graph per receive area, each holding the whole step (push and device
                # fence included); they alternate like the areas do
                graph, (rows, locs, found, st) = self._graphs[self._g_next]
                self._g_next = (self._g_next + 1) % len(self._graphs)
                graph.replay()
            else:
                # local part from the graph, the push and its fence launched eagerly (the NCCL
                # fence is a collective), owner update from the graph captured for that area
                graph, (rows, locs, found, st, hot_ids, hot_rows, hot_cnt) = self._graphs[0]
                graph.replay()
                parity = self.px.push(hot_ids, hot_rows, hot_cnt, st.split_counts[HOT:HOT + 1])
                self.px.fence()
                self._graphs[1 + parity][0].replay()
                self._fence_shards()
            st.flushed = 0
            self._after_step(st)
            return rows, locs, found, st
        rows, locs, found = self.forward(ids, out_rows, defer_touch=True)
        st = self.backward(ids, grads, locs)
        return rows, locs, found, st

    def capture(self, ids_buf: torch.Tensor, grads: torch.Tensor, out_rows: torch.Tensor) -> None:
        """Capture the per-step work of ``step`` in CUDA graphs over the caller's buffers; later
        ``step(ids, grads, out_rows)`` calls with the same ``grads`` and ``out_rows`` replay them
        (``ids`` is copied into ``ids_buf`` unless it is that tensor).  Call it after a few eager
        steps: every lazy allocation of the library has to have happened.

        One GPU: one graph holds the whole step (the periodic flush stays eager).  Several GPUs
        with the peer-memory exchange and its device-side fence: two graphs, one per receive
        area, each holding the whole step; they are replayed alternately.  With the NCCL fence
        the collective is not captured: one graph for everything before the exchange and one
        per receive area for the owner update, push and fence launched eagerly between them.
        Not available with the NCCL all-to-all, which reads sizes on the host."""
        if self.world > 1 and self.px is None:
            raise RuntimeError("the NCCL all-to-all exchange reads sizes on the host and cannot be captured")
        graphs = []
        self._whole_step_graphs = self.world == 1 or self.px.fence_kind == "device"
        if self._whole_step_graphs:
            for _ in range(1 if self.world == 1 else 2):  # the push picks the areas in turn
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    rows, locs, found = self.forward(ids_buf, out_rows, defer_touch=True)
                    st = self._backward_core(ids_buf, grads, locs)
                graphs.append((g, (rows, locs, found, st)))
        else:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                rows, locs, found = self.forward(ids_buf, out_rows, defer_touch=True)
                st, hot_ids, hot_rows, hot_cnt = self._backward_local(ids_buf, grads, locs)
            graphs.append((g, (rows, locs, found, st, hot_ids, hot_rows, hot_cnt)))
            for parity in (0, 1):
                gp = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gp):
                    self._owner_update_from_slabs(parity)
                graphs.append((gp, None))
        self._graphs, self._g_ids, self._g_grads, self._g_out, self._g_next = graphs, ids_buf, grads, out_rows, 0


    # ---- forward and backward as separate graphs (a model runs between them) -------------------
    def capture_split(self, ids_buf: torch.Tensor, grads_buf: torch.Tensor, out_rows: torch.Tensor) -> None:
        """Capture the forward fetch and the backward path as separate CUDA graphs over the
        caller's buffers, for use with a model between them (``forward_replay`` /
        ``backward_replay``).  Same conditions as ``capture``; several GPUs need the peer-memory
        exchange with the device-side fence (one backward graph per receive area)."""
        if self.world > 1 and (self.px is None or self.px.fence_kind != "device"):
            raise RuntimeError("split capture on several GPUs needs the peer-memory exchange with the device fence")
        fg = torch.cuda.CUDAGraph()
        with torch.cuda.graph(fg):
            rows, locs, found = self.forward(ids_buf, out_rows, defer_touch=True)
        back = []
        for _ in range(1 if self.world == 1 else 2):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                st = self._backward_core(ids_buf, grads_buf, locs)
            back.append((g, st))
        self._split = dict(fwd=fg, back=back, next=0, ids=ids_buf, grads=grads_buf, out=(rows, locs, found))

    def forward_replay(self, ids: torch.Tensor):
        sp = self._split
        if ids is not sp["ids"]:
            sp["ids"].copy_(ids, non_blocking=True)
        sp["fwd"].replay()
        return sp["out"]

    def backward_replay(self, grads: torch.Tensor) -> StepStats:
        """Backward for the ids of the last ``forward_replay``."""
        sp = self._split
        if grads is not sp["grads"]:
            sp["grads"].copy_(grads, non_blocking=True)
        g, st = sp["back"][sp["next"]]
        sp["next"] = (sp["next"] + 1) % len(sp["back"])
        g.replay()
        st.flushed = 0
        self._after_step(st)
        return st

    # ---- save / resume ---------------------------------------------------------------------------
    def state_dict(self) -> dict:
        """Everything a resumed run needs to continue bit for bit: index lines and LRU counters,
        cached rows, staging buffers, optimiser state, table / owner shard, step counter.  (The
        reference keeps all of this in server shared memory and DGL DistTensors and has no
        save path; python/EmbCache/server.py:76-175.)"""
        line_ids, lru = self.cold.index.export_state()
        r = self.cold.remote
        opt = {k: v.clone() for k, v in vars(self.opt).items() if isinstance(v, torch.Tensor)}
        sd = {"step_no": self.step_no, "index_ids": line_ids, "index_lru": lru, "cache_emb": self.cold.emb.clone(),
              "staging": {"grad": r.grad.clone(), "cnt": r.cnt.clone(), "idx": r.idx.clone(),
                          "iter_count": r.iter_count.clone(), "iter_threshold": r.iter_threshold.clone()},
              "dropped": self.cold.dropped.clone(), "optimizer": opt, "weight": self.opt.emb.weight.clone()}
        if self.table is not None and self.opt.emb.weight is not self.table:
            sd["table"] = self.table.clone()
        return sd

    def load_state_dict(self, sd: dict) -> None:
        """In place (buffer addresses are kept, so captured graphs stay valid)."""
        self.step_no = int(sd["step_no"])
        self.cold.index.import_state(sd["index_ids"], sd["index_lru"])
        self.cold.emb.copy_(sd["cache_emb"])
        r = self.cold.remote
        for k, v in sd["staging"].items():
            getattr(r, k).copy_(v)
        self.cold.dropped.copy_(sd["dropped"])
        for k, v in sd["optimizer"].items():
            getattr(self.opt, k).copy_(v)
        self.opt.emb.weight.copy_(sd["weight"])
        if "table" in sd:
            self.table.copy_(sd["table"])


def _warm_collectives(world: int, device, group) -> None:
    """NCCL sets up its send/receive connections on first use (about a second); do it at
    set-up, not inside the first flush."""
    if world > 1:
        import torch.distributed as dist

        t = torch.zeros(world, dtype=torch.int64, device=device)
        dist.all_to_all_single(torch.empty_like(t), t, group=group)
        dist.all_reduce(t, group=group)
        torch.cuda.synchronize()


def _peer_exchange(rank, world, cap, dim, device, group, fence="device"):
    """The peer-memory exchange, or None when it cannot be set up on every rank."""
    import torch.distributed as dist

    from .exchange import PeerExchange

    try:
        px = PeerExchange(rank, world, cap, dim, torch.float32, device, group, fence)
        ok = 1
    except Exception as e:  # noqa: BLE001  (e.g. CUDA IPC not permitted between these processes)
        import warnings

        warnings.warn(f"peer-memory exchange unavailable ({e}); using the NCCL all-to-all")
        px, ok = None, 0
    agree = torch.tensor([ok], dtype=torch.int32, device=device)  # every rank must use the same exchange
    dist.all_reduce(agree, op=dist.ReduceOp.MIN, group=group)
    return px if int(agree.item()) == 1 else None


def assemble_path(name: str, table: torch.Tensor, class_table: torch.Tensor, cache_ids: torch.Tensor,
                  hot_per_owner_max: int, rank: int, world: int, device, optimizer: str, flush_every: int,
                  lookup_mode: int, mover: int, touch_lru: bool, group, exchange: str,
                  cache_entries: int, table_dtype=torch.float32, table_sigma: float = 0.01,
                  generator=None) -> EmbeddingPath:
    """Cold cache filled with `cache_ids` (rows from `table`), optimiser shard, exchange."""
    rows_total, dim = table.shape
    cold = ColdCache(f"{name}_r{rank}", cache_entries, dim, threshold=None, cnt_threshold=16,
                     default_threshold=0, num_clients=world, lookup_mode=lookup_mode, device=device)
    rows = torch.empty((cache_ids.numel(), dim), dtype=torch.float32, device=device)
    E.cudaFetch2(table, cache_ids, rows)
    cold.insert(cache_ids, rows)
    del rows
    share = world > 1 and table_dtype == torch.float32
    shard = ShardedEmbedding(rows_total, dim, rank, world, dtype=table_dtype, device=device, shared=share,
                             group=group)
    if world == 1 and table_dtype == torch.float32:
        shard.weight = table  # one GPU: the backing table is the owner shard
    else:
        # every rank generated the same table; it keeps the rows it owns
        shard.weight.copy_(table[rank::world])
        if share:
            table = None  # cache misses read the owners' shards
            import torch.distributed as dist

            torch.cuda.synchronize()
            dist.barrier(group=group)  # every shard is filled before anyone reads it
    opt = SparseAdam(shard, lr=0.01) if optimizer == "adam" else SparseAdagrad(shard, lr=0.01)
    id_bits = max(int(rows_total).bit_length() + 1, 8)
    _warm_collectives(world, device, group)
    px = None
    if world > 1 and exchange in ("push", "push_nccl_fence"):
        px = _peer_exchange(rank, world, hot_per_owner_max, dim, device, group,
                            "device" if exchange == "push" else "nccl")
    path = EmbeddingPath(table, class_table, cold, opt, rank, world, flush_every, id_bits,
                         lookup_mode, mover, touch_lru, group, px)
    path.cache_fill_ids = cache_ids  # what the cold cache was filled with, in insertion order
    return path


def build_path(cfg, rank: int = 0, world: int = 1, device=None, optimizer: str = "adam",
               hot_fraction: float = 0.01, lookup_mode: int = E.LOOKUP_SETASSOC,
               mover: int = E.MOVER_AUTO, touch_lru: bool = True, table_dtype=torch.float32,
               seed_config: int | None = None, group=None, exchange: str = "push") -> EmbeddingPath:
    """Build the state of one trainer for a cached-fetch configuration (``synth.CacheFetchConfig``):
    backing table, hot cache filled with the most popular ids, class table (the top
    ``hot_fraction`` of the popularity ranking is HOT), cold cache and optimiser shard."""
    import numpy as np

    from . import synth

    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    gen = torch.Generator(device=device)
    gen.manual_seed(1000 * (seed_config or cfg.config))  # the same table on every rank
    table = torch.empty((cfg.table_rows, cfg.dim), dtype=torch.float32, device=device)
    table.normal_(0.0, cfg.table_sigma, generator=gen)
    n_hot = max(int(cfg.table_rows * hot_fraction), 1)
    hot_ranked = synth.rank_to_id(np.arange(n_hot, dtype=np.int64), cfg.table_rows)
    cls = np.full(cfg.table_rows, COLD, dtype=np.int8)
    cls[hot_ranked] = HOT
    class_table = torch.from_numpy(cls).to(device)
    cache_ids = torch.from_numpy(synth.hot_ids(cfg.table_rows, cfg.cache_entries)).to(device)
    # a rank can receive from one source at most the hot ids it owns
    cap = int(np.bincount(hot_ranked % world, minlength=world).max())
    return assemble_path(cfg.name, table, class_table, cache_ids, cap, rank, world, device, optimizer,
                         cfg.flush_every, lookup_mode, mover, touch_lru, group, exchange,
                         cfg.cache_entries, table_dtype, cfg.table_sigma, gen)


def build_rmat_path(cfg, rank: int = 0, world: int = 1, device=None, optimizer: str = "adam",
                    lookup_mode: int = E.LOOKUP_SETASSOC, mover: int = E.MOVER_AUTO,
                    touch_lru: bool = True, group=None, exchange: str = "push") -> EmbeddingPath:
    """State of one trainer for the sampled-GraphSAGE configuration (``synth.RmatConfig``).
    Under R-MAT a vertex is the more popular the fewer one-bits its id has, so the HOT class
    is ``popcount(id) <= cfg.hot_popcount`` and the cold cache starts with the most popular
    cold vertices (popcount hot_popcount+1, +2, ... in id order)."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    n, dim = cfg.num_nodes, cfg.dim
    need = n * dim * 4 * (1 if world > 1 else 0) + (n // world + 1) * dim * 4 * (3 if optimizer == "adam" else 2)
    need += 2 * (cfg.cache_entries + 8) * dim * 4 + n * 2
    total = torch.cuda.get_device_properties(device).total_memory
    if need > 0.9 * total:
        raise RuntimeError(f"configuration {cfg.name} needs about {need / 2**30:.0f} GiB per GPU with "
                           f"{world} rank(s) and optimizer={optimizer}; this GPU has {total / 2**30:.0f} GiB")
    gen = torch.Generator(device=device)
    gen.manual_seed(1000 * cfg.config)  # the same table on every rank
    table = torch.empty((n, dim), dtype=torch.float32, device=device)
    table.normal_(0.0, cfg.table_sigma, generator=gen)
    ids = torch.arange(n, dtype=torch.int32, device=device)
    x = ids - ((ids >> 1) & 0x55555555)                      # popcount of a 32-bit word
    x = (x & 0x33333333) + ((x >> 2) & 0x33333333)
    x = (x + (x >> 4)) & 0x0F0F0F0F
    pc = ((x * 0x01010101) >> 24).to(torch.int8)
    del ids, x
    class_table = torch.where(pc <= cfg.hot_popcount, torch.tensor(HOT, dtype=torch.int8, device=device),
                              torch.tensor(COLD, dtype=torch.int8, device=device))
    picked, have, k = [], 0, cfg.hot_popcount + 1
    while have < cfg.cache_entries and k <= cfg.bits:
        level = torch.nonzero(pc == k).flatten()[: cfg.cache_entries - have]
        picked.append(level)
        have += level.numel()
        k += 1
    cache_ids = torch.cat(picked).to(torch.int64)
    hot = torch.nonzero(pc <= cfg.hot_popcount).flatten()
    cap = int(torch.bincount(hot % world, minlength=world).max().item())
    del pc, hot
    return assemble_path(cfg.name, table, class_table, cache_ids, cap, rank, world, device, optimizer,
                         cfg.flush_every, lookup_mode, mover, touch_lru, group, exchange,
                         cfg.cache_entries, torch.float32, cfg.table_sigma, gen)
