"""One trainer's embedding hot path on one GPU, end to end:

    forward   sort the batch once -> cache lookup + cached fetch over the runs of equal ids
              (each distinct id looked up and read once per warp) -> LRU ageing of the lookup
              -> the cold ids that missed go into the cache with the rows just fetched
    backward  local aggregation over the same runs -> hot rows to their owners (exchange,
              merge, optimiser update) while the cold rows are staged in the cold cache;
              every ``flush_every`` steps the stale staged rows leave for their owners too

It strings together what ``DistEmb.__call__`` (python/EmbCache/dist_emb.py:167-292),
``DistembSparseGradOptimizer.step`` (python/EmbCache/sparse_optim.py:212-448) and the cache
server loop (python/EmbCache/server.py:259-298) do across three processes in the reference.

Which rows the cache may serve: only ids of the COLD class are ever cached (the cache is
filled with cold ids and only cold misses are inserted), exactly the ids whose updates the
reference defers (dist_emb.py:179-212).  HOT ids always miss and are read from the authoritative
table -- this GPU's table with one trainer, the owner's shard (``peer_table.PeerTable``) with
several -- so a hot row updated in step t is what step t+1 fetches.  A cached cold row keeps
the value it was inserted with until a flush evicts it (server.py:413) and a later miss brings
the updated row back (server.py:499-544), as in the reference.

Everything is ordered on the current CUDA stream (cache insert and cold accumulate run on a
side stream and join before the step ends); no step reads a size on the host unless NCCL
carries the exchange.
"""
from __future__ import annotations

import contextlib
from dataclasses import dataclass, field

import torch

from . import EmbCacheLib as E
from .cold_cache import ColdCache, flush_thresholds
from .sparse_optim import ShardedEmbedding, SparseAdam, SparseAdagrad, exchange_packed

HOT, COLD = 1, 2  # classes of the per-node table (remote hot / remote cold, src/cuda/split.cu:39-43)


@dataclass
class StepStats:
    """Device-side counters of one step (read them only when needed: each is a host sync)."""
    num_unique: torch.Tensor | None = None
    split_counts: torch.Tensor | None = None
    sent_counts: torch.Tensor | None = None
    flushed_dev: torch.Tensor | None = None   # stale rows the flush of this step found
    flush_cap: int = 0
    extra: dict = field(default_factory=dict)

    @property
    def flushed(self) -> int:
        """Rows the flush of this step sent (0 on other steps); one host read."""
        if self.flushed_dev is None:
            return 0
        n = int(self.flushed_dev.sum().item())
        return min(n, self.flush_cap) if self.flush_cap else n


class EmbeddingPath:
    def __init__(self, table: torch.Tensor, class_table: torch.Tensor, cold: ColdCache,
                 optimizer, rank: int = 0, world: int = 1, flush_every: int = 8, id_bits: int = 64,
                 lookup_mode: int = E.LOOKUP_SETASSOC, mover: int = E.MOVER_AUTO,
                 touch_lru: bool = True, group=None, peer_exchange=None, flush_exchange=None,
                 insert_misses: bool = True, miss_cap: int = 1 << 17, flush_cap: int = 1 << 19,
                 want_locs: bool = True, overlap_fetch: bool = False, request_exchange=None,
                 fetch_stages=None):
        """table: backing rows for cache misses, [num_nodes, dim] fp32 on this GPU; None when the
        optimiser's shard is a ``PeerTable`` (misses then read the owners' shards).
        class_table: int8 per node, HOT or COLD.  optimizer: SparseAdam / SparseAdagrad on this
        rank's shard (owner = id % world).  peer_exchange / flush_exchange: ``PeerExchange`` for
        the per-step hot rows and for the flushed rows (None: NCCL all-to-all, sizes read on the
        host).  insert_misses: cold ids that miss the cache are inserted in the forward pass (at
        most miss_cap distinct ids per step; the rest stay uncached until they miss again).
        flush_cap: rows one flush can send (the other stale rows wait for the next flush).
        want_locs: ``forward`` also returns the slots by batch position (False: None; the path
        itself uses the slot of every run).  overlap_fetch: ``step`` runs the fetch of a batch beside
        the aggregation of the same batch's gradients (both need only the sort)."""
        self.overlap_fetch = bool(overlap_fetch)
        # several GPUs, owners deliver the remote rows of the forward fetch: the exchange that
        # carries the requests and the stages (one per rank, mapped by all) the owners store into
        self.px_req, self.fetch_stages = request_exchange, fetch_stages
        self.table, self.class_table, self.cold, self.opt = table, class_table, cold, optimizer
        self.rank, self.world = rank, world
        self.flush_every, self.id_bits = flush_every, id_bits
        self.lookup_mode, self.mover, self.touch_lru = lookup_mode, mover, touch_lru
        self.group = group
        self.px = peer_exchange
        self.px_flush = flush_exchange
        self.insert_misses = insert_misses
        self.want_locs = want_locs
        self.miss_cap = int(miss_cap)
        self.flush_cap = int(min(flush_cap, cold.remote.slots))
        self.step_no = 0
        self._graphs, self._g_ids, self._g_grads, self._g_out, self._g_next = [], None, None, None, 0
        self._whole_step_graphs = True
        self._flush_graphs, self._flush_next = [], 0
        # unique hot ids of a batch cannot outnumber the hot ids of the table
        self.num_hot_ids = int((class_table == HOT).sum().item())
        self.num_nodes, self.dim, self.row_dtype = class_table.numel(), cold.dim, cold.emb.dtype
        self.device = class_table.device
        # owner shards that every GPU can read: cache misses fetch the authoritative row from the
        # owner (table is then None); otherwise misses read `table` on this GPU
        self.shared = getattr(optimizer.emb, "peer_table", None)
        self._token = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._side = None
        self._maint = None
        self._req_parity = 0
        self._evt_resolved = self._evt_expanded = None  # where a fetch beside the backward pass stands
        self._side_done, self._side_refs = None, []
        self._runs_ws, self._side_ws, self._fetch_ws = None, None, None
        self._last = None  # (BatchRuns, locs) of the last forward pass

    # ---- streams ---------------------------------------------------------------------------
    def _on_side(self):
        """Context: the side stream, ordered after everything the current stream holds so far."""
        if self._side is None:
            self._side = torch.cuda.Stream(device=self.device)
        forked = torch.cuda.Event()
        forked.record(torch.cuda.current_stream())
        self._side.wait_event(forked)
        return torch.cuda.stream(self._side)

    def _side_finished(self, *refs) -> None:
        """Called inside ``_on_side``: note where the side stream stands and keep what it reads
        (buffers of the main stream's allocator) until the join."""
        self._side_done = torch.cuda.Event()
        self._side_done.record(self._side)
        self._side_refs.append(refs)

    def _join_side(self) -> None:
        if self._side_done is not None:
            torch.cuda.current_stream().wait_event(self._side_done)
            self._side_done, self._side_refs = None, []

    def _ws(self, which: str, nbytes: int) -> torch.Tensor:
        """Scratch that belongs to this path (the library-wide scratch is used by whatever runs
        on the main stream meanwhile)."""
        cur = getattr(self, which)
        if cur is None or cur.numel() < nbytes:
            cur = torch.empty(int(nbytes), dtype=torch.uint8, device=self.device)
            setattr(self, which, cur)
        return cur

    # ---- forward -------------------------------------------------------------------------
    def forward(self, ids: torch.Tensor, out_rows: torch.Tensor | None = None, join: bool = True,
                on_side: bool = False):
        """(rows, locs, found) at the batch positions.  join=False leaves the cache insert
        running on the side stream (``backward`` joins it).  on_side=True (``step`` with
        overlap_fetch): everything after the sort runs on the side stream and the rows are
        complete only after the join at the end of the backward pass."""
        lib = E._lib.load()
        n = ids.numel()
        runs = E.cudaRunsBuild(ids, self.id_bits, self.class_table, keep=(False, True, True),
                               caps=(None, self.num_hot_ids, None),
                               ws=self._ws("_runs_ws", lib.hb_runs_workspace_bytes(n)))
        self._runs_ws = runs.ws
        sharded = self.shared is not None and self.world > 1
        fetch_ws = self._ws("_fetch_ws", lib.hb_lookup_fetch_runs_workspace_bytes(
            n, self.dim * self.cold.emb.element_size(), int(sharded)))
        if n == 0:
            rows, locs, found = E.cudaLookupFetchRuns(self.cold.index, runs, self.cold.emb, self.table, self.shared,
                                                      out_rows, self.lookup_mode, want_locs=self.want_locs,
                                                      ws=fetch_ws)
            self._last = (runs, locs)
            return rows, locs, found
        # on_side: the whole fetch leaves the main stream, which goes on to the aggregation of the
        # same batch (it needs the sort only); the main stream joins before it returns the rows.
        with (self._on_side() if on_side else contextlib.nullcontext()):
            fetch_stream = torch.cuda.current_stream()
            other_rows = self._resolve(runs, fetch_ws)
            if on_side:
                # this GPU's reads of other GPUs' shards (pull) are done: the backward pass waits for
                # this before it tells the owners, through the exchange's fence, that they may update
                self._evt_resolved = torch.cuda.Event()
                self._evt_resolved.record(fetch_stream)
            maintain = self.touch_lru or self.insert_misses
            pending = None
            if maintain:
                # What the index needs from this lookup -- the LRU ageing (cache.h:101), the list of
                # uncached cold ids and their add() (dist_emb.py:218-259 -> server.py:499-544) --
                # needs the slots only: it runs beside the expansion, on a stream of its own.
                resolved = torch.cuda.Event()
                resolved.record(fetch_stream)
                if self._maint is None:
                    self._maint = torch.cuda.Stream(device=self.device)
                self._maint.wait_event(resolved)
                with torch.cuda.stream(self._maint):
                    pending = self._index_maintenance(runs, n, lib)
            rows, locs, found = self._expand(runs, out_rows, other_rows)
            if on_side:
                # every read of this GPU's own shard by this fetch (rows of ids it owns, rows served to
                # the peers) is done: the owner update of the same step waits for this
                self._evt_expanded = torch.cuda.Event()
                self._evt_expanded.record(fetch_stream)
            if maintain:
                expanded = torch.cuda.Event()
                expanded.record(fetch_stream)
                with torch.cuda.stream(self._maint):
                    self._maint.wait_event(expanded)
                    if pending is not None:
                        # the rows of the inserted ids are taken from the output that has just fetched them
                        self.cold.insert_rows(rows, pending[1], pending[2], pending[3])
                    maintained = torch.cuda.Event()
                    maintained.record(self._maint)
                # the side stream carries on from here (the cold accumulate looks the cache up)
                if self._side is None:
                    self._side = torch.cuda.Stream(device=self.device)
                self._side.wait_event(maintained)
                if not on_side:
                    self._side.wait_event(expanded)
                self._side_done = torch.cuda.Event()
                self._side_done.record(self._side)
                self._side_refs.append((pending, rows, runs))
        if on_side and not torch.cuda.is_current_stream_capturing():
            for t in (rows, locs, found):  # allocated under the side stream, read on this one
                if t is not None:
                    t.record_stream(torch.cuda.current_stream())
        if on_side and not maintain:
            self._side_finished(rows, runs)
        if join:
            self._join_side()
        self._last = (runs, locs)
        return rows, locs, found

    def _fetch(self, runs, out_rows, fetch_ws):
        """Lookup per distinct id + rows to the batch positions, on the current stream (no index
        maintenance: what ``forward`` does without its other streams; used to time the fetch)."""
        if runs.n == 0:
            return E.cudaLookupFetchRuns(self.cold.index, runs, self.cold.emb, self.table, self.shared, out_rows,
                                         self.lookup_mode, want_locs=self.want_locs, ws=fetch_ws)
        return self._expand(runs, out_rows, self._resolve(runs, fetch_ws))

    def _resolve(self, runs, fetch_ws):
        """The per-distinct-id launch of the fetch on the current stream: slots into runs.slots,
        where every run's row is read from; rows of other GPUs' shards copied (pull) or asked for
        (deliver).  Returns the buffer ``_expand`` names as the other source of rows."""
        if self.px_req is None or self.world == 1:
            E.cudaLookupFetchRuns(self.cold.index, runs, self.cold.emb, self.table, self.shared, None,
                                  self.lookup_mode, ws=fetch_ws, resolve_only=True)
            return self.table
        # The owners deliver: the lookup stores an (id, run) request for every remote run straight into
        # the owner's receive area, every owner stores the rows it was asked for into the
        # requesters' stages, and the expansion reads local memory only.  Two fences: requests
        # complete before they are served, rows complete before they are read.
        stage = self.fetch_stages.weight
        self._req_parity = E.cudaRunsResolveRequests(self.cold.index, runs, self.cold.emb, self.shared, stage,
                                                     self.px_req, self.lookup_mode, ws=fetch_ws)
        return stage

    def _expand(self, runs, out_rows, other_rows):
        """The rest of the fetch: (deliver: fence, serve, fence) rows to their batch positions."""
        sharded = self.shared is not None and self.world > 1
        if self.px_req is not None and self.world > 1:
            self.px_req.fence()
            r_ids, _, r_runs, seg_counts = self.px_req.received(self._req_parity)
            self.shared.serve(self.fetch_stages, r_ids, r_runs, seg_counts, self.px_req.cap)
            self.px_req.fence()
        return E.cudaRunsExpand(runs, self.cold.emb, other_rows, out_rows, want_locs=self.want_locs,
                                peer_sources=sharded)

    def _index_maintenance(self, runs, n: int, lib):
        """On the maintenance stream, after the per-distinct-id launch: LRU ageing of the lookup,
        cold misses added to the index.  Returns what ``insert_rows`` needs, or None."""
        if self.touch_lru:
            self.cold.index.cuda_touch_lru_runs(runs.slots, runs, locs_kind=2)
        if not self.insert_misses:
            return None
        need = max(lib.hb_runs_miss_list_workspace_bytes(n), lib.hb_staging_insert_workspace_bytes(self.miss_cap))
        ws = self._ws("_side_ws", need)
        miss_ids, miss_src, miss_n = E.cudaRunsMissList(runs, runs.slots, COLD, self.miss_cap, ws=ws, locs_kind=2)
        locs, last_writer = self.cold.insert_index(miss_ids, ws)
        return miss_ids, miss_src, locs, last_writer, miss_n

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
        """Bucket by owner and deliver to the owners over NCCL.  Returns (ids, rows, cnt, sent)."""
        p_ids, p_rows, p_cnt, counts = E.cudaBucketPack(ids, rows, cnt, self.world, n_dev=n_dev)
        r_ids, r_rows, r_cnt = exchange_packed(p_ids, p_rows, p_cnt, counts, self.group)
        return r_ids, r_rows, r_cnt, counts

    # ---- backward ------------------------------------------------------------------------
    def backward(self, ids: torch.Tensor, grads: torch.Tensor, locs: torch.Tensor | None = None) -> StepStats:
        """ids: the ids the gradients belong to.  When they are the batch of the last ``forward``
        its sort is reused; otherwise (several forward calls before one step) they are sorted
        here.  locs is accepted for callers of the earlier interface and not used: every
        forward pass ages the LRU counters of its own lookup."""
        st = self._backward_core(ids, grads)
        self._after_step(st)
        return st

    def _after_step(self, st: StepStats, replaying: bool = False) -> None:
        self.step_no += 1
        st.flushed_dev = None
        if self.flush_every > 0 and self.step_no % self.flush_every == 0:
            if replaying and self._flush_graphs:
                # the flush has no host read either: one graph per receive area of its exchange
                graph, (counts, cap) = self._flush_graphs[self._flush_next]
                self._flush_next = (self._flush_next + 1) % len(self._flush_graphs)
                graph.replay()
                st.flushed_dev, st.flush_cap = counts, cap
            else:
                self.flush(st)

    def _runs_for(self, ids: torch.Tensor) -> E.BatchRuns:
        if self._last is not None and self._last[0].matches(ids):
            return self._last[0]
        lib = E._lib.load()
        return E.cudaRunsBuild(ids, self.id_bits, self.class_table, keep=(False, True, True),
                               caps=(None, self.num_hot_ids, None),
                               ws=self._ws("_runs_ws", lib.hb_runs_workspace_bytes(ids.numel())))

    def _backward_local(self, ids, grads, join: bool = True):
        """Backward up to the exchange: aggregation over the runs with the hot / cold selects
        (only_unique_grads, sparse_optim.py:132-139; the selects of :243-259) fused into its
        output, and the cold accumulate.  No host read and no collective.  Returns (stats, hot
        ids, rows, cnt).

        The cold accumulate touches only the staging table and the index, the hot rows' way to
        their owners only the exchange buffers and the optimiser state, so the former runs on
        the side stream (behind this step's cache insert); join=False leaves the join to the
        caller (``_join_side``)."""
        st = StepStats()
        runs = self._runs_for(ids)
        outs = E.cudaSegSumRuns(runs, grads, split_keep=(False, True, True))
        st.num_unique = runs.num_unique
        st.split_counts = runs.class_counts
        hot_ids, (hot_rows, hot_cnt) = runs.class_ids[HOT], outs[HOT]
        cold_ids, (cold_rows, _) = runs.class_ids[COLD], outs[COLD]
        with self._on_side():
            self.cold.accumulate_remote(cold_ids, cold_rows, n_dev=runs.class_counts[COLD:COLD + 1],
                                        touch_lru=self.touch_lru)
            self._side_finished(outs, runs)
        if join:
            self._join_side()
        return st, hot_ids, hot_rows, hot_cnt

    def _owner_update_from_slabs(self, parity: int) -> None:
        """Owner side after a peer-memory push: merge the senders' slabs and update."""
        r_ids, r_rows, r_cnt, seg_counts = self.px.received(parity)
        # every slab holds the sorted unique hot ids of its sender (stable bucketing): a merge
        self.opt.update(r_ids, r_rows, r_cnt, is_unique=False, id_bits=self.id_bits,
                        seg_counts=seg_counts, seg_cap=self.px.cap, sorted_segments=True)

    def _after_fetch_event(self, which: str) -> None:
        """The current stream waits for that point of a fetch that runs beside this backward pass."""
        evt = getattr(self, which)
        if evt is not None:
            torch.cuda.current_stream().wait_event(evt)
            setattr(self, which, None)

    def _backward_core(self, ids, grads) -> StepStats:
        """Everything of the backward path that runs every step (no host read unless NCCL
        carries the exchange).  When the fetch of the same batch runs beside it (``step`` with
        overlap_fetch), the exchange waits until that fetch has read what it needs from the other
        GPUs' shards, and the owner update until it has read what it needs from this GPU's shard:
        a fetch returns the rows as they were before the step's update."""
        st, hot_ids, hot_rows, hot_cnt = self._backward_local(ids, grads, join=False)
        n_hot = st.split_counts[HOT:HOT + 1]
        if self.world > 1:
            self._after_fetch_event("_evt_resolved")
        # hot rows go to their owners now
        if self.world == 1:
            # One trainer: bucketing by owner is the identity (the reference skips the exchange
            # too, sparse_optim.py:263,320), and the hot ids are already unique and ascending, so
            # unique_grads (sparse_optim.py:142-157) reduces to its division by 1 + cnt.
            st.sent_counts = n_hot
            self._after_fetch_event("_evt_expanded")
            self.opt.update(hot_ids, hot_rows, hot_cnt + 1, is_unique=True, n_dev=n_hot)
        elif self.px is not None:
            parity = self.px.push(hot_ids, hot_rows, hot_cnt, n_hot)
            self.px.fence()
            self._after_fetch_event("_evt_expanded")
            self._owner_update_from_slabs(parity)
        else:
            r_ids, r_rows, r_cnt, sent = self._exchange(hot_ids, hot_rows, hot_cnt, n_hot)
            st.sent_counts = sent
            # owner: merge the senders' rows (unique_grads with counts) and update
            self._after_fetch_event("_evt_expanded")
            self.opt.update(r_ids, r_rows, r_cnt, is_unique=False, id_bits=self.id_bits)
        self._join_side()
        self._fence_shards()
        return st

    def flush(self, st: StepStats | None = None) -> None:
        """Stale cold rows leave for their owners; their cache entries are evicted by the flush
        (server.py:413) and come back, with the owner's current row, when a later forward pass
        misses them (server.py:499-544).  No host read: the flush fills a buffer of
        ``flush_cap`` rows and hands the count over on the device."""
        if self.world > 1 and self.px_flush is None:
            return self._flush_nccl(st)
        f_ids, f_rows, f_cnt, counts = self.cold.flush_remote(sync=False, out_cap=self.flush_cap)
        if st is not None:
            st.flushed_dev, st.flush_cap = counts, self.flush_cap
        if self.world == 1:
            # one trainer: every flushed row is its own (is_unique=True, sparse_optim.py:405-421)
            self.opt.update(f_ids, f_rows, f_cnt, is_unique=True, n_dev=counts)
        else:
            # owner = id % world: the push buckets; what arrives is in slot order, so the owner
            # sorts (unique_grads, sparse_optim.py:142-157) instead of merging
            parity = self.px_flush.push(f_ids, f_rows, f_cnt, counts)
            self.px_flush.fence()
            r_ids, r_rows, r_cnt, seg_counts = self.px_flush.received(parity)
            self.opt.update(r_ids, r_rows, r_cnt, is_unique=False, id_bits=self.id_bits, seg_counts=seg_counts,
                            seg_cap=self.px_flush.cap)
            self._fence_shards()
        if self.lookup_mode == E.LOOKUP_SORTED:
            self.cold.index.build_sorted()  # the flush reset entries: captured steps expect a fresh view

    def _flush_nccl(self, st: StepStats | None) -> None:
        """The flush over NCCL all_to_all_single (sizes read on the host, as the reference's
        swap_gradients does, sparse_optim.py:55,77)."""
        f_ids, f_rows, f_cnt, counts = self.cold.flush_remote(sync=True)
        if st is not None:
            st.flushed_dev, st.flush_cap = counts, 0
        r_ids, r_rows, r_cnt = exchange_packed(f_ids, f_rows, f_cnt, counts, self.group,
                                               counts_host=self.cold.remote.last_counts_host)
        self.opt.update(r_ids, r_rows, r_cnt, is_unique=False, id_bits=self.id_bits)
        self._fence_shards()
        if self.lookup_mode == E.LOOKUP_SORTED:
            self.cold.index.build_sorted()

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
            self._after_step(st, replaying=True)
            return rows, locs, found, st
        rows, locs, found = self.forward(ids, out_rows, join=False, on_side=self.overlap_fetch)
        st = self.backward(ids, grads)
        return rows, locs, found, st

    def capture(self, ids_buf: torch.Tensor, grads: torch.Tensor, out_rows: torch.Tensor) -> None:
        """Capture the per-step work of ``step`` in CUDA graphs over the caller's buffers; later
        ``step(ids, grads, out_rows)`` calls with the same ``grads`` and ``out_rows`` replay them
        (``ids`` is copied into ``ids_buf`` unless it is that tensor).  Call it after a few eager
        steps: every lazy allocation of the library has to have happened.

        One GPU: one graph holds the whole step, one more the periodic flush.  Several GPUs
        with the peer-memory exchange and its device-side fence: two graphs, one per receive
        area, each holding the whole step; they are replayed alternately.  With the NCCL fence
        the collective is not captured: one graph for everything before the exchange and one
        per receive area for the owner update, push and fence launched eagerly between them.
        Not available with the NCCL all-to-all, which reads sizes on the host."""
        if self.world > 1 and self.px is None:
            raise RuntimeError("the NCCL all-to-all exchange reads sizes on the host and cannot be captured")
        graphs = []
        self._whole_step_graphs = self.world == 1 or self.px.fence_kind == "device"
        # the graph that fills receive area 0 (where an exchange starts again after a reset)
        self._g_area0 = self.px.next_parity if (self.world > 1 and self._whole_step_graphs) else 0
        if self._whole_step_graphs:
            for _ in range(1 if self.world == 1 else 2):  # the push picks the areas in turn
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    rows, locs, found = self.forward(ids_buf, out_rows, join=False, on_side=self.overlap_fetch)
                    st = self._backward_core(ids_buf, grads)
                graphs.append((g, (rows, locs, found, st)))
        else:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                rows, locs, found = self.forward(ids_buf, out_rows, join=False)
                st, hot_ids, hot_rows, hot_cnt = self._backward_local(ids_buf, grads)
            graphs.append((g, (rows, locs, found, st, hot_ids, hot_rows, hot_cnt)))
            for parity in (0, 1):
                gp = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gp):
                    self._owner_update_from_slabs(parity)
                graphs.append((gp, None))
        self._graphs, self._g_ids, self._g_grads, self._g_out, self._g_next = graphs, ids_buf, grads, out_rows, 0
        # the periodic flush as graphs of its own (it reads nothing on the host): with several GPUs
        # one per receive area of the flush exchange.  Not with the sorted lookup view (rebuilt on
        # the host side after a flush), tiered optimiser state, or the NCCL flush.
        self._flush_graphs, self._flush_next = [], 0
        capturable = (self._whole_step_graphs and self.flush_every > 0 and self.lookup_mode != E.LOOKUP_SORTED
                      and getattr(self.opt, "state_cache", None) is None
                      and (self.world == 1 or (self.px_flush is not None and self.px_flush.fence_kind == "device")))
        self._flush_area0 = self.px_flush.next_parity if (capturable and self.world > 1) else 0
        if capturable:
            for _ in range(1 if self.world == 1 else 2):
                g = torch.cuda.CUDAGraph()
                holder = StepStats()
                with torch.cuda.graph(g):
                    self.flush(holder)
                self._flush_graphs.append((g, (holder.flushed_dev, holder.flush_cap)))

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
            rows, locs, found = self.forward(ids_buf, out_rows, join=True)
        back = []
        area0 = self.px.next_parity if self.world > 1 else 0
        for _ in range(1 if self.world == 1 else 2):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                st = self._backward_core(ids_buf, grads_buf)
            back.append((g, st))
        self._split = dict(fwd=fg, back=back, next=0, area0=area0, ids=ids_buf, grads=grads_buf,
                           out=(rows, locs, found))

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
        self._after_step(st)
        return st

    def reset_exchange(self) -> None:
        """After a fence timed out on a missing peer and the host side has agreed that every rank
        is back: all ranks call this (a collective; host barriers inside), then go on stepping."""
        import torch.distributed as dist

        for px in (self.px, self.px_flush, self.px_req):
            if px is not None:
                px.reset()
        self._g_next = getattr(self, "_g_area0", 0) if len(self._graphs) == 2 else 0
        self._flush_next = getattr(self, "_flush_area0", 0) if len(self._flush_graphs) == 2 else 0
        if getattr(self, "_split", None):
            self._split["next"] = self._split.get("area0", 0) if len(self._split["back"]) == 2 else 0
        if self.world > 1:
            dist.barrier(group=self.group)

    def close(self) -> None:
        """Release what this path shares with the other ranks (exchange areas, the owner shard);
        every rank calls it, after its last step.  The path cannot step afterwards."""
        torch.cuda.synchronize()
        self._graphs, self._split, self._flush_graphs = [], None, []
        for obj in (self.px, self.px_flush, self.px_req, self.fetch_stages, self.shared):
            if obj is not None:
                obj.close()
        self.px = self.px_flush = self.px_req = self.fetch_stages = None

    # ---- save / resume ---------------------------------------------------------------------------
    def state_dict(self) -> dict:
        """Everything a resumed run needs to continue bit for bit: index lines and LRU counters,
        cached rows, staging buffers, optimiser state, table / owner shard, step counter.  (The
        reference keeps all of this in server shared memory and DGL DistTensors and has no
        save path; python/EmbCache/server.py:76-175.)"""
        line_ids, lru = self.cold.index.export_state()
        r = self.cold.remote
        if getattr(self.opt, "state_cache", None) is not None:
            self.opt.sync_state_to_backing()  # the saved tensors are the pinned backing ones
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
        if getattr(self.opt, "state_cache", None) is not None:
            self.opt.reload_state_cache()
        self.opt.emb.weight.copy_(sd["weight"])
        if "table" in sd:
            self.table.copy_(sd["table"])
        self._last = None


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
                  generator=None, threshold: torch.Tensor | None = None, default_threshold: int = 0,
                  cnt_threshold: int = 16, insert_misses: bool = True, flush_cap: int = 1 << 19,
                  miss_cap: int = 1 << 17, state_budget_bytes: int | None = None,
                  hotness: torch.Tensor | None = None, remote_fetch: str = "auto",
                  fetch_stage_rows: int = 0) -> EmbeddingPath:
    """Cold cache filled with `cache_ids` (rows from `table`), optimiser shard, exchange.
    remote_fetch: who brings the rows of other GPUs' shards in the forward fetch: "pull" (this GPU
    reads them, once per distinct id), "deliver" (the owners store them into this GPU's stage of
    fetch_stage_rows rows; needs the peer-memory exchange with the device fence), "auto": deliver
    (scattered peer loads collapse once a GPU reads several peers at a time while all of them read
    it; with two GPUs the two forms measure within 2 % of each other).
    state_budget_bytes / hotness: see ``SparseAdam`` (state tiered between HBM and pinned host
    memory when it does not fit the budget; hotness per node of the whole table).
    threshold: int32 per-node flush period (``cold_cache.flush_thresholds`` of the presampled
    hotness, server.py:87-88); None: every staged row is stale at every flush."""
    rows_total, dim = table.shape
    _warm_collectives(world, device, group)
    slots = -(-int(cache_entries) // 8) * 8  # the index rounds its capacity up to whole lines
    flush_cap = int(min(flush_cap, slots))
    px = px_flush = None
    if world > 1 and exchange in ("push", "push_nccl_fence"):
        fence = "device" if exchange == "push" else "nccl"
        px = _peer_exchange(rank, world, hot_per_owner_max, dim, device, group, fence)
        if px is not None:
            # a rank may find all its stale rows owned by one peer: a slab holds a whole flush
            px_flush = _peer_exchange(rank, world, flush_cap, dim, device, group, fence)
            if px_flush is None:
                px = None
    push = px is not None
    cold = ColdCache(f"{name}_r{rank}", cache_entries, dim, threshold=threshold, cnt_threshold=cnt_threshold,
                     default_threshold=default_threshold, num_clients=1 if (world == 1 or push) else world,
                     lookup_mode=lookup_mode, device=device)
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
    if optimizer == "adam":
        opt = SparseAdam(shard, lr=0.01, state_budget_bytes=state_budget_bytes,
                         hotness=None if hotness is None else hotness[rank::world].float().cpu())
    else:
        opt = SparseAdagrad(shard, lr=0.01)
    id_bits = max(int(rows_total).bit_length() + 1, 8)
    px_req = stages = None
    deliver = remote_fetch == "deliver" or (remote_fetch == "auto" and world > 1)
    if deliver and share and px is not None and px.fence_kind == "device" and fetch_stage_rows > 0:
        from .peer_table import PeerTable

        # a requester asks one owner for at most the rows that owner has, and for at most one per stage row
        req_cap = int(min(fetch_stage_rows, -(-rows_total // world)))
        px_req = _peer_exchange(rank, world, req_cap, 4, device, group, "device")
        if px_req is not None:
            stages = PeerTable(world * int(fetch_stage_rows), dim, rank, world, dtype=torch.float32, device=device,
                               group=group)
    path = EmbeddingPath(table, class_table, cold, opt, rank, world, flush_every, id_bits,
                         lookup_mode, mover, touch_lru, group, px, px_flush, insert_misses=insert_misses,
                         miss_cap=miss_cap, flush_cap=flush_cap, request_exchange=px_req, fetch_stages=stages)
    path.cache_fill_ids = cache_ids  # what the cold cache was filled with, in insertion order
    return path


def build_path(cfg, rank: int = 0, world: int = 1, device=None, optimizer: str = "adam",
               hot_fraction: float = 0.01, lookup_mode: int = E.LOOKUP_SETASSOC,
               mover: int = E.MOVER_AUTO, touch_lru: bool = True, table_dtype=torch.float32,
               seed_config: int | None = None, group=None, exchange: str = "push",
               hotness: torch.Tensor | None = None, hot_threshold: float | None = None,
               cnt_threshold: int = 16, insert_misses: bool = True, flush_cap: int = 1 << 19,
               miss_cap: int = 1 << 17, state_budget_bytes: int | None = None,
               remote_fetch: str = "auto", fetch_stage_rows: int | None = None) -> EmbeddingPath:
    """Build the state of one trainer for a cached-fetch configuration (``synth.CacheFetchConfig``):
    backing table, class table, cold cache filled with the most popular COLD ids, optimiser shard.

    Without `hotness` the popularity ranking of the synthetic stream stands in for it: the top
    ``hot_fraction`` of the ranking is HOT, the cache holds the next ``cache_entries`` ids, and
    every staged row is stale at every flush.  With `hotness` (float32 per node, accesses per
    sampled batch: ``hotness.presampling``) everything is derived from it as the reference
    does: HOT = hotness >= hot_threshold (dist_emb.py:108-120), per-node flush periods
    ceil(1 / (0.001 + hotness)) capped at 100 (server.py:87-88) with the count threshold
    `cnt_threshold` (dist_emb.py:139), and the cache starts with the hottest COLD ids."""
    import numpy as np

    from . import hotness as H
    from . import synth

    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    gen = torch.Generator(device=device)
    gen.manual_seed(1000 * (seed_config or cfg.config))  # the same table on every rank
    table = torch.empty((cfg.table_rows, cfg.dim), dtype=torch.float32, device=device)
    table.normal_(0.0, cfg.table_sigma, generator=gen)
    threshold, default_threshold = None, 0
    if hotness is not None:
        hotness = hotness.to(device=device, dtype=torch.float32)
        if hot_threshold is None:
            # the value that makes about hot_fraction of the nodes hot
            k = max(int(cfg.table_rows * hot_fraction), 1)
            hot_threshold = float(torch.topk(hotness, k).values[-1].item())
        class_table = H.class_table(hotness, hot_threshold)
        threshold = flush_thresholds(hotness)
        cache_ids = H.hottest_ids(hotness, class_table == COLD, cfg.cache_entries)
        hot_owner = torch.nonzero(class_table == HOT).flatten() % world
        cap = int(torch.bincount(hot_owner, minlength=world).max().item()) if hot_owner.numel() else 1
    else:
        n_hot = max(int(cfg.table_rows * hot_fraction), 1)
        hot_ranked = synth.rank_to_id(np.arange(n_hot, dtype=np.int64), cfg.table_rows)
        cls = np.full(cfg.table_rows, COLD, dtype=np.int8)
        cls[hot_ranked] = HOT
        class_table = torch.from_numpy(cls).to(device)
        # the most popular ids that are not hot, in popularity order
        last = min(n_hot + cfg.cache_entries, cfg.table_rows)
        cache_ids = torch.from_numpy(synth.rank_to_id(np.arange(n_hot, last, dtype=np.int64), cfg.table_rows)).to(device)
        # a rank can receive from one source at most the hot ids it owns
        cap = int(np.bincount(hot_ranked % world, minlength=world).max())
    return assemble_path(cfg.name, table, class_table, cache_ids, max(cap, 1), rank, world, device, optimizer,
                         cfg.flush_every, lookup_mode, mover, touch_lru, group, exchange,
                         cfg.cache_entries, table_dtype, cfg.table_sigma, gen, threshold, default_threshold,
                         cnt_threshold, insert_misses, flush_cap, miss_cap, state_budget_bytes, hotness,
                         remote_fetch, cfg.batch if fetch_stage_rows is None else fetch_stage_rows)


def build_rmat_path(cfg, rank: int = 0, world: int = 1, device=None, optimizer: str = "adam",
                    lookup_mode: int = E.LOOKUP_SETASSOC, mover: int = E.MOVER_AUTO,
                    touch_lru: bool = True, group=None, exchange: str = "push",
                    insert_misses: bool = True, remote_fetch: str = "auto") -> EmbeddingPath:
    """State of one trainer for the sampled-GraphSAGE configuration (``synth.RmatConfig``).
    Under R-MAT a vertex is the more popular the fewer one-bits its id has, so the HOT class
    is ``popcount(id) <= cfg.hot_popcount`` and the cold cache starts with the most popular
    cold vertices (popcount hot_popcount+1, +2, ... in id order)."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    n, dim = cfg.num_nodes, cfg.dim
    frontier, layer = cfg.seeds, cfg.seeds  # ids one step fetches: seeds + 1-hop + 2-hop samples
    for f in cfg.fanout:
        layer *= f
        frontier += layer
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
                         cfg.cache_entries, torch.float32, cfg.table_sigma, gen, insert_misses=insert_misses,
                         remote_fetch=remote_fetch, fetch_stage_rows=frontier)
