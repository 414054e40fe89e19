"""TEST INFRASTRUCTURE -- not part of the product.  The whole per-step embedding path of `world`
trainers composed from the oracle's restatements (oracle/oracle.py), in numpy on the host: what
``DistEmb.__call__`` (python/EmbCache/dist_emb.py:167-292), ``DistembSparseGradOptimizer.step``
(python/EmbCache/sparse_optim.py:212-448) and the cache-server loop (python/EmbCache/server.py:
259-298) compute for one step, with every trainer's cold cache, one table and one optimiser
state for the whole box.  hades_b200.pipeline.EmbeddingPath is compared with it (tests, the
benchmark's untimed self-check)."""
from __future__ import annotations

import numpy as np

HOT, COLD = 1, 2


class PipelineOracle:
    def __init__(self, om, table, class_table, cache_entries, cache_fill_ids, world=1, flush_every=8, lr=0.01,
                 optimizer="adam", threshold=None, default_threshold=0, cnt_threshold=16, insert_misses=True,
                 miss_cap=1 << 17, flush_cap=1 << 19, touch_lru=True):
        self.om, self.world, self.flush_every, self.lr, self.optimizer = om, world, flush_every, lr, optimizer
        self.table = np.array(table, dtype=np.float32, copy=True)
        self.cls = np.asarray(class_table)
        self.threshold, self.default_threshold = threshold, default_threshold
        self.insert_misses, self.miss_cap, self.touch_lru = insert_misses, miss_cap, touch_lru
        n, dim = self.table.shape
        self.dim = dim
        self.step_state = np.zeros(n, np.float32)
        self.mem = np.zeros((n, dim), np.float32)
        self.power = np.zeros((n, dim), np.float32)   # Adagrad: the sum of squares
        self.ranks = []
        for _ in range(world):
            ix = om.OracleIndex(cache_entries)
            slots = ix.get_capacity()
            st = om.OracleStaging(slots, dim, cnt_threshold=cnt_threshold)
            cache = np.zeros((slots, dim), np.float32)
            fill = np.asarray(cache_fill_ids, np.int64)
            st.insert(ix, fill, self.table[fill], cache)
            self.ranks.append(dict(index=ix, staging=st, cache=cache, dropped=0))
        self.flush_cap = min(flush_cap, self.ranks[0]["index"].get_capacity())
        self.step_no = 0

    def _update(self, ids, grads, cnt=None):
        if ids.size == 0:
            return
        if self.optimizer == "adam":
            self.om.sparse_adam_update(ids, grads, self.step_state, self.mem, self.power, self.table, self.lr, cnt=cnt)
        else:
            self.om.sparse_adagrad_update(ids, grads, self.power, self.table, self.lr, cnt=cnt)

    def step(self, ids_per_rank, grads_per_rank):
        """One step of every trainer.  Returns per rank (rows, locs, found) and the rows each
        rank's flush sent (0 when this is no flush step)."""
        om = self.om
        outs = []
        # forward: every trainer reads the table as the previous step left it
        for r, ids in zip(self.ranks, ids_per_rank):
            ids = np.asarray(ids, np.int64)
            rows = np.zeros((ids.size, self.dim), np.float32)
            locs, hit = om.lookup_fetch(r["index"], ids, r["cache"], self.table, rows)
            if self.touch_lru:
                r["index"].touch(locs)
            if self.insert_misses and ids.size:
                u, first = np.unique(ids, return_index=True)
                miss = u[(self.cls[u] == COLD) & (locs[first] < 0)][: self.miss_cap]
                r["staging"].insert(r["index"], miss, self.table[miss], r["cache"])
            outs.append((rows, locs, hit))
        # backward: local aggregation, cold rows staged, hot rows to their owners
        hot_parts = []
        for r, ids, grads in zip(self.ranks, ids_per_rank, grads_per_rank):
            u, s, c = om.only_unique_grads(np.asarray(ids, np.int64), grads)
            kind = self.cls[u]
            cold = kind == COLD
            if self.touch_lru:
                r["dropped"] += r["staging"].accumulate_cached(r["index"], u[cold], s[cold], self.threshold,
                                                               self.default_threshold)
            else:
                r["dropped"] += _accumulate_no_touch(om, r, u[cold], s[cold], self.threshold, self.default_threshold)
            hot_parts.append((u[kind == HOT], s[kind == HOT], c[kind == HOT]))
        if self.world == 1:
            hu, hs, hc = hot_parts[0]
            self._update(hu, hs, cnt=hc + 1)   # unique_grads of unique ids: the division by 1 + cnt
        else:
            hu, hm, _ = om.unique_grads(np.concatenate([p[0] for p in hot_parts]),
                                        np.concatenate([p[1] for p in hot_parts]),
                                        np.concatenate([p[2] for p in hot_parts]))
            self._update(hu, hm)
        self.step_no += 1
        flushed = [0] * self.world
        if self.flush_every > 0 and self.step_no % self.flush_every == 0:
            parts = []
            for k, r in enumerate(self.ranks):
                fi, fr, fc, _ = r["staging"].flush(r["index"], 1, out_cap=self.flush_cap)
                flushed[k] = fi.size
                parts.append((fi, fr, fc))
            if self.world == 1:
                self._update(parts[0][0], parts[0][1], cnt=parts[0][2])
            else:
                fu, fm, _ = om.unique_grads(np.concatenate([p[0] for p in parts]),
                                            np.concatenate([p[1] for p in parts]),
                                            np.concatenate([p[2] for p in parts]))
                self._update(fu, fm)
        return outs, flushed


def _accumulate_no_touch(om, r, ids, grads, threshold, default_threshold):
    st, ix = r["staging"], r["index"]
    locs = ix.lookup(ids, touch=False)
    hit = np.nonzero(locs >= 0)[0]
    if hit.size:
        s = locs[hit]
        st.idx[s] = ids[hit]
        st.iter_threshold[s] = threshold[ids[hit]] if threshold is not None else default_threshold
        st.grad[s] += grads[hit]
        st.cnt[s] += 1
    return int((locs < 0).sum())


def compare_rank(path, oracle: PipelineOracle, rank: int, where="", rtol=1e-4):
    """Assert that an EmbeddingPath's state equals the oracle's for `rank`: index lines and LRU
    counters, staging counters and ids bit-exact; staged gradient sums within 1e-5 of their
    terms; optimiser state within `rtol`; table and cached rows within `rtol` plus 1e-3 of the
    learning rate (an early Adam step moves a weight by about lr whatever the gradient's size,
    lr * g / (|g| + eps), so where the duplicates of an id nearly cancel, the rounding of their
    mean is amplified by 1 / |mean|: the bound is relative to lr, not to the weight)."""
    atol_w = 1e-3 * oracle.lr
    r = oracle.ranks[rank]
    gi, gl = path.cold.index.export_state()
    oi, ol = r["index"].export()
    assert np.array_equal(gi.cpu().numpy(), oi), f"index ids differ {where}"
    assert np.array_equal(gl.cpu().numpy(), ol), f"LRU counters differ {where}"
    st = path.cold.remote
    assert np.array_equal(st.cnt.cpu().numpy(), r["staging"].cnt), f"staging cnt differs {where}"
    assert np.array_equal(st.idx.cpu().numpy(), r["staging"].idx), f"staging idx differs {where}"
    assert np.array_equal(st.iter_count.cpu().numpy(), r["staging"].iter_count), f"iter_count differs {where}"
    np.testing.assert_allclose(st.grad.cpu().numpy(), r["staging"].grad, rtol=1e-5, atol=1e-9,
                               err_msg=f"staged gradients differ {where}")
    np.testing.assert_allclose(path.cold.emb.cpu().numpy(), r["cache"], rtol=rtol, atol=atol_w,
                               err_msg=f"cached rows differ {where}")
    assert int(path.cold.dropped.item()) == r["dropped"], f"dropped count differs {where}"
    w, world = path.opt.emb.weight.float().cpu().numpy(), oracle.world
    np.testing.assert_allclose(w, oracle.table[rank::world], rtol=rtol, atol=atol_w,
                               err_msg=f"owned table rows differ {where}")
    if hasattr(path.opt, "state_step"):
        assert np.array_equal(path.opt.state_step.cpu().numpy(), oracle.step_state[rank::world]), f"Adam step {where}"
        np.testing.assert_allclose(path.opt.state_mem.cpu().numpy(), oracle.mem[rank::world], rtol=rtol, atol=1e-9,
                                   err_msg=f"Adam first moment differs {where}")
    else:
        np.testing.assert_allclose(path.opt.state_sum.cpu().numpy(), oracle.power[rank::world], rtol=rtol, atol=1e-12,
                                   err_msg=f"Adagrad sum differs {where}")
