"""Replay of tests/golden/server_golden.npz (recorded from the reference's own cache-server
methods, tests/golden/make_golden_server.py) against a cold-cache implementation: the numpy
oracle on CPU or the CUDA library.  A backend offers flush_remote / flush_local / insert /
accumulate_remote / accumulate_local and state()."""
import numpy as np


class OracleBackend:
    def __init__(self, om, g, name, compat_no_clear):
        k = lambda f: g[f"{name}_{f}"]
        self.om = om
        self.clients = int(k("clients"))
        self.thr = om.flush_thresholds(k("hotness"))
        self.ps, self.pn = int(k("part_start")), int(k("part_nodes"))
        dim = int(k("dim"))
        self.ix = om.OracleIndex(int(k("cache_entries")))
        slots = self.ix.get_capacity()
        assert slots == int(k("slots"))
        self.cache = np.zeros((slots, dim), np.float32)
        ct = int(k("cnt_threshold"))
        self.rem = om.OracleStaging(slots, dim, cnt_threshold=ct, compat_no_clear=compat_no_clear)
        self.loc = om.OracleStaging(self.pn, dim, cnt_threshold=ct, compat_no_clear=compat_no_clear,
                                    iter_threshold=self.thr[self.ps:self.ps + self.pn])

    def flush_remote(self):
        return self.rem.flush(self.ix, self.clients)

    def flush_local(self):
        return self.loc.flush(None, self.clients)

    def insert(self, ids, embs):
        return self.rem.insert(self.ix, ids, embs, self.cache)

    def accumulate_remote(self, ids, grads):
        self.rem.accumulate_cached(self.ix, ids, grads, self.thr, 1)

    def accumulate_local(self, ids, grads):
        self.loc.accumulate_direct(ids, grads, self.ps, 1)

    def state(self):
        n = self.ix.get_valid_entries_num()
        gi, gl = self.ix.getall(n)
        return dict(index_ids=gi, index_locs=gl, cnt=self.rem.cnt, idx=self.rem.idx, iter_count=self.rem.iter_count,
                    grad=self.rem.grad, emb=self.cache, local_cnt=self.loc.cnt,
                    local_iter_count=self.loc.iter_count, local_grad=self.loc.grad)


def replay(g, name, be, rows_exact: bool, buffers_exact: bool):
    """rows_exact: the rows a flush sends are compared (bit-exact); buffers_exact: the gradient
    buffers themselves are compared too (only an implementation that, like the reference,
    never clears them can match in a scenario that stages into a flushed slot again)."""
    k = lambda f: g[f"{name}_{f}"]
    clients = int(k("clients"))
    for it in range(int(k("iters"))):
        for kind, fn in (("remote", be.flush_remote), ("local", be.flush_local)):
            ids, rows, cnt, counts = fn()
            where = (name, it, kind)
            assert np.array_equal(np.asarray(counts), k(f"it{it}_sent_{kind}_counts")), where
            assert np.array_equal(np.asarray(ids), k(f"it{it}_sent_{kind}_ids")), where
            assert np.array_equal(np.asarray(cnt), k(f"it{it}_sent_{kind}_cnt")), where
            if rows_exact:
                assert np.array_equal(np.asarray(rows), k(f"it{it}_sent_{kind}_rows")), where
        sizes = k(f"it{it}_ins_sizes")
        ids_all, embs_all = k(f"it{it}_ins_ids"), k(f"it{it}_ins_embs")
        o = 0
        for c in range(clients):  # one client's message after the other, server.py:501
            if sizes[c]:
                be.insert(ids_all[o:o + sizes[c]], embs_all[o:o + sizes[c]])
            o += sizes[c]
        for c in range(clients):
            be.accumulate_remote(k(f"it{it}_c{c}_rid"), k(f"it{it}_c{c}_rg"))
            be.accumulate_local(k(f"it{it}_c{c}_lid"), k(f"it{it}_c{c}_lg"))
        st = be.state()
        for f in ("index_ids", "index_locs", "cnt", "idx", "iter_count", "emb", "local_cnt", "local_iter_count"):
            assert np.array_equal(np.asarray(st[f]), k(f"it{it}_{f}")), (name, it, f)
        if buffers_exact:
            for f in ("grad", "local_grad"):
                assert np.array_equal(np.asarray(st[f]), k(f"it{it}_{f}")), (name, it, f)
