"""The sort-once operators (hb_runs_build, hb_lookup_fetch_runs, hb_segsum_runs_f32,
hb_runs_miss_list, hb_staging_insert_gather) against numpy restatements of what the reference
computes per call (torch.unique of python/EmbCache/sparse_optim.py:133, the cached fetch of
dist_emb.py:184-243, the uncached cold ids of dist_emb.py:218-259) and against this library's
unsorted operators: bit-exact ids, counts, classes, slots, found masks and rows."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _ids(rng, n, space, skew=True):
    if skew:
        return np.minimum((rng.pareto(1.05, n) * 3).astype(np.int64), space - 1)
    return rng.integers(0, space, n, dtype=np.int64)


@pytest.mark.parametrize("n,space,id_bits", [(1, 10, 8), (31, 7, 8), (2048, 300, 16), (2049, 50_000, 17),
                                             (70_000, 1_000_000, 21), (70_000, 5 * 10**9, 40), (300_000, 90, 64)])
def test_runs_build_matches_numpy_unique(cuda_lib, n, space, id_bits):
    from hades_b200 import EmbCacheLib as E

    rng = np.random.default_rng(n + id_bits)
    ids = _ids(rng, n, space, skew=n % 2 == 0)
    table_len = min(space, 1 << 22)
    table = rng.integers(0, 4, table_len).astype(np.int8)  # class 3 = no class
    runs = E.cudaRunsBuild(_t(ids), id_bits, _t(table), want_uniq=True)
    u, first, counts = np.unique(ids, return_index=True, return_counts=True)
    U = int(runs.num_unique.item())
    assert U == u.size
    assert np.array_equal(runs.uniq_ids[:U].cpu().numpy(), u)
    cls = np.where(u < table_len, table[np.minimum(u, table_len - 1)], 3)
    cc = runs.class_counts.cpu().numpy()
    for c in range(3):
        assert cc[c] == (cls == c).sum()
        assert np.array_equal(runs.class_ids[c][: cc[c]].cpu().numpy(), u[cls == c])
    # the grouping itself, read back through the descriptor
    from hades_b200.exchange import _as_tensor

    dev = torch.device("cuda", torch.cuda.current_device())
    perm = _as_tensor(runs.desc.perm, (n,), "<i4", dev).cpu().numpy().astype(np.int64)
    run_start = _as_tensor(runs.desc.run_start, (U + 1,), "<i8", dev).cpu().numpy()
    head = _as_tensor(runs.desc.head, (n,), "|u1", dev).cpu().numpy()
    assert np.array_equal(perm, np.argsort(ids, kind="stable"))
    assert np.array_equal(np.diff(run_start), counts) and run_start[U] == n
    assert head.sum() == U and np.array_equal(np.nonzero(head)[0], run_start[:U])


def test_runs_build_prefix_count_and_segments(cuda_lib):
    from hades_b200 import EmbCacheLib as E

    rng = np.random.default_rng(5)
    ids = _ids(rng, 10_000, 4000)
    n_dev = torch.tensor([6_111], dtype=torch.int64, device="cuda")
    runs = E.cudaRunsBuild(_t(ids), 16, n_dev=n_dev, want_uniq=True)
    u = np.unique(ids[:6_111])
    assert int(runs.num_unique.item()) == u.size and np.array_equal(runs.uniq_ids[: u.size].cpu().numpy(), u)
    seg = torch.tensor([100, 0, 2500, 7], dtype=torch.int64, device="cuda")
    runs = E.cudaRunsBuild(_t(ids), 16, seg_counts=seg, seg_cap=2500, want_uniq=True)
    valid = np.concatenate([ids[0:100], ids[5000:7500], ids[7500:7507]])
    u = np.unique(valid)
    assert int(runs.num_unique.item()) == u.size and np.array_equal(runs.uniq_ids[: u.size].cpu().numpy(), u)


def test_out_of_range_id_raises_the_status_word(cuda_lib):
    """An id that does not fit below 2^id_bits - 1 would collide with the padding key: the
    device status word reports HB_ERR_INVALID (the guard reads nothing out of range)."""
    from hades_b200 import EmbCacheLib as E, _lib

    assert _lib.device_status() == 0
    ids = np.array([3, 1, 70_000, 3, 2], np.int64)
    runs = E.cudaRunsBuild(_t(ids), 16, want_uniq=True)
    torch.cuda.synchronize()
    assert _lib.device_status() != 0 and _lib.device_status() == 0  # reported once, then cleared
    assert int(runs.num_unique.item()) == 4  # 1, 2, 3 and the key the bad id was given


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("dim,dtype", [(128, np.float32), (64, np.float32), (3, np.float32), (200, np.float32),
                                       (16, np.float64)])
def test_lookup_fetch_runs_equals_unsorted_fetch(cuda_lib, oracle_mod, mode, dim, dtype):
    from hades_b200 import EmbCacheLib as E, synth

    cfg = synth.scaled(synth.CONFIG1, 0.1)
    rng = synth.rng_for(1, 0, dim)
    table = synth.normal_rows(rng, cfg.table_rows, dim, cfg.table_sigma).astype(dtype)
    ix = E.IndexCache(cfg.cache_entries, f"lfr{mode}{dim}", True, False, lookup_mode=mode)
    ora = oracle_mod.OracleIndex(cfg.cache_entries)
    hot = synth.hot_ids(cfg.table_rows, cfg.cache_entries)
    locs = ix.add(torch.from_numpy(hot)).numpy()
    assert np.array_equal(locs, ora.add(hot))
    cache = np.zeros((ix.get_capacity(), dim), dtype)
    cache[locs[locs >= 0]] = table[hot[locs >= 0]] * 2.0
    q = synth.ZipfSampler(cfg.table_rows, cfg.zipf_s).ids(rng, cfg.batch + 5)
    want = np.full((q.size, dim), -7.0, dtype)
    want_locs, want_hit = oracle_mod.lookup_fetch(ora, q, cache, table, want)
    runs = E.cudaRunsBuild(_t(q), 21)
    pre = torch.full((q.size, dim), -7.0, device="cuda", dtype=torch.from_numpy(want).dtype)
    out, locs_g, found = E.cudaLookupFetchRuns(ix, runs, _t(cache), _t(table), out_rows=pre)
    assert np.array_equal(locs_g.cpu().numpy(), want_locs)
    assert np.array_equal(found.cpu().numpy(), want_hit)
    assert np.array_equal(out.cpu().numpy(), want)
    assert 0 < want_hit.sum() < q.size
    # the slot of every run (distinct id) is the per-position slot of the run's first entry
    from hades_b200.exchange import _as_tensor

    U = int(runs.num_unique.item())
    perm = _as_tensor(runs.desc.perm, (q.size,), "<i4", locs_g.device).long()
    run_start = _as_tensor(runs.desc.run_start, (U,), "<i8", locs_g.device)
    assert torch.equal(runs.slots[:U], locs_g[perm[run_start]])
    out2, none_locs, found2 = E.cudaLookupFetchRuns(ix, runs, _t(cache), _t(table), want_locs=False)
    assert none_locs is None and torch.equal(out2, out) and torch.equal(found2, found)
    # the two launches as separate calls (work that needs only the slots can run between them)
    runs3 = E.cudaRunsBuild(_t(q), 21)
    cache_t, table_t = _t(cache), _t(table)  # the first call leaves addresses of their rows behind
    assert E.cudaLookupFetchRuns(ix, runs3, cache_t, table_t, resolve_only=True) == (None, None, None)
    assert torch.equal(runs3.slots[:U], runs.slots[:U])
    pre = torch.full((q.size, dim), -7.0, device="cuda", dtype=pre.dtype)
    out3, locs3, found3 = E.cudaRunsExpand(runs3, cache_t, table_t, out_rows=pre, peer_sources=False)
    assert torch.equal(out3, out) and torch.equal(locs3, locs_g) and torch.equal(found3, found)
    # without a backing table a miss leaves the output row untouched
    want1 = np.full((q.size, dim), -7.0, dtype)
    oracle_mod.lookup_fetch(ora, q, cache, None, want1)
    pre = torch.full((q.size, dim), -7.0, device="cuda", dtype=pre.dtype)
    E.cudaLookupFetchRuns(ix, runs, _t(cache), None, out_rows=pre)
    assert np.array_equal(pre.cpu().numpy(), want1)


def test_lookup_fetch_runs_bounds_a_bad_id(cuda_lib):
    """A miss whose id has no row in the table leaves its output row untouched and raises the
    status word; nothing is read out of range."""
    from hades_b200 import EmbCacheLib as E, _lib

    ix = E.IndexCache(64, "lfr_bounds", True, False)
    table = torch.arange(40, dtype=torch.float32, device="cuda").reshape(10, 4)
    cache = torch.zeros((ix.get_capacity(), 4), device="cuda")
    q = torch.tensor([2, 12, 2, 9], dtype=torch.int64, device="cuda")
    runs = E.cudaRunsBuild(q, 8)
    pre = torch.full((4, 4), -1.0, device="cuda")
    out, locs, found = E.cudaLookupFetchRuns(ix, runs, cache, table, out_rows=pre)
    torch.cuda.synchronize()
    assert _lib.device_status() != 0
    assert torch.equal(out[0], table[2]) and torch.equal(out[2], table[2]) and torch.equal(out[3], table[9])
    assert torch.equal(out[1], torch.full((4,), -1.0, device="cuda")) and not found.any()


@pytest.mark.parametrize("dim", [1, 4, 128, 130])
def test_segsum_runs_equals_unique_segsum(cuda_lib, oracle_mod, dim):
    from hades_b200 import EmbCacheLib as E

    rng = np.random.default_rng(dim)
    n = 60_000
    ids = _ids(rng, n, 20_000)
    grads = (rng.standard_normal((n, dim)) * 1e-3).astype(np.float32)
    table = rng.integers(0, 3, 20_000).astype(np.int8)
    runs = E.cudaRunsBuild(_t(ids), 16, _t(table), want_uniq=True)
    outs = E.cudaSegSumRuns(runs, _t(grads), split_keep=(True, True, True))
    sums, counts = E.cudaSegSumRuns(runs, _t(grads))
    ref_u, ref_s, ref_c = E.cudaUniqueSegSum(_t(ids), _t(grads), id_bits=16)
    U = ref_u.numel()
    assert torch.equal(runs.uniq_ids[:U], ref_u) and torch.equal(counts[:U], ref_c)
    assert torch.equal(sums[:U], ref_s)  # the same additions in the same order
    u, s, c = oracle_mod.only_unique_grads(ids, grads)
    scale = np.zeros_like(s)
    np.add.at(scale, np.unique(ids, return_inverse=True)[1], np.abs(grads))
    assert (np.abs(sums[:U].cpu().numpy() - s) <= 1e-5 * np.maximum(scale, 1e-30)).all()
    cls = table[u]
    cc = runs.class_counts.cpu().numpy()
    for k in range(3):
        assert torch.equal(outs[k][0][: cc[k]], ref_s[_t(np.nonzero(cls == k)[0])])
        assert np.array_equal(outs[k][1][: cc[k]].cpu().numpy(), c[cls == k])


def test_miss_list_and_gathered_insert(cuda_lib, oracle_mod):
    """Cold ids that missed the lookup, ascending, capped; inserted from the rows the fetch wrote
    (dist_emb.py:218-259 -> server.py:499-544) with the same slots and cache contents as the
    oracle's insert of the same ids."""
    from hades_b200 import EmbCacheLib as E
    from hades_b200.cold_cache import ColdCache

    rng = np.random.default_rng(77)
    nodes, dim, entries = 30_000, 16, 2_000
    table = (rng.standard_normal((nodes, dim)) * 0.01).astype(np.float32)
    cls = np.where(rng.random(nodes) < 0.1, 1, 2).astype(np.int8)
    cc = ColdCache("misslist", entries, dim)
    ox = oracle_mod.OracleIndex(entries)
    ocache = np.zeros((ox.get_capacity(), dim), np.float32)
    ost = oracle_mod.OracleStaging(ox.get_capacity(), dim)
    first = rng.permutation(nodes)[:1500].astype(np.int64)
    cc.insert(_t(first), _t(table[first]))
    ost.insert(ox, first, table[first], ocache)
    for cap in (1 << 12, 300):
        q = _ids(rng, 9_000, nodes, skew=False)
        runs = E.cudaRunsBuild(_t(q), 16, _t(cls))
        rows, locs, found = E.cudaLookupFetchRuns(cc.index, runs, cc.emb, _t(table))
        wl = ox.lookup(q, touch=False)
        assert np.array_equal(locs.cpu().numpy(), wl)
        cc.index.cuda_touch_lru_runs(locs, runs)
        ox.touch(wl)
        miss_ids, miss_src, miss_n = E.cudaRunsMissList(runs, locs, 2, cap)
        ms_ids, ms_src, ms_n = E.cudaRunsMissList(runs, runs.slots, 2, cap, locs_kind=2)
        assert torch.equal(ms_ids, miss_ids) and torch.equal(ms_src, miss_src) and torch.equal(ms_n, miss_n)
        u, fi = np.unique(q, return_index=True)
        want = u[(cls[u] == 2) & (wl[fi] < 0)][:cap]
        m = int(miss_n.item())
        assert m == want.size and np.array_equal(miss_ids[:m].cpu().numpy(), want)
        assert (miss_ids[m:] == -1).all()
        assert np.array_equal(q[miss_src[:m].cpu().numpy()], want)
        glocs = cc.insert_gather(miss_ids, rows, miss_src)
        wlocs = ost.insert(ox, want, table[want], ocache)
        assert np.array_equal(glocs[:m].cpu().numpy(), wlocs) and (glocs[m:] == -1).all()
        assert np.array_equal(cc.emb.cpu().numpy(), ocache)
        gi, gl = cc.index.export_state()
        oi, ol = ox.export()
        assert np.array_equal(gi.cpu().numpy(), oi) and np.array_equal(gl.cpu().numpy(), ol)
