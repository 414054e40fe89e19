"""Row movers through the reference-facing API against the oracle: copies are bit-exact.
Shapes follow the reference's own test scripts (test/test_fetch.py, test_cached_fetch.py,
test_cached_set.py, test_combine.py and their 1-D variants) at reduced row counts, plus odd
dimensions, both index widths and both float widths."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DIMS = [1, 3, 64, 128, 257]


def _case(rng, rows, n, dim, fdtype, idtype, unique=True):
    src = rng.standard_normal((rows, dim)).astype(fdtype)
    idx = (rng.permutation(rows)[:n] if unique else rng.integers(0, rows, n)).astype(idtype)
    return src, idx


@pytest.mark.parametrize("dim", DIMS)
@pytest.mark.parametrize("fdtype,idtype", [(np.float32, np.int64), (np.float64, np.int32)])
def test_fetch_and_fetch2(cuda_lib, oracle_mod, dim, fdtype, idtype):
    from hades_b200 import EmbCacheLib as E

    rng = np.random.default_rng(dim)
    src, si = _case(rng, 40_000, 10_000, dim, fdtype, idtype, unique=False)
    di = rng.permutation(12_000)[:10_000].astype(idtype)
    dst0 = rng.standard_normal((12_000, dim)).astype(fdtype)
    want = oracle_mod.rows_gather(src, si, dst0.copy(), di)
    dst = torch.from_numpy(dst0.copy()).cuda()
    E.cudaFetch(torch.from_numpy(src).cuda(), torch.from_numpy(si).cuda(), dst, torch.from_numpy(di).cuda())
    assert np.array_equal(dst.cpu().numpy(), want)
    want2 = oracle_mod.rows_gather(src, si, dst0.copy(), None)
    for mover in (E.MOVER_AUTO, E.MOVER_LSU):
        dst = torch.from_numpy(dst0.copy()).cuda()
        E.cudaFetch2(torch.from_numpy(src).cuda(), torch.from_numpy(si).cuda(), dst, mover=mover)
        assert np.array_equal(dst.cpu().numpy(), want2)


@pytest.mark.parametrize("dim,fdtype", [(4, np.float32), (64, np.float32), (128, np.float32),
                                        (132, np.float32), (128, np.float64), (1024, np.float32),
                                        (4096, np.float32)])
@pytest.mark.parametrize("n", [1, 31, 32, 33, 5000])
def test_bulk_movers(cuda_lib, oracle_mod, dim, fdtype, n):
    """cp.async.bulk path: same bytes as the oracle for full and ragged stages."""
    from hades_b200 import EmbCacheLib as E

    rng = np.random.default_rng(dim * 7 + n)
    rows = 9000
    src, si = _case(rng, rows, n, dim, fdtype, np.int64, unique=False)
    dst0 = np.zeros((n + 3, dim), fdtype)
    want = oracle_mod.rows_gather(src, si, dst0.copy(), None)
    dst = torch.from_numpy(dst0.copy()).cuda()
    E.cudaFetch2(torch.from_numpy(src).cuda(), torch.from_numpy(si).cuda(), dst, mover=E.MOVER_BULK)
    assert np.array_equal(dst.cpu().numpy(), want)
    # scatter
    di = rng.permutation(rows)[:n].astype(np.int64)
    payload = rng.standard_normal((n, dim)).astype(fdtype)
    table0 = rng.standard_normal((rows, dim)).astype(fdtype)
    want = oracle_mod.rows_scatter(payload, table0.copy(), di)
    table = torch.from_numpy(table0.copy()).cuda()
    E.cudaSet(torch.from_numpy(payload).cuda(), table, torch.from_numpy(di).cuda(), mover=E.MOVER_BULK)
    assert np.array_equal(table.cpu().numpy(), want)


def test_bulk_rejects_unaligned(cuda_lib):
    from hades_b200 import EmbCacheLib as E

    src = torch.zeros((10, 3), device="cuda")
    dst = torch.zeros((4, 3), device="cuda")
    with pytest.raises(RuntimeError, match="bulk"):
        E.cudaFetch2(src, torch.arange(4, device="cuda"), dst, mover=E.MOVER_BULK)


@pytest.mark.parametrize("dim", DIMS)
def test_set_and_combine(cuda_lib, oracle_mod, dim):
    from hades_b200 import EmbCacheLib as E

    rng = np.random.default_rng(dim + 100)
    payload, di = _case(rng, 30_000, 8_000, dim, np.float32, np.int64)
    payload = payload[:8_000]
    table0 = rng.standard_normal((30_000, dim)).astype(np.float32)
    want = oracle_mod.rows_scatter(payload, table0.copy(), di)
    for fn in (E.cudaSet, E.cudaCombine):
        table = torch.from_numpy(table0.copy()).cuda()
        fn(torch.from_numpy(payload).cuda(), table, torch.from_numpy(di).cuda())
        assert np.array_equal(table.cpu().numpy(), want)


def test_1d_fetch_and_set(cuda_lib, oracle_mod):
    from hades_b200 import EmbCacheLib as E

    rng = np.random.default_rng(11)
    src = rng.standard_normal(50_000).astype(np.float32)
    idx = rng.permutation(50_000)[:7_777].astype(np.int64)
    dst = torch.zeros(7_777, device="cuda")
    E.cudaFetch2(torch.from_numpy(src).cuda(), torch.from_numpy(idx).cuda(), dst)
    assert np.array_equal(dst.cpu().numpy(), src[idx])
    table = torch.from_numpy(src.copy()).cuda()
    vals = rng.standard_normal(7_777).astype(np.float32)
    E.cudaSet(torch.from_numpy(vals).cuda(), table, torch.from_numpy(idx).cuda())
    want = src.copy()
    want[idx] = vals
    assert np.array_equal(table.cpu().numpy(), want)


@pytest.mark.parametrize("dim", [1, 3, 128])
@pytest.mark.parametrize("idtype", [np.int64, np.int32])
def test_cached_fetch_and_set(cuda_lib, oracle_mod, dim, idtype):
    """test/test_cached_fetch.py / test_cached_set.py: half of the table cached, dense map."""
    from hades_b200 import EmbCacheLib as E

    rng = np.random.default_rng(dim + 7)
    rows, cached_n, n = 40_000, 20_000, 10_000
    shape = (rows,) if dim == 1 else (rows, dim)
    backing = rng.standard_normal(shape).astype(np.float32)
    cached_idx = rng.permutation(rows)[:cached_n]
    index_map = np.full(rows, -1, dtype=idtype)
    index_map[cached_idx] = np.arange(cached_n, dtype=idtype)
    cached = backing[cached_idx] + 1.0  # differ from the backing copy to see the routing
    index = rng.permutation(rows)[:n].astype(idtype)
    dst0 = np.zeros((n,) if dim == 1 else (n, dim), np.float32)
    want, hit = oracle_mod.rows_gather_cached(backing, cached, index, index_map, dst0.copy())
    dst = torch.from_numpy(dst0.copy()).cuda()
    found = torch.zeros(n, dtype=torch.bool, device="cuda")
    E.cudaFetchWithCache2(torch.from_numpy(backing).cuda(), torch.from_numpy(cached).cuda(),
                          torch.from_numpy(index).cuda(), torch.from_numpy(index_map).cuda(), dst, found)
    assert np.array_equal(dst.cpu().numpy(), want)
    assert np.array_equal(found.cpu().numpy(), hit)
    # cached set
    payload = rng.standard_normal(dst0.shape).astype(np.float32)
    wb, wc = oracle_mod.rows_scatter_cached(payload, backing.copy(), cached.copy(), index, index_map)
    b = torch.from_numpy(backing.copy()).cuda()
    c = torch.from_numpy(cached.copy()).cuda()
    E.cudaSetWithCache(torch.from_numpy(payload).cuda(), b, c, torch.from_numpy(index).cuda(),
                       torch.from_numpy(index_map).cuda())
    assert np.array_equal(b.cpu().numpy(), wb) and np.array_equal(c.cpu().numpy(), wc)


def test_pinned_host_source(cuda_lib, oracle_mod):
    """The reference's UVA use: the source table stays in pinned host memory."""
    from hades_b200 import EmbCacheLib as E

    rng = np.random.default_rng(2)
    src = torch.from_numpy(rng.standard_normal((5000, 64)).astype(np.float32))
    E.cudaPin(src)
    try:
        idx = torch.from_numpy(rng.permutation(5000)[:1000]).cuda()
        dst = torch.zeros((1000, 64), device="cuda")
        E.cudaFetch2(src, idx, dst)
        torch.cuda.synchronize()
        assert torch.equal(dst.cpu(), src[idx.cpu()])
    finally:
        E.cudaUnpin(src)


def test_accumulate(cuda_lib, oracle_mod):
    from hades_b200 import EmbCacheLib as E

    rng = np.random.default_rng(9)
    for dim in (3, 64, 128):
        table0 = rng.standard_normal((20_000, dim)).astype(np.float32)
        cnt0 = rng.integers(0, 5, 20_000).astype(np.int32)
        idx = rng.permutation(20_000)[:6_000].astype(np.int64)
        g = rng.standard_normal((6_000, dim)).astype(np.float32)
        want_cnt = cnt0.copy()
        want = oracle_mod.rows_accumulate(g, table0.copy(), idx, want_cnt)
        t = torch.from_numpy(table0.copy()).cuda()
        c = torch.from_numpy(cnt0.copy()).cuda()
        E.cudaAccumulate(torch.from_numpy(g).cuda(), t, torch.from_numpy(idx).cuda(), c)
        assert np.array_equal(t.cpu().numpy(), want)  # one add per element: exact
        assert np.array_equal(c.cpu().numpy(), want_cnt)


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("mover", [1, 2])
@pytest.mark.parametrize("dim", [4, 64, 128])
def test_lookup_fetch_fused(cuda_lib, oracle_mod, mode, mover, dim):
    """Configuration-1 shapes scaled down: Zipf queries with duplicates against a hot cache;
    slots and found masks bit-exact, rows bit-exact, for every lookup mode and mover."""
    from hades_b200 import EmbCacheLib as E, synth

    cfg = synth.scaled(synth.CONFIG1, 0.1)
    rng = synth.rng_for(1, 0)
    table = synth.normal_rows(rng, cfg.table_rows, dim, cfg.table_sigma)
    ix = E.IndexCache(cfg.cache_entries, f"lf{mode}{mover}{dim}", True, False, lookup_mode=mode)
    ora = oracle_mod.OracleIndex(cfg.cache_entries)
    hot = synth.hot_ids(cfg.table_rows, cfg.cache_entries)
    locs = ix.add(torch.from_numpy(hot)).numpy()
    assert np.array_equal(locs, ora.add(hot))
    cache = np.zeros((ix.get_capacity(), dim), np.float32)
    cache[locs[locs >= 0]] = table[hot[locs >= 0]] * 2.0
    q = synth.ZipfSampler(cfg.table_rows, cfg.zipf_s).ids(rng, cfg.batch + 5)
    out0 = np.full((q.size, dim), -7.0, np.float32)
    want_locs, want_hit = oracle_mod.lookup_fetch(ora, q, cache, table, out0)
    out, locs_g, found = E.cudaLookupFetch(ix, torch.from_numpy(q).cuda(), torch.from_numpy(cache).cuda(),
                                           torch.from_numpy(table).cuda(), mover=mover)
    assert np.array_equal(locs_g.cpu().numpy(), want_locs)
    assert np.array_equal(found.cpu().numpy(), want_hit)
    assert np.array_equal(out.cpu().numpy(), out0)
    assert 0 < want_hit.sum() < q.size
    # without a backing table a miss leaves the output row untouched
    out1 = np.full((q.size, dim), -7.0, np.float32)
    oracle_mod.lookup_fetch(ora, q, cache, None, out1)
    pre = torch.full((q.size, dim), -7.0, device="cuda")
    E.cudaLookupFetch(ix, torch.from_numpy(q).cuda(), torch.from_numpy(cache).cuda(), None,
                      out_rows=pre, mover=mover)
    assert np.array_equal(pre.cpu().numpy(), out1)


def test_shape_errors_raise_like_check():
    from hades_b200 import EmbCacheLib as E

    a = torch.zeros((4, 3))
    b = torch.zeros((4, 5))
    i = torch.zeros(4, dtype=torch.int64)
    with pytest.raises(RuntimeError, match="Check failed"):
        E.cudaFetch(a, i, b, i)
    with pytest.raises(RuntimeError, match="Check failed"):
        E.cudaSet(a, b, i)
    with pytest.raises(RuntimeError, match="float or double"):
        E.cudaFetch2(a.int(), i, a.int())
