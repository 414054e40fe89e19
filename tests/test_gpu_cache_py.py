"""The Python mirrors of python/EmbCache/cache.py: LocalCache and the hotness-ranked optimiser
state cache (cached fetch / cached set through a dense index map, pinned-host backing)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_local_cache_wrapper(cuda_lib, oracle_mod):
    from hades_b200.cache import LocalCache

    c = LocalCache("lc_test", 1000, create=True)
    ora = oracle_mod.OracleIndex(1000)
    ids = np.random.default_rng(1).integers(0, 5000, 3000, dtype=np.int64)
    assert np.array_equal(c.add(torch.from_numpy(ids)).numpy(), ora.add(ids))
    assert np.array_equal(c.lookup(torch.from_numpy(ids)).numpy(), ora.lookup(ids))
    assert np.array_equal(c.cudalookup(torch.from_numpy(ids).cuda()).cpu().numpy(), ora.lookup(ids, touch=False))
    assert c.get_num_entries() == 1000
    c.reset(torch.from_numpy(ids[:10]))
    ora.reset(ids[:10])
    assert np.array_equal(c.lookup(torch.from_numpy(ids)).numpy(), ora.lookup(ids))


@pytest.mark.parametrize("backing", ["pinned_host", "device"])
def test_state_cache_fetch_set(cuda_lib, backing):
    """create_cache picks the hottest owned ids (cache.py:149-171); __getitem__/__setitem__ route
    rows to the HBM copy or the backing tensors exactly like the dense-map kernels."""
    from hades_b200.cache import LocalSparseAdamStateCache

    rng = np.random.default_rng(3)
    n, dim, start, world, rank = 30_000, 32, 1000, 2, 1
    step = torch.from_numpy(rng.random(n).astype(np.float32))
    mem = torch.from_numpy(rng.standard_normal((n, dim)).astype(np.float32))
    power = torch.from_numpy(rng.random((n, dim)).astype(np.float32))
    if backing == "device":
        step, mem, power = step.cuda(), mem.cuda(), power.cuda()
    hotness = torch.from_numpy(rng.random(start + n).astype(np.float32))
    ref = [t.clone().cpu().numpy() for t in (step, mem, power)]
    sc = LocalSparseAdamStateCache(step, mem, power, hotness, start, rank, world, count_hit=True)
    item = 4 + 8 * dim
    used = sc.create_cache(4000 * item + 8 * n)
    assert sc.has_cached and used == 4000 * item + 8 * n
    # the cached set = the 4000 hottest among ids with id % world == rank
    gids = np.arange(n) + start
    owned = gids[gids % world == rank]
    want = owned[np.argsort(-hotness.numpy()[owned], kind="stable")][:4000] - start
    got = torch.nonzero(sc.idx_map != -1).flatten().cpu().numpy()
    assert np.array_equal(np.sort(want), got)
    assert np.array_equal(sc.idx_map.cpu().numpy()[want], np.arange(4000))
    # fetch
    q = torch.from_numpy(rng.permutation(n)[:5000] + start).cuda()
    s, m, p = sc[q]
    qi = q.cpu().numpy() - start
    assert np.array_equal(s.cpu().numpy(), ref[0][qi])
    assert np.array_equal(m.cpu().numpy(), ref[1][qi]) and np.array_equal(p.cpu().numpy(), ref[2][qi])
    # set, then read back through the cache and check where the rows went
    ns = torch.from_numpy(rng.random(5000).astype(np.float32)).cuda()
    nm = torch.from_numpy(rng.standard_normal((5000, dim)).astype(np.float32)).cuda()
    npow = torch.from_numpy(rng.random((5000, dim)).astype(np.float32)).cuda()
    sc[q] = (ns, nm, npow)
    torch.cuda.synchronize()
    s2, m2, p2 = sc[q]
    assert torch.equal(s2, ns) and torch.equal(m2, nm) and torch.equal(p2, npow)
    cached_mask = sc.idx_map.cpu().numpy()[qi] != -1
    backing_mem = sc.local_state[1].cpu().numpy()
    # rows of cached ids stay untouched in the backing tensor, the others are written there
    assert np.array_equal(backing_mem[qi[cached_mask]], ref[1][qi[cached_mask]])
    assert np.array_equal(backing_mem[qi[~cached_mask]], nm.cpu().numpy()[~cached_mask])
    assert 0 < sc.get_hit_rate() < 1
    del sc
