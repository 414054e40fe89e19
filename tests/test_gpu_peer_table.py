"""hb_peer_table_*: a table sharded by id % world whose shards all GPUs read.  Here the shards of
four "ranks" live on one GPU (pointers handed over with set_peer), which exercises the owner
arithmetic and the fused lookup + fetch with sharded misses against the oracle."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _tables(num_rows, dim, world, dtype=torch.float32):
    from hades_b200.peer_table import PeerTable

    tabs = [PeerTable(num_rows, dim, r, world, dtype, connect=False) for r in range(world)]
    for a in tabs:
        for b in tabs:
            if a is not b:
                a.set_peer(b.rank, b.weight)
    return tabs


@pytest.mark.parametrize("world,num_rows,dim", [(1, 1000, 128), (4, 100_003, 128), (3, 5000, 32), (4, 6, 4)])
def test_gather_reads_the_owner(cuda_lib, world, num_rows, dim):
    tabs = _tables(num_rows, dim, world)
    full = torch.randn(num_rows, dim, device="cuda")
    for t in tabs:
        assert t.rows_local == len(range(t.rank, num_rows, world))
        t.weight.copy_(full[t.rank::world])
    g = torch.Generator(device="cuda").manual_seed(5)
    ids = torch.randint(0, num_rows, (20_011,), device="cuda", generator=g)
    for t in tabs:
        assert torch.equal(t.gather(ids), full[ids])
    # device-side count: rows beyond it stay untouched
    out = torch.full((ids.numel(), dim), -7.0, device="cuda")
    n_dev = torch.tensor([1234], dtype=torch.int64, device="cuda")
    tabs[0].gather(ids, n_dev, out)
    assert torch.equal(out[:1234], full[ids[:1234]]) and bool((out[1234:] == -7.0).all())
    assert tabs[0].gather(ids[:0]).shape == (0, dim)


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("dim", [128, 64, 12])
def test_lookup_fetch_sharded_matches_oracle(cuda_lib, oracle_mod, mode, dim):
    from hades_b200 import EmbCacheLib as E

    world, num_rows, entries = 4, 50_000, 6_000
    rng = np.random.default_rng(11)
    full = rng.standard_normal((num_rows, dim)).astype(np.float32)
    tabs = _tables(num_rows, dim, world)
    for t in tabs:
        t.weight.copy_(torch.from_numpy(full[t.rank::world]))
    fill = rng.permutation(num_rows)[:entries].astype(np.int64)
    ox = oracle_mod.OracleIndex(entries)
    locs0 = ox.add(fill)
    cache = np.zeros((ox.get_capacity(), dim), np.float32)
    ok = locs0 >= 0
    cache[locs0[ok]] = rng.standard_normal((int(ok.sum()), dim)).astype(np.float32)  # differs from the table
    index = E.IndexCache(entries, f"pt_{mode}_{dim}", True, False, lookup_mode=mode)
    assert np.array_equal(index.cuda_add(torch.from_numpy(fill).cuda()).cpu().numpy(), locs0)
    ids = rng.integers(0, num_rows, 33_333).astype(np.int64)
    want = np.full((ids.size, dim), 3.0, np.float32)
    wl, wf = oracle_mod.lookup_fetch(ox, ids, cache, full, want)
    for t in tabs[:2]:
        out = torch.full((ids.size, dim), 3.0, device="cuda")
        rows, locs, found = t.lookup_fetch(index, torch.from_numpy(ids).cuda(), torch.from_numpy(cache).cuda(), out, mode)
        assert np.array_equal(locs.cpu().numpy(), wl) and np.array_equal(found.cpu().numpy(), wf)
        assert np.array_equal(rows.cpu().numpy(), want)


def test_unmapped_peer_is_an_error(cuda_lib):
    from hades_b200.peer_table import PeerTable

    t = PeerTable(100, 16, 0, 2, connect=False)
    with pytest.raises(RuntimeError, match="not mapped"):
        t.gather(torch.zeros(4, dtype=torch.int64, device="cuda"))
    with pytest.raises(RuntimeError, match="multiple of 16"):
        PeerTable(100, 3, 0, 1)
