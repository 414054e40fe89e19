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


def test_owner_serves_requested_rows_into_the_requesters_stages(cuda_lib):
    """hb_fetch_serve (the owner's half of a forward fetch in which the owners deliver): requests
    (id, stage row) in per-requester segments; every requested row of the owner's shard lands in
    the stage of its requester; a request for a row of another owner, beyond the table or beyond the
    stage is skipped and raises the status word."""
    from hades_b200 import _lib

    world, num_rows, dim, stage_rows, cap = 3, 10_001, 32, 64, 40
    tabs = _tables(num_rows, dim, world)
    stages = _tables(world * stage_rows, dim, world)
    full = torch.randn(num_rows, dim, device="cuda")
    for t in tabs:
        t.weight.copy_(full[t.rank::world])
    for owner in range(world):
        for s in stages:
            s.weight.fill_(-1.0)
        g = torch.Generator().manual_seed(10 + owner)
        req_ids = torch.full((world * cap,), -5, dtype=torch.int64)
        req_rows = torch.full((world * cap,), -5, dtype=torch.int64)
        counts = torch.zeros(world, dtype=torch.int64)
        want = {}
        for s in range(world):
            k = [0, 17, cap][s]  # an empty segment, a partly filled one, a full one
            owned = torch.arange(owner, num_rows, world)
            ids = owned[torch.randperm(owned.numel(), generator=g)[:k]]
            rows = torch.randperm(stage_rows, generator=g)[:k]
            req_ids[s * cap: s * cap + k], req_rows[s * cap: s * cap + k], counts[s] = ids, rows, k
            want[s] = (ids, rows)
        assert _lib.device_status() == 0
        tabs[owner].serve(stages[owner], req_ids.cuda(), req_rows.cuda(), counts.cuda(), cap)
        torch.cuda.synchronize()
        assert _lib.device_status() == 0
        for s in range(world):
            ids, rows = want[s]
            got = stages[s].weight
            assert torch.equal(got[rows.cuda()], full[ids.cuda()])
            untouched = torch.ones(stage_rows, dtype=torch.bool)
            untouched[rows] = False
            assert bool((got[untouched.cuda()] == -1.0).all())
    # bad requests: not this owner's id, no such id, no such stage row -> skipped, status word raised
    for s in stages:
        s.weight.fill_(-1.0)
    req_ids = torch.tensor([1, num_rows + 3 - (num_rows % 3), 0, 3], dtype=torch.int64)  # owner 0 is asked
    req_rows = torch.tensor([0, 1, stage_rows, 2], dtype=torch.int64)
    pad_i = torch.full((world * 4,), -5, dtype=torch.int64)
    pad_r = torch.full((world * 4,), -5, dtype=torch.int64)
    pad_i[4:8], pad_r[4:8] = req_ids, req_rows  # all from requester 1
    counts = torch.tensor([0, 4, 0], dtype=torch.int64)
    tabs[0].serve(stages[0], pad_i.cuda(), pad_r.cuda(), counts.cuda(), 4)
    torch.cuda.synchronize()
    assert _lib.device_status() == 1  # HB_ERR_INVALID, cleared by the read
    assert torch.equal(stages[1].weight[2], full[3])  # the one good request was served
    assert bool((stages[1].weight[:2] == -1.0).all()) and bool((stages[0].weight == -1.0).all())
