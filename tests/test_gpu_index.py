"""Cache index on the GPU (through the C ABI) against the oracle and the golden vectors:
slots, found masks, valid counts, enumeration order and the complete state including the
LRU counters must be bit-exact."""
import numpy as np
import pytest
import torch

from .conftest import GOLDEN
from .test_oracle_pins import replay

pytestmark = pytest.mark.gpu


class GpuIndexAdapter:
    """EmbCacheLib.IndexCache with numpy in/out, so that the golden replay reads like the
    reference's own usage (CPU tensors in, CPU tensors out)."""

    def __init__(self, cache_size, mode):
        from hades_b200 import EmbCacheLib

        self.ix = EmbCacheLib.IndexCache(cache_size, f"t{id(self)}", True, False, lookup_mode=mode)

    def add(self, ids):
        return self.ix.add(torch.from_numpy(np.ascontiguousarray(ids))).numpy()

    def lookup(self, ids):
        return self.ix.lookup(torch.from_numpy(np.ascontiguousarray(ids))).numpy()

    def reset(self, ids):
        self.ix.reset(torch.from_numpy(np.ascontiguousarray(ids)))

    def get_valid_entries_num(self):
        return self.ix.get_valid_entries_num()

    def getall(self, n):
        a, b = self.ix.getall(n)
        return a.numpy(), b.numpy()


def _eq(a, b, where):
    a, b = np.asarray(a), np.asarray(b)
    assert a.shape == b.shape, where
    bad = np.nonzero(a != b)[0]
    assert bad.size == 0, (where, bad[:5], a[bad[:5]], b[bad[:5]])


@pytest.mark.parametrize("mode", [0, 1])
def test_golden_replay(cuda_lib, mode):
    golden = np.load(GOLDEN / "index_golden.npz")
    for i in range(int(golden["num_scenarios"])):
        ix = GpuIndexAdapter(int(golden[f"s{i}_cache_size"]), mode)
        assert ix.ix.get_capacity() == int(golden[f"s{i}_capacity"])
        assert ix.ix.get_size() == int(golden[f"s{i}_capacity"])
        assert ix.ix.get_space() == int(golden[f"s{i}_space"])
        replay(ix, golden, i, _eq)


def test_known_answers(cuda_lib):
    ix = GpuIndexAdapter(30, 0)
    assert ix.add(np.arange(10)).tolist() == [7, 15, 23, 31, 6, 14, 22, 30, 5, 13]
    assert ix.lookup(np.array([0, 1, 4, 5, 8, 9, 11, 40])).tolist() == [7, 15, 6, 14, 5, 13, -1, -1]
    assert ix.add(np.arange(0, 41, 4)).tolist() == [7, 6, 5, 4, 3, 2, 1, 0, 7, 6, -1]


@pytest.mark.parametrize("cache_size,id_range,batch", [(8, 40, 64), (1000, 3000, 5000),
                                                        (100_000, 1_000_000, 65_536)])
def test_state_matches_oracle(cuda_lib, oracle_mod, cache_size, id_range, batch):
    """Random add / lookup / reset rounds with duplicates inside a batch; after every round
    the exported line ids and LRU counters equal the oracle's."""
    rng = np.random.default_rng(cache_size)
    gpu = GpuIndexAdapter(cache_size, 0)
    ora = oracle_mod.OracleIndex(cache_size)
    for step in range(12):
        n = int(rng.integers(1, batch + 1))
        ids = rng.integers(0, id_range, n, dtype=np.int64)
        if step % 3 == 0:
            ids[: n // 4] = ids[0]  # a hot id, many duplicates
        kind = ["add", "lookup", "lookup", "add", "reset", "lookup"][step % 6]
        if kind == "add":
            _eq(gpu.add(ids), ora.add(ids), (step, kind))
        elif kind == "lookup":
            _eq(gpu.lookup(ids), ora.lookup(ids, touch=True), (step, kind))
        else:
            gpu.reset(ids)
            ora.reset(ids)
        gi, gl = gpu.ix.export_state()
        oi, ol = ora.export()
        _eq(gi.cpu().numpy(), oi, (step, kind, "line ids"))
        _eq(gl.cpu().numpy(), ol, (step, kind, "lru"))


@pytest.mark.parametrize("cache_size", [8, 100, 20_000, 300_000])
def test_lookup_modes_agree(cuda_lib, oracle_mod, cache_size):
    """The sorted-view search and the set-associative probe return the same slots and found
    masks as the oracle, for hits, misses, negative ids and an empty index."""
    from hades_b200 import EmbCacheLib

    rng = np.random.default_rng(cache_size + 1)
    ix = EmbCacheLib.IndexCache(cache_size, f"modes{cache_size}", True, False)
    ora = oracle_mod.OracleIndex(cache_size)
    q = torch.from_numpy(rng.integers(0, cache_size * 4, 10_000, dtype=np.int64)).cuda()
    for mode in (0, 1):  # empty index
        locs, found = ix.cuda_lookup_found(q, mode)
        assert (locs == -1).all() and not found.any()
    ids = rng.integers(0, cache_size * 4, cache_size * 2, dtype=np.int64)
    _eq(ix.add(torch.from_numpy(ids)).numpy(), ora.add(ids), "add")
    qn = rng.integers(-5, cache_size * 4, 50_001, dtype=np.int64)
    want = ora.lookup(qn, touch=False)
    for mode in (0, 1):
        locs, found = ix.cuda_lookup_found(torch.from_numpy(qn).cuda(), mode)
        _eq(locs.cpu().numpy(), want, ("mode", mode))
        _eq(found.cpu().numpy(), want >= 0, ("found", mode))
    # the view follows later changes
    ix.reset(torch.from_numpy(ids[:100]))
    ora.reset(ids[:100])
    want = ora.lookup(qn, touch=False)
    locs, _ = ix.cuda_lookup_found(torch.from_numpy(qn).cuda(), 1)
    _eq(locs.cpu().numpy(), want, "after reset")


def test_open_by_name_and_empty_batches(cuda_lib):
    from hades_b200 import EmbCacheLib

    a = EmbCacheLib.IndexCache(64, "shared_name", True, False)
    b = EmbCacheLib.IndexCache(64, "shared_name", False, False)
    a.add(torch.arange(10))
    assert b.get_valid_entries_num() == 10
    assert b.lookup(torch.arange(3)).tolist() == a.lookup(torch.arange(3)).tolist()
    assert a.add(torch.empty(0, dtype=torch.int64)).numel() == 0
    assert a.lookup(torch.empty(0, dtype=torch.int64)).numel() == 0
    a.reset(torch.empty(0, dtype=torch.int64))
    with pytest.raises(RuntimeError):
        EmbCacheLib.IndexCache(64, "never_created", False, False)


@pytest.mark.parametrize("cache_size,id_range,n", [(64, 300, 5000), (20_000, 60_000, 200_000)])
def test_touch_lru_from_runs(cuda_lib, oracle_mod, cache_size, id_range, n):
    """The run-based LRU ageing (grouping taken from the aggregation's sort) leaves the same
    counters as the sequential rule, for batches with heavy duplication and for unique ids."""
    from hades_b200 import EmbCacheLib as E

    rng = np.random.default_rng(cache_size + n)
    ix = E.IndexCache(cache_size, f"runs{cache_size}", True, False)
    ora = oracle_mod.OracleIndex(cache_size)
    seed_ids = rng.integers(0, id_range, cache_size * 2, dtype=np.int64)
    assert np.array_equal(ix.add(torch.from_numpy(seed_ids)).numpy(), ora.add(seed_ids))
    for rnd in range(3):
        q = rng.integers(0, id_range, n, dtype=np.int64)
        q[: n // 3] = q[0]  # one very hot id
        rng.shuffle(q)
        want = ora.lookup(q, touch=True)
        qd = torch.from_numpy(q).cuda()
        locs = ix.cudalookup(qd)
        assert np.array_equal(locs.cpu().numpy(), want)
        g = torch.zeros((n, 4), device="cuda")
        *_, runs = E.cudaUniqueSegSum(qd, g, id_bits=32, sync=False, want_runs=True)
        ix.cuda_touch_lru_runs(locs, runs)
        assert np.array_equal(ix.export_state()[1].cpu().numpy(), ora.export()[1]), rnd
        # unique ids: every position its own run, with a device-side count
        uq = np.unique(rng.integers(0, id_range, n // 4, dtype=np.int64))
        rng.shuffle(uq)
        want = ora.lookup(uq, touch=True)
        padded = np.concatenate([uq, np.full(100, 7, dtype=np.int64)])  # ignored tail
        locs = ix.cudalookup(torch.from_numpy(padded).cuda())
        ix.cuda_touch_lru_runs(locs, None, torch.tensor([uq.size], device="cuda"))
        assert np.array_equal(locs.cpu().numpy()[: uq.size], want)
        assert np.array_equal(ix.export_state()[1].cpu().numpy(), ora.export()[1]), rnd
