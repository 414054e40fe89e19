"""Host-side logic that needs no GPU: argument checks of the EmbCacheLib mirror (they raise like
the reference's CHECKs before any CUDA work), the named shared-memory helpers, and the seeded
synthetic generators."""
import os

import numpy as np
import pytest
import torch


def test_shape_and_dtype_checks_raise_without_gpu():
    from hades_b200 import EmbCacheLib as E

    a, b = torch.zeros((4, 3)), torch.zeros((4, 5))
    i = torch.zeros(4, dtype=torch.int64)
    with pytest.raises(RuntimeError, match="Check failed"):
        E.cudaFetch(a, i, b, i)
    with pytest.raises(RuntimeError, match="Check failed"):
        E.cudaSet(a, b, i)
    with pytest.raises(RuntimeError, match="Check failed"):
        E.cudaCombine(a, b, i)
    with pytest.raises(RuntimeError, match="float or double"):
        E.cudaFetch2(a.int(), i, a.int())
    with pytest.raises(RuntimeError, match="Check failed"):
        E.cudaFetchWithCache2(a, b, i, i, a)
    with pytest.raises(RuntimeError, match="pinned host memory"):
        E.cudaFetch2(a, i, a.clone())  # unpinned host tensors are not reachable from the device


def test_shared_memory_round_trip():
    from hades_b200 import EmbCacheLib as E

    name = f"hades_b200_test_{os.getpid()}"
    ptr, fd = E.create_shared_mem(name, 4096, pin_memory=False)
    try:
        t = E.open_shared_tensor(ptr, torch.float32, (16, 8))
        t[:] = torch.arange(128, dtype=torch.float32).view(16, 8)
        ptr2, fd2 = E.open_shared_mem(name, 4096, pin_memory=False)
        t2 = E.open_shared_tensor(ptr2, torch.float32, (16, 8))
        assert torch.equal(t, t2) and ptr != ptr2
        t2[3, 4] = -1.0
        assert t[3, 4] == -1.0
        del t2
        E._SHM.pop(ptr2)[0]  # drop the second mapping's bookkeeping; unlink happens below
        os.close(fd2)
    finally:
        del t
        E.release_shared_mem(name, 4096, ptr, fd, pin_memory=False)
    assert not os.path.exists("/dev/shm/" + name)
    with pytest.raises(RuntimeError, match="fail to open"):
        E.open_shared_mem(name, 4096, pin_memory=False)


def test_synthetic_generators_are_seeded_and_sane():
    from hades_b200 import synth

    perm = synth.rank_to_id(np.arange(100_000), 100_000)
    assert np.array_equal(np.sort(perm), np.arange(100_000))  # a permutation
    s = synth.ZipfSampler(1_000_000, 1.1)
    a = s.ids(synth.rng_for(1, 0), 65_536)
    b = s.ids(synth.rng_for(1, 0), 65_536)
    c = s.ids(synth.rng_for(1, 1), 65_536)
    assert np.array_equal(a, b) and not np.array_equal(a, c)
    st = synth.stream_stats(a)
    assert 0.3 < st["duplicate_fraction"] < 0.95 and a.min() >= 0 and a.max() < 1_000_000
    u = s.unique_ids(synth.rng_for(4, 0), 10_000)
    assert np.unique(u).size == 10_000
    hot = synth.hot_ids(1_000_000, 100)
    assert np.array_equal(hot, synth.rank_to_id(np.arange(100), 1_000_000))
    rows = synth.normal_rows(synth.rng_for(1, 0), 1000, 128, 0.01)
    assert rows.dtype == np.float32 and abs(float(rows.std()) - 0.01) < 1e-3
    small = synth.scaled(synth.CONFIG2, 0.01)
    assert small.table_rows == 200_000 and small.batch == 20_000 and small.dim == 128
    # a ranking cut to its head, spread over a larger id space (configuration 4's 2.4e8 ids)
    w = synth.ZipfSampler(5000, 1.1).unique_ids(synth.rng_for(4, 1), 2000, id_space=10**7)
    assert np.unique(w).size == 2000 and w.max() >= 5000 and w.max() < 10**7
    # the sampled 2-hop frontier of configuration 5, on a small R-MAT graph
    cfg = synth.scaled_rmat(synth.CONFIG5, 14, seeds=16)
    f1, f2 = synth.rmat_frontier(cfg, synth.rng_for(5, 0)), synth.rmat_frontier(cfg, synth.rng_for(5, 0))
    assert np.array_equal(f1, f2) and f1.size == cfg.batch == 16 * (1 + 25 + 250)
    assert f1.min() >= 0 and f1.max() < cfg.num_nodes
    # R-MAT favours vertices with few one-bits: the sampled neighbours have fewer than uniform ids would
    pop = np.array([bin(int(v)).count("1") for v in f1[16:]])
    assert pop.mean() < 0.5 * cfg.bits - 1.0


class _FakePath:
    """Stands in for EmbeddingPath: records what the layer and the optimiser hand over."""

    def __init__(self, nodes=50, dim=4):
        self.table = torch.arange(nodes * dim, dtype=torch.float32).reshape(nodes, dim)
        self.num_nodes, self.dim, self.row_dtype, self.device = nodes, dim, torch.float32, torch.device("cpu")
        self.shared, self.calls = None, []

    def forward(self, ids, out_rows=None):
        return self.table[ids].clone(), ids * 10, torch.ones_like(ids, dtype=torch.bool)

    def backward(self, ids, grads):
        self.calls.append((ids.clone(), grads.clone()))
        return "stats"


def test_layer_trace_and_optimizer_step_follow_the_reference_protocol():
    """zero_grad only arms the clearing of the trace at the next step (sparse_optim.py:350-354,
    468-470); a step hands the concatenated (ids, grads) of every traced call to the path."""
    from hades_b200.dist_emb import DistEmb, DistembSparseGradOptimizer

    path = _FakePath()
    layer = DistEmb(path)
    opt = DistembSparseGradOptimizer([layer.sparse_emb])
    a, b = torch.tensor([3, 5, 3]), torch.tensor([7])
    ha, hb = layer(a), layer(b)
    assert ha.requires_grad and ha.is_leaf and torch.equal(ha.detach(), path.table[a])
    opt.zero_grad()
    (ha.sum() * 2 + hb.sum() * 3).backward()
    opt.step()
    ids, grads = path.calls[-1]
    assert torch.equal(ids, torch.tensor([3, 5, 3, 7]))
    assert torch.equal(grads, torch.cat([torch.full((3, 4), 2.0), torch.full((1, 4), 3.0)]))
    assert layer.sparse_emb.trace == [] and opt.last_stats[layer.sparse_emb.name] == "stats"
    # without zero_grad the trace stays and the next step applies it again, as in the reference
    hc = layer(torch.tensor([1]))
    hc.sum().backward()
    opt.step()
    opt.step()
    assert len(path.calls) == 3 and torch.equal(path.calls[1][0], path.calls[2][0])
    # calls whose rows received no gradient are left out; no_grad calls are not traced
    opt.zero_grad()
    opt.step()
    with torch.no_grad():
        layer(torch.tensor([2]))
    assert layer.sparse_emb.trace == []
    layer(torch.tensor([4]))
    opt.step()
    assert len(path.calls) == 4


def test_presampled_hotness_class_table_and_cache_fill():
    from hades_b200 import hotness as H

    batches = [torch.tensor([1, 2, 2, 7]), torch.tensor([2, 7, 9]), torch.tensor([7]), torch.tensor([0, 7])]
    heat = H.presampling(batches, 12)
    want = torch.zeros(12)
    want[[0, 1, 9]] = 0.25
    want[2] = 0.5   # twice in the first batch still counts once for that batch
    want[7] = 1.0
    assert torch.equal(heat, want)
    local = torch.zeros(12, dtype=torch.bool)
    local[[0, 7]] = True
    table = H.class_table(heat, 0.5, local)
    assert table.dtype == torch.int8
    assert table.tolist() == [0, 2, 1, 2, 2, 2, 2, 0, 2, 2, 2, 2]
    assert H.class_table(heat, 0.5).tolist() == [2, 2, 1, 2, 2, 2, 2, 1, 2, 2, 2, 2]
    assert H.hottest_ids(heat, table == 2, 3).tolist() == [1, 9, 3]     # ties by ascending id
    thr = H.flush_thresholds(heat)                                       # ceil(1 / (0.001 + heat)) capped at 100
    assert thr[7].item() == 1 and thr[2].item() == 2 and thr[1].item() == 4 and thr[3].item() == 100
