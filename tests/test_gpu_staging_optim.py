"""Cold-gradient staging table (insert / accumulate / flush) and the sparse optimiser updates
against the oracle's restatement of python/EmbCache/server.py and sparse_optim.py."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

RTOL = 1e-5


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("dim", [3, 64, 128])
def test_cold_cache_rounds(cuda_lib, oracle_mod, mode, dim):
    """Several server iterations: flush, insert uncached rows, accumulate remote and local cold
    gradients.  Ids / counts / slot state bit-exact; rows exact too (every slot receives the
    same fp32 additions in the same order as the oracle)."""
    from hades_b200.cold_cache import ColdCache

    rng = np.random.default_rng(dim * 10 + mode)
    num_nodes, entries, clients, local_nodes = 20_000, 2_000, 4, 3_000
    hotness = rng.random(num_nodes).astype(np.float32) * 0.2
    thr = oracle_mod.flush_thresholds(hotness)
    thr = np.minimum(thr, 3).astype(np.int32)  # short periods so that rows do flush
    cc = ColdCache(f"cc{mode}{dim}", entries, dim, threshold=_t(thr), cnt_threshold=3, num_clients=clients,
                   local_nodes=local_nodes, local_start=1000, lookup_mode=mode)
    ox = oracle_mod.OracleIndex(entries)
    slots = ox.get_capacity()
    ocache = np.zeros((slots, dim), np.float32)
    orem = oracle_mod.OracleStaging(slots, dim, cnt_threshold=3)
    oloc = oracle_mod.OracleStaging(local_nodes, dim, cnt_threshold=3, iter_threshold=thr[1000:1000 + local_nodes])
    for it in range(7):
        # step 0: flush
        gi, gr, gc, gcounts = cc.flush_remote()
        wi, wr, wc, wcounts = orem.flush(ox, clients)
        assert np.array_equal(gcounts.cpu().numpy(), wcounts), it
        assert np.array_equal(gi.cpu().numpy(), wi) and np.array_equal(gc.cpu().numpy(), wc), it
        assert np.array_equal(gr.cpu().numpy(), wr), it
        gi, gr, gc, gcounts = cc.flush_local()
        wi, wr, wc, wcounts = oloc.flush(None, clients)
        assert np.array_equal(gcounts.cpu().numpy(), wcounts), it
        assert np.array_equal(gi.cpu().numpy(), wi) and np.array_equal(gr.cpu().numpy(), wr), it
        assert np.array_equal(gc.cpu().numpy(), wc), it
        # step 2: insert uncached embeddings
        new_ids = rng.integers(0, num_nodes, 900, dtype=np.int64)
        embs = rng.standard_normal((900, dim)).astype(np.float32)
        # duplicate ids inside a batch carry the same row
        uniq_rows = {}
        for k, i in enumerate(new_ids):
            uniq_rows.setdefault(int(i), embs[k])
            embs[k] = uniq_rows[int(i)]
        glocs = cc.insert(_t(new_ids), _t(embs))
        wlocs = orem.insert(ox, new_ids, embs, ocache)
        assert np.array_equal(glocs.cpu().numpy(), wlocs), it
        assert np.array_equal(cc.emb.cpu().numpy(), ocache), it
        # step 3: accumulate, two "clients", unique ids per message
        for c in range(2):
            ids = rng.permutation(num_nodes)[:1500].astype(np.int64)
            g = (rng.standard_normal((1500, dim)) * 1e-3).astype(np.float32)
            cc.accumulate_remote(_t(ids), _t(g))
            orem.accumulate_cached(ox, ids, g, thr, 1)
            lids = (1000 + rng.permutation(local_nodes)[:700]).astype(np.int64)
            lg = (rng.standard_normal((700, dim)) * 1e-3).astype(np.float32)
            cc.accumulate_local(_t(lids), _t(lg))
            oloc.accumulate_direct(lids, lg, 1000, 1)
        for name, gs, os_ in (("remote", cc.remote, orem), ("local", cc.local, oloc)):
            assert np.array_equal(gs.cnt.cpu().numpy(), os_.cnt), (it, name)
            assert np.array_equal(gs.idx.cpu().numpy(), os_.idx), (it, name)
            assert np.array_equal(gs.iter_count.cpu().numpy(), os_.iter_count), (it, name)
            assert np.array_equal(gs.iter_threshold.cpu().numpy(), os_.iter_threshold), (it, name)
            assert np.array_equal(gs.grad.cpu().numpy(), os_.grad), (it, name)
        gi, gl = cc.index.export_state()
        oi, ol = ox.export()
        assert np.array_equal(gi.cpu().numpy(), oi) and np.array_equal(gl.cpu().numpy(), ol), it
    assert int(cc.dropped.item()) > 0


@pytest.mark.parametrize("emb_dtype", [np.float32, np.float16])
@pytest.mark.parametrize("dim", [3, 64, 128])
def test_sparse_adam(cuda_lib, oracle_mod, emb_dtype, dim):
    """Three steps of SparseAdam on an owner shard (id % 4 == 1): state and embedding within
    1e-5 relative of the fp32 restatement (fp16 tables: within one fp16 rounding)."""
    from hades_b200.sparse_optim import ShardedEmbedding, SparseAdam

    rng = np.random.default_rng(dim)
    num, world, rank = 40_000, 4, 1
    emb = ShardedEmbedding(num, dim, rank, world, dtype=torch.float16 if emb_dtype == np.float16 else torch.float32)
    w0 = (rng.standard_normal((emb.rows, dim)) * 0.01).astype(emb_dtype)
    emb.weight.copy_(_t(w0))
    opt = SparseAdam(emb, lr=0.01)
    step = np.zeros(emb.rows, np.float32)
    mem = np.zeros((emb.rows, dim), np.float32)
    power = np.zeros((emb.rows, dim), np.float32)
    w = w0.copy()
    for it in range(3):
        local_rows = rng.permutation(emb.rows)[:3000]
        ids = (local_rows * world + rank).astype(np.int64)
        g = (rng.standard_normal((3000, dim)) * 1e-3).astype(np.float32)
        cnt = rng.integers(1, 5, 3000, dtype=np.int64) if it == 1 else None
        opt.update(_t(ids), _t(g), None if cnt is None else _t(cnt), is_unique=True)
        oracle_mod.sparse_adam_update(ids, g, step, mem, power, w, 0.01, cnt=cnt, id_offset=rank, id_stride=world)
        assert np.array_equal(opt.state_step.cpu().numpy(), step)
        # 1e-5 relative to the size of the operands: a sum of two terms of opposite sign can
        # cancel, so the bound is on |a| + |b| (gradients ~1e-3, updates ~lr = 1e-2), not on the result
        np.testing.assert_allclose(opt.state_mem.cpu().numpy(), mem, rtol=RTOL, atol=RTOL * 1e-3)
        np.testing.assert_allclose(opt.state_power.cpu().numpy(), power, rtol=RTOL, atol=RTOL * 1e-6)
        if emb_dtype == np.float32:
            np.testing.assert_allclose(emb.weight.cpu().numpy(), w, rtol=RTOL, atol=RTOL * 2e-2)
        else:
            got = emb.weight.float().cpu().numpy()
            assert np.abs(got - w.astype(np.float32)).max() <= 2e-5  # one fp16 ulp near 0.03
            w = emb.weight.cpu().numpy().copy()  # keep the two tables from drifting apart by roundings


def test_sparse_adam_not_unique_uses_mean(cuda_lib, oracle_mod):
    from hades_b200.sparse_optim import ShardedEmbedding, SparseAdam

    rng = np.random.default_rng(1)
    emb = ShardedEmbedding(5000, 32)
    opt = SparseAdam(emb, lr=0.05)
    ids = rng.integers(0, 5000, 20_000, dtype=np.int64)
    g = (rng.standard_normal((20_000, 32)) * 1e-3).astype(np.float32)
    opt.update(_t(ids), _t(g), id_bits=16)
    u, mean, _ = oracle_mod.unique_grads(ids, g)
    step = np.zeros(5000, np.float32)
    mem = np.zeros((5000, 32), np.float32)
    power = np.zeros((5000, 32), np.float32)
    w = np.zeros((5000, 32), np.float32)
    oracle_mod.sparse_adam_update(u, mean, step, mem, power, w, 0.05)
    assert np.array_equal(opt.state_step.cpu().numpy(), step)
    # the first Adam step is lr * g / (|g| + eps): where the duplicates of an id nearly cancel,
    # the rounding of the mean is amplified by 1/|g|, so the bound is relative to lr
    np.testing.assert_allclose(emb.weight.cpu().numpy(), w, rtol=1e-4, atol=0.05 * 1e-3)


@pytest.mark.parametrize("emb_dtype", [np.float32, np.float16])
def test_sparse_adagrad(cuda_lib, oracle_mod, emb_dtype):
    """Configuration-4 shapes scaled down: 64-dim fp32 gradients, fp16 table sharded id % 8."""
    from hades_b200.sparse_optim import ShardedEmbedding, SparseAdagrad

    rng = np.random.default_rng(3)
    num, world, rank, dim = 80_000, 8, 5, 64
    emb = ShardedEmbedding(num, dim, rank, world, dtype=torch.float16 if emb_dtype == np.float16 else torch.float32)
    w = (rng.standard_normal((emb.rows, dim)) * 0.01).astype(emb_dtype)
    emb.weight.copy_(_t(w))
    opt = SparseAdagrad(emb, lr=0.01)
    ssum = np.zeros((emb.rows, dim), np.float32)
    for it in range(3):
        rows = rng.permutation(emb.rows)[:4000]
        ids = (rows * world + rank).astype(np.int64)
        g = (rng.standard_normal((4000, dim)) * 1e-3).astype(np.float32)
        opt.update(_t(ids), _t(g), is_unique=True)
        oracle_mod.sparse_adagrad_update(ids, g, ssum, w, 0.01, id_offset=rank, id_stride=world)
        np.testing.assert_allclose(opt.state_sum.cpu().numpy(), ssum, rtol=RTOL, atol=RTOL * 1e-6)
        if emb_dtype == np.float32:
            np.testing.assert_allclose(emb.weight.cpu().numpy(), w, rtol=RTOL, atol=RTOL * 2e-2)
        else:
            got = emb.weight.float().cpu().numpy()
            assert np.abs(got - w.astype(np.float32)).max() <= 2e-5
            w = emb.weight.cpu().numpy().copy()


@pytest.mark.parametrize("unique", [True, False])
def test_sparse_adam_state_through_the_tiered_cache(cuda_lib, unique):
    """Optimiser state in pinned host memory behind LocalSparseAdamStateCache (a third of the
    rows cached in HBM, python/EmbCache/cache.py:66-194 used at sparse_optim.py:621-668) against
    the all-HBM optimiser on the same updates: the same kernel runs on the same numbers, so
    state and weights are bit-exact."""
    from hades_b200.sparse_optim import ShardedEmbedding, SparseAdam

    rng = np.random.default_rng(11)
    num, dim, world, rank = 24_000, 32, 2, 1
    ea, eb = ShardedEmbedding(num, dim, rank, world), ShardedEmbedding(num, dim, rank, world)
    w0 = (rng.standard_normal((ea.rows, dim)) * 0.01).astype(np.float32)
    ea.weight.copy_(_t(w0))
    eb.weight.copy_(_t(w0))
    full = ea.rows * (4 + 8 * dim)
    hot = torch.from_numpy(rng.random(ea.rows).astype(np.float32))
    a = SparseAdam(ea, lr=0.01)
    b = SparseAdam(eb, lr=0.01, state_budget_bytes=full // 3, hotness=hot)
    assert a.state_cache is None and b.state_cache is not None and b.state_cache.has_cached
    assert not b.state_mem.is_cuda and b.state_mem.is_pinned()
    cached_rows = int((b.state_cache.idx_map != -1).sum().item())
    assert 0 < cached_rows < ea.rows
    for it in range(4):
        if unique:
            ids = (rng.permutation(ea.rows)[:3000] * world + rank).astype(np.int64)
        else:
            ids = (rng.integers(0, ea.rows, 5000) * world + rank).astype(np.int64)
        g = (rng.standard_normal((ids.size, dim)) * 1e-3).astype(np.float32)
        cnt = rng.integers(1, 5, ids.size, dtype=np.int64) if it % 2 else None
        for opt in (a, b):
            opt.update(_t(ids), _t(g), None if cnt is None else _t(cnt), is_unique=unique, id_bits=20)
        for x, y in zip(a.full_state(), b.full_state()):
            assert torch.equal(x, y), it
        assert torch.equal(ea.weight, eb.weight), it
    # the backing tensors hold the rows that are not cached, the HBM copy the others
    idx_map = b.state_cache.idx_map.cpu()
    uncached = torch.nonzero(idx_map == -1).flatten()
    assert torch.equal(b.state_mem[uncached], a.state_mem.cpu()[uncached])
