"""The whole per-step path (sorted forward fetch, LRU ageing, insertion of the cold misses, local
aggregation, hot/cold split, cold-cache accumulate, owner update, periodic flush) on one GPU against
the same steps composed from the oracle's functions (oracle/pipeline_oracle.py): slots, found
masks, index state, LRU counters and staging counters bit-exact, optimiser state and table within
1e-4 relative (they carry Adam updates whose first steps amplify roundings of nearly cancelling
means by 1 / |mean|)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _oracle_for(path, oracle_mod, cfg, **kw):
    from oracle.pipeline_oracle import PipelineOracle

    table = (path.table if path.table is not None else path.opt.emb.weight).cpu().numpy()
    return PipelineOracle(oracle_mod, table, path.class_table.cpu().numpy(), cfg.cache_entries,
                          path.cache_fill_ids.cpu().numpy(), world=1, flush_every=cfg.flush_every,
                          miss_cap=path.miss_cap, flush_cap=path.flush_cap, **kw)


def _check_step(path, orc, ids, grads, it):
    from oracle.pipeline_oracle import compare_rank

    rows, locs, found, st = path.step(torch.from_numpy(ids).cuda(), torch.from_numpy(grads).cuda())
    (outs,), (wflushed,) = orc.step([ids], [grads])
    wout, wlocs, whit = outs
    assert np.array_equal(locs.cpu().numpy(), wlocs), it
    assert np.array_equal(found.cpu().numpy(), whit), it
    np.testing.assert_allclose(rows.cpu().numpy(), wout, rtol=1e-4, atol=1e-5)
    assert st.flushed == wflushed, it
    compare_rank(path, orc, 0, where=f"step {it}")
    return wflushed, int(whit.sum())


@pytest.mark.parametrize("mode,overlap", [(0, False), (1, False), (0, True)])
def test_pipeline_matches_oracle(cuda_lib, oracle_mod, mode, overlap):
    """overlap: the fetch of a step runs on the side stream beside the aggregation of the same step."""
    from hades_b200 import pipeline, synth

    cfg = synth.scaled(synth.CONFIG1, 0.05, "pipe_test")
    cfg = synth.CacheFetchConfig(cfg.name, cfg.config, cfg.table_rows, 64, cfg.cache_entries // 4, cfg.batch,
                                 cfg.zipf_s, flush_every=3)
    path = pipeline.build_path(cfg, lookup_mode=mode, hot_fraction=0.02)
    path.overlap_fetch = overlap
    orc = _oracle_for(path, oracle_mod, cfg)
    cls = path.class_table.cpu().numpy()
    fill = path.cache_fill_ids.cpu().numpy()
    assert (cls[fill] == 2).all(), "the cold cache is filled with cold ids only"
    assert np.array_equal(path.cold.emb.cpu().numpy(), orc.ranks[0]["cache"])
    rng = synth.rng_for(1, 0, 7)
    sampler = synth.ZipfSampler(cfg.table_rows, cfg.zipf_s)
    total_flushed = hits = 0
    valid0 = path.cold.index.get_valid_entries_num()
    for it in range(1, 8):
        ids = sampler.ids(rng, cfg.batch)
        grads = synth.normal_rows(rng, cfg.batch, cfg.dim, cfg.grad_sigma)
        f, h = _check_step(path, orc, ids, grads, it)
        total_flushed += f
        hits += h
    assert total_flushed > 0 and hits > 0
    # cold misses were inserted (the small cache evicts by LRU and refuses where no way was ever hit)
    assert path.cold.index.get_valid_entries_num() != valid0 or int(path.cold.dropped.item()) > 0


def test_hot_rows_are_fresh_and_cold_rows_wait_for_the_flush(cuda_lib):
    """A HOT id is never served from the cache: the row fetched after an update is the updated
    one.  A cached COLD id keeps its row until the flush that applies its staged gradient evicts
    it; the next fetch then misses, reads the updated row and caches it again."""
    from hades_b200 import pipeline, synth

    base = synth.scaled(synth.CONFIG1, 0.05, "fresh_test")
    cfg = synth.CacheFetchConfig(base.name, base.config, base.table_rows, 32, base.cache_entries, 4096, base.zipf_s,
                                 flush_every=2)
    path = pipeline.build_path(cfg, hot_fraction=0.02)
    cls = path.class_table.cpu().numpy()
    hot_id = int(np.nonzero(cls == 1)[0][0])
    cold_id = int(path.cache_fill_ids[0].item())
    ids = torch.tensor([hot_id, cold_id] * 8, dtype=torch.int64, device="cuda")
    g = torch.full((16, cfg.dim), 1e-3, device="cuda")
    r1, _, f1, _ = path.step(ids, g)
    assert not bool(f1[0]) and bool(f1[1]), "hot ids miss the cache by construction, cached cold ids hit"
    hot_before, cold_before = r1[0].clone(), r1[1].clone()
    r2, _, f2, st2 = path.step(ids, g)          # step 2 ends with a flush
    assert not torch.equal(r2[0], hot_before), "the hot row carries the update of step 1"
    assert torch.equal(r2[1], cold_before) and bool(f2[1]), "the cold row is served from the cache until the flush"
    assert st2.flushed == 1
    r3, _, f3, _ = path.step(ids, g)
    assert not bool(f3[1]), "the flush evicted the cold id"
    assert not torch.equal(r3[1], cold_before), "its staged gradient reached the table"
    assert torch.equal(r3[1], path.table[cold_id])
    r4, _, f4, _ = path.step(ids, g)
    assert bool(f4[1]), "the miss of step 3 put it back into the cache"


def test_presampled_hotness_drives_classes_periods_and_fill(cuda_lib, oracle_mod):
    """A path built from presampled hotness as the reference builds its own: HOT = hotness >=
    threshold, per-node flush periods ceil(1 / (0.001 + hotness)) capped at 100 with count
    threshold 3, cache filled with the hottest cold ids; stepped against the oracle with the same
    tables."""
    from hades_b200 import hotness as H
    from hades_b200 import pipeline, synth

    base = synth.scaled(synth.CONFIG1, 0.03, "hotness_test")
    cfg = synth.CacheFetchConfig(base.name, base.config, base.table_rows, 32, base.cache_entries, base.batch,
                                 base.zipf_s, flush_every=1)
    sampler = synth.ZipfSampler(cfg.table_rows, cfg.zipf_s)
    rng = synth.rng_for(1, 0, 9)
    heat = H.presampling([torch.from_numpy(sampler.ids(rng, cfg.batch)) for _ in range(6)], cfg.table_rows)
    path = pipeline.build_path(cfg, hotness=heat, hot_threshold=0.99, cnt_threshold=3)
    cls = path.class_table.cpu().numpy()
    assert np.array_equal(cls == 1, heat.numpy() >= 0.99) and (cls == 1).sum() > 0
    thr = oracle_mod.flush_thresholds(heat.numpy())
    assert np.array_equal(path.cold.threshold.cpu().numpy(), thr)
    assert thr.min() == 1 and thr.max() == 100 and ((thr > 1) & (thr < 100)).any()
    orc = _oracle_for(path, oracle_mod, cfg, threshold=thr, cnt_threshold=3)
    flushed = []
    for it in range(1, 9):
        ids = sampler.ids(rng, cfg.batch)
        grads = synth.normal_rows(rng, cfg.batch, cfg.dim, cfg.grad_sigma)
        flushed.append(_check_step(path, orc, ids, grads, it)[0])
    assert sum(flushed) > 0 and flushed[0] == 0, "rows wait for their period (or three messages) before they leave"
    assert int((path.cold.remote.cnt > 0).sum().item()) > 0, "colder rows are still staged"


def test_flush_cap_leaves_the_rest_staged(cuda_lib, oracle_mod):
    from hades_b200 import pipeline, synth

    base = synth.scaled(synth.CONFIG1, 0.05, "cap_test")
    cfg = synth.CacheFetchConfig(base.name, base.config, base.table_rows, 16, base.cache_entries, base.batch,
                                 base.zipf_s, flush_every=2)
    path = pipeline.build_path(cfg, flush_cap=100)
    orc = _oracle_for(path, oracle_mod, cfg)
    assert path.flush_cap == 100 == orc.flush_cap
    rng = synth.rng_for(1, 0, 13)
    sampler = synth.ZipfSampler(cfg.table_rows, cfg.zipf_s)
    sent = []
    for it in range(1, 7):
        ids = sampler.ids(rng, cfg.batch)
        grads = synth.normal_rows(rng, cfg.batch, cfg.dim, cfg.grad_sigma)
        sent.append(_check_step(path, orc, ids, grads, it)[0])
    assert sent == [0, 100, 0, 100, 0, 100]


def test_graph_replay_equals_eager(cuda_lib):
    """The captured CUDA graph of the per-step path leaves exactly the bytes the eager launches
    leave (same kernels, same order), across flush steps."""
    from hades_b200 import pipeline, synth

    base = synth.scaled(synth.CONFIG1, 0.05, "graph_test")
    cfg = synth.CacheFetchConfig(base.name, base.config, base.table_rows, 128, base.cache_entries // 4, base.batch,
                                 base.zipf_s, flush_every=3)
    paths = [pipeline.build_path(synth.CacheFetchConfig(cfg.name + str(i), *list(cfg.__dict__.values())[1:]))
             for i in range(2)]
    sampler = synth.ZipfSampler(cfg.table_rows, cfg.zipf_s)
    rng = synth.rng_for(1, 0, 11)
    batches = [torch.from_numpy(sampler.ids(rng, cfg.batch)).cuda() for _ in range(9)]
    grads = torch.from_numpy(synth.normal_rows(rng, cfg.batch, cfg.dim, cfg.grad_sigma)).cuda()
    outs = [torch.empty((cfg.batch, cfg.dim), device="cuda") for _ in range(2)]
    ids_buf = torch.empty(cfg.batch, dtype=torch.int64, device="cuda")
    for k in range(2):
        for p, o in zip(paths, outs):
            p.step(batches[k], grads, o)
    torch.cuda.synchronize()
    paths[1].capture(ids_buf, grads, outs[1])
    flushed_total = 0
    for k in range(2, 9):
        r0 = paths[0].step(batches[k], grads, outs[0])
        r1 = paths[1].step(batches[k], grads, outs[1])
        assert torch.equal(r0[0], r1[0]) and torch.equal(r0[1], r1[1]) and torch.equal(r0[2], r1[2]), k
        assert r0[3].flushed == r1[3].flushed
        flushed_total += r1[3].flushed
        assert int(r0[3].num_unique.item()) == int(r1[3].num_unique.item())
    assert len(paths[1]._graphs) == 1 and len(paths[1]._flush_graphs) == 1
    assert flushed_total > 0  # the flush steps (replayed from a graph of their own) did flush rows
    assert torch.equal(paths[0].table, paths[1].table)
    assert torch.equal(paths[0].opt.state_mem, paths[1].opt.state_mem)
    assert torch.equal(paths[0].cold.remote.grad, paths[1].cold.remote.grad)
    assert torch.equal(paths[0].cold.emb, paths[1].cold.emb)
    for a, b in zip(paths[0].cold.index.export_state(), paths[1].cold.index.export_state()):
        assert torch.equal(a, b)


def test_rmat_frontier_path_matches_oracle(cuda_lib, oracle_mod):
    """Configuration-5 shapes scaled down: frontier ids of a sampled 2-hop expansion on a small
    R-MAT graph, hot class by popcount, through the same step as above."""
    from hades_b200 import pipeline, synth

    cfg = synth.scaled_rmat(synth.CONFIG5, 16, seeds=64)
    cfg = synth.RmatConfig(**{**cfg.__dict__, "dim": 32, "flush_every": 2})
    path = pipeline.build_rmat_path(cfg)
    cls = path.class_table.cpu().numpy()
    pop = np.array([bin(int(i)).count("1") for i in np.arange(cfg.num_nodes)])
    assert np.array_equal(cls == 1, pop <= cfg.hot_popcount)
    fill = path.cache_fill_ids.cpu().numpy()
    assert (pop[fill] > cfg.hot_popcount).all() and fill.size == min(cfg.cache_entries, (pop > cfg.hot_popcount).sum())
    orc = _oracle_for(path, oracle_mod, cfg)
    rng = synth.rng_for(5, 0, 1)
    for it in range(1, 5):
        ids = synth.rmat_frontier(cfg, rng)
        assert ids.size == cfg.batch
        grads = synth.normal_rows(rng, ids.size, cfg.dim, cfg.grad_sigma)
        _check_step(path, orc, ids, grads, it)


def test_path_with_tiered_optimizer_state_equals_all_hbm(cuda_lib):
    """The same steps with the optimiser state in HBM and with it tiered (pinned host memory + an
    HBM copy of the hottest rows, python/EmbCache/cache.py:66-194): tables bit-exact."""
    from hades_b200 import hotness as H
    from hades_b200 import pipeline, synth

    base = synth.scaled(synth.CONFIG1, 0.03, "tier_a")
    mk = lambda name: synth.CacheFetchConfig(name, base.config, base.table_rows, 32, base.cache_entries, base.batch,
                                             base.zipf_s, flush_every=2)
    sampler = synth.ZipfSampler(base.table_rows, base.zipf_s)
    rng = synth.rng_for(1, 0, 31)
    heat = H.presampling([torch.from_numpy(sampler.ids(rng, base.batch)) for _ in range(4)], base.table_rows)
    full = base.table_rows * (4 + 8 * 32)
    pa = pipeline.build_path(mk("tier_a"), hotness=heat, hot_threshold=0.7)
    pb = pipeline.build_path(mk("tier_b"), hotness=heat, hot_threshold=0.7, state_budget_bytes=full // 4)
    assert pa.opt.state_cache is None and pb.opt.state_cache is not None
    for it in range(5):
        ids = torch.from_numpy(sampler.ids(rng, base.batch)).cuda()
        g = torch.from_numpy(synth.normal_rows(rng, base.batch, 32, 1e-3)).cuda()
        ra, rb = pa.step(ids, g), pb.step(ids, g)
        assert torch.equal(ra[0], rb[0]) and torch.equal(ra[2], rb[2]), it
    assert torch.equal(pa.table, pb.table)
    for x, y in zip(pa.opt.full_state(), pb.opt.full_state()):
        assert torch.equal(x, y)
    hit = pb.opt.state_cache.idx_map != -1
    assert 0 < int(hit.sum().item()) < base.table_rows
