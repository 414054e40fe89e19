"""The whole per-step path (forward fetch, local aggregation, hot/cold split, cold-cache
accumulate, owner update, periodic flush and refill) on one GPU against the same steps composed
from the oracle's functions: index state, staging state and found masks bit-exact, optimiser
state and table within 1e-5 relative."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _oracle_step(o, ids, grads, step_no, flush_every):
    om = o["mod"]
    # forward
    out = np.zeros((ids.size, o["dim"]), np.float32)
    locs, hit = om.lookup_fetch(o["index"], ids, o["cache"], o["table"], out)
    o["index"].touch(locs)
    # backward
    u, s, c = om.only_unique_grads(ids, grads)
    cls = o["cls"][u]
    hot, cold = cls == 1, cls == 2
    o["staging"].accumulate_cached(o["index"], u[cold], s[cold], None, 0)
    hu, hm, _ = om.unique_grads(u[hot], s[hot], c[hot])
    om.sparse_adam_update(hu, hm, o["step"], o["mem"], o["power"], o["table"], 0.01)
    flushed = 0
    if step_no % flush_every == 0:
        fi, fr, fc, _ = o["staging"].flush(o["index"], 1)
        flushed = fi.size
        if flushed:
            om.sparse_adam_update(fi, fr, o["step"], o["mem"], o["power"], o["table"], 0.01, cnt=fc)
            o["staging"].insert(o["index"], fi, o["table"][fi], o["cache"])
    return out, locs, hit, flushed


@pytest.mark.parametrize("mode,mover", [(0, 1), (1, 2)])
def test_pipeline_matches_oracle(cuda_lib, oracle_mod, mode, mover):
    from hades_b200 import pipeline, synth

    cfg = synth.scaled(synth.CONFIG1, 0.05, "pipe_test")
    cfg = synth.CacheFetchConfig(cfg.name, cfg.config, cfg.table_rows, 64, cfg.cache_entries, cfg.batch,
                                 cfg.zipf_s, flush_every=3)
    path = pipeline.build_path(cfg, lookup_mode=mode, mover=mover, hot_fraction=0.02)
    # oracle state from the same initial table
    table = path.table.cpu().numpy().copy()
    ox = oracle_mod.OracleIndex(cfg.cache_entries)
    slots = ox.get_capacity()
    staging = oracle_mod.OracleStaging(slots, cfg.dim, cnt_threshold=16)
    cache = np.zeros((slots, cfg.dim), np.float32)
    hot_ids = synth.hot_ids(cfg.table_rows, cfg.cache_entries)
    staging.insert(ox, hot_ids, table[hot_ids], cache)
    o = dict(mod=oracle_mod, index=ox, cache=cache, table=table, staging=staging, dim=cfg.dim,
             cls=path.class_table.cpu().numpy(), step=np.zeros(cfg.table_rows, np.float32),
             mem=np.zeros((cfg.table_rows, cfg.dim), np.float32),
             power=np.zeros((cfg.table_rows, cfg.dim), np.float32))
    assert np.array_equal(path.cold.emb.cpu().numpy(), cache)
    rng = synth.rng_for(1, 0, 7)
    sampler = synth.ZipfSampler(cfg.table_rows, cfg.zipf_s)
    total_flushed = 0
    for it in range(1, 8):
        ids = sampler.ids(rng, cfg.batch)
        grads = synth.normal_rows(rng, cfg.batch, cfg.dim, cfg.grad_sigma)
        rows, locs, found, st = path.step(torch.from_numpy(ids).cuda(), torch.from_numpy(grads).cuda())
        wout, wlocs, whit, wflushed = _oracle_step(o, ids, grads, it, cfg.flush_every)
        assert np.array_equal(locs.cpu().numpy(), wlocs), it
        assert np.array_equal(found.cpu().numpy(), whit), it
        np.testing.assert_allclose(rows.cpu().numpy(), wout, rtol=1e-4, atol=1e-6)  # rows carry Adam updates
        assert st.flushed == wflushed, it
        total_flushed += wflushed
        gi, gl = path.cold.index.export_state()
        oi, ol = ox.export()
        assert np.array_equal(gi.cpu().numpy(), oi), it
        assert np.array_equal(gl.cpu().numpy(), ol), it
        assert np.array_equal(path.cold.remote.cnt.cpu().numpy(), staging.cnt), it
        assert np.array_equal(path.cold.remote.idx.cpu().numpy(), staging.idx), it
        np.testing.assert_allclose(path.cold.remote.grad.cpu().numpy(), staging.grad, rtol=1e-5, atol=1e-10)
        assert np.array_equal(path.opt.state_step.cpu().numpy(), o["step"]), it
        np.testing.assert_allclose(path.opt.state_mem.cpu().numpy(), o["mem"], rtol=1e-4, atol=1e-10)
        np.testing.assert_allclose(path.table.cpu().numpy(), o["table"], rtol=1e-4, atol=1e-7)
    assert total_flushed > 0
    assert int(path.cold.dropped.item()) > 0


def test_graph_replay_equals_eager(cuda_lib):
    """The captured CUDA graph of the per-step path leaves exactly the bytes the eager launches
    leave (same kernels, same order), across flush steps."""
    from hades_b200 import pipeline, synth

    base = synth.scaled(synth.CONFIG1, 0.05, "graph_test")
    cfg = synth.CacheFetchConfig(base.name, base.config, base.table_rows, 128, base.cache_entries, base.batch,
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
    for k in range(2, 9):
        r0 = paths[0].step(batches[k], grads, outs[0])
        r1 = paths[1].step(batches[k], grads, outs[1])
        assert torch.equal(r0[0], r1[0]) and torch.equal(r0[1], r1[1]) and torch.equal(r0[2], r1[2]), k
        assert r0[3].flushed == r1[3].flushed
        assert int(r0[3].num_unique.item()) == int(r1[3].num_unique.item())
    assert len(paths[1]._graphs) == 1
    assert torch.equal(paths[0].table, paths[1].table)
    assert torch.equal(paths[0].opt.state_mem, paths[1].opt.state_mem)
    assert torch.equal(paths[0].cold.remote.grad, paths[1].cold.remote.grad)
    for a, b in zip(paths[0].cold.index.export_state(), paths[1].cold.index.export_state()):
        assert torch.equal(a, b)


def test_rmat_frontier_path_matches_oracle(cuda_lib, oracle_mod):
    """Configuration-5 shapes scaled down: frontier ids of a sampled 2-hop expansion on a small
    R-MAT graph, hot class by popcount, through the same step as above."""
    from hades_b200 import pipeline, synth

    cfg = synth.scaled_rmat(synth.CONFIG5, 16, seeds=64)
    cfg = synth.RmatConfig(**{**cfg.__dict__, "dim": 32, "flush_every": 2})
    path = pipeline.build_rmat_path(cfg)
    table = path.table.cpu().numpy().copy()
    cls = path.class_table.cpu().numpy()
    ids_all = np.arange(cfg.num_nodes)
    pop = np.array([bin(int(i)).count("1") for i in ids_all])
    assert np.array_equal(cls == 1, pop <= cfg.hot_popcount)
    fill = path.cache_fill_ids.cpu().numpy()
    assert (pop[fill] > cfg.hot_popcount).all() and fill.size == min(cfg.cache_entries, (pop > cfg.hot_popcount).sum())
    ox = oracle_mod.OracleIndex(cfg.cache_entries)
    slots = ox.get_capacity()
    staging = oracle_mod.OracleStaging(slots, cfg.dim, cnt_threshold=16)
    cache = np.zeros((slots, cfg.dim), np.float32)
    staging.insert(ox, fill, table[fill], cache)
    o = dict(mod=oracle_mod, index=ox, cache=cache, table=table, staging=staging, dim=cfg.dim, cls=cls,
             step=np.zeros(cfg.table_rows, np.float32), mem=np.zeros((cfg.table_rows, cfg.dim), np.float32),
             power=np.zeros((cfg.table_rows, cfg.dim), np.float32))
    rng = synth.rng_for(5, 0, 1)
    for it in range(1, 5):
        ids = synth.rmat_frontier(cfg, rng)
        assert ids.size == cfg.batch
        grads = synth.normal_rows(rng, ids.size, cfg.dim, cfg.grad_sigma)
        rows, locs, found, st = path.step(torch.from_numpy(ids).cuda(), torch.from_numpy(grads).cuda())
        wout, wlocs, whit, wflushed = _oracle_step(o, ids, grads, it, cfg.flush_every)
        assert np.array_equal(locs.cpu().numpy(), wlocs) and np.array_equal(found.cpu().numpy(), whit), it
        assert st.flushed == wflushed, it
        # fetched rows carry earlier Adam updates (lr = 1e-2), whose first step lr*g/(|g|+eps)
        # amplifies the rounding of a nearly cancelling mean: bound relative to lr
        np.testing.assert_allclose(rows.cpu().numpy(), wout, rtol=1e-4, atol=1e-6)
        assert np.array_equal(path.opt.state_step.cpu().numpy(), o["step"]), it
        np.testing.assert_allclose(path.table.cpu().numpy(), o["table"], rtol=1e-4, atol=1e-6)
        gi, gl = path.cold.index.export_state()
        oi, ol = ox.export()
        assert np.array_equal(gi.cpu().numpy(), oi) and np.array_equal(gl.cpu().numpy(), ol), it
