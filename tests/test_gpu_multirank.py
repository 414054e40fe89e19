"""Two ranks on two GPUs over NCCL: the owner-partitioned exchange and the whole backward path
against a numpy simulation of both ranks built from the oracle's functions.  Skipped when fewer
than two GPUs are visible."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
WORLD = 2


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _cfg():
    from hades_b200 import synth

    c = synth.scaled(synth.CONFIG1, 0.05, "mr_test")
    return synth.CacheFetchConfig(c.name, c.config, c.table_rows, 64, c.cache_entries, c.batch, c.zipf_s,
                                  flush_every=2)


def _batch(cfg, rank, it):
    from hades_b200 import synth

    rng = synth.rng_for(7, rank, it)
    ids = synth.ZipfSampler(cfg.table_rows, cfg.zipf_s).ids(rng, cfg.batch)
    grads = synth.normal_rows(rng, cfg.batch, cfg.dim, cfg.grad_sigma)
    return ids, grads


def _worker(rank, port, exchange):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=WORLD, device_id=torch.device("cuda", rank))
    from hades_b200 import pipeline, synth
    from hades_b200.sparse_optim import swap_gradients
    from oracle import oracle as om

    # --- swap_gradients alone -------------------------------------------------------------
    rng = np.random.default_rng(50 + rank)
    n = 20_000 if rank == 0 else 7_000
    ids = rng.integers(0, 10**7, n, dtype=np.int64)
    rows = rng.standard_normal((n, 32)).astype(np.float32)
    cnt = rng.integers(1, 5, n, dtype=np.int64)
    r_ids, r_rows, r_cnt = swap_gradients(torch.from_numpy(ids).cuda(), torch.from_numpy(rows).cuda(), None, 1,
                                          WORLD, torch.device("cuda", rank), torch.from_numpy(cnt).cuda())
    want = []
    for src in range(WORLD):
        g = np.random.default_rng(50 + src)
        m = 20_000 if src == 0 else 7_000
        s_ids = g.integers(0, 10**7, m, dtype=np.int64)
        s_rows = g.standard_normal((m, 32)).astype(np.float32)
        s_cnt = g.integers(1, 5, m, dtype=np.int64)
        mine = s_ids % WORLD == rank
        want.append((s_ids[mine], s_rows[mine], s_cnt[mine]))
    assert np.array_equal(r_ids.cpu().numpy(), np.concatenate([w[0] for w in want]))
    assert np.array_equal(r_rows.cpu().numpy(), np.concatenate([w[1] for w in want]))
    assert np.array_equal(r_cnt.cpu().numpy(), np.concatenate([w[2] for w in want]))

    # --- the whole step on both ranks vs a simulation of both -------------------------------
    # The table is sharded by owner and every GPU reads every shard: cache misses of the
    # forward fetch and the refill after a flush see the owners' current rows.
    cfg = _cfg()
    path = pipeline.build_path(cfg, rank, WORLD, hot_fraction=0.02,
                               exchange={"nccl": "nccl", "push": "push", "push_graph": "push",
                                         "push_nccl_fence_graph": "push_nccl_fence"}[exchange])
    assert (path.px is not None) == exchange.startswith("push")
    assert path.shared is not None and path.table is None
    cls = path.class_table.cpu().numpy()
    # the whole table from the shards, through the same reads the kernels do
    all_ids = torch.arange(cfg.table_rows, dtype=torch.int64, device="cuda")
    w = path.shared.gather(all_ids).cpu().numpy()
    assert np.array_equal(w[rank::WORLD], path.opt.emb.weight.cpu().numpy())
    step = np.zeros(cfg.table_rows, np.float32)
    mem = np.zeros((cfg.table_rows, cfg.dim), np.float32)
    power = np.zeros((cfg.table_rows, cfg.dim), np.float32)
    # cold state (index, cached rows, staging) of BOTH ranks
    sim = []
    hot_ids = synth.hot_ids(cfg.table_rows, cfg.cache_entries)
    for r in range(WORLD):
        ox = om.OracleIndex(cfg.cache_entries)
        stg = om.OracleStaging(ox.get_capacity(), cfg.dim, cnt_threshold=16)
        cache = np.zeros((ox.get_capacity(), cfg.dim), np.float32)
        stg.insert(ox, hot_ids, w[hot_ids], cache)
        sim.append((ox, stg, cache))
    use_graph = exchange.endswith("_graph")
    g_ids = torch.empty(cfg.batch, dtype=torch.int64, device="cuda")
    g_grads = torch.empty((cfg.batch, cfg.dim), device="cuda")
    g_out = torch.empty((cfg.batch, cfg.dim), device="cuda")
    for it in range(1, 6):
        ids, grads = _batch(cfg, rank, it)
        if use_graph and it == 2:  # one eager step first, then the captured graphs
            torch.cuda.synchronize()
            path.capture(g_ids, g_grads, g_out)
        g_grads.copy_(torch.from_numpy(grads))
        rows, locs, found, st = path.step(torch.from_numpy(ids).cuda(), g_grads, g_out)
        rows, locs, found = rows.cpu().numpy(), locs.cpu().numpy(), found.cpu().numpy()
        # every rank's forward reads the table as the previous step left it
        uniq = []
        for r in range(WORLD):
            i_r, g_r = _batch(cfg, r, it)
            ox, stg, cache = sim[r]
            out = np.zeros((i_r.size, cfg.dim), np.float32)
            l_r, hit_r = om.lookup_fetch(ox, i_r, cache, w, out)
            ox.touch(l_r)
            if r == rank:
                assert np.array_equal(locs, l_r) and np.array_equal(found, hit_r), (rank, it)
                np.testing.assert_allclose(rows, out, rtol=1e-4, atol=2e-6)
            u, s, c = om.only_unique_grads(i_r, g_r)
            k = cls[u]
            stg.accumulate_cached(ox, u[k == 2], s[k == 2], None, 0)
            uniq.append((u[k == 1], s[k == 1], c[k == 1]))
        for owner in range(WORLD):
            inbox = [(u[u % WORLD == owner], s[u % WORLD == owner], c[u % WORLD == owner]) for u, s, c in uniq]
            hu, hm, _ = om.unique_grads(*[np.concatenate([x[j] for x in inbox]) for j in range(3)])
            om.sparse_adam_update(hu, hm, step, mem, power, w, 0.01)
        if it % cfg.flush_every == 0:
            flushed = []
            for r in range(WORLD):
                ox, stg, cache = sim[r]
                fi, fr, fc, _ = stg.flush(ox, WORLD)
                flushed.append((fi, fr, fc))
            for owner in range(WORLD):
                inbox = [(fi[fi % WORLD == owner], fr[fi % WORLD == owner], fc[fi % WORLD == owner])
                         for fi, fr, fc in flushed]
                fu, fm, _ = om.unique_grads(*[np.concatenate([x[j] for x in inbox]) for j in range(3)])
                om.sparse_adam_update(fu, fm, step, mem, power, w, 0.01)
            for r in range(WORLD):  # refill with the rows every owner has just written
                ox, stg, cache = sim[r]
                stg.insert(ox, flushed[r][0], w[flushed[r][0]], cache)
        assert np.array_equal(path.opt.state_step.cpu().numpy(), step[rank::WORLD]), (rank, it)
        np.testing.assert_allclose(path.opt.state_mem.cpu().numpy(), mem[rank::WORLD], rtol=1e-4, atol=1e-9)
        np.testing.assert_allclose(path.opt.emb.weight.cpu().numpy(), w[rank::WORLD], rtol=1e-4, atol=2e-6)
        gi, gl = path.cold.index.export_state()
        oi, ol = sim[rank][0].export()
        assert np.array_equal(gi.cpu().numpy(), oi) and np.array_equal(gl.cpu().numpy(), ol), (rank, it)
        np.testing.assert_allclose(path.cold.emb.cpu().numpy(), sim[rank][2], rtol=1e-4, atol=2e-6)
    assert path.step_no == 5
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("exchange", ["nccl", "push", "push_graph", "push_nccl_fence_graph"])
def test_two_ranks(exchange):
    """exchange = "nccl": ragged all_to_all_single; "push": the fused pack+push kernel over
    peer memory with the device-side fence (plain stores, NVLS off); "push_graph": the same
    replayed from two whole-step CUDA graphs; "push_nccl_fence_graph": NCCL all-reduce as the
    fence, graphs around the eagerly launched exchange."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < WORLD:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    from oracle import build_oracle

    build_oracle.build_oracle()
    mp.spawn(_worker, args=(_free_port(), exchange), nprocs=WORLD, join=True)
