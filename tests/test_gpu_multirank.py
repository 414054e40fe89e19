"""Two ranks on two GPUs: the owner-partitioned exchange (NCCL and peer-memory push) and the whole
step against a numpy simulation of both ranks built from the oracle's functions
(oracle/pipeline_oracle.py).  Skipped when fewer than two GPUs are visible."""
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
    # forward fetch (hot ids always, cold ids until they are inserted) see the owners' rows.
    from oracle.pipeline_oracle import PipelineOracle, compare_rank

    cfg = _cfg()
    path = pipeline.build_path(cfg, rank, WORLD, hot_fraction=0.02,
                               exchange={"nccl": "nccl", "push": "push", "push_graph": "push",
                                         "push_overlap": "push", "push_overlap_graph": "push",
                                         "push_deliver": "push", "push_deliver_overlap_graph": "push",
                                         "push_nccl_fence_graph": "push_nccl_fence"}[exchange],
                               remote_fetch="deliver" if "deliver" in exchange else "pull")
    assert (path.px_req is not None) == ("deliver" in exchange)
    path.overlap_fetch = "overlap" in exchange
    assert (path.px is not None) == exchange.startswith("push")
    assert (path.px_flush is not None) == exchange.startswith("push")
    assert path.shared is not None and path.table is None
    # the whole table from the shards, through the same reads the kernels do
    all_ids = torch.arange(cfg.table_rows, dtype=torch.int64, device="cuda")
    w = path.shared.gather(all_ids).cpu().numpy()
    assert np.array_equal(w[rank::WORLD], path.opt.emb.weight.cpu().numpy())
    orc = PipelineOracle(om, w, path.class_table.cpu().numpy(), cfg.cache_entries,
                         path.cache_fill_ids.cpu().numpy(), world=WORLD, flush_every=cfg.flush_every,
                         miss_cap=path.miss_cap, flush_cap=path.flush_cap)
    use_graph = exchange.endswith("_graph")
    g_ids = torch.empty(cfg.batch, dtype=torch.int64, device="cuda")
    g_grads = torch.empty((cfg.batch, cfg.dim), device="cuda")
    g_out = torch.empty((cfg.batch, cfg.dim), device="cuda")
    flushed_total = 0
    for it in range(1, 6):
        ids, grads = _batch(cfg, rank, it)
        if use_graph and it == 2:  # one eager step first, then the captured graphs
            torch.cuda.synchronize()
            path.capture(g_ids, g_grads, g_out)
        g_grads.copy_(torch.from_numpy(grads))
        rows, locs, found, st = path.step(torch.from_numpy(ids).cuda(), g_grads, g_out)
        rows, locs, found = rows.cpu().numpy(), locs.cpu().numpy(), found.cpu().numpy()
        both = [_batch(cfg, r, it) for r in range(WORLD)]
        outs, flushed = orc.step([b[0] for b in both], [b[1] for b in both])
        out, l_r, hit_r = outs[rank]
        assert np.array_equal(locs, l_r) and np.array_equal(found, hit_r), (rank, it)
        np.testing.assert_allclose(rows, out, rtol=1e-4, atol=1e-5)
        assert st.flushed == flushed[rank], (rank, it)
        flushed_total += flushed[rank]
        compare_rank(path, orc, rank, where=f"rank {rank} step {it}")
    assert flushed_total > 0
    assert path.step_no == 5
    path.close()
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("exchange", ["nccl", "push", "push_graph", "push_nccl_fence_graph", "push_overlap",
                                      "push_overlap_graph", "push_deliver", "push_deliver_overlap_graph"])
def test_two_ranks(exchange):
    """exchange = "nccl": ragged all_to_all_single; "push": the fused pack+push kernel over
    peer memory with the device-side fence (plain stores, NVLS off); "push_graph": the same
    replayed from two whole-step CUDA graphs; "push_nccl_fence_graph": NCCL all-reduce as the
    fence, graphs around the eagerly launched exchange; "..._overlap": the forward fetch of a step
    (remote rows included) on the side stream beside the aggregation of the same step;
    "..._deliver": the owners store the remote rows of the forward fetch into the requester's stage
    (requests through a third exchange, two fences) instead of the requester reading them."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < WORLD:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    from oracle import build_oracle

    build_oracle.build_oracle()
    mp.spawn(_worker, args=(_free_port(), exchange), nprocs=WORLD, join=True)


def _deliver_worker(rank, port):
    """The three calls of a forward fetch whose remote rows the owners deliver, on two GPUs, with a
    request exchange that is too small on purpose: the requests that do not fit are refused with a
    status code (HB_ERR_CAPACITY), nothing is written out of bounds, what fitted is served."""
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=WORLD, device_id=torch.device("cuda", rank))
    from hades_b200 import EmbCacheLib as E
    from hades_b200 import _lib
    from hades_b200.exchange import PeerExchange
    from hades_b200.peer_table import PeerTable

    num_rows, dim, n = 1000, 8, 200
    table = PeerTable(num_rows, dim, rank, WORLD)
    full = torch.arange(num_rows * dim, dtype=torch.float32, device="cuda").reshape(num_rows, dim)
    table.weight.copy_(full[rank::WORLD])
    stages = PeerTable(WORLD * n, dim, rank, WORLD)
    stages.weight.fill_(-1.0)
    torch.cuda.synchronize()
    dist.barrier()
    index = E.IndexCache(64, f"deliver_r{rank}", True, False)  # empty: every id misses
    cache = torch.zeros((index.get_capacity(), dim), device="cuda")
    ids = torch.arange(n, dtype=torch.int64, device="cuda")    # 100 of them live on the other GPU
    for cap, want_status in ((8, 6), (128, 0)):                 # HB_ERR_CAPACITY, then room for all
        px = PeerExchange(rank, WORLD, cap, 4)
        runs = E.cudaRunsBuild(ids, 12)
        parity = E.cudaRunsResolveRequests(index, runs, cache, table, stages.weight, px)
        px.fence()
        r_ids, _, r_runs, seg = px.received(parity)
        table.serve(stages, r_ids, r_runs, seg, px.cap)
        px.fence()
        out = torch.full((n, dim), -7.0, device="cuda")
        rows, locs, found = E.cudaRunsExpand(runs, cache, stages.weight, out)
        torch.cuda.synchronize()
        assert _lib.device_status() == want_status, (rank, cap)
        assert int(seg[1 - rank].item()) == min(cap, n // 2) and int(seg[rank].item()) == 0
        assert not bool(found.any()) and bool((locs == -1).all())
        mine = ids % WORLD == rank
        assert torch.equal(rows[mine], full[ids[mine]])          # own rows: read from the local shard
        theirs = rows[~mine]
        delivered = (theirs == full[ids[~mine]]).all(dim=1)
        stale = (theirs == -1.0).all(dim=1)                      # the stage row nobody filled
        assert bool((delivered | stale).all())
        assert int(delivered.sum().item()) == min(cap, n // 2), (rank, cap, int(delivered.sum().item()))
        px.close()
        stages.weight.fill_(-1.0)
        torch.cuda.synchronize()
        dist.barrier()
    stages.close()
    table.close()
    dist.destroy_process_group()


def test_delivery_refuses_requests_beyond_the_slab():
    if not torch.cuda.is_available() or torch.cuda.device_count() < WORLD:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    mp.spawn(_deliver_worker, args=(_free_port(),), nprocs=WORLD, join=True)
