#!/usr/bin/env python
"""Benchmark of the embedding-cache / sparse-gradient hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload ...]

One "step" = one pass of the whole path over one batch of synthetic ids on every GPU: the batch
is sorted once; fused cache lookup + cached fetch over the runs of equal ids, LRU ageing, insertion
of the cold ids that missed; local aggregation (segment-sum over the same runs), hot/cold split,
cold-cache accumulate, owner-partitioned exchange of the hot rows + optimiser update on the owner;
every 8th step the stale rows of the cold cache leave for their owners too.  The workload is
configuration 2 of the baseline (20M x 128 fp32 table, 4M-entry cold cache, 2M Zipf(1.2) ids per
step and GPU); per-GPU work is fixed as N grows ("weak" scaling).

Prints ONE JSON line (rank 0).  `value` is timed with the batch already in HBM; `e2e` times the
same step with the ids arriving from pinned host memory and the found mask read back to the host.
`parity_check` is an untimed self-check against the CPU checkers under oracle/ made before the
timed region (a mismatch ends the run with a non-zero exit code).  `extra` holds short legs on the
other baseline configurations at the same N.  `--impl reference` times the reference's CPU path
(its compiled index + the torch CPU expressions of its call sites) on the same configuration.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "embedding_rows_per_s_lookup_fetch_aggregate_sync"
UNIT = "rows/s"
WORKLOAD = "config2: table 20M x 128 fp32, cold cache 4M, batch 2M Zipf(1.2) per GPU, flush every 8 steps"
HBM_NOMINAL_GBS = 8000.0      # the figure the north-star target is quoted on
NVLINK_NOMINAL_GBS = 900.0    # per direction per GPU
NVLINK_MEASURED_GBS = 770.0   # peer copy measured on this pool (cudaMemcpyPeer, 1 GiB)

# DRAM bytes of ONE launch of the fused lookup+fetch kernel at configuration 2, from an ncu capture
# (dram__bytes_read.sum + dram__bytes_write.sum).  Tied to the kernel source it was taken on: when
# that source changes the figure is withheld (traffic = null) until it is captured again.
TRAFFIC_CAPTURE = {
    "kernel_sources": ["hades_b200/csrc/runs.cu", "hades_b200/csrc/index.cuh"],
    "sha256": "946dcb7ba44aa64ec78f9adbd91048d4ce8b226e941bcff7084d467b91d4912b",
    "bytes_per_launch": 1_092_927_488,
    "source": "ncu --metrics dram__bytes_read.sum,dram__bytes_write.sum --clock-control none (1 pass) over "
              "bench.py --steps 8 --warmup 3 --no-graph at full configuration 2 on one B200: runs_resolve_kernel "
              "17.8 MB read + runs_expand_kernel 105.9 MB read, 969.2 MB written, mean of 3 calls",
}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--scale", type=float, default=1.0, help="shrink the workload (profiling captures)")
    ap.add_argument("--lookup", default="setassoc", choices=["setassoc", "sorted"])
    ap.add_argument("--no-lru", action="store_true", help="skip the LRU ageing passes")
    ap.add_argument("--no-insert", action="store_true", help="do not insert the cold ids that miss the cache")
    ap.add_argument("--workload", default="config2",
                    choices=["config2", "c1", "c3", "c4_exchange", "c5", "ref_kernels", "micro", "micro_update"],
                    help="config2: the whole path (default); c1: lookup + fetch + set / accumulate at "
                         "configuration-1 shapes (1M x 128 table, 100k-entry cache, 65,536 ids); c3: hot-node local "
                         "aggregation + reduction of the hot ids across GPUs (524,288 ids per GPU, Zipf(1.2) over "
                         "1e8); c4_exchange: the owner-partitioned sync at configuration-4 shapes (1,048,576 unique "
                         "ids x 64 fp32 per rank) and the Adagrad update on the fp16 shard; c5: the whole path on "
                         "the frontier of a sampled 2-layer GraphSAGE step over a synthetic R-MAT graph (1e8 nodes, "
                         "1,024 seeds, fanout [25, 10], per GPU); ref_kernels: the reference's own CUDA operators "
                         "beside this library's at configuration-2 shapes; micro / micro_update: single operators")
    ap.add_argument("--optimizer", default="adam", choices=["adam", "adagrad"])
    ap.add_argument("--rmat-bits", type=int, default=0, help="c5 on a smaller graph of 2**bits vertices")
    ap.add_argument("--exchange", default="push", choices=["push", "push_nccl_fence", "nccl"],
                    help="N>1: fused pack+push over peer memory with the device-side fence (default) or "
                         "with an NCCL all-reduce as the fence, or NCCL all_to_all_single")
    ap.add_argument("--remote-fetch", default="auto", choices=["auto", "pull", "deliver"],
                    help="N > 1, rows of other GPUs' shards in the forward fetch: read by this GPU once per distinct "
                         "id (pull) or stored into this GPU's stage by their owners (deliver, the default of auto)")
    ap.add_argument("--overlap-fetch", default="on", choices=["on", "off"],
                    help="run the forward fetch of a step beside the aggregation of the same step (default on)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the legs on the other configurations")
    ap.add_argument("--no-parity", action="store_true", help="skip the untimed self-check")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel eagerly (no CUDA graph)")
    return ap.parse_args()


def measured_peaks() -> dict:
    pk = ROOT / "MEASURED_PEAKS.json"
    return json.loads(pk.read_text()) if pk.exists() else {}


def traffic_capture():
    """(bytes per launch, provenance) of the recorded ncu capture, or (None, why)."""
    h = hashlib.sha256()
    for rel in TRAFFIC_CAPTURE["kernel_sources"]:
        h.update((ROOT / rel).read_bytes())
    sha = h.hexdigest()
    if TRAFFIC_CAPTURE["bytes_per_launch"] is None:
        return None, {"traffic_source": None, "traffic_kernel_sha": sha, "why_null": "no capture recorded"}
    if TRAFFIC_CAPTURE["sha256"] != sha:
        return None, {"traffic_source": TRAFFIC_CAPTURE["source"], "traffic_kernel_sha": sha,
                      "why_null": "the kernel source changed since the capture"}
    return TRAFFIC_CAPTURE["bytes_per_launch"], {"traffic_source": TRAFFIC_CAPTURE["source"],
                                                 "traffic_kernel_sha": sha}


# --------------------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and the clock-event (throttle) reasons of one GPU through NVML from a
    background thread while the timed region runs.  Read-only."""

    REASONS = {
        "hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20,
        "hw_thermal_slowdown": 0x40, "hw_power_brake_slowdown": 0x80,
    }

    def __init__(self, index: int, period_s: float = 0.02):
        self.index, self.period = index, period_s
        self.sm, self.bits, self.max_sm, self.err = [], 0, None, None
        self._stop = None
        self._thread = None

    def start(self):
        import threading

        try:
            import pynvml

            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_sm = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
        except Exception as e:  # noqa: BLE001
            self.err = f"nvml unavailable: {e}"
            return
        self._stop = threading.Event()

        def loop():
            while not self._stop.is_set():
                try:
                    self.sm.append(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
                    self.bits |= int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(h))
                except Exception as e:  # noqa: BLE001
                    self.err = str(e)
                    break
                self._stop.wait(self.period)

        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()

    def stop(self) -> dict:
        if self._thread is not None:
            self._stop.set()
            self._thread.join(timeout=2)
        sm = sorted(self.sm)
        out = {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.max_sm,
               "samples": len(sm),
               "reasons": sorted(k for k, bit in self.REASONS.items() if self.bits & bit)}
        if self.err:
            out["error"] = self.err
        return out


# --------------------------------------------------------------------------------------
# reference arm / CPU baseline: the reference's own CPU path
# --------------------------------------------------------------------------------------
def cpu_reference_run(steps: int, warmup: int, scale: float, threads: int | None = None) -> dict:
    """The path as the reference runs it on CPU tensors, step for step what the GPU arm does:
    the split of the ids by class (dist_emb.py:174-180), IndexCache.lookup of the cold ids (its
    compiled C++ index, OpenMP; dist_emb.py:184-186), torch CPU gathers for the fetch
    (test/test_cached_fetch.py:33-36), IndexCache.add of the uncached cold ids with their rows
    (server.py:499-544), only_unique_grads (sparse_optim.py:132-139), the server's accumulate and
    flush (server.py:346-574) and SparseAdam.update (:590-685).  oracle/ is used here as the thing
    measured ONLY in this baseline leg."""
    import numpy as np
    import torch

    from hades_b200 import synth
    from oracle import oracle as om

    cfg = synth.CONFIG2 if scale == 1.0 else synth.scaled(synth.CONFIG2, scale, "config2_cpu_sample")
    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    use_ref = om.RefIndex.available()
    if use_ref:
        om.RefIndex.set_threads(threads)
        index = om.RefIndex(cfg.cache_entries)
    else:
        index = om.OracleIndex(cfg.cache_entries)
    g = torch.Generator().manual_seed(2000)
    table = torch.empty((cfg.table_rows, cfg.dim)).normal_(0, cfg.table_sigma, generator=g)
    n_hot = max(int(cfg.table_rows * 0.01), 1)
    cls = torch.full((cfg.table_rows,), 2, dtype=torch.int8)
    cls[torch.from_numpy(synth.rank_to_id(np.arange(n_hot, dtype=np.int64), cfg.table_rows))] = 1
    fill = synth.rank_to_id(np.arange(n_hot, min(n_hot + cfg.cache_entries, cfg.table_rows), dtype=np.int64),
                            cfg.table_rows)
    if use_ref:
        om.RefIndex.set_threads(1)  # add() depends on thread timing otherwise
    locs = index.add(fill)
    slots = index.get_capacity()
    cache = torch.zeros((slots, cfg.dim))
    ok = torch.from_numpy(locs >= 0)
    cache[torch.from_numpy(locs)[ok]] = table[torch.from_numpy(fill)[ok]]
    if use_ref:
        om.RefIndex.set_threads(threads)
    grad_buf = torch.zeros((slots, cfg.dim))
    cnt_buf = torch.zeros(slots, dtype=torch.int32)
    idx_buf = torch.full((slots,), -1, dtype=torch.int64)
    step_s = torch.zeros(cfg.table_rows)
    mem = torch.zeros((cfg.table_rows, cfg.dim))
    power = torch.zeros((cfg.table_rows, cfg.dim))
    sampler = synth.ZipfSampler(cfg.table_rows, cfg.zipf_s)
    rng = synth.rng_for(2, 0, 1)
    batches = [torch.from_numpy(sampler.ids(rng, cfg.batch)) for _ in range(4)]
    grads = torch.empty((cfg.batch, cfg.dim)).normal_(0, cfg.grad_sigma, generator=g)

    def adam(idx, gv):
        t = step_s[idx] + 1
        m = 0.9 * mem[idx] + (1.0 - 0.9) * gv
        v = 0.999 * power[idx] + (1.0 - 0.999) * gv * gv
        mc = m / (1.0 - torch.pow(torch.tensor(0.9), t)).unsqueeze(1)
        vc = v / (1.0 - torch.pow(torch.tensor(0.999), t)).unsqueeze(1)
        step_s[idx] = t
        mem[idx] = m
        power[idx] = v
        table[idx] -= 0.01 * mc / (torch.sqrt(vc) + 1e-8)

    def one_step(k: int):
        ids = batches[k % len(batches)]
        cold_pos = torch.nonzero(cls[ids] == 2).flatten()
        cold_ids = ids[cold_pos]
        l = torch.from_numpy(index.lookup(cold_ids.numpy()))
        hit = l >= 0
        out = table[ids]                                  # authoritative rows (hot ids, uncached cold ids)
        out[cold_pos[hit]] = cache[l[hit]]                # cold rows the cache holds
        miss_ids = torch.unique(cold_ids[~hit])
        if miss_ids.numel():
            nl = torch.from_numpy(index.add(miss_ids.numpy()))  # all threads: timed, not compared
            okk = nl >= 0
            cache[nl[okk]] = table[miss_ids[okk]]
            cnt_buf[nl[okk]] = 0
            idx_buf[nl[okk]] = -1
            grad_buf[nl[okk]] = 0
        u, inv, c = torch.unique(ids, return_inverse=True, return_counts=True)
        s = torch.zeros((u.numel(), cfg.dim))
        s.index_add_(0, inv, grads)
        kind = cls[u]
        hu, hs, hc = u[kind == 1], s[kind == 1], c[kind == 1]
        cu, cs = u[kind == 2], s[kind == 2]
        cl = torch.from_numpy(index.lookup(cu.numpy()))
        chit = cl >= 0
        sl = cl[chit]
        idx_buf[sl] = cu[chit]
        grad_buf[sl] += cs[chit]
        cnt_buf[sl] += 1
        adam(hu, hs / (1 + hc).unsqueeze(1))
        if (k + 1) % cfg.flush_every == 0:
            live = torch.nonzero(cnt_buf > 0).flatten()
            fid, frow, fcnt = idx_buf[live], grad_buf[live], cnt_buf[live]
            index.reset(fid.numpy())
            grad_buf[live] = 0
            cnt_buf[live] = 0
            if live.numel():
                adam(fid, frow / fcnt.unsqueeze(1))
        return out

    for k in range(warmup):
        one_step(k)
    t0 = time.perf_counter()
    for k in range(warmup, warmup + steps):
        one_step(k)
    dt = time.perf_counter() - t0
    return {"value": cfg.batch * steps / dt, "unit": UNIT, "cores": threads,
            "kind": "reference" if use_ref else "port",
            "sample": (f"config2 {'at full size' if scale == 1.0 else f'scaled by {scale:g}'} (table "
                       f"{cfg.table_rows} x {cfg.dim}, cache {cfg.cache_entries}, batch {cfg.batch}), {steps} "
                       f"steps after {warmup} warm-up; the reference's compiled CPU index + the torch CPU "
                       "expressions of its Python call sites"),
            "same_config": scale == 1.0, "ms_per_step": dt / steps * 1e3}


def cpu_sample_scale() -> tuple[float, str]:
    """Configuration 2 at full size needs about 47 GB of host memory (table, two Adam moments,
    cache, staging); run it when the host has that to spare, else a 1/8 sample."""
    try:
        import psutil

        avail = psutil.virtual_memory().available
    except Exception:  # noqa: BLE001
        avail = 0
    if avail > 80 * 2**30:
        return 1.0, f"host has {avail / 2**30:.0f} GiB available"
    return 1.0 / 8.0, f"host has only {avail / 2**30:.0f} GiB available: 1/8 sample"


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    scale, why = cpu_sample_scale()
    steps = min(max(args.steps, 1), 10 if scale == 1.0 else 40)  # bounded: each full-size step is ~0.5 s of CPU
    warm = min(max(args.warmup, 1), 2)
    r = cpu_reference_run(steps, warm, scale)
    line = {
        "impl": "reference", "metric": METRIC, "value": r["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warm, "ms_per_step": r["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": r["sample"], "same_config": r["same_config"], "memory": why,
                   "processes": "ONE CPU process on rank 0 whatever --gpus says: at N > 1 the ratio to the GPU "
                                "arm divides N GPUs by one host"},
        "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": r["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------------------
# set-up shared by the GPU legs
# --------------------------------------------------------------------------------------
_DIST = {}


def dist_setup():
    """(rank, world, device, timed).  timed(fn, steps) -> ms per step: CUDA events on the current
    stream, a barrier + synchronize on both sides, max over ranks."""
    if _DIST:
        return _DIST["v"]
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)

    def timed(fn, steps, first=0, tail=None, total=False):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for k in range(first, first + steps):
            fn(k)
        if tail:
            tail()
        b.record()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ms = torch.tensor([a.elapsed_time(b)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()) if total else float(ms.item()) / steps

    _DIST["v"] = (rank, world, dev, timed)
    return _DIST["v"]


def time_local(fn, reps=5):
    """ms per call of a single-GPU operation, CUDA events, after one warm-up call."""
    import torch

    fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps


# --------------------------------------------------------------------------------------
# untimed self-checks against the CPU checkers
# --------------------------------------------------------------------------------------
def parity_full_size(path, ids_dev, ids_host) -> dict:
    """Configuration 2 at full size, before any step: the slots and found mask of one whole batch
    against IndexCache.lookup of the reference's compiled CPU index (filled by the same add()
    calls), the fetched rows against the torch expression of the reference's tests, unique ids and
    counts against numpy."""
    import numpy as np
    import torch

    from hades_b200 import EmbCacheLib as E
    from hades_b200.exchange import _as_tensor
    from oracle import build_oracle
    from oracle import oracle as om

    build_oracle.build_oracle()
    use_ref = om.RefIndex.available()
    if use_ref:
        om.RefIndex.set_threads(1)
    ref = (om.RefIndex if use_ref else om.OracleIndex)(path.cold.index.get_size())
    fill = path.cache_fill_ids.cpu().numpy()
    fill_locs = ref.add(fill)
    if use_ref:
        om.RefIndex.set_threads(os.cpu_count() or 1)
    want = ref.lookup(ids_host.numpy())
    runs = E.cudaRunsBuild(ids_dev, path.id_bits, path.class_table, want_uniq=True)
    table = path.table if path.table is not None else None
    rows, locs, found = E.cudaLookupFetchRuns(path.cold.index, runs, path.cold.emb, table, path.shared, mode=path.lookup_mode)
    ok_locs = bool(np.array_equal(locs.cpu().numpy(), want))
    ok_found = bool(np.array_equal(found.cpu().numpy(), want >= 0))
    ok_rows = None
    if table is not None:
        expect = table[ids_dev]
        hit = locs >= 0
        expect[hit] = path.cold.emb[locs[hit]]
        ok_rows = bool(torch.equal(rows, expect))
        del expect
    u, c = np.unique(ids_host.numpy(), return_counts=True)
    U = int(runs.num_unique.item())
    ok_uniq = U == u.size and bool(np.array_equal(runs.uniq_ids[:U].cpu().numpy(), u))
    rs = _as_tensor(runs.desc.run_start, (U + 1,), "<i8", ids_dev.device).cpu().numpy()
    ok_counts = bool(np.array_equal(np.diff(rs), c))
    ok = ok_locs and ok_found and ok_uniq and ok_counts and ok_rows is not False
    return {"ok": ok, "what": f"one batch of {ids_host.numel()} ids at full size before the first step: slots and "
                              f"found mask vs the {'reference compiled CPU index' if use_ref else 'oracle index'} "
                              f"after add() of the {fill.size} cache-fill ids ({int((fill_locs >= 0).sum())} inserted), "
                              "fetched rows vs the torch gather expression, unique ids and counts vs numpy.unique",
            "slots": ok_locs, "found": ok_found, "rows": ok_rows, "unique_ids": ok_uniq, "counts": ok_counts,
            "found_fraction": float((want >= 0).mean())}


def parity_steps(rank, world, dev, exchange, lookup_mode, overlap_fetch=False, remote_fetch="auto") -> dict:
    """Four steps (the second and fourth end with a flush) of a small configuration through the
    same EmbeddingPath on every rank against a numpy simulation of all ranks
    (oracle/pipeline_oracle.py): slots, found masks, index and LRU state, staging state, optimiser
    state and owned table rows."""
    import numpy as np
    import torch
    import torch.distributed as dist

    from hades_b200 import pipeline, synth
    from oracle import build_oracle

    build_oracle.build_oracle()
    from oracle import oracle as om
    from oracle.pipeline_oracle import PipelineOracle, compare_rank

    base = synth.scaled(synth.CONFIG2, 1.0 / 400.0, "parity_small")
    cfg = synth.CacheFetchConfig(base.name, base.config, base.table_rows, 64, base.cache_entries, base.batch,
                                 base.zipf_s, flush_every=2)
    path = pipeline.build_path(cfg, rank, world, dev, lookup_mode=lookup_mode, exchange=exchange, hot_fraction=0.02,
                               remote_fetch=remote_fetch)
    path.overlap_fetch = overlap_fetch
    if path.shared is not None:
        w = path.shared.gather(torch.arange(cfg.table_rows, dtype=torch.int64, device=dev)).cpu().numpy()
    else:
        w = path.table.cpu().numpy()
    orc = PipelineOracle(om, w, path.class_table.cpu().numpy(), cfg.cache_entries, path.cache_fill_ids.cpu().numpy(),
                         world=world, flush_every=cfg.flush_every, miss_cap=path.miss_cap, flush_cap=path.flush_cap)
    sampler = synth.ZipfSampler(cfg.table_rows, cfg.zipf_s)
    err, flushed_total = None, 0
    try:
        for it in range(1, 5):
            both = []
            for r in range(world):
                rng = synth.rng_for(9, r, it)
                both.append((sampler.ids(rng, cfg.batch), synth.normal_rows(rng, cfg.batch, cfg.dim, cfg.grad_sigma)))
            rows, locs, found, st = path.step(torch.from_numpy(both[rank][0]).to(dev),
                                              torch.from_numpy(both[rank][1]).to(dev))
            outs, flushed = orc.step([b[0] for b in both], [b[1] for b in both])
            assert np.array_equal(locs.cpu().numpy(), outs[rank][1]), f"slots differ at step {it}"
            assert np.array_equal(found.cpu().numpy(), outs[rank][2]), f"found mask differs at step {it}"
            np.testing.assert_allclose(rows.cpu().numpy(), outs[rank][0], rtol=1e-4, atol=1e-5)
            assert st.flushed == flushed[rank], f"flushed rows differ at step {it}"
            flushed_total += flushed[rank]
            compare_rank(path, orc, rank, where=f"rank {rank} step {it}")
    except AssertionError as e:
        err = str(e)[:300]
    ok = torch.tensor([0 if err else 1], dtype=torch.int32, device=dev)
    if world > 1:
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    out = {"ok": bool(ok.item()), "what": f"4 steps (2 flushes) of config 2 scaled by 1/400 (dim 64) on {world} "
                                          f"rank(s) vs a numpy simulation of all ranks: slots, found masks, index / LRU "
                                          f"/ staging state bit-exact, optimiser state and owned rows within 1e-4",
           "rows_flushed_rank0": flushed_total}
    if err:
        out["error_rank0"] = err
    path.close()
    del path
    torch.cuda.empty_cache()
    return out


# --------------------------------------------------------------------------------------
# the whole path (config 2 / config 5)
# --------------------------------------------------------------------------------------
def run_path(args, workload: str, steps: int, warmup: int, main_line: bool) -> dict:
    import numpy as np
    import torch
    import torch.distributed as dist

    from hades_b200 import EmbCacheLib as E
    from hades_b200 import _lib, pipeline, synth

    rank, world, dev, timed = dist_setup()
    local_rank = dev.index
    _lib.load()
    mode = E.LOOKUP_SORTED if args.lookup == "sorted" else E.LOOKUP_SETASSOC
    c5 = workload == "c5"
    if c5:
        cfg = synth.CONFIG5 if not args.rmat_bits else synth.scaled_rmat(synth.CONFIG5, args.rmat_bits)
        path = pipeline.build_rmat_path(cfg, rank, world, dev, optimizer=args.optimizer, lookup_mode=mode,
                                        touch_lru=not args.no_lru, exchange=args.exchange,
                                        insert_misses=not args.no_insert, remote_fetch=args.remote_fetch)
        rng = synth.rng_for(5, rank, 1)
        host_batches = [torch.from_numpy(synth.rmat_frontier(cfg, rng)).pin_memory() for _ in range(4)]
    else:
        cfg = synth.CONFIG2 if args.scale == 1.0 else synth.scaled(synth.CONFIG2, args.scale, "config2_scaled")
        path = pipeline.build_path(cfg, rank, world, dev, optimizer=args.optimizer, lookup_mode=mode,
                                   touch_lru=not args.no_lru, exchange=args.exchange,
                                   insert_misses=not args.no_insert, remote_fetch=args.remote_fetch)
        sampler = synth.ZipfSampler(cfg.table_rows, cfg.zipf_s)
        rng = synth.rng_for(2, rank, 1)
        host_batches = [torch.from_numpy(sampler.ids(rng, cfg.batch)).pin_memory() for _ in range(4)]
    path.want_locs = False  # the step needs the slots in sorted order only (a coalesced write)
    # the fetch of a batch beside the aggregation of its gradients: pays when part of the fetch is
    # bound by NVLink round trips (remote rows: 3 % of the step at N = 2, 7 % on configuration 5);
    # neutral on one GPU, where both are HBM-bound
    path.overlap_fetch = args.overlap_fetch != "off"
    dev_batches = [b.to(dev) for b in host_batches]
    gen = torch.Generator(device=dev)
    gen.manual_seed(2000 + rank)
    grads = torch.empty((cfg.batch, cfg.dim), dtype=torch.float32, device=dev)
    grads.normal_(0.0, cfg.grad_sigma, generator=gen)
    out_rows = torch.empty((cfg.batch, cfg.dim), dtype=torch.float32, device=dev)
    stats = synth.stream_stats(host_batches[0].numpy())
    host_found = torch.empty(cfg.batch, dtype=torch.bool).pin_memory()
    ids_stage = torch.empty(cfg.batch, dtype=torch.int64, device=dev)

    parity = None
    if main_line and not args.no_parity:
        if world == 1 and not c5 and args.scale == 1.0:
            parity = parity_full_size(path, dev_batches[0], host_batches[0])
            small = parity_steps(rank, world, dev, args.exchange, mode, path.overlap_fetch, args.remote_fetch)
            parity = {"ok": parity["ok"] and small["ok"], "full_size_batch": parity, "steps_small": small}
        else:
            parity = parity_steps(rank, world, dev, args.exchange, mode, path.overlap_fetch, args.remote_fetch)
        if not parity["ok"]:
            if rank == 0:
                print(json.dumps({"metric": METRIC, "parity_check": parity, "error": "parity self-check failed"}))
            raise SystemExit(3)

    last = {}

    def step_resident(k):
        ids_stage.copy_(dev_batches[k % len(dev_batches)], non_blocking=True)  # 16 MB device copy
        rows, locs, found, st = path.step(ids_stage, grads, out_rows)
        last["found"], last["st"] = found, st

    # e2e: the ids of step k+1 cross PCIe on a copy stream while step k computes, and the found
    # mask of step k-1 goes back on another; every step still pays its own H2D and D2H inside the
    # timed region
    h2d_stream, d2h_stream = torch.cuda.Stream(), torch.cuda.Stream()
    ids_e2e = [torch.empty(cfg.batch, dtype=torch.int64, device=dev) for _ in range(2)]
    h2d_done = [torch.cuda.Event(), torch.cuda.Event()]
    consumed = [torch.cuda.Event(), torch.cuda.Event()]
    pending = {"k": None}
    found_buf = [torch.empty(cfg.batch, dtype=torch.bool, device=dev) for _ in range(2)]
    d2h_done = [torch.cuda.Event(), torch.cuda.Event()]

    def e2e_prefetch(k):
        slot = k % 2
        with torch.cuda.stream(h2d_stream):
            h2d_stream.wait_event(consumed[slot])  # the step that used this buffer has read it
            ids_e2e[slot].copy_(host_batches[k % len(host_batches)], non_blocking=True)
            h2d_done[slot].record(h2d_stream)
        pending["k"] = k

    def step_e2e(k):
        if pending["k"] != k:
            e2e_prefetch(k)
        slot = k % 2
        main = torch.cuda.current_stream()
        main.wait_event(h2d_done[slot])
        e2e_prefetch(k + 1)
        ids_stage.copy_(ids_e2e[slot], non_blocking=True)
        rows, locs, found, st = path.step(ids_stage, grads, out_rows)
        consumed[slot].record(main)
        main.wait_event(d2h_done[slot])  # the read-back of step k-2 has left this result buffer
        found_buf[slot].copy_(found, non_blocking=True)
        done = torch.cuda.Event()
        done.record(main)
        with torch.cuda.stream(d2h_stream):
            d2h_stream.wait_event(done)
            host_found.copy_(found_buf[slot], non_blocking=True)
            d2h_done[slot].record(d2h_stream)

    K = max(steps, 1)
    if cfg.flush_every > 0:
        # a whole number of flush periods: where the window falls cannot bias ms_per_step
        K = max(cfg.flush_every, (K // cfg.flush_every) * cfg.flush_every)
    W = max(warmup, 3)
    launches_eager0 = _lib.launch_count()
    for k in range(W):
        step_resident(k)
    launches_per_step = (_lib.launch_count() - launches_eager0) / W
    use_graph = not args.no_graph and (world == 1 or path.px is not None)
    if use_graph:
        torch.cuda.synchronize()
        path.capture(ids_stage, grads, out_rows)
    # Untimed settling steps in the form that is timed: a GPU that sat idle through the set-up has
    # been seen to run its first few dozen steps up to 12 % slower.  They end on a flush boundary.
    settle = 24
    if cfg.flush_every > 0:
        settle += (-(W + settle)) % cfg.flush_every
    for k in range(W, W + settle):
        step_resident(k)
    sampler_clk = ClockSampler(local_rank)
    if rank == 0 and main_line:
        sampler_clk.start()
    launches0 = _lib.launch_count()
    ms_step = timed(step_resident, K, W + settle)
    launches = _lib.launch_count() - launches0
    if use_graph:
        # kernels replayed from the graph are not seen by the launch counter: count them from
        # the eager warm-up steps (same kernels), plus the eagerly launched flush steps
        launches += int(launches_per_step * K)
    found_frac = float(last["found"].float().mean().item())
    num_unique = int(last["st"].num_unique.item())
    split_counts = last["st"].split_counts.tolist()

    # flush cost: the same number of steps with the flush switched off, right after
    flush_ms = None
    if cfg.flush_every > 0:
        saved = path.flush_every
        path.flush_every = 0
        ms_noflush = timed(step_resident, K, W + settle + K)
        path.flush_every = saved
        path.step_no = 0
        flush_ms = (ms_step - ms_noflush) * cfg.flush_every

    # forward and backward on their own, eager, every rank in step with the others (with several
    # GPUs the forward pass reads the peers' shards while the peers do the same)
    saved = path.flush_every
    path.flush_every = 0

    def fwd_only(k):
        path.forward(ids_stage, out_rows, join=True)

    def bwd_only(k):
        path.backward(ids_stage, grads)

    fwd_only(0)
    breakdown = {"forward_ms": timed(fwd_only, 10), "backward_ms": timed(bwd_only, 10),
                 "what": "eager launches, all ranks in step; forward = sort + lookup/fetch (+ LRU ageing and cache insert "
                         "on the side stream, joined); backward = aggregation, cold accumulate, exchange, owner update"}
    path.flush_every = saved
    path.step_no = 0

    e2e = None
    if not args.no_e2e:
        for k in range(2):
            step_e2e(k)
        torch.cuda.synchronize()
        path.step_no = 0
        pending["k"] = None  # the first timed step pays its own, unhidden, H2D
        e2e_ms = timed(step_e2e, K, W + K, tail=lambda: torch.cuda.current_stream().wait_stream(d2h_stream))
        e2e = {"value": world * cfg.batch / (e2e_ms * 1e-3), "unit": UNIT,
               "h2d_bytes_per_step": cfg.batch * 8, "d2h_bytes_per_step": cfg.batch,
               "ms_per_step": e2e_ms,
               "note": "ids from pinned host memory, found mask read back, both on copy streams overlapped with the "
                       f"previous/next step; the {cfg.batch * cfg.dim * 4} bytes of fetched rows per step are NOT copied "
                       "to the host: they stay on the device for the model, as in the reference (its emb is a CUDA "
                       "tensor, dist_emb.py:199-212); gradients are produced on the device by the backward pass"}
    clocks = sampler_clk.stop() if (rank == 0 and main_line) else None

    # per-stage timing of the dominant kernels, on the launching stream (local kernels only)
    ids0 = dev_batches[0]
    runs0 = E.cudaRunsBuild(ids0, path.id_bits, path.class_table, keep=(False, True, True),
                            caps=(None, path.num_hot_ids, None))
    lib = E._lib.load()
    sharded = path.shared is not None and world > 1
    fetch_ws = path._ws("_fetch_ws", lib.hb_lookup_fetch_runs_workspace_bytes(
        cfg.batch, cfg.dim * 4, int(sharded)))
    st_ms = {
        "sort_runs": time_local(lambda: E.cudaRunsBuild(ids0, path.id_bits, path.class_table, keep=(False, True, True),
                                                        caps=(None, path.num_hot_ids, None), ws=runs0.ws)),
        "segsum": time_local(lambda: E.cudaSegSumRuns(runs0, grads, split_keep=(False, True, True))),
    }
    resolve_ms = None
    if path.px_req is not None:
        # the owners deliver the remote rows: requests, two fences and the owners' stores are part
        # of the fetch, so every rank runs it at the same time (max over ranks)
        path._fetch(runs0, out_rows, fetch_ws)
        st_ms["lookup_fetch"] = timed(lambda k: path._fetch(runs0, out_rows, fetch_ws), 10)
    else:
        st_ms["lookup_fetch"] = time_local(lambda: E.cudaLookupFetchRuns(
            path.cold.index, runs0, path.cold.emb, path.table, path.shared, out_rows, mode, want_locs=False))
        # the per-distinct-id launch alone: index probe (+ at N > 1 remote rows copied once into this GPU's stage)
        resolve_ms = time_local(lambda: E.cudaLookupFetchRuns(path.cold.index, runs0, path.cold.emb, path.table,
                                                              path.shared, None, mode, resolve_only=True))
    no_reuse_ms = None
    if path.shared is None and main_line:
        unif = torch.randint(0, cfg.table_rows, (cfg.batch,), device=dev, generator=gen)
        runs_u = E.cudaRunsBuild(unif, path.id_bits)
        no_reuse_ms = time_local(lambda: E.cudaLookupFetchRuns(path.cold.index, runs_u, path.cold.emb, path.table,
                                                               None, out_rows, mode, want_locs=False))
        del runs_u, unif
    nvlink = None
    if world > 1 and path.px is not None:
        # the per-step push of the hot rows alone: every rank pushes what its last step aggregated
        outs = E.cudaSegSumRuns(runs0, grads, split_keep=(False, True, True))
        h_ids, (h_rows, h_cnt), n_hot = runs0.class_ids[1], outs[1], runs0.class_counts[1:2]
        sent = torch.zeros(world, dtype=torch.int64, device=dev)

        def push(_k):
            path.px.push(h_ids, h_rows, h_cnt, n_hot, sent_counts=sent)
            path.px.fence()

        for k in range(3):
            push(k)
        push_ms = timed(push, 20)
        sent_h = sent.tolist()
        out_bytes = (sum(sent_h) - sent_h[rank]) * (16 + cfg.dim * 4)
        gbs = out_bytes / (push_ms * 1e-3) / 1e9
        nvlink = {"what": "fused pack+push of one step's hot rows to their owners + device fence, rank 0's bytes",
                  "bytes_leaving_gpu": out_bytes, "ms": push_ms, "achieved": gbs, "unit": "GB/s",
                  "frac_of_nominal_900": gbs / NVLINK_NOMINAL_GBS, "frac_of_measured_770": gbs / NVLINK_MEASURED_GBS,
                  "peak_measured_how": "cudaMemcpyPeer of 1 GiB between two GPUs of this pool, per direction",
                  "note": "a few MB per step: bound by the launches of the partition and the fence, not by the links; "
                          "extra.c4_exchange is the bandwidth case"}
    status = _lib.device_status()
    if status != 0:
        raise SystemExit(f"device-side error status {status}")
    dropped = int(path.cold.dropped.item())

    line = None
    if rank == 0:
        peaks = measured_peaks()
        peak = float(peaks.get("hbm_gbs", 6650.0))
        row_bytes = cfg.dim * 4
        lf_bytes = cfg.batch * (8 + 8 + 1) + 2 * cfg.batch * row_bytes
        achieved = lf_bytes / (st_ms["lookup_fetch"] * 1e-3) / 1e9
        seg_bytes = cfg.batch * (8 + row_bytes) + num_unique * (8 + 8 + row_bytes)
        traffic, prov = traffic_capture() if (not c5 and args.scale == 1.0 and args.lookup == "setassoc"
                                              and world == 1) else (None, {"why_null": "captured on config 2, one GPU"})
        stage_ms = st_ms["sort_runs"] + st_ms["lookup_fetch"] + st_ms["segsum"]
        stage_gbs = (lf_bytes + seg_bytes) / (stage_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": world * cfg.batch / (ms_step * 1e-3), "unit": UNIT,
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": (f"config5: R-MAT(0.57,0.19,0.19) 2^{cfg.bits} ({cfg.num_nodes} nodes), "
                                    f"{cfg.seeds} seeds x fanout {list(cfg.fanout)} per GPU, dim {cfg.dim} fp32") if c5
                       else (WORKLOAD if args.scale == 1.0 else f"config2 scaled by {args.scale:g}"),
                       "table_rows": cfg.table_rows, "dim": cfg.dim, "cache_entries": cfg.cache_entries,
                       "batch_per_gpu": cfg.batch, "zipf_s": None if c5 else cfg.zipf_s,
                       "flush_every": cfg.flush_every, "steps_with_flush": K // cfg.flush_every if cfg.flush_every else 0,
                       "flush_ms": flush_ms, "breakdown": breakdown,
                       "lookup": args.lookup, "lru_ageing": not args.no_lru, "insert_cold_misses": not args.no_insert,
                       "cuda_graph": use_graph, "untimed_settling_steps_after_warmup": settle,
                       "fetch_beside_aggregation": path.overlap_fetch,
                       "remote_rows_of_the_fetch": (None if world == 1 else
                                                    "delivered by their owners (requests pushed, rows stored into the "
                                                    "requester's stage, two device fences)" if path.px_req is not None
                                                    else "read by this GPU from the owners' shards, once per distinct id"),
                       "optimizer": "SparseAdam fp32" if args.optimizer == "adam" else "SparseAdagrad fp32",
                       "exchange": "local" if world == 1 else (
                           "nccl all_to_all" if path.px is None else
                           f"fused pack+push over peer memory, {path.px.fence_kind} fence (hot rows and flushed rows)"),
                       "l2": ("145 MB of rows read and written per step (just above L2), 4 frontier batches rotate"
                              if c5 else
                              "inputs larger than L2: 1.0 GB of rows written per step, 4 id batches rotate"),
                       "stream": stats, "found_fraction": found_frac, "unique_per_batch": num_unique,
                       "hot_cold_unique": split_counts[1:3],
                       "cold_gradient_rows_dropped_total": dropped,
                       "note": "found = served by the cold cache: HOT ids (top 1 % of the popularity ranking) are "
                               "never cached and read the authoritative table / owner shard"},
            "roofline": {"bound": "hbm", "kernel": "runs_resolve_kernel + runs_expand_kernel (hb_lookup_fetch_runs: cache "
                                                   "lookup per distinct id + cached fetch over the sorted batch)",
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": "measured" if peaks else "fallback",
                         "algorithmic_bytes": lf_bytes, "ms": st_ms["lookup_fetch"], "traffic": traffic, **prov,
                         "frac_dram": (traffic / (st_ms["lookup_fetch"] * 1e-3) / 1e9 / peak) if traffic else None,
                         "frac_no_reuse": (lf_bytes / (no_reuse_ms * 1e-3) / 1e9 / peak) if no_reuse_ms else None,
                         "no_reuse_ms": no_reuse_ms,
                         "note": "frac counts the duplicate ids of the Zipf stream as algorithmic bytes although "
                                 "their row reads never reach HBM (a duplicate takes its predecessor's registers); "
                                 "frac_dram is what reached HBM over the same time, frac_no_reuse the same kernel on "
                                 "uniform ids (every row read from HBM)",
                         "stage": {"what": "north-star stage: sort of the batch + lookup+fetch + aggregation, summed "
                                           "CUDA-event times of the three calls",
                                   "algorithmic_bytes": lf_bytes + seg_bytes, "ms": stage_ms,
                                   "sort_runs_ms": st_ms["sort_runs"], "lookup_fetch_ms": st_ms["lookup_fetch"],
                                   "resolve_part_of_lookup_fetch_ms": resolve_ms,
                                   "segsum_ms": st_ms["segsum"], "achieved": stage_gbs,
                                   "frac_of_measured": stage_gbs / peak, "frac_of_nominal_8TBs": stage_gbs / HBM_NOMINAL_GBS},
                         "also": {"segsum_gbs": seg_bytes / (st_ms["segsum"] * 1e-3) / 1e9,
                                  "segsum_frac": seg_bytes / (st_ms["segsum"] * 1e-3) / 1e9 / peak}},
            "clocks": clocks, "gpu_launches": int(launches),
        }
        if nvlink:
            line["roofline"]["nvlink"] = nvlink
        if e2e:
            line["e2e"] = e2e
        if parity is not None:
            line["parity_check"] = parity
    path.close()
    del path
    torch.cuda.empty_cache()
    return line


# --------------------------------------------------------------------------------------
# configuration 1
# --------------------------------------------------------------------------------------
def run_c1(args, steps: int, warmup: int) -> dict:
    """Configuration 1 (the case the reference runs on its CPU path): 1,000,000 x 128 fp32 table,
    100,000-entry cache index, 65,536 Zipf(1.1) ids per query: lookup + cached fetch, then the
    set step both ways (overwrite = cudaSet of the reference; accumulate = scatter-add).  The
    whole working set (67 MB of rows per query) fits L2, so the ids are regenerated (4 batches
    rotate) and the numbers are launch- and L2-bound, not HBM-bound."""
    import numpy as np
    import torch

    from hades_b200 import EmbCacheLib as E
    from hades_b200 import _lib, synth

    rank, world, dev, timed = dist_setup()
    cfg = synth.CONFIG1
    rng = synth.rng_for(1, rank, 0)
    table = torch.empty((cfg.table_rows, cfg.dim), device=dev).normal_(0, cfg.table_sigma)
    ix = E.IndexCache(cfg.cache_entries, f"bench_c1_r{rank}", True, False)
    hot = torch.from_numpy(synth.hot_ids(cfg.table_rows, cfg.cache_entries)).to(dev)
    locs = ix.cuda_add(hot)
    cache = torch.zeros((ix.get_capacity(), cfg.dim), device=dev)
    ok = locs >= 0
    cache[locs[ok]] = table[hot[ok]]
    sampler = synth.ZipfSampler(cfg.table_rows, cfg.zipf_s)
    batches = [torch.from_numpy(sampler.ids(rng, cfg.batch)).to(dev) for _ in range(4)]
    stats = synth.stream_stats(batches[0].cpu().numpy())
    grad = torch.empty((cfg.batch, cfg.dim), device=dev).normal_(0, cfg.grad_sigma)
    out = torch.empty((cfg.batch, cfg.dim), device=dev)
    staging = torch.zeros((cfg.table_rows, cfg.dim), device=dev)
    cnt = torch.zeros(cfg.table_rows, dtype=torch.int32, device=dev)
    state = {}

    def fetch(k):
        state["o"] = E.cudaLookupFetch(ix, batches[k % 4], cache, table, out_rows=out)

    def fetch_touch(k):
        rows, l, f = E.cudaLookupFetch(ix, batches[k % 4], cache, table, out_rows=out)
        ix.cuda_touch_lru(l)

    def set_overwrite(k):
        E.cudaSet(grad, staging, batches[k % 4])

    uniq = [torch.unique(b) for b in batches]

    def accumulate(k):
        # scatter-add needs unique destinations: aggregate the duplicates first, then add
        ids = batches[k % 4]
        u, s, c, num = E.cudaUniqueSegSum(ids, grad, id_bits=21, sync=False)
        E.cudaAccumulate(s[: uniq[k % 4].numel()], staging, u[: uniq[k % 4].numel()], cnt)

    W, K = max(warmup, 3), max(steps, 1)
    res = {}
    for name, fn in (("lookup_fetch", fetch), ("lookup_fetch_lru", fetch_touch), ("set_overwrite", set_overwrite),
                     ("aggregate_accumulate", accumulate)):
        for k in range(W):
            fn(k)
        res[name] = timed(fn, K)
    found = float(state["o"][2].float().mean().item())
    status = _lib.device_status()
    row = cfg.dim * 4
    lf_bytes = cfg.batch * 17 + 2 * cfg.batch * row
    return {"workload": "config1: 1,000,000 x 128 fp32 table, 100,000-entry cache, 65,536 Zipf(1.1) ids per query",
            "stream": stats, "found_fraction": found,
            "lookup_fetch_us": res["lookup_fetch"] * 1e3, "lookup_fetch_plus_lru_us": res["lookup_fetch_lru"] * 1e3,
            "set_overwrite_us": res["set_overwrite"] * 1e3, "aggregate_accumulate_us": res["aggregate_accumulate"] * 1e3,
            "rows_per_s_lookup_fetch": world * cfg.batch / (res["lookup_fetch"] * 1e-3),
            "lookup_fetch_algorithmic_gbs": lf_bytes / (res["lookup_fetch"] * 1e-3) / 1e9,
            "note": "67 MB of rows per query fit the 126 MB L2: 4 id batches rotate, numbers are launch- and L2-bound",
            "device_status": status}


# --------------------------------------------------------------------------------------
# configuration 4: the exchange
# --------------------------------------------------------------------------------------
def run_exchange(args, steps: int, warmup: int) -> dict:
    """Configuration 4: owner-partitioned sparse-gradient sync + sparse Adagrad on an fp16 table
    sharded by id % world.  Times the all-to-all alone against the NVLink roofline (bytes that
    leave a GPU / 770 GB/s measured peer copy on this pool; 900 GB/s nominal), three ways, and
    the whole sync (exchange + owner-side merge + Adagrad update on the owning shard)."""
    import numpy as np
    import torch
    import torch.distributed as dist

    from hades_b200 import _lib, synth
    from hades_b200.exchange import PeerExchange
    from hades_b200.sparse_optim import ShardedEmbedding, SparseAdagrad, swap_gradients

    rank, world, dev, timed = dist_setup()
    n, dim = int(1_048_576 * args.scale), 64
    table_rows = int(240_000_000 * args.scale)
    # distinct ids, Zipf(1.1) without replacement, ascending as a rank's local aggregation emits them.
    # The ranking is cut after its 4M most popular ids and spread over the 2.4e8 ids (the exact CDF of
    # the whole table would take 2 GB of host memory in each of 8 processes); rank 0 builds the sampler's
    # table once and the others receive it.
    head = min(table_rows, 4_000_000)
    if world > 1:
        cdf = torch.empty(head, dtype=torch.float64, device=dev)
        if rank == 0:
            cdf.copy_(torch.from_numpy(synth.ZipfSampler(head, 1.1).cdf))
        dist.broadcast(cdf, 0)
        sampler = synth.ZipfSampler.__new__(synth.ZipfSampler)
        sampler.cdf, sampler.num_ids = cdf.cpu().numpy(), head
        del cdf
    else:
        sampler = synth.ZipfSampler(head, 1.1)
    rng = synth.rng_for(4, rank, 0)
    ids_np = np.sort(sampler.unique_ids(rng, n, id_space=table_rows))
    del sampler
    ids = torch.from_numpy(ids_np).to(dev)
    rows = torch.empty((n, dim), device=dev).normal_(0, 1e-3)
    cnt = torch.ones(n, dtype=torch.int64, device=dev)
    sent_to_others = int((ids_np % world != rank).sum())
    bytes_out = sent_to_others * (8 + 8 + dim * 4)
    cap_t = torch.tensor([int(np.bincount(ids_np % world, minlength=world).max() * 1.05) + 16], device=dev)
    if world > 1:
        dist.all_reduce(cap_t, op=dist.ReduceOp.MAX)  # the slabs have one size on every rank
    cap = int(cap_t.item())
    px = PeerExchange(rank, world, cap, dim, torch.float32, dev)                    # device-side fence
    px_nf = PeerExchange(rank, world, cap, dim, torch.float32, dev, fence="nccl")   # all-reduce as the fence
    shard = ShardedEmbedding(table_rows, dim, rank, world, dtype=torch.float16, device=dev, init_sigma=0.01, seed=4)
    opt = SparseAdagrad(shard, lr=0.01)
    id_bits = max(table_rows.bit_length() + 1, 8)

    def do_push(_k):
        px.push(ids, rows, cnt)
        px.fence()

    def do_push_nccl_fence(_k):
        px_nf.push(ids, rows, cnt)
        px_nf.fence()

    def do_nccl(_k):
        swap_gradients(ids, rows, None, 1, world, dev, cnt)

    def do_sync_update(_k):
        parity = px.push(ids, rows, cnt)
        px.fence()
        r_ids, r_rows, r_cnt, seg = px.received(parity)
        opt.update(r_ids, r_rows, r_cnt, is_unique=False, id_bits=id_bits, seg_counts=seg, seg_cap=px.cap,
                   sorted_segments=True)

    W, K = max(warmup, 3), max(steps, 1)
    out = {}
    for name, fn in (("push", do_push), ("push_nccl_fence", do_push_nccl_fence), ("nccl", do_nccl),
                     ("sync_update", do_sync_update)):
        for k in range(W):
            fn(k)
        out[name] = timed(fn, K)
    status = _lib.device_status()
    res = {"workload": "config4: 1,048,576 unique ids x 64 fp32 (+8 B id, 8 B cnt) per rank, "
                       f"fp16 table of {table_rows} x 64 sharded id % world, sparse Adagrad fp32 state",
           "rows_per_rank": n, "bytes_leaving_each_gpu": bytes_out,
           "push_ms": out["push"], "push_nccl_fence_ms": out["push_nccl_fence"], "nccl_ms": out["nccl"],
           "sync_update_ms": out["sync_update"],
           "sync_update_rows_per_s": world * n / (out["sync_update"] * 1e-3), "device_status": status}
    if world > 1:
        res["push_gbs_out_of_each_gpu"] = bytes_out / (out["push"] * 1e-3) / 1e9
        res["nccl_gbs_out_of_each_gpu"] = bytes_out / (out["nccl"] * 1e-3) / 1e9
        res["roofline"] = {"bound": "nvlink", "achieved": res["push_gbs_out_of_each_gpu"], "peak": NVLINK_MEASURED_GBS,
                           "unit": "GB/s", "frac": res["push_gbs_out_of_each_gpu"] / NVLINK_MEASURED_GBS,
                           "peak_source": "measured peer copy on this pool (cudaMemcpyPeer, 1 GiB, per direction)",
                           "nominal_peak": NVLINK_NOMINAL_GBS,
                           "frac_of_nominal": res["push_gbs_out_of_each_gpu"] / NVLINK_NOMINAL_GBS, "traffic": None}
    px.close()
    px_nf.close()
    del px, px_nf, shard, opt
    torch.cuda.empty_cache()
    return res


# --------------------------------------------------------------------------------------
# configuration 3: hot-node local aggregation
# --------------------------------------------------------------------------------------
def run_hot_aggregation(args, steps: int, warmup: int) -> dict:
    """Configuration 3: hot-node local aggregation.  Every GPU holds 524,288 gradient ids,
    Zipf(1.2) over [0, 1e8), with 128-dim fp32 gradients; per GPU sort / unique / segment-sum;
    the rows of the hot ids (top 1 % of the popularity ranking) then go to their owners
    (id % world), which merge what the ranks sent (unique_grads with counts)."""
    import numpy as np
    import torch
    import torch.distributed as dist

    from hades_b200 import EmbCacheLib as E
    from hades_b200 import _lib, synth
    from hades_b200.exchange import PeerExchange

    rank, world, dev, timed = dist_setup()
    nodes = int(100_000_000 * args.scale)
    n, dim = int(524_288 * args.scale), 128
    # the exact CDF over 1e8 ranks is 800 MB: rank 0 builds it, the ids of every rank come from it
    rng = synth.rng_for(3, rank, 0)
    if world > 1:
        buf = torch.empty((4, n), dtype=torch.int64, device=dev)
        if rank == 0:
            sampler = synth.ZipfSampler(nodes, 1.2)
            every = [torch.from_numpy(np.stack([sampler.ids(synth.rng_for(3, r, 0), n) for _ in range(4)]))
                     for r in range(world)]
            del sampler
            for r in range(1, world):
                dist.send(every[r].to(dev), r)
            buf.copy_(every[0])
        else:
            dist.recv(buf, 0)
        batches = [buf[k] for k in range(4)]
    else:
        sampler = synth.ZipfSampler(nodes, 1.2)
        batches = [torch.from_numpy(sampler.ids(rng, n)).to(dev) for _ in range(4)]
        del sampler
    stats = synth.stream_stats(batches[0].cpu().numpy())
    grads = torch.empty((n, dim), device=dev).normal_(0, 1e-3)
    n_hot = max(nodes // 100, 1)
    hot_ranked = synth.rank_to_id(np.arange(n_hot, dtype=np.int64), nodes)
    cls = np.full(nodes, 2, dtype=np.int8)
    cls[hot_ranked] = 1
    table = torch.from_numpy(cls).to(dev)
    cap = int(np.bincount(hot_ranked % world, minlength=world).max())
    cap = min(cap, n)
    del cls, hot_ranked
    px = PeerExchange(rank, world, cap, dim, torch.float32, dev) if world > 1 else None
    id_bits = max(nodes.bit_length() + 1, 8)
    state = {"k": 0}
    ws = None

    ids_buf = torch.empty(n, dtype=torch.int64, device=dev)

    def local_body():
        runs = E.cudaRunsBuild(ids_buf, id_bits, table, keep=(False, True, False), caps=(None, min(n_hot, n), None),
                               ws=state.get("ws"))
        state["ws"] = runs.ws
        outs = E.cudaSegSumRuns(runs, grads, split_keep=(False, True, False))
        state["runs"], state["hot"] = runs, outs[1]

    def local_only(_k):
        # the dozen launches of the local aggregation are replayed from a CUDA graph once it exists
        ids_buf.copy_(batches[state["k"] % 4], non_blocking=True)
        state["k"] += 1
        if state.get("graph") is not None:
            state["graph"].replay()
        else:
            local_body()

    def with_reduction(_k):
        local_only(_k)
        runs = state["runs"]
        h_ids, (h_rows, h_cnt), n_h = runs.class_ids[1], state["hot"], runs.class_counts[1:2]
        if px is None:
            state["merged"] = E.cudaUniqueSegSum(h_ids, h_rows, h_cnt, mean=True, id_bits=id_bits, sync=False, n_dev=n_h)
        else:
            parity = px.push(h_ids, h_rows, h_cnt, n_h)
            px.fence()
            r_ids, r_rows, r_cnt, seg = px.received(parity)
            # every slab holds its sender's ascending unique hot ids: a merge, not a sort
            state["merged"] = E.cudaMergeSortedSlabs(r_ids, r_rows, r_cnt, seg, px.cap, mean=True)

    W, K = max(warmup, 3), max(steps, 1)
    out = {}
    for k in range(W):  # eager first: every lazy allocation happens before the capture
        local_only(k)
    torch.cuda.synchronize()
    if not args.no_graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            local_body()
        state["graph"] = g
    for name, fn in (("local", local_only), ("local_plus_hot_reduction", with_reduction)):
        for k in range(W):
            fn(k)
        out[name] = timed(fn, K)
    uniq = int(state["runs"].num_unique.item())
    hot_u = int(state["runs"].class_counts[1].item())
    merged = int(state["merged"][3].item())
    status = _lib.device_status()
    peaks = measured_peaks()
    peak = float(peaks.get("hbm_gbs", 6650.0))
    alg = n * (8 + dim * 4) + uniq * 16 + hot_u * dim * 4
    res = {"workload": f"config3: {n} ids per GPU, Zipf(1.2) over {nodes}, dim 128 fp32, hot = top 1 %",
           "rows_per_s": world * n / (out["local_plus_hot_reduction"] * 1e-3),
           "ms_per_step": out["local_plus_hot_reduction"], "local_aggregation_ms": out["local"],
           "stream": stats, "unique": uniq, "hot_unique": hot_u, "owned_after_reduction": merged,
           "exchange": "local" if world == 1 else "fused pack+push over peer memory, device fence",
           "cuda_graph": "local aggregation replayed from a graph" if state.get("graph") is not None else "none",
           "roofline": {"bound": "hbm", "kernel": "local aggregation (sort + run heads + segment-sum, hot rows kept)",
                        "achieved": alg / (out["local"] * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                        "frac": alg / (out["local"] * 1e-3) / 1e9 / peak,
                        "peak_source": "measured" if peaks else "fallback", "traffic": None},
           "device_status": status}
    if px is not None:
        px.close()
    state.clear()
    del px, table, state
    torch.cuda.empty_cache()
    return res


# --------------------------------------------------------------------------------------
# the reference's own CUDA operators beside this library's
# --------------------------------------------------------------------------------------
def run_ref_kernels(args) -> dict:
    """The reference's CUDA operators (src/cuda/uva_fetch.cu, uva_set.cu, split.cu), compiled from its
    own sources for sm_100a (oracle/build_oracle.py), against this library's on the same GPU, same
    inputs, configuration-2 shapes: CUDA events (the reference launches on the legacy default stream,
    which is torch's default stream), outputs compared bit for bit."""
    import torch

    from hades_b200 import EmbCacheLib as E
    from hades_b200 import synth
    from oracle import oracle as om

    if not om.RefCuda.available():
        return {"unavailable": "oracle/_ref/libhades_ref_cuda.so is not built (run oracle/build_oracle.py where the "
                               "reference checkout is present)"}
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    cfg = synth.CONFIG2 if args.scale == 1.0 else synth.scaled(synth.CONFIG2, args.scale)
    n, d, rows = cfg.batch, cfg.dim, cfg.table_rows
    g = torch.Generator(device=dev).manual_seed(7)
    table = torch.randn((rows, d), device=dev, generator=g)
    cached = torch.randn((cfg.cache_entries, d), device=dev, generator=g)
    index_map = torch.full((rows,), -1, dtype=torch.int64, device=dev)
    index_map[torch.randperm(rows, device=dev, generator=g)[: cfg.cache_entries]] = torch.arange(cfg.cache_entries, device=dev)
    idx = torch.randperm(rows, device=dev, generator=g)[:n]          # unique, as the reference's tests use
    di = torch.randperm(n, device=dev, generator=g)
    src = torch.randn((n, d), device=dev, generator=g)
    mask = torch.randint(0, 3, (rows,), device=dev, generator=g).to(torch.int8)
    zipf = torch.from_numpy(synth.ZipfSampler(rows, cfg.zipf_s).ids(synth.rng_for(2, 0, 1), n)).to(dev)
    out_a, out_b = torch.zeros((n, d), device=dev), torch.zeros((n, d), device=dev)
    res = {}

    def both(name, ours, theirs, check, nbytes):
        ok = check()
        ms_o, ms_r = time_local(ours, 10), time_local(theirs, 10)
        res[name] = {"ours_us": ms_o * 1e3, "reference_us": ms_r * 1e3, "speedup": ms_r / ms_o, "bit_exact": bool(ok),
                     "ours_gbs": nbytes / (ms_o * 1e-3) / 1e9, "reference_gbs": nbytes / (ms_r * 1e-3) / 1e9}

    lib = om.RefCuda._load()
    P = om.RefCuda._p
    import ctypes as C

    def ref_call(name, *a):  # no synchronisation: timed with events on the default stream
        getattr(lib, f"ref_cuda_{name}")(*a)

    i64, i32 = C.c_int64, C.c_int
    row = 2 * n * d * 4

    def chk_fetch2():
        E.cudaFetch2(table, idx, out_a)
        om.RefCuda.fetch2(table, idx, out_b)
        return torch.equal(out_a, out_b)

    both("cudaFetch2 (unique random rows)", lambda: E.cudaFetch2(table, idx, out_a),
         lambda: ref_call("fetch2", P(table), i64(rows), P(idx), P(out_b), i64(n), i64(d), i32(4), i32(8)),
         chk_fetch2, row + n * 8)

    def chk_fetch():
        out_a.zero_(); out_b.zero_()
        E.cudaFetch(table, idx, out_a, di)
        om.RefCuda.fetch(table, idx, out_b, di)
        return torch.equal(out_a, out_b)

    both("cudaFetch (src and dst index)", lambda: E.cudaFetch(table, idx, out_a, di),
         lambda: ref_call("fetch", P(table), i64(rows), P(idx), P(out_b), i64(n), P(di), i64(n), i64(d), i32(4), i32(8)),
         chk_fetch, row + n * 16)

    def chk_cached():
        E.cudaFetchWithCache2(table, cached, zipf, index_map, out_a)
        om.RefCuda.fetch_with_cache2(table, cached, zipf, index_map, out_b)
        return torch.equal(out_a, out_b)

    both("cudaFetchWithCache2 (Zipf ids, dense index map)",
         lambda: E.cudaFetchWithCache2(table, cached, zipf, index_map, out_a),
         lambda: ref_call("fetch_with_cache2", P(table), i64(rows), P(cached), i64(cfg.cache_entries), P(zipf),
                          P(index_map), P(out_b), i64(n), i64(d), i32(4), i32(8)),
         chk_cached, row + n * 16)
    ta, tb = table.clone(), table.clone()

    def chk_set():
        E.cudaSet(src, ta, idx)
        om.RefCuda.set(src, tb, idx)
        return torch.equal(ta, tb)

    both("cudaSet (unique random rows)", lambda: E.cudaSet(src, ta, idx),
         lambda: ref_call("set", P(src), P(tb), i64(rows), P(idx), i64(n), i64(d), i32(4), i32(8)),
         chk_set, row + n * 8)

    def chk_combine():
        E.cudaCombine(src, out_a, di)
        om.RefCuda.combine(src, out_b, di)
        return torch.equal(out_a, out_b)

    both("cudaCombine", lambda: E.cudaCombine(src, out_a, di),
         lambda: ref_call("combine", P(src), P(out_b), i64(n), P(di), i64(n), i64(d), i32(4), i32(8)),
         chk_combine, row + n * 8)
    del ta, tb
    masks_r = [torch.zeros(n, dtype=torch.bool, device=dev) for _ in range(3)]

    def chk_split():
        return all(torch.equal(x, y) for x, y in zip(E.cudaSplit(zipf, mask), om.RefCuda.split(zipf, mask)))

    both("cudaSplit (three masks)", lambda: E.cudaSplit(zipf, mask),
         lambda: ref_call("split", P(zipf), i64(n), P(mask), i64(rows), P(masks_r[0]), P(masks_r[1]), P(masks_r[2])),
         chk_split, n * 12)
    return {"workload": f"reference CUDA operators vs this library, {n} rows of {d} fp32, table {rows} rows",
            "operators": res,
            "cudalookup": {"unavailable": "lanes of the reference's lookupkernel2 return before a warp-wide "
                                          "cooperative-groups reduce (src/cache/lookup.cu:28,36): undefined behaviour, "
                                          "not run on a shared GPU"}}


# --------------------------------------------------------------------------------------
# single operators
# --------------------------------------------------------------------------------------
def run_micro(update_only: bool) -> None:
    """Single operators at configuration-2 shapes (2M rows of 128 fp32), CUDA events, 20 repetitions
    after a warm-up call; prints a table, not a JSON line.  `micro_update`: only the small cases
    (sparse Adam on 84,000 random rows, the flush of a 4M-slot staging table with 6 % stale rows,
    the owner-side merge of 8 sorted slabs against the sorting path); a few GB on the device."""
    import torch

    from hades_b200 import EmbCacheLib as E
    from hades_b200 import _lib, synth

    torch.cuda.set_device(0)
    dev = "cuda"
    _time = lambda fn: time_local(fn, 20)
    if update_only:
        from hades_b200.cold_cache import StagingTable
        from hades_b200.sparse_optim import ShardedEmbedding, SparseAdam

        g = torch.Generator(device=dev).manual_seed(1)
        rows, dim, n = 2_000_000, 128, 84_000
        opt = SparseAdam(ShardedEmbedding(rows, dim, init_sigma=0.01), lr=0.01)
        ids = torch.sort(torch.randperm(rows, device=dev, generator=g)[:n])[0]
        grads = torch.empty((n, dim), device=dev).normal_(0, 1e-3, generator=g)
        cnt = torch.randint(1, 5, (n,), device=dev, generator=g)
        flush = torch.empty(64 << 20, dtype=torch.float32, device=dev)
        best = 1e9
        for k in range(5):
            flush.fill_(k)  # 256 MB written: nothing of the table is left in L2
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            opt.update(ids, grads, cnt, is_unique=True)
            b.record()
            torch.cuda.synchronize()
            if k:
                best = min(best, a.elapsed_time(b))
        print(f"sparse Adam, {n} rows of {dim} fp32      {best * 1e3:8.1f} us  {n * (dim * 4 * 7 + 24) / best / 1e6:8.0f} GB/s")
        del opt, flush
        slots = 4_000_000
        st = StagingTable(slots, dim, dev)
        stale = torch.randperm(slots, device=dev, generator=g)[: slots * 6 // 100]
        best = 1e9
        for k in range(4):
            st.cnt[stale] = 20
            st.idx[stale] = stale
            st.grad[stale] = 1.0
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            out = st.flush(None, 16, 1, sync=False, out_cap=1 << 19)
            b.record()
            torch.cuda.synchronize()
            if k:
                best = min(best, a.elapsed_time(b))
        m = int(out[3].sum().item())
        print(f"staging flush, {m} of {slots} slots stale  {best * 1e3:8.1f} us  "
              f"{(m * (3 * dim * 4 + 16) + slots * 12) / best / 1e6:8.0f} GB/s   (includes the allocation of the outputs)")
        del st, out
        w, cap = 8, 25_000
        s_ids = torch.full((w, cap), -1, dtype=torch.int64, device=dev)
        counts = torch.randint(cap * 3 // 4, cap + 1, (w,), device=dev, generator=g)
        for s in range(w):
            c = int(counts[s])
            s_ids[s, :c] = torch.sort(torch.randperm(200_000, device=dev, generator=g)[:c])[0]
        s_rows = torch.randn((w * cap, dim), device=dev, generator=g)
        s_cnt = torch.randint(1, 5, (w * cap,), device=dev, generator=g)
        ms_merge = _time(lambda: E.cudaMergeSortedSlabs(s_ids.view(-1), s_rows, s_cnt, counts, cap))
        ms_sort = _time(lambda: E.cudaUniqueSegSum(s_ids.view(-1), s_rows, s_cnt, mean=True, id_bits=20, sync=False,
                                                   seg_counts=counts, seg_cap=cap))
        print(f"owner merge of {w} sorted slabs ({int(counts.sum())} rows): merge {ms_merge * 1e3:.1f} us, "
              f"sorting path {ms_sort * 1e3:.1f} us")
        print("device status", _lib.device_status())
        return
    cfg = synth.CONFIG2
    n, d = cfg.batch, cfg.dim
    row = d * 4
    table = torch.randn((cfg.table_rows, d), device=dev)
    out = torch.empty((n, d), device=dev)
    src = torch.randn((n, d), device=dev)
    idx = torch.randperm(cfg.table_rows, device=dev)[:n]
    print(f"shapes: n={n} rows of {row} B, table {cfg.table_rows} rows, cache {cfg.cache_entries} entries")
    ms = _time(lambda: out.copy_(src))
    print(f"torch copy (sequential)            {ms * 1e3:8.1f} us  {2 * n * row / ms / 1e6:8.0f} GB/s")
    for name, mv in (("lsu", E.MOVER_LSU), ("bulk", E.MOVER_BULK)):
        ms = _time(lambda: E.cudaFetch2(table, idx, out, mover=mv))
        print(f"gather unique random rows, {name:4s}     {ms * 1e3:8.1f} us  {2 * n * row / ms / 1e6:8.0f} GB/s")
        ms = _time(lambda: E.cudaSet(src, table, idx, mover=mv))
        print(f"scatter unique random rows, {name:4s}    {ms * 1e3:8.1f} us  {2 * n * row / ms / 1e6:8.0f} GB/s")
    ix = E.IndexCache(cfg.cache_entries, "microbench", True, False)
    ix.cuda_add(torch.from_numpy(synth.hot_ids(cfg.table_rows, cfg.cache_entries)).to(dev))
    ix.build_sorted()
    cache = torch.randn((ix.get_capacity(), d), device=dev)
    zipf = torch.from_numpy(synth.ZipfSampler(cfg.table_rows, cfg.zipf_s).ids(synth.rng_for(2, 0, 1), n)).to(dev)
    unif = torch.randint(0, cfg.table_rows, (n,), device=dev)
    grads = torch.randn((n, d), device=dev) * 1e-3
    bits = int(cfg.table_rows).bit_length() + 1
    for qn, q in (("zipf(1.2)", zipf), ("uniform", unif)):
        for mode, mname in ((E.LOOKUP_SETASSOC, "set-assoc"), (E.LOOKUP_SORTED, "sorted")):
            ms = _time(lambda: ix.cuda_lookup_found(q, mode))
            print(f"lookup {qn:9s} {mname:9s}               {ms * 1e3:8.1f} us  {n / ms / 1e6:8.2f} G ids/s")
            ms = _time(lambda: E.cudaLookupFetch(ix, q, cache, table, out_rows=out, mode=mode, mover=E.MOVER_LSU))
            print(f"lookup+fetch {qn:9s} {mname:9s}         {ms * 1e3:8.1f} us  {(n * 17 + 2 * n * row) / ms / 1e6:8.0f} GB/s")
            runs = E.cudaRunsBuild(q, bits)
            ms = _time(lambda: E.cudaLookupFetchRuns(ix, runs, cache, table, out_rows=out, mode=mode))
            print(f"lookup+fetch over runs {qn:9s} {mname:9s} {ms * 1e3:6.1f} us  {(n * 17 + 2 * n * row) / ms / 1e6:8.0f} GB/s")
        ms = _time(lambda: E.cudaRunsBuild(q, bits, ws=runs.ws))
        print(f"sort + run heads {qn:9s}                 {ms * 1e3:8.1f} us")
        ms = _time(lambda: E.cudaSegSumRuns(runs, grads))
        print(f"segment-sum over runs {qn:9s}            {ms * 1e3:8.1f} us")
        ms = _time(lambda: E.cudaUniqueSegSum(q, grads, id_bits=bits, sync=False))
        print(f"unique+segment-sum {qn:9s}               {ms * 1e3:8.1f} us")
        locs = ix.cudalookup(q)
        ms = _time(lambda: ix.cuda_touch_lru(locs))
        print(f"LRU ageing by sort {qn:9s}               {ms * 1e3:8.1f} us")
        ms = _time(lambda: ix.cuda_touch_lru_runs(locs, runs))
        print(f"LRU ageing from runs {qn:9s}             {ms * 1e3:8.1f} us  (grouping taken from the step's sort)")
    print("device status", _lib.device_status())


# --------------------------------------------------------------------------------------
def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    rank, world, dev, timed = dist_setup()
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    wl = args.workload
    if wl in ("config2", "c5"):
        line = run_path(args, wl, args.steps, args.warmup, main_line=True)
        if wl == "config2" and not args.no_extra and args.scale == 1.0:
            extra = {}
            short = argparse.Namespace(**{**vars(args), "no_e2e": True})
            for name, fn in (("c1", lambda: run_c1(args, 50, 5)),
                             ("c3", lambda: run_hot_aggregation(args, 30, 5)),
                             ("c4_exchange", lambda: run_exchange(args, 20, 5)),
                             ("c5", lambda: run_path(short, "c5", 40, 5, main_line=False))):
                try:
                    t0 = time.perf_counter()
                    r = fn()
                    if rank == 0 and r is not None:
                        if name == "c5":  # keep the leg's headline figures
                            r = {"workload": r["config"]["workload"], "rows_per_s": r["value"],
                                 "ms_per_step": r["ms_per_step"], "found_fraction": r["config"]["found_fraction"],
                                 "unique_per_batch": r["config"]["unique_per_batch"],
                                 "lookup_fetch_frac_of_measured_hbm": r["roofline"]["frac"],
                                 "flush_ms": r["config"]["flush_ms"]}
                        r["leg_wall_s"] = time.perf_counter() - t0
                        extra[name] = r
                except Exception as e:  # noqa: BLE001  (a leg must not take the headline down)
                    if rank == 0:
                        extra[name] = {"error": f"{type(e).__name__}: {e}"[:300]}
                    if world > 1:
                        # ranks would fall out of step with one another: stop here, but not without the
                        # headline that has already been measured
                        if rank == 0:
                            line["extra"] = extra
                            print(json.dumps(line), flush=True)
                        raise
            if rank == 0:
                line["extra"] = extra
        if rank == 0:
            if world == 1 and not args.no_cpu_baseline and wl == "config2":
                scale, why = cpu_sample_scale()
                r = cpu_reference_run(3 if scale == 1.0 else 4, 1, scale)
                line["cpu_baseline"] = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")}
            print(json.dumps(line))
    else:
        fn = {"c1": run_c1, "c3": run_hot_aggregation, "c4_exchange": run_exchange}[wl]
        r = fn(args, args.steps, args.warmup)
        if rank == 0:
            head = {"c1": ("lookup_fetch_rows_per_s_config1", "rows/s", r.get("rows_per_s_lookup_fetch")),
                    "c3": ("gradient_rows_per_s_local_aggregation_plus_hot_reduction", "rows/s", r.get("rows_per_s")),
                    "c4_exchange": ("sparse_grad_all_to_all_GBps_per_gpu_out", "GB/s",
                                    r.get("push_gbs_out_of_each_gpu"))}[wl]
            print(json.dumps({"metric": head[0], "unit": head[1], "value": head[2], "n_gpus": world,
                              "steps": args.steps, "warmup": max(args.warmup, 3), "higher_is_better": True,
                              "scaling": "weak", "data": "synthetic", "dtype": "f32", "config": {"workload": r["workload"]},
                              **{k: v for k, v in r.items() if k != "workload"}}))
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "ref_kernels":
        print(json.dumps(run_ref_kernels(args)))
    elif args.workload in ("micro", "micro_update"):
        run_micro(args.workload == "micro_update")
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
