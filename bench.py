#!/usr/bin/env python
"""Benchmark of the embedding-cache / sparse-gradient hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" = one pass of the whole path over one batch of synthetic ids on every GPU:
fused cache lookup + cached fetch (+ LRU ageing), local aggregation (sort / unique /
segment-sum), hot/cold split, cold-cache accumulate, owner-partitioned exchange of the hot
rows + optimiser update on the owner, and every 8th step the cold-cache flush and refill.
The workload is configuration 2 of the baseline (20M x 128 fp32 table, 4M-entry hot cache,
2M Zipf(1.2) ids per step and GPU); per-GPU work is fixed as N grows ("weak" scaling).

Prints ONE JSON line (rank 0).  `value` is timed with the batch already in HBM; `e2e` times
the same step with the ids arriving from pinned host memory and the found mask and slots
read back to the host.  `--impl reference` times the reference's own CPU path (its compiled
index + the torch CPU expressions it uses) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "embedding_rows_per_s_lookup_fetch_aggregate_sync"
UNIT = "rows/s"
WORKLOAD = "config2: table 20M x 128 fp32, hot cache 4M, batch 2M Zipf(1.2) per GPU, flush every 8 steps"
CPU_SAMPLE_SCALE = 1.0 / 8.0


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--scale", type=float, default=1.0, help="shrink the workload (profiling captures)")
    ap.add_argument("--lookup", default="setassoc", choices=["setassoc", "sorted"])
    ap.add_argument("--mover", default="auto", choices=["auto", "lsu", "bulk"])
    ap.add_argument("--no-lru", action="store_true", help="skip the LRU ageing passes")
    ap.add_argument("--workload", default="config2", choices=["config2", "c3", "c4_exchange", "c5"],
                    help="config2: the whole path (default); c3: hot-node local aggregation + reduction of "
                         "the hot ids across GPUs (524,288 ids per GPU, Zipf(1.2) over 1e8); c4_exchange: the "
                         "owner-partitioned sync at configuration-4 shapes (1,048,576 unique ids x 64 fp32 per "
                         "rank) and the Adagrad update on the fp16 shard; "
                         "c5: the whole path on the frontier of a sampled 2-layer GraphSAGE step over a "
                         "synthetic R-MAT graph (1e8 nodes, 1,024 seeds, fanout [25, 10], per GPU)")
    ap.add_argument("--optimizer", default="adam", choices=["adam", "adagrad"])
    ap.add_argument("--rmat-bits", type=int, default=0, help="c5 on a smaller graph of 2**bits vertices")
    ap.add_argument("--exchange", default="push", choices=["push", "push_nccl_fence", "nccl"],
                    help="N>1: fused pack+push over peer memory with the device-side fence (default) or "
                         "with an NCCL all-reduce as the fence, or NCCL all_to_all_single")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel eagerly (no CUDA graph)")
    return ap.parse_args()


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
    """The path as the reference runs it on CPU tensors: IndexCache.lookup (its compiled C++
    index, OpenMP), torch CPU gathers for the fetch (test/test_cached_fetch.py:33-36),
    only_unique_grads (python/EmbCache/sparse_optim.py:132-139), the server's accumulate
    and flush (python/EmbCache/server.py:346-574) and SparseAdam.update (:590-685).
    oracle/ is used here as the thing measured ONLY in this baseline leg."""
    import numpy as np
    import torch

    from hades_b200 import synth
    from oracle import oracle as om

    cfg = synth.scaled(synth.CONFIG2, scale, "config2_cpu_sample")
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
    hot = synth.hot_ids(cfg.table_rows, cfg.cache_entries)
    if use_ref:
        om.RefIndex.set_threads(1)  # add() depends on thread timing otherwise
    locs = index.add(hot)
    if use_ref:
        om.RefIndex.set_threads(threads)
    slots = index.get_capacity()
    cache = torch.zeros((slots, cfg.dim))
    ok = torch.from_numpy(locs >= 0)
    cache[torch.from_numpy(locs)[ok]] = table[torch.from_numpy(hot)[ok]]
    n_hot = max(int(cfg.table_rows * 0.01), 1)
    cls = torch.full((cfg.table_rows,), 2, dtype=torch.int8)
    cls[torch.from_numpy(synth.rank_to_id(np.arange(n_hot, dtype=np.int64), cfg.table_rows))] = 1
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
        l = torch.from_numpy(index.lookup(ids.numpy()))
        found = l >= 0
        out = torch.empty((ids.numel(), cfg.dim))
        out[found] = cache[l[found]]
        out[~found] = table[ids[~found]]
        u, inv, c = torch.unique(ids, return_inverse=True, return_counts=True)
        s = torch.zeros((u.numel(), cfg.dim))
        s.index_add_(0, inv, grads)
        kind = cls[u]
        hu, hs, hc = u[kind == 1], s[kind == 1], c[kind == 1]
        cu, cs = u[kind == 2], s[kind == 2]
        cl = torch.from_numpy(index.lookup(cu.numpy()))
        hit = cl >= 0
        sl = cl[hit]
        idx_buf[sl] = cu[hit]
        grad_buf[sl] += cs[hit]
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
                nl = torch.from_numpy(index.add(fid.numpy()))
                okk = nl >= 0
                cache[nl[okk]] = table[fid[okk]]
        return out

    for k in range(warmup):
        one_step(k)
    t0 = time.perf_counter()
    for k in range(warmup, warmup + steps):
        one_step(k)
    dt = time.perf_counter() - t0
    return {"value": cfg.batch * steps / dt, "unit": UNIT, "cores": threads,
            "kind": "reference" if use_ref else "port",
            "sample": f"config2 scaled by {scale:g} (table {cfg.table_rows} x {cfg.dim}, cache "
                      f"{cfg.cache_entries}, batch {cfg.batch}), {steps} steps after {warmup} warm-up",
            "ms_per_step": dt / steps * 1e3}


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = min(max(args.steps, 1), 40)  # each step is a bounded CPU sample; keep the run to minutes
    r = cpu_reference_run(steps, max(args.warmup, 1), CPU_SAMPLE_SCALE)
    line = {
        "impl": "reference", "metric": METRIC, "value": r["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": max(args.warmup, 1), "ms_per_step": r["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": WORKLOAD, "sample": r["sample"]},
        "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": r["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------
def run_ours(args) -> None:
    import numpy as np
    import torch
    import torch.distributed as dist

    from hades_b200 import EmbCacheLib as E
    from hades_b200 import _lib, pipeline, synth

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.load()

    mode = E.LOOKUP_SORTED if args.lookup == "sorted" else E.LOOKUP_SETASSOC
    mover = {"auto": E.MOVER_AUTO, "lsu": E.MOVER_LSU, "bulk": E.MOVER_BULK}[args.mover]
    c5 = args.workload == "c5"
    if c5:
        cfg = synth.CONFIG5 if not args.rmat_bits else synth.scaled_rmat(synth.CONFIG5, args.rmat_bits)
        path = pipeline.build_rmat_path(cfg, rank, world, dev, optimizer=args.optimizer, lookup_mode=mode,
                                        mover=mover, touch_lru=not args.no_lru, exchange=args.exchange)
        rng = synth.rng_for(5, rank, 1)
        host_batches = [torch.from_numpy(synth.rmat_frontier(cfg, rng)).pin_memory() for _ in range(4)]
    else:
        cfg = synth.CONFIG2 if args.scale == 1.0 else synth.scaled(synth.CONFIG2, args.scale, "config2_scaled")
        path = pipeline.build_path(cfg, rank, world, dev, optimizer=args.optimizer, lookup_mode=mode, mover=mover,
                                   touch_lru=not args.no_lru, exchange=args.exchange)
        sampler = synth.ZipfSampler(cfg.table_rows, cfg.zipf_s)
        rng = synth.rng_for(2, rank, 1)
        host_batches = [torch.from_numpy(sampler.ids(rng, cfg.batch)).pin_memory() for _ in range(4)]
    dev_batches = [b.to(dev) for b in host_batches]
    gen = torch.Generator(device=dev)
    gen.manual_seed(2000 + rank)
    grads = torch.empty((cfg.batch, cfg.dim), dtype=torch.float32, device=dev)
    grads.normal_(0.0, cfg.grad_sigma, generator=gen)
    out_rows = torch.empty((cfg.batch, cfg.dim), dtype=torch.float32, device=dev)
    stats = synth.stream_stats(host_batches[0].numpy())
    host_found = torch.empty(cfg.batch, dtype=torch.bool).pin_memory()
    ids_stage = torch.empty(cfg.batch, dtype=torch.int64, device=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, first, tail=None):
        """K steps between CUDA events on the current stream, barrier + synchronize on both
        sides; returns the max over ranks in ms.  tail: joins side streams before the end event."""
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for k in range(first, first + steps):
            fn(k)
        if tail:
            tail()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    last = {}

    def step_resident(k):
        ids_stage.copy_(dev_batches[k % len(dev_batches)], non_blocking=True)  # 16 MB device copy
        rows, locs, found, st = path.step(ids_stage, grads, out_rows)
        last["found"], last["st"] = found, st

    # e2e: the ids of step k+1 cross PCIe on a copy stream while step k computes, and the found
    # mask and slots of step k-1 go back on another; every step still pays its own H2D and D2H
    # inside the timed region
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
        rows, locs, found, st = path.step(ids_e2e[slot], grads, out_rows)
        consumed[slot].record(main)
        main.wait_event(d2h_done[slot])  # the read-back of step k-2 has left this result buffer
        found_buf[slot].copy_(found, non_blocking=True)
        done = torch.cuda.Event()
        done.record(main)
        with torch.cuda.stream(d2h_stream):
            d2h_stream.wait_event(done)
            host_found.copy_(found_buf[slot], non_blocking=True)
            d2h_done[slot].record(d2h_stream)

    # per-stage timing of the dominant kernels, on the launching stream
    def stage_times(k, reps=5):
        ids = dev_batches[k % len(dev_batches)]
        out = {}
        ev = lambda: torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        for name, fn in (
            ("lookup_fetch", (lambda: path.shared.lookup_fetch(path.cold.index, ids, path.cold.emb, out_rows, mode))
             if path.shared is not None else
             (lambda: E.cudaLookupFetch(path.cold.index, ids, path.cold.emb, path.table,
                                        out_rows=out_rows, mode=mode, mover=mover))),
            ("unique_segsum", lambda: E.cudaUniqueSegSum(ids, grads, id_bits=path.id_bits, sync=False)),
        ):
            fn()
            a, b = ev(), ev()
            a.record()
            for _ in range(reps):
                fn()
            b.record()
            torch.cuda.synchronize()
            out[name] = a.elapsed_time(b) / reps
        return out

    W, K = max(args.warmup, 3), max(args.steps, 1)
    launches_eager0 = _lib.launch_count()
    for k in range(W):
        step_resident(k)
    launches_per_step = (_lib.launch_count() - launches_eager0) / W
    # N > 1: graphs around the exchange, the push and its fence stay eager (see EmbeddingPath.capture)
    use_graph = not args.no_graph and (world == 1 or path.px is not None)
    if use_graph:
        torch.cuda.synchronize()
        path.capture(ids_stage, grads, out_rows)
    # Untimed settling steps in the form that is timed (graph replays when graphs are used): the
    # timed region is a fraction of a second, and a GPU that sat idle through the set-up has been
    # seen to run its first few dozen steps up to 12 % slower.
    settle = 24
    for k in range(W, W + settle):
        step_resident(k)
    sampler_clk = ClockSampler(local_rank)
    if rank == 0:
        sampler_clk.start()
    launches0 = _lib.launch_count()
    total_ms = timed(step_resident, K, W + settle)
    launches = _lib.launch_count() - launches0
    if use_graph:
        # kernels replayed from the graph are not seen by the launch counter: count them from
        # the eager warm-up steps (same kernels), plus the eagerly launched flush steps
        launches += int(launches_per_step * K)
    found_frac = float(last["found"].float().mean().item())
    num_unique = int(last["st"].num_unique.item())
    split_counts = last["st"].split_counts.tolist()

    e2e = None
    if not args.no_e2e:
        for k in range(2):
            step_e2e(k)
        torch.cuda.synchronize()
        pending["k"] = None  # the first timed step pays its own, unhidden, H2D
        e2e_ms = timed(step_e2e, K, W + K,
                       tail=lambda: torch.cuda.current_stream().wait_stream(d2h_stream))
        e2e = {"value": world * cfg.batch * K / (e2e_ms * 1e-3), "unit": UNIT,
               "h2d_bytes_per_step": cfg.batch * 8, "d2h_bytes_per_step": cfg.batch,
               "ms_per_step": e2e_ms / K,
               "note": "ids from pinned host memory, found mask read back (the fetched rows stay on the device for the model, as in the reference), both on copy streams "
                       "overlapped with the previous/next step; gradients are produced on the device by the "
                       "backward pass and stay there"}

    clocks = sampler_clk.stop() if rank == 0 else None  # covers both timed loops
    st_ms = stage_times(0)
    status = _lib.device_status()
    if status != 0:
        raise SystemExit(f"device-side error status {status}")

    if rank == 0:
        peaks = {}
        pk = ROOT / "MEASURED_PEAKS.json"
        if pk.exists():
            peaks = json.loads(pk.read_text())
        peak = float(peaks.get("hbm_gbs", 6650.0))
        row_bytes = cfg.dim * 4
        # dram__bytes_read.sum + dram__bytes_write.sum of one lookup_fetch launch at full size
        # (one-pass ncu capture, profiles/lookup_fetch512_kernel_config2.md); only for that workload
        traffic = 1.136e9 if (not c5 and args.scale == 1.0 and args.lookup == "setassoc" and cfg.dim == 128) else None
        lf_bytes = cfg.batch * (8 + 8 + 1) + 2 * cfg.batch * row_bytes
        achieved = lf_bytes / (st_ms["lookup_fetch"] * 1e-3) / 1e9
        seg_bytes = cfg.batch * (8 + row_bytes) + num_unique * (8 + 8 + row_bytes)
        line = {
            "metric": METRIC, "value": world * cfg.batch * K / (total_ms * 1e-3), "unit": UNIT,
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": total_ms / K,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": (f"config5: R-MAT(0.57,0.19,0.19) 2^{cfg.bits} ({cfg.num_nodes} nodes), "
                                    f"{cfg.seeds} seeds x fanout {list(cfg.fanout)} per GPU, dim {cfg.dim} fp32") if c5
                       else (WORKLOAD if args.scale == 1.0 else f"config2 scaled by {args.scale:g}"),
                       "table_rows": cfg.table_rows, "dim": cfg.dim, "cache_entries": cfg.cache_entries,
                       "batch_per_gpu": cfg.batch, "zipf_s": None if c5 else cfg.zipf_s,
                       "flush_every": cfg.flush_every,
                       "lookup": args.lookup, "mover": args.mover, "lru_ageing": not args.no_lru,
                       "cuda_graph": use_graph, "untimed_settling_steps_after_warmup": settle,
                       "optimizer": "SparseAdam fp32" if args.optimizer == "adam" else "SparseAdagrad fp32",
                       "exchange": "local" if world == 1 else (
                           "nccl all_to_all" if path.px is None else
                           f"fused pack+push over peer memory, {path.px.fence_kind} fence (hot rows); "
                           "nccl all_to_all (flush)"),
                       "l2": ("145 MB of rows read and written per step (just above L2), 4 frontier batches rotate"
                              if c5 else
                              "inputs larger than L2: 1.0 GB of rows read and written per step, 4 id batches rotate"),
                       "stream": stats, "found_fraction": found_frac, "unique_per_batch": num_unique,
                       "hot_cold_unique": split_counts[1:]},
            "roofline": {"bound": "hbm", "kernel": "lookup_fetch (fused cache lookup + cached fetch)",
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": "measured" if peaks else "fallback",
                         "algorithmic_bytes": lf_bytes, "ms": st_ms["lookup_fetch"], "traffic": traffic,
                         "dram_frac": (traffic / (st_ms["lookup_fetch"] * 1e-3) / 1e9 / peak) if traffic else None,
                         "note": "algorithmic bytes count the duplicate ids of the Zipf stream, whose row reads "
                                 "hit L2; traffic is what reached HBM",
                         "also": {"unique_segsum_ms": st_ms["unique_segsum"],
                                  "unique_segsum_gbs": seg_bytes / (st_ms["unique_segsum"] * 1e-3) / 1e9}},
            "clocks": clocks, "gpu_launches": int(launches),
        }
        if e2e:
            line["e2e"] = e2e
        if world == 1 and not args.no_cpu_baseline and not c5:
            r = cpu_reference_run(4, 1, CPU_SAMPLE_SCALE)
            line["cpu_baseline"] = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def _dist_setup():
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def timed(fn, steps):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ms = torch.tensor([a.elapsed_time(b) / steps], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    return rank, world, dev, timed


def run_exchange(args) -> None:
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

    rank, world, dev, timed = _dist_setup()
    n, dim = int(1_048_576 * args.scale), 64
    table_rows = int(240_000_000 * args.scale)
    rng = synth.rng_for(4, rank, 0)
    # distinct ids, Zipf(1.1) without replacement, ascending as a rank's local aggregation emits them
    # (the ranking is cut after its 30M most popular ids, 96 % of the Zipf(1.1) mass over 2.4e8: the
    # exact CDF of the whole table would take 4 GB of host memory in each of 8 processes)
    ids_np = np.sort(synth.ZipfSampler(min(table_rows, 30_000_000), 1.1).unique_ids(rng, n, id_space=table_rows))
    ids = torch.from_numpy(ids_np).to(dev)
    rows = torch.empty((n, dim), device=dev).normal_(0, 1e-3)
    cnt = torch.ones(n, dtype=torch.int64, device=dev)
    sent_to_others = int((ids_np % world != rank).sum())
    bytes_out = sent_to_others * (8 + 8 + dim * 4)
    cap = int(np.bincount(ids_np % world, minlength=world).max() * 1.05) + 16
    px = PeerExchange(rank, world, cap, dim, torch.float32, dev)                    # device-side fence
    px_nf = PeerExchange(rank, world, cap, dim, torch.float32, dev, fence="nccl")   # all-reduce as the fence
    shard = ShardedEmbedding(table_rows, dim, rank, world, dtype=torch.float16, device=dev, init_sigma=0.01, seed=4)
    opt = SparseAdagrad(shard, lr=0.01)
    id_bits = max(table_rows.bit_length() + 1, 8)

    def do_push():
        px.push(ids, rows, cnt)
        px.fence()

    def do_push_nccl_fence():
        px_nf.push(ids, rows, cnt)
        px_nf.fence()

    def do_nccl():
        swap_gradients(ids, rows, None, 1, world, dev, cnt)

    def do_sync_update():
        parity = px.push(ids, rows, cnt)
        px.fence()
        r_ids, r_rows, r_cnt, seg = px.received(parity)
        opt.update(r_ids, r_rows, r_cnt, is_unique=False, id_bits=id_bits, seg_counts=seg, seg_cap=px.cap,
                   sorted_segments=True)

    W, K = max(args.warmup, 3), max(args.steps, 1)
    out = {}
    for name, fn in (("push", do_push), ("push_nccl_fence", do_push_nccl_fence), ("nccl", do_nccl),
                     ("sync_update", do_sync_update)):
        for _ in range(W):
            fn()
        out[name] = timed(fn, K)
    status = _lib.device_status()
    if rank == 0:
        line = {"metric": "sparse_grad_all_to_all_GBps_per_gpu_out", "unit": "GB/s", "n_gpus": world,
                "steps": K, "warmup": W, "higher_is_better": True, "data": "synthetic", "dtype": "f32",
                "config": {"workload": "config4: 1,048,576 unique ids x 64 fp32 (+8 B id, 8 B cnt) per rank, "
                                       f"fp16 table of {table_rows} x 64 sharded id % world, sparse Adagrad fp32 state",
                           "rows_per_rank": n, "bytes_leaving_each_gpu": bytes_out},
                "push_ms": out["push"], "push_nccl_fence_ms": out["push_nccl_fence"], "nccl_ms": out["nccl"],
                "sync_update_ms": out["sync_update"],
                "sync_update_rows_per_s": world * n / (out["sync_update"] * 1e-3), "device_status": status}
        if world > 1:
            line["value"] = bytes_out / (out["push"] * 1e-3) / 1e9
            line["nccl_value"] = bytes_out / (out["nccl"] * 1e-3) / 1e9
            line["roofline"] = {"bound": "nvlink", "achieved": line["value"], "peak": 770.0, "unit": "GB/s",
                                "frac": line["value"] / 770.0, "peak_source": "measured peer copy on this pool",
                                "nominal_peak": 900.0, "traffic": None}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_hot_aggregation(args) -> None:
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

    rank, world, dev, timed = _dist_setup()
    nodes = int(100_000_000 * args.scale)
    n, dim = int(524_288 * args.scale), 128
    sampler = synth.ZipfSampler(nodes, 1.2)
    rng = synth.rng_for(3, rank, 0)
    batches = [torch.from_numpy(sampler.ids(rng, n)).to(dev) for _ in range(4)]
    stats = synth.stream_stats(batches[0].cpu().numpy())
    grads = torch.empty((n, dim), device=dev).normal_(0, 1e-3)
    n_hot = max(nodes // 100, 1)
    hot_ranked = synth.rank_to_id(np.arange(n_hot, dtype=np.int64), nodes)
    cls = np.full(nodes, 2, dtype=np.int8)
    cls[hot_ranked] = 1
    table = torch.from_numpy(cls).to(dev)
    cap = int(np.bincount(hot_ranked % world, minlength=world).max())
    cap = min(cap, n)
    px = PeerExchange(rank, world, cap, dim, torch.float32, dev) if world > 1 else None
    id_bits = max(nodes.bit_length() + 1, 8)
    state = {"k": 0, "u": None, "hot": None, "merged": None}

    def local_only():
        ids = batches[state["k"] % 4]
        state["k"] += 1
        outs, cc, num = E.cudaUniqueSegSumSplit(ids, grads, table, keep=(False, True, False),
                                                caps=(None, min(n_hot, n), None), id_bits=id_bits)
        state["u"], state["hot"], state["cc"] = num, outs[1], cc

    def with_reduction():
        local_only()
        h_ids, h_rows, h_cnt = state["hot"]
        if px is None:
            state["merged"] = E.cudaUniqueSegSum(h_ids, h_rows, h_cnt, mean=True, id_bits=id_bits, sync=False,
                                                 n_dev=state["cc"][1:2])
        else:
            parity = px.push(h_ids, h_rows, h_cnt, state["cc"][1:2])
            px.fence()
            r_ids, r_rows, r_cnt, seg = px.received(parity)
            # every slab holds its sender's ascending unique hot ids: a merge, not a sort
            state["merged"] = E.cudaMergeSortedSlabs(r_ids, r_rows, r_cnt, seg, px.cap, mean=True)

    W, K = max(args.warmup, 3), max(args.steps, 1)
    out = {}
    for name, fn in (("local", local_only), ("local_plus_hot_reduction", with_reduction)):
        for _ in range(W):
            fn()
        out[name] = timed(fn, K)
    uniq = int(state["u"].item())
    hot_u = int(state["cc"][1].item())
    merged = int(state["merged"][3].item())
    status = _lib.device_status()
    if rank == 0:
        peaks = {}
        pk = ROOT / "MEASURED_PEAKS.json"
        if pk.exists():
            peaks = json.loads(pk.read_text())
        peak = float(peaks.get("hbm_gbs", 6650.0))
        alg = n * (8 + dim * 4) + uniq * 16 + hot_u * dim * 4
        line = {"metric": "gradient_rows_per_s_local_aggregation_plus_hot_reduction", "unit": "rows/s",
                "value": world * n / (out["local_plus_hot_reduction"] * 1e-3), "n_gpus": world, "steps": K,
                "warmup": W, "higher_is_better": True, "scaling": "weak", "data": "synthetic", "dtype": "f32",
                "ms_per_step": out["local_plus_hot_reduction"], "local_aggregation_ms": out["local"],
                "config": {"workload": f"config3: {n} ids per GPU, Zipf(1.2) over {nodes}, dim 128 fp32, hot = top 1 %",
                           "stream": stats, "unique": uniq, "hot_unique": hot_u, "owned_after_reduction": merged,
                           "exchange": "local" if world == 1 else "fused pack+push over peer memory, device fence"},
                "roofline": {"bound": "hbm", "kernel": "local aggregation (sort + run heads + segment-sum, hot rows kept)",
                             "achieved": alg / (out["local"] * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                             "frac": alg / (out["local"] * 1e-3) / 1e9 / peak,
                             "peak_source": "measured" if peaks else "fallback", "traffic": None},
                "device_status": status}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "c4_exchange":
        run_exchange(args)
    elif args.workload == "c3":
        run_hot_aggregation(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
