"""Micro-benchmarks of the individual operators at configuration-2 shapes (2M rows of 128 fp32):

    python -m hades_b200.microbench              every operator
    python -m hades_b200.microbench update       only the small cases below (a few GB on the device)

Row movers (LSU vs bulk-copy path), the two lookup algorithms, the fused lookup+fetch on a
Zipf(1.2) stream (91 % duplicates, reads mostly served by L2) and on uniform ids (no reuse),
local aggregation, and the two LRU ageing forms.  CUDA events, 20 repetitions after a warm-up
call; algorithmic bytes as defined in include/hades_b200.h.

``update``: the sparse Adam row update on 84,000 random rows of a 2M x 128 table, the flush of a
4M-slot staging table with 6 % stale rows, and the owner-side merge of 8 sorted slabs against the
sorting path; L2 is flushed between repetitions of the Adam case.
"""
from __future__ import annotations

import torch

from . import EmbCacheLib as E
from . import _lib, synth


def _time(fn, reps: int = 20) -> float:
    fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps


def small_cases() -> None:
    from .cold_cache import StagingTable
    from .sparse_optim import ShardedEmbedding, SparseAdam

    torch.cuda.set_device(0)
    dev = "cuda"
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
        out = st.flush(None, 16, 1, sync=False)
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


def main() -> None:
    import sys

    if len(sys.argv) > 1 and sys.argv[1] == "update":
        return small_cases()
    torch.cuda.set_device(0)
    dev = "cuda"
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
            print(f"lookup {qn:9s} {mname:9s}         {ms * 1e3:8.1f} us  {n / ms / 1e6:8.2f} G ids/s")
            ms = _time(lambda: E.cudaLookupFetch(ix, q, cache, table, out_rows=out, mode=mode, mover=E.MOVER_LSU))
            print(f"lookup+fetch {qn:9s} {mname:9s}   {ms * 1e3:8.1f} us  {(n * 17 + 2 * n * row) / ms / 1e6:8.0f} GB/s")
        ms = _time(lambda: E.cudaUniqueSegSum(q, grads, id_bits=bits, sync=False))
        print(f"unique+segment-sum {qn:9s}         {ms * 1e3:8.1f} us")
        locs = ix.cudalookup(q)
        ms = _time(lambda: ix.cuda_touch_lru(locs))
        print(f"LRU ageing by sort {qn:9s}         {ms * 1e3:8.1f} us")

        def runs_touch():
            *_, runs = E.cudaUniqueSegSum(q, grads[:, :4].contiguous(), id_bits=bits, sync=False, want_runs=True)
            ix.cuda_touch_lru_runs(locs, runs)

        g4 = grads[:, :4].contiguous()
        *_, runs = E.cudaUniqueSegSum(q, g4, id_bits=bits, sync=False, want_runs=True)
        ms = _time(lambda: ix.cuda_touch_lru_runs(locs, runs))
        print(f"LRU ageing from runs {qn:9s}       {ms * 1e3:8.1f} us  (grouping taken from the aggregation's sort)")
    print("device status", _lib.device_status())


if __name__ == "__main__":
    main()
