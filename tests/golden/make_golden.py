"""Generate tests/golden/index_golden.npz from the REFERENCE's own compiled CPU index
(oracle/_ref/libhades_ref.so, built by oracle/build_oracle.py from the reference sources
where they lie; OMP threads = 1, the parity configuration).

Run where the reference checkout is present:  python tests/golden/make_golden.py
The .npz holds, per scenario, the op sequence with its inputs and the reference's outputs.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from oracle import build_oracle  # noqa: E402
from oracle.oracle import RefIndex  # noqa: E402

OUT = Path(__file__).resolve().parent / "index_golden.npz"


def scenario(seed: int, cache_size: int, id_range: int, steps: int, batch: int, zipf: bool):
    """add / lookup / reset / getall interleaved; lookups drive the LRU state that later
    adds evict by."""
    rng = np.random.default_rng(seed)
    ref = RefIndex(cache_size)
    rec = {"cache_size": np.int64(cache_size), "capacity": np.int64(ref.get_capacity()),
           "space": np.int64(ref.get_space())}
    ops = []
    for s in range(steps):
        op = ["add", "lookup", "lookup", "add", "reset", "lookup", "add"][s % 7]
        n = int(rng.integers(1, batch + 1))
        if zipf:
            ids = np.minimum((rng.pareto(1.1, n) * 3).astype(np.int64), id_range - 1)
        else:
            ids = rng.integers(0, id_range, n, dtype=np.int64)
        rec[f"op{s}_ids"] = ids
        if op == "add":
            rec[f"op{s}_out"] = ref.add(ids)
        elif op == "lookup":
            rec[f"op{s}_out"] = ref.lookup(ids)
        else:
            ref.reset(ids)
        rec[f"op{s}_valid"] = np.int64(ref.get_valid_entries_num())
        ops.append(op)
    valid = ref.get_valid_entries_num()
    gi, gl = ref.getall(valid)
    rec["final_ids"], rec["final_locs"] = gi, gl
    rec["ops"] = np.array(ops)
    return rec


def main():
    build_oracle.build_oracle()
    if build_oracle.build_ref() is None:
        raise SystemExit("reference sources not found; cannot generate golden vectors")
    RefIndex.set_threads(1)
    out = {}
    # the small known-answer case: IndexCache(30) -> 4 lines
    ref = RefIndex(30)
    out["ka_add1"] = ref.add(np.arange(10))
    out["ka_lookup"] = ref.lookup(np.array([0, 1, 4, 5, 8, 9, 11, 40]))
    out["ka_add2"] = ref.add(np.arange(0, 41, 4))
    scen = [
        (1, 64, 200, 28, 60, False),      # tiny, heavy overflow and eviction
        (2, 1000, 5000, 35, 400, False),  # moderate load
        (3, 1000, 100000, 35, 700, True), # skewed ids, many duplicates in a batch
        (4, 8, 50, 21, 30, False),        # a single line
        (5, 100_000, 1_000_000, 7, 30_000, False),
    ]
    for i, args in enumerate(scen):
        for k, v in scenario(*args).items():
            out[f"s{i}_{k}"] = v
    out["num_scenarios"] = np.int64(len(scen))
    np.savez_compressed(OUT, **out)
    print(OUT, OUT.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
