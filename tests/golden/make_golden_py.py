"""Generate tests/golden/aggregation_golden.npz by running the REFERENCE's own Python
functions ``only_unique_grads`` and ``unique_grads`` (python/EmbCache/sparse_optim.py:132-157)
on CPU tensors.  The reference package imports DGL and its compiled extension at import time;
neither is needed by these two functions, so DGL is stubbed and ``EmbCacheLib`` is served by this
repository's mirror (which is not called on this path).

Run where the reference checkout is present:
    HADES_REFERENCE_ROOT=<checkout> python tests/golden/make_golden_py.py
"""
from __future__ import annotations

import os
import sys
import types
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from oracle.build_oracle import reference_root  # noqa: E402

# the reference checkout: first argument, else $HADES_REFERENCE_ROOT, else a checkout named
# `reference` beside this repository
REFERENCE = reference_root(sys.argv[1] if len(sys.argv) > 1 else None)
if REFERENCE is None:
    raise SystemExit("set HADES_REFERENCE_ROOT (or pass the checkout as the first argument)")
OUT = Path(__file__).resolve().parent / "aggregation_golden.npz"


def import_reference_sparse_optim():
    sys.path.insert(0, str(ROOT))
    for name in ("dgl", "dgl.distributed", "dgl.distributed.dist_tensor", "dgl.backend"):
        sys.modules.setdefault(name, types.ModuleType(name))
    sys.modules["dgl.distributed.dist_tensor"].DistTensor = object
    sys.modules["dgl.distributed"].DistTensor = object
    import hades_b200.EmbCacheLib as mirror

    sys.modules["EmbCacheLib"] = mirror
    sys.path.insert(0, str(REFERENCE / "python"))
    import importlib.util

    pkg = types.ModuleType("EmbCache")
    pkg.__path__ = [str(REFERENCE / "python" / "EmbCache")]
    sys.modules["EmbCache"] = pkg
    for sub in ("common", "utils", "cache"):
        spec = importlib.util.spec_from_file_location(f"EmbCache.{sub}", REFERENCE / "python" / "EmbCache" / f"{sub}.py")
        mod = importlib.util.module_from_spec(spec)
        sys.modules[f"EmbCache.{sub}"] = mod
        spec.loader.exec_module(mod)
    spec = importlib.util.spec_from_file_location("EmbCache.sparse_optim",
                                                  REFERENCE / "python" / "EmbCache" / "sparse_optim.py")
    mod = importlib.util.module_from_spec(spec)
    sys.modules["EmbCache.sparse_optim"] = mod
    spec.loader.exec_module(mod)
    return mod


def main():
    ref = import_reference_sparse_optim()
    rng = np.random.default_rng(20240)
    out = {}
    cases = [(1, 4, 5), (300, 8, 40), (3000, 16, 500), (512, 128, 900), (6000, 3, 50)]
    for k, (n, dim, id_range) in enumerate(cases):
        idx = rng.integers(0, id_range, n, dtype=np.int64)
        if n > 100:
            idx[: n // 3] = idx[0]
            rng.shuffle(idx)
        grad = (rng.standard_normal((n, dim)) * 1e-3).astype(np.float32)
        cnt = rng.integers(1, 17, n, dtype=np.int64)
        ti, tg, tc = torch.from_numpy(idx), torch.from_numpy(grad), torch.from_numpy(cnt)
        u, s, c = ref.only_unique_grads(ti, tg)
        mu, mv = ref.unique_grads(ti, tg)
        cu, cv = ref.unique_grads(ti, tg, tc)
        out.update({f"c{k}_idx": idx, f"c{k}_grad": grad, f"c{k}_cnt": cnt,
                    f"c{k}_sum_ids": u.numpy(), f"c{k}_sum_vals": s.numpy(), f"c{k}_sum_counts": c.numpy(),
                    f"c{k}_mean_ids": mu.numpy(), f"c{k}_mean_vals": mv.numpy(),
                    f"c{k}_cntmean_ids": cu.numpy(), f"c{k}_cntmean_vals": cv.numpy()})
    out["num_cases"] = np.int64(len(cases))
    np.savez_compressed(OUT, **out)
    print(OUT, OUT.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
