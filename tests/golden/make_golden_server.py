"""Generate tests/golden/server_golden.npz and tests/golden/adam_golden.npz by running the
REFERENCE's own Python on CPU tensors:

* the cache server's arithmetic -- ``_accumulate_gradients_cold_remote/_local``
  (python/EmbCache/server.py:546-574), ``_send_staled_gradients`` (:346-497) and
  ``_update_cache`` (:499-544) -- as bound methods of a bare ``EmbCacheServer`` object (no
  sockets, no shared memory: ``_create_shm_tensor`` hands out plain tensors and the
  ``_send_shm_tensor_*`` methods record what would have been sent), with the reference's own
  compiled CPU index (oracle/_ref/libhades_ref.so, OMP threads = 1) as ``_idx_cache``;
* ``SparseAdam.update`` (python/EmbCache/sparse_optim.py:590-685) on a bare ``SparseAdam`` with a
  dictionary-backed state holder.  That method builds ``torch.tensor(beta, device='cuda')``
  (:650-653); the module's ``torch`` name is replaced by a proxy that drops the device argument
  and stubs ``torch.cuda.Event``, so the same expressions run on CPU tensors.

The reference never clears its gradient rows after a flush or an insert (server.py:414,489,537
zero a temporary copy), so the rows it sends are running sums.  Scenario ``once`` never
accumulates into a slot again after that slot was flushed, so its outputs are also those of the
intended read-and-zero behaviour; scenario ``again`` does, and pins the reference's literal
behaviour (the oracle's ``compat_no_clear=True``).

Run where the reference checkout is present:
    HADES_REFERENCE_ROOT=<checkout> python tests/golden/make_golden_server.py
"""
from __future__ import annotations

import importlib.util
import os
import sys
import types
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from oracle import build_oracle  # noqa: E402

HERE = Path(__file__).resolve().parent


def import_reference(modules=("common", "utils", "cache", "base", "server", "sparse_optim")):
    """The reference's EmbCache package with DGL stubbed and this repository's EmbCacheLib mirror
    in place of its compiled extension (neither is called on the paths recorded here)."""
    ref_root = build_oracle.reference_root(sys.argv[1] if len(sys.argv) > 1 else None)
    if ref_root is None:
        raise SystemExit("set HADES_REFERENCE_ROOT (or pass the checkout as the first argument)")
    for name in ("dgl", "dgl.distributed", "dgl.distributed.dist_tensor", "dgl.backend"):
        sys.modules.setdefault(name, types.ModuleType(name))
    sys.modules["dgl.distributed.dist_tensor"].DistTensor = object
    sys.modules["dgl.distributed"].DistTensor = object
    import hades_b200.EmbCacheLib as mirror

    sys.modules["EmbCacheLib"] = mirror
    pkg = types.ModuleType("EmbCache")
    pkg.__path__ = [str(ref_root / "python" / "EmbCache")]
    sys.modules["EmbCache"] = pkg
    out = {}
    for sub in modules:
        spec = importlib.util.spec_from_file_location(f"EmbCache.{sub}", ref_root / "python" / "EmbCache" / f"{sub}.py")
        mod = importlib.util.module_from_spec(spec)
        sys.modules[f"EmbCache.{sub}"] = mod
        spec.loader.exec_module(mod)
        out[sub] = mod
    return out


class RefIndexAdapter:
    """The reference's compiled CPU index behind the tensor interface LocalCache offers
    (python/EmbCache/cache.py:6-31)."""

    def __init__(self, cache_size: int):
        from oracle.oracle import RefIndex

        RefIndex.set_threads(1)
        self.ref = RefIndex(cache_size)

    def get_num_entries(self):
        return self.ref.get_capacity()

    def add(self, ids):
        return torch.from_numpy(self.ref.add(ids.numpy().astype(np.int64)))

    def lookup(self, ids):
        return torch.from_numpy(self.ref.lookup(ids.numpy().astype(np.int64)))

    def reset(self, ids):
        self.ref.reset(ids.numpy().astype(np.int64))

    def state(self):
        n = self.ref.get_valid_entries_num()
        return self.ref.getall(n)


def bare_server(ref, cache_entries, dim, num_clients, hotness, part_nodes, part_start, cnt_threshold):
    """An EmbCacheServer with the state _create_cache builds (server.py:76-175), no process
    plumbing."""
    S = ref["server"].EmbCacheServer
    srv = object.__new__(S)
    srv.num_clients = num_clients
    srv._shm_tensor_meta, srv._create_tensor_count, srv._pin_memory = {}, 0, False
    srv._check_iters = 50
    srv._reset_recorder()
    srv.hotness = torch.from_numpy(hotness)
    srv.cnt_threshold = int(cnt_threshold)
    srv.threshold = (1 / (0.001 + srv.hotness)).ceil().int().clamp(max=100)  # server.py:87-88
    srv._idx_cache = RefIndexAdapter(cache_entries)
    slots = srv._idx_cache.get_num_entries()
    srv._idx_dtype, srv._emb_dtype, srv._emb_dim = torch.int64, torch.float32, dim
    srv._emb_cache_buff = torch.zeros((slots, dim))
    srv._grad_cache_buff = torch.zeros((slots, dim))
    srv._grad_cnt_cache_buff = torch.zeros(slots, dtype=torch.int32)
    srv._grad_iter_count = torch.zeros(slots, dtype=torch.int32)
    srv._grad_iter_threshold = torch.zeros(slots, dtype=torch.int32)
    srv._grad_idx_cache_buff = torch.full((slots,), -1, dtype=torch.int64)
    srv._part_nnodes, srv._part_start = part_nodes, part_start
    srv._local_grad_buff = torch.zeros((part_nodes, dim))
    srv._local_grad_cnt_buff = torch.zeros(part_nodes, dtype=torch.int32)
    srv._local_grad_iter_count = torch.zeros(part_nodes, dtype=torch.int32)
    srv._local_grad_iter_threshold = srv.threshold[part_start:part_start + part_nodes]
    sent = []  # (tensor name or EMPTY, rank or None)
    held = {}

    def create(name, dtype, shape):
        t = torch.empty(tuple(shape), dtype=dtype)
        held[name] = t
        return t

    srv._create_shm_tensor = create
    srv._send_shm_tensor_to_one = lambda name, rank: sent.append((name, rank, held.get(name)))
    srv._send_shm_tensor_to_all = lambda name: sent.append((name, None, held.get(name)))
    return srv, sent


def collect_sent(sent, num_clients, kind):
    """What one _send_staled_gradients call sent to every client for `kind` ('remote' or
    'local'): ids, rows and counts, clients in order."""
    ids, rows, cnt, counts = [], [], [], np.zeros(num_clients, np.int64)
    for name, rank, t in sent:
        if t is None or f"_{kind}_staled_" not in name:
            continue
        if "_staled_id_" in name:
            ids.append((rank, t.clone().numpy()))
            counts[rank] = t.numel()
        elif "_staled_grad_cnt_" in name:
            cnt.append((rank, t.clone().numpy()))
        elif "_staled_grad_" in name:
            rows.append((rank, t.clone().numpy()))
    cat = lambda parts, empty: (np.concatenate([p for _, p in sorted(parts, key=lambda x: x[0])])
                                if parts else empty)
    return cat(ids, np.empty(0, np.int64)), cat(rows, None), cat(cnt, np.empty(0, np.int64)), counts


def server_scenario(ref, name, seed, again: bool):
    rng = np.random.default_rng(seed)
    nodes, dim, cache_entries, clients, iters, cnt_threshold = 4000, 8, 160, 3, 9, 3
    part_start, part_nodes = 1000, 600
    hot = rng.random(nodes).astype(np.float32)
    hot[rng.random(nodes) < 0.5] *= 0.02   # flush periods from 1 to 50 iterations
    hot[rng.random(nodes) < 0.3] = 5.0     # period 1
    srv, sent = bare_server(ref, cache_entries, dim, clients, hot, part_nodes, part_start, cnt_threshold)
    rec = {"nodes": nodes, "dim": dim, "cache_entries": cache_entries, "clients": clients, "iters": iters,
           "cnt_threshold": cnt_threshold, "part_start": part_start, "part_nodes": part_nodes, "hotness": hot,
           "slots": srv._idx_cache.get_num_entries()}
    remote_pool = rng.permutation(np.setdiff1d(np.arange(nodes), np.arange(part_start, part_start + part_nodes)))
    used_remote = np.zeros(nodes, bool)
    used_local = np.zeros(nodes, bool)
    for it in range(iters):
        del sent[:]
        srv._send_staled_gradients()                                         # step 0
        for kind in ("remote", "local"):
            i, r, c, k = collect_sent(sent, clients, kind)
            rec[f"it{it}_sent_{kind}_ids"], rec[f"it{it}_sent_{kind}_cnt"] = i, c
            rec[f"it{it}_sent_{kind}_counts"] = k
            rec[f"it{it}_sent_{kind}_rows"] = r if r is not None else np.zeros((0, dim), np.float32)
        # step 2: uncached embeddings of every client, inserted one client after the other
        ids_list, embs_list = [], []
        for c in range(clients):
            n = int(rng.integers(20, 60)) if it < 6 else int(rng.integers(0, 12))
            if not again and it > 0:
                n = 0  # a slot that was flushed is not handed to another id in this scenario
            ids = rng.choice(remote_pool[:900], n, replace=True).astype(np.int64)
            embs = (rng.standard_normal((n, dim)) * 0.01).astype(np.float32)
            first = {}
            for k, i in enumerate(ids):  # the copies of an id inside one message carry the same row
                embs[k] = embs[first.setdefault(int(i), k)]
            ids_list.append(torch.from_numpy(ids))
            embs_list.append(torch.from_numpy(embs))
        rec[f"it{it}_ins_ids"] = np.concatenate([t.numpy() for t in ids_list])
        rec[f"it{it}_ins_embs"] = np.concatenate([t.numpy() for t in embs_list])
        rec[f"it{it}_ins_sizes"] = np.array([t.numel() for t in ids_list], np.int64)
        # _update_cache asks for valid_index.max(): every client's batch must insert something
        srv._update_cache(ids_list, embs_list)
        # step 3: cold gradients, unique ids per message (server.py:547)
        for c in range(clients):
            pool = remote_pool[:900] if again else remote_pool[:900][~used_remote[remote_pool[:900]]]
            n = min(int(rng.integers(30, 90)), pool.size)
            rid = rng.choice(pool, n, replace=False).astype(np.int64)
            rg = (rng.standard_normal((n, dim)) * 1e-3).astype(np.float32)
            srv._accumulate_gradients_cold_remote(torch.from_numpy(rid), torch.from_numpy(rg))
            lpool = np.arange(part_start, part_start + part_nodes)
            if not again:
                lpool = lpool[~used_local[lpool]]
            m = min(int(rng.integers(10, 50)), lpool.size)
            lid = rng.choice(lpool, m, replace=False).astype(np.int64)
            lg = (rng.standard_normal((m, dim)) * 1e-3).astype(np.float32)
            srv._accumulate_gradients_cold_local(torch.from_numpy(lid), torch.from_numpy(lg))
            if not again:
                # an id whose slot may be flushed later is not given a gradient again
                used_remote[rid] = True
                used_local[lid] = True
            rec[f"it{it}_c{c}_rid"], rec[f"it{it}_c{c}_rg"] = rid, rg
            rec[f"it{it}_c{c}_lid"], rec[f"it{it}_c{c}_lg"] = lid, lg
        srv._iter_cnt += 1
        gi, gl = srv._idx_cache.state()
        rec[f"it{it}_index_ids"], rec[f"it{it}_index_locs"] = gi, gl
        rec[f"it{it}_cnt"] = srv._grad_cnt_cache_buff.numpy().copy()
        rec[f"it{it}_idx"] = srv._grad_idx_cache_buff.numpy().copy()
        rec[f"it{it}_iter_count"] = srv._grad_iter_count.numpy().copy()
        rec[f"it{it}_grad"] = srv._grad_cache_buff.numpy().copy()
        rec[f"it{it}_emb"] = srv._emb_cache_buff.numpy().copy()
        rec[f"it{it}_local_cnt"] = srv._local_grad_cnt_buff.numpy().copy()
        rec[f"it{it}_local_iter_count"] = srv._local_grad_iter_count.numpy().copy()
        rec[f"it{it}_local_grad"] = srv._local_grad_buff.numpy().copy()
    return {f"{name}_{k}": np.asarray(v) for k, v in rec.items()}


class _TorchOnCpu:
    """Stands in for the module-level name ``torch`` of sparse_optim.py: ``tensor(..., device=)``
    loses its device and ``cuda.Event`` is a no-op; everything else is torch."""

    class _Event:
        def record(self):
            pass

        def wait(self):
            pass

        def synchronize(self):
            pass

    class _Cuda:
        Event = None

    def __init__(self):
        self.cuda = _TorchOnCpu._Cuda()
        self.cuda.Event = _TorchOnCpu._Event

    def tensor(self, *a, device=None, **k):
        return torch.tensor(*a, **k)

    def __getattr__(self, name):
        return getattr(torch, name)


class _State:
    """What LocalSparseAdamStateCache offers to update(): state[idx] -> (step, mem, power) and
    state[idx] = (step, mem, power) (python/EmbCache/cache.py:66-131), all rows in one place."""

    def __init__(self, rows, dim):
        self.step = torch.zeros(rows)
        self.mem = torch.zeros((rows, dim))
        self.power = torch.zeros((rows, dim))

    def __getitem__(self, idx):
        return self.step[idx], self.mem[idx], self.power[idx]

    def __setitem__(self, idx, val):
        self.step[idx], self.mem[idx], self.power[idx] = val


def adam_cases(ref):
    so = ref["sparse_optim"]
    so.torch = _TorchOnCpu()
    rng = np.random.default_rng(777)
    out = {}
    cases = [(50, 4, 12, False), (300, 16, 200, False), (300, 16, 200, True), (256, 128, 300, False),
             (64, 3, 64, True)]
    for k, (rows, dim, n, unique) in enumerate(cases):
        opt = object.__new__(so.SparseAdam)
        opt._beta1, opt._beta2, opt._eps, opt._lr = 0.9, 0.999, 1e-8, 0.01
        emb = types.SimpleNamespace(name="emb", tensor=torch.from_numpy(
            (rng.standard_normal((rows, dim)) * 0.01).astype(np.float32)))
        opt._state = {"emb": _State(rows, dim)}
        out[f"a{k}_emb0"] = emb.tensor.numpy().copy()
        rounds = 3
        for r in range(rounds):
            if unique:
                idx = rng.choice(rows, min(n, rows), replace=False).astype(np.int64)
            else:
                idx = rng.integers(0, rows, n, dtype=np.int64)
            grad = (rng.standard_normal((idx.size, dim)) * 1e-3).astype(np.float32)
            cnt = rng.integers(1, 9, idx.size, dtype=np.int64) if r != 1 else None
            opt.update(torch.from_numpy(idx), torch.from_numpy(grad), emb,
                       cnt=None if cnt is None else torch.from_numpy(cnt), is_unique=unique)
            out[f"a{k}_r{r}_idx"], out[f"a{k}_r{r}_grad"] = idx, grad
            out[f"a{k}_r{r}_cnt"] = cnt if cnt is not None else np.empty(0, np.int64)
            st = opt._state["emb"]
            out[f"a{k}_r{r}_emb"] = emb.tensor.numpy().copy()
            out[f"a{k}_r{r}_step"] = st.step.numpy().copy()
            out[f"a{k}_r{r}_mem"] = st.mem.numpy().copy()
            out[f"a{k}_r{r}_power"] = st.power.numpy().copy()
        out[f"a{k}_meta"] = np.array([rows, dim, int(unique), rounds], np.int64)
    out["num_cases"] = np.int64(len(cases))
    return out


def main():
    build_oracle.build_oracle()
    if build_oracle.build_ref() is None:
        raise SystemExit("the reference's compiled index is needed (oracle/_ref/libhades_ref.so)")
    ref = import_reference()
    out = {}
    out.update(server_scenario(ref, "once", 11, again=False))
    out.update(server_scenario(ref, "again", 12, again=True))
    path = HERE / "server_golden.npz"
    np.savez_compressed(path, **out)
    print(path, path.stat().st_size, "bytes")
    path = HERE / "adam_golden.npz"
    np.savez_compressed(path, **adam_cases(ref))
    print(path, path.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
