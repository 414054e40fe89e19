"""This library's operators against the REFERENCE's own CUDA operators (src/cuda/ops.h:9-41),
compiled from the reference's .cu files into oracle/_ref/libhades_ref_cuda.so
(oracle/build_oracle.py) and run on the same GPU with the same inputs: bit-exact outputs.
Shapes follow the reference's scripts (test/test_fetch.py:6-38, test_cached_fetch.py:6-76,
test_cached_set.py:6-74, test_combine.py:6-40, test_split.py:6-52, test_binaryserach.py).
The reference's cudalookup is left out: lanes of lookupkernel2 return before a warp-wide reduce
(src/cache/lookup.cu:28,36), which is undefined behaviour, so it does not run here."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref(oracle_mod):
    if not oracle_mod.RefCuda.available():
        pytest.skip("oracle/_ref/libhades_ref_cuda.so is not built")
    return oracle_mod.RefCuda


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("idx", [torch.int64, torch.int32])
def test_fetch_set_combine(cuda_lib, ref, dtype, idx):
    from hades_b200 import EmbCacheLib as E

    g = torch.Generator(device="cuda").manual_seed(42)
    rows, dim, n = 400_000, 128, 100_000
    src = torch.randn((rows, dim), dtype=dtype, device="cuda", generator=g)
    si = torch.randperm(rows, device="cuda", generator=g)[:n].to(idx)
    di = torch.randperm(rows, device="cuda", generator=g)[:n].to(idx)
    a, b = torch.zeros_like(src), torch.zeros_like(src)
    E.cudaFetch(src, si, a, di)
    ref.fetch(src, si, b, di)
    assert torch.equal(a, b)
    a, b = torch.zeros((n, dim), dtype=dtype, device="cuda"), torch.zeros((n, dim), dtype=dtype, device="cuda")
    E.cudaFetch2(src, si, a)
    ref.fetch2(src, si, b)
    assert torch.equal(a, b)
    v = torch.randn(rows, dtype=dtype, device="cuda", generator=g)
    a1, b1 = torch.zeros(n, dtype=dtype, device="cuda"), torch.zeros(n, dtype=dtype, device="cuda")
    E.cudaFetch2(v, si, a1)
    ref.fetch2(v, si, b1)
    assert torch.equal(a1, b1)
    upd = torch.randn((n, dim), dtype=dtype, device="cuda", generator=g)
    a, b = src.clone(), src.clone()
    E.cudaSet(upd, a, di)
    ref.set(upd, b, di)
    assert torch.equal(a, b)
    a, b = src.clone(), src.clone()
    E.cudaCombine(upd, a, di)
    ref.combine(upd, b, di)
    assert torch.equal(a, b)


@pytest.mark.parametrize("dim", [1, 128])
def test_cached_fetch_and_set(cuda_lib, ref, dim):
    from hades_b200 import EmbCacheLib as E

    g = torch.Generator(device="cuda").manual_seed(7)
    rows, cached_rows, n = 400_000, 200_000, 150_000
    shape = (lambda r: (r,)) if dim == 1 else (lambda r: (r, dim))
    backing = torch.randn(shape(rows), device="cuda", generator=g)
    cached = torch.randn(shape(cached_rows), device="cuda", generator=g)
    index_map = torch.full((rows,), -1, dtype=torch.int64, device="cuda")
    hot = torch.randperm(rows, device="cuda", generator=g)[:cached_rows]
    index_map[hot] = torch.arange(cached_rows, device="cuda")
    idx = torch.randperm(rows, device="cuda", generator=g)[:n]
    a, b = torch.zeros(shape(n), device="cuda"), torch.zeros(shape(n), device="cuda")
    E.cudaFetchWithCache2(backing, cached, idx, index_map, a)
    ref.fetch_with_cache2(backing, cached, idx, index_map, b)
    assert torch.equal(a, b)
    upd = torch.randn(shape(n), device="cuda", generator=g)
    ba, ca, bb, cb = backing.clone(), cached.clone(), backing.clone(), cached.clone()
    E.cudaSetWithCache(upd, ba, ca, idx, index_map)
    ref.set_with_cache(upd, bb, cb, idx, index_map)
    assert torch.equal(ba, bb) and torch.equal(ca, cb)


def test_split_and_owner_search(cuda_lib, ref):
    from hades_b200 import EmbCacheLib as E

    g = torch.Generator(device="cuda").manual_seed(42)
    nodes, n = 1_000_000, 300_000
    mask = torch.randint(0, 3, (nodes,), device="cuda", generator=g).to(torch.int8)
    ids = torch.randint(0, nodes, (n,), device="cuda", generator=g)
    for x, y in zip(E.cudaSplit(ids, mask), ref.split(ids, mask)):
        assert torch.equal(x, y)
    for dt in (torch.int64, torch.int32):
        v = ids.to(dt)
        assert torch.equal(E.cudaReminder(v, 8), ref.reminder(v, 8))
        part = torch.tensor([0, 150_000, 420_000, 700_000, nodes], dtype=dt, device="cuda")
        assert torch.equal(E.cudaBinarySearch(v, part, 4), ref.binary_search(v, part, 4))
        owners = torch.sort(E.cudaReminder(v, 8)).values
        r = torch.arange(8, dtype=dt, device="cuda")
        assert torch.equal(E.cudaBinarySearch2(r, owners), ref.binary_search2(r, owners))
