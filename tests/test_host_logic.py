"""Host-side logic that needs no GPU: argument checks of the EmbCacheLib mirror (they raise like
the reference's CHECKs before any CUDA work), the named shared-memory helpers, and the seeded
synthetic generators."""
import os

import numpy as np
import pytest
import torch


def test_shape_and_dtype_checks_raise_without_gpu():
    from hades_b200 import EmbCacheLib as E

    a, b = torch.zeros((4, 3)), torch.zeros((4, 5))
    i = torch.zeros(4, dtype=torch.int64)
    with pytest.raises(RuntimeError, match="Check failed"):
        E.cudaFetch(a, i, b, i)
    with pytest.raises(RuntimeError, match="Check failed"):
        E.cudaSet(a, b, i)
    with pytest.raises(RuntimeError, match="Check failed"):
        E.cudaCombine(a, b, i)
    with pytest.raises(RuntimeError, match="float or double"):
        E.cudaFetch2(a.int(), i, a.int())
    with pytest.raises(RuntimeError, match="Check failed"):
        E.cudaFetchWithCache2(a, b, i, i, a)
    with pytest.raises(RuntimeError, match="pinned host memory"):
        E.cudaFetch2(a, i, a.clone())  # unpinned host tensors are not reachable from the device


def test_shared_memory_round_trip():
    from hades_b200 import EmbCacheLib as E

    name = f"hades_b200_test_{os.getpid()}"
    ptr, fd = E.create_shared_mem(name, 4096, pin_memory=False)
    try:
        t = E.open_shared_tensor(ptr, torch.float32, (16, 8))
        t[:] = torch.arange(128, dtype=torch.float32).view(16, 8)
        ptr2, fd2 = E.open_shared_mem(name, 4096, pin_memory=False)
        t2 = E.open_shared_tensor(ptr2, torch.float32, (16, 8))
        assert torch.equal(t, t2) and ptr != ptr2
        t2[3, 4] = -1.0
        assert t[3, 4] == -1.0
        del t2
        E._SHM.pop(ptr2)[0]  # drop the second mapping's bookkeeping; unlink happens below
        os.close(fd2)
    finally:
        del t
        E.release_shared_mem(name, 4096, ptr, fd, pin_memory=False)
    assert not os.path.exists("/dev/shm/" + name)
    with pytest.raises(RuntimeError, match="fail to open"):
        E.open_shared_mem(name, 4096, pin_memory=False)


def test_synthetic_generators_are_seeded_and_sane():
    from hades_b200 import synth

    perm = synth.rank_to_id(np.arange(100_000), 100_000)
    assert np.array_equal(np.sort(perm), np.arange(100_000))  # a permutation
    s = synth.ZipfSampler(1_000_000, 1.1)
    a = s.ids(synth.rng_for(1, 0), 65_536)
    b = s.ids(synth.rng_for(1, 0), 65_536)
    c = s.ids(synth.rng_for(1, 1), 65_536)
    assert np.array_equal(a, b) and not np.array_equal(a, c)
    st = synth.stream_stats(a)
    assert 0.3 < st["duplicate_fraction"] < 0.95 and a.min() >= 0 and a.max() < 1_000_000
    u = s.unique_ids(synth.rng_for(4, 0), 10_000)
    assert np.unique(u).size == 10_000
    hot = synth.hot_ids(1_000_000, 100)
    assert np.array_equal(hot, synth.rank_to_id(np.arange(100), 1_000_000))
    rows = synth.normal_rows(synth.rng_for(1, 0), 1000, 128, 0.01)
    assert rows.dtype == np.float32 and abs(float(rows.std()) - 0.01) < 1e-3
    small = synth.scaled(synth.CONFIG2, 0.01)
    assert small.table_rows == 200_000 and small.batch == 20_000 and small.dim == 128
