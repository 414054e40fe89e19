"""Split, owner search, owner bucketing and the 3-way gradient split against the oracle:
all outputs are integers or row copies, so everything is bit-exact."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [0, 1, 255, 2048, 2049, 100_003])
def test_split_and_compact(cuda_lib, oracle_mod, n):
    from hades_b200 import EmbCacheLib as E

    rng = np.random.default_rng(n)
    table = rng.integers(0, 3, 50_000).astype(np.int8)
    table[::97] = 5  # a value outside {0,1,2} leaves every mask false
    ids = rng.integers(0, 50_000, n, dtype=np.int64)
    want_masks, want_index, want_counts = oracle_mod.split_compact(ids, table)
    masks = E.cudaSplit(torch.from_numpy(ids).cuda(), torch.from_numpy(table).cuda())
    for m, w in zip(masks, want_masks):
        assert m.dtype == torch.bool and np.array_equal(m.cpu().numpy(), w)
    masks2, index, counts = E.cudaSplitCompact(torch.from_numpy(ids).cuda(), torch.from_numpy(table).cuda())
    assert np.array_equal(counts.cpu().numpy(), want_counts)
    assert np.array_equal(index.cpu().numpy()[: want_index.size], want_index)
    for m, w in zip(masks2, want_masks):
        assert np.array_equal(m.cpu().numpy(), w)


@pytest.mark.parametrize("dtype", [np.int64, np.int32])
def test_owner_search(cuda_lib, oracle_mod, dtype):
    """test/test_binaryserach.py and test_binarysearch2.py: NUM_PART=2, LOCAL_NUM_GPU=4."""
    from hades_b200 import EmbCacheLib as E

    rng = np.random.default_rng(4)
    ids = rng.integers(0, 3_000_000, 100_000).astype(dtype)
    rp = np.array([i * 3_000_000 // 2 for i in range(3)], dtype=dtype)
    got = E.cudaReminder(torch.from_numpy(ids).cuda(), 4)
    assert np.array_equal(got.cpu().numpy(), oracle_mod.owner_mod(ids, 4))
    split = E.cudaBinarySearch(torch.from_numpy(ids).cuda(), torch.from_numpy(rp).cuda(), 4)
    want = oracle_mod.owner_range(ids, rp, 4).astype(dtype)
    assert np.array_equal(split.cpu().numpy(), want)
    value = np.sort(want)
    pr = np.arange(8, dtype=dtype)
    got = E.cudaBinarySearch2(torch.from_numpy(pr).cuda(), torch.from_numpy(value).cuda())
    assert np.array_equal(got.cpu().numpy(), oracle_mod.upper_bound(pr, value))


@pytest.mark.parametrize("W", [1, 2, 8, 64])
@pytest.mark.parametrize("n,dim", [(0, 8), (1, 8), (5000, 3), (70_001, 64), (20_000, 128)])
def test_bucket_pack(cuda_lib, oracle_mod, W, n, dim):
    from hades_b200 import EmbCacheLib as E

    rng = np.random.default_rng(W * 1000 + n)
    ids = rng.integers(0, 10_000_000, n, dtype=np.int64)
    rows = rng.standard_normal((n, dim)).astype(np.float32)
    cnt = rng.integers(1, 9, n, dtype=np.int64)
    wi, wr, wc, wcounts = oracle_mod.bucket_pack(ids, rows, cnt, W)
    gi, gr, gc, gcounts = E.cudaBucketPack(torch.from_numpy(ids).cuda(), torch.from_numpy(rows).cuda(),
                                           torch.from_numpy(cnt).cuda(), W)
    assert np.array_equal(gcounts.cpu().numpy(), wcounts)
    assert np.array_equal(gi.cpu().numpy(), wi)
    assert np.array_equal(gc.cpu().numpy(), wc)
    assert np.array_equal(gr.cpu().numpy(), wr)


def test_bucket_pack_range_partition(cuda_lib, oracle_mod):
    from hades_b200 import EmbCacheLib as E

    rng = np.random.default_rng(77)
    n = 30_000
    ids = rng.integers(0, 4_000_000, n, dtype=np.int64)
    rows = rng.standard_normal((n, 16)).astype(np.float32)
    rp = np.array([0, 1_000_000, 2_500_000, 4_000_000], dtype=np.int64)
    wi, wr, _, wcounts = oracle_mod.bucket_pack(ids, rows, None, 6, rp, 2)
    gi, gr, _, gcounts = E.cudaBucketPack(torch.from_numpy(ids).cuda(), torch.from_numpy(rows).cuda(), None,
                                          6, torch.from_numpy(rp).cuda(), 2)
    assert np.array_equal(gcounts.cpu().numpy(), wcounts)
    assert np.array_equal(gi.cpu().numpy(), wi) and np.array_equal(gr.cpu().numpy(), wr)


@pytest.mark.parametrize("n", [0, 7, 40_000])
def test_grad_split3(cuda_lib, oracle_mod, n):
    from hades_b200 import EmbCacheLib as E

    rng = np.random.default_rng(n + 5)
    ids = rng.integers(0, 1_000_000, n, dtype=np.int64)
    rows = rng.standard_normal((n, 128)).astype(np.float32)
    hot = rng.random(n) < 0.3
    local = rng.random(n) < 0.5
    wi, wr, wc = oracle_mod.grad_split3(ids, rows, hot, local)
    gi, gr, gc = E.cudaGradSplit3(torch.from_numpy(ids).cuda(), torch.from_numpy(rows).cuda(),
                                  torch.from_numpy(hot).cuda(), torch.from_numpy(local).cuda())
    assert np.array_equal(gc.cpu().numpy(), wc)
    assert np.array_equal(gi.cpu().numpy(), wi) and np.array_equal(gr.cpu().numpy(), wr)
