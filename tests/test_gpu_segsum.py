"""Hot-node local aggregation against the oracle's restatement of only_unique_grads /
unique_grads: unique ids and counts bit-exact, fp32 sums within 1e-5 relative (the
summation order differs from index_add_'s), and bitwise reproducible run to run."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

RTOL = 1e-5  # relative error bound on fp32 gradient sums


def _close(got, want, scale):
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    assert err.max(initial=0.0) <= RTOL * scale, err.max()


def _ids(rng, n, kind):
    if kind == "zipf":
        from hades_b200 import synth

        return synth.ZipfSampler(1_000_000, 1.2).ids(rng, n)
    if kind == "one":
        return np.full(n, 42, dtype=np.int64)
    if kind == "unique":
        return rng.permutation(n * 3)[:n].astype(np.int64)
    return rng.integers(0, max(n // 3, 1), n, dtype=np.int64)


@pytest.mark.parametrize("kind", ["zipf", "uniform", "one", "unique"])
@pytest.mark.parametrize("n,dim", [(1, 128), (33, 128), (5000, 128), (70_000, 64), (40_000, 3),
                                   (30_000, 257), (9_000, 640), (524_288, 128)])
def test_only_unique_grads(cuda_lib, oracle_mod, kind, n, dim):
    from hades_b200 import EmbCacheLib as E

    if n > 100_000 and kind not in ("zipf",):
        pytest.skip("large case runs on the Zipf stream only")
    rng = np.random.default_rng(n * 13 + dim)
    ids = _ids(rng, n, kind)
    grad = (rng.standard_normal((n, dim)) * 1e-3).astype(np.float32)
    wu, wv, wc = oracle_mod.only_unique_grads(ids, grad)
    gu, gv, gc = E.cudaUniqueSegSum(torch.from_numpy(ids).cuda(), torch.from_numpy(grad).cuda(), id_bits=40)
    assert np.array_equal(gu.cpu().numpy(), wu)
    assert np.array_equal(gc.cpu().numpy(), wc)
    # scale: the sum of magnitudes bounds the rounding error of any summation order
    absum = np.zeros_like(wv)
    np.add.at(absum, np.unique(ids, return_inverse=True)[1], np.abs(grad))
    err = np.abs(gv.cpu().numpy().astype(np.float64) - wv.astype(np.float64))
    assert (err <= RTOL * np.maximum(absum, 1e-30)).all(), err.max()
    # deterministic: same bits on a second run
    gu2, gv2, gc2 = E.cudaUniqueSegSum(torch.from_numpy(ids).cuda(), torch.from_numpy(grad).cuda(), id_bits=40)
    assert torch.equal(gv, gv2) and torch.equal(gu, gu2) and torch.equal(gc, gc2)


@pytest.mark.parametrize("with_cnt", [False, True])
def test_unique_grads_mean(cuda_lib, oracle_mod, with_cnt):
    from hades_b200 import EmbCacheLib as E

    rng = np.random.default_rng(21 + with_cnt)
    n, dim = 60_000, 128
    ids = _ids(rng, n, "zipf")
    grad = (rng.standard_normal((n, dim)) * 1e-3).astype(np.float32)
    cnt = rng.integers(1, 17, n, dtype=np.int64) if with_cnt else None
    wu, wv, wc = oracle_mod.unique_grads(ids, grad, cnt)
    gu, gv, gc = E.cudaUniqueSegSum(torch.from_numpy(ids).cuda(), torch.from_numpy(grad).cuda(),
                                    None if cnt is None else torch.from_numpy(cnt).cuda(), mean=True, id_bits=32)
    assert np.array_equal(gu.cpu().numpy(), wu)
    assert np.array_equal(gc.cpu().numpy(), wc)  # 1 + sum(cnt) when cnt is given
    absum = np.zeros_like(wv)
    np.add.at(absum, np.unique(ids, return_inverse=True)[1], np.abs(grad))
    err = np.abs(gv.cpu().numpy().astype(np.float64) - wv.astype(np.float64))
    assert (err <= RTOL * np.maximum(absum / wc[:, None], 1e-30)).all()


def test_empty(cuda_lib):
    from hades_b200 import EmbCacheLib as E

    u, v, c = E.cudaUniqueSegSum(torch.empty(0, dtype=torch.int64, device="cuda"),
                                 torch.empty((0, 8), device="cuda"))
    assert u.numel() == 0 and v.shape == (0, 8) and c.numel() == 0


@pytest.mark.parametrize("n,dim", [(1, 8), (5000, 128), (200_000, 64), (60_000, 257)])
def test_unique_segsum_with_class_split(cuda_lib, oracle_mod, n, dim):
    """Aggregation with the hot/cold selects fused into its output: every class buffer holds
    the ids (ascending), counts and sums that selecting from only_unique_grads' output gives;
    a dropped class is only counted; ids whose table value is outside {0,1,2} vanish."""
    from hades_b200 import EmbCacheLib as E

    rng = np.random.default_rng(n + dim)
    nodes = 50_000
    table = rng.integers(0, 3, nodes).astype(np.int8)
    table[::53] = 7
    ids = _ids(rng, n, "uniform") % nodes
    grad = (rng.standard_normal((n, dim)) * 1e-3).astype(np.float32)
    u, s, c = oracle_mod.only_unique_grads(ids, grad)
    outs, class_counts, num = E.cudaUniqueSegSumSplit(torch.from_numpy(ids).cuda(), torch.from_numpy(grad).cuda(),
                                                      torch.from_numpy(table).cuda(), keep=(True, False, True),
                                                      id_bits=20)
    assert int(num.item()) == u.size
    cc = class_counts.cpu().numpy()
    for k in range(3):
        sel = table[u] == k
        assert cc[k] == sel.sum()
        if k == 1:
            assert outs[k] is None
            continue
        gi, gr, gc = (t[: cc[k]].cpu().numpy() for t in outs[k])
        assert np.array_equal(gi, u[sel]) and np.array_equal(gc, c[sel])
        np.testing.assert_allclose(gr, s[sel], rtol=1e-4, atol=1e-8)


@pytest.mark.parametrize("num_seg,cap,dim,universe", [(1, 500, 128, 2000), (2, 3000, 128, 5000), (3, 1000, 20, 1500),
                                                       (8, 2000, 64, 6000), (8, 40, 7, 60), (40, 64, 32, 300)])
@pytest.mark.parametrize("with_cnt,mean", [(True, True), (False, True), (False, False)])
def test_merge_sorted_slabs_equals_sorting_path(cuda_lib, oracle_mod, num_seg, cap, dim, universe, with_cnt, mean):
    """Slabs of ascending unique ids (ragged, one of them empty): the merge gives what the
    sorting path gives on the same slabs, and what the oracle's unique_grads gives."""
    from hades_b200 import EmbCacheLib as E

    rng = np.random.default_rng(num_seg * 1000 + cap)
    ids = np.full((num_seg, cap), -1, np.int64)
    rows = rng.standard_normal((num_seg, cap, dim)).astype(np.float32)
    cnt = rng.integers(1, 6, (num_seg, cap)).astype(np.int64)
    counts = rng.integers(0, cap + 1, num_seg).astype(np.int64)
    counts[rng.integers(0, num_seg)] = 0 if num_seg > 1 else cap
    counts = np.minimum(counts, universe)
    if num_seg > 2:
        counts[1] = min(cap, universe)  # one full slab
    for s in range(num_seg):
        ids[s, :counts[s]] = np.sort(rng.choice(universe, counts[s], replace=False))
    d_ids, d_rows = torch.from_numpy(ids.reshape(-1)).cuda(), torch.from_numpy(rows.reshape(-1, dim)).cuda()
    d_cnt = torch.from_numpy(cnt.reshape(-1)).cuda() if with_cnt else None
    d_counts = torch.from_numpy(counts).cuda()
    u, r, c, num = E.cudaMergeSortedSlabs(d_ids, d_rows, d_cnt, d_counts, cap, mean=mean)
    u2, r2, c2, num2 = E.cudaUniqueSegSum(d_ids, d_rows, d_cnt, mean=mean, id_bits=20, sync=False,
                                          seg_counts=d_counts, seg_cap=cap)
    k = int(num.item())
    assert k == int(num2.item())
    assert torch.equal(u[:k], u2[:k]) and torch.equal(c[:k], c2[:k])
    # the sorting path may add a long run in another order
    torch.testing.assert_close(r[:k], r2[:k], rtol=1e-5, atol=1e-5)
    valid = np.concatenate([np.arange(s * cap, s * cap + counts[s]) for s in range(num_seg)]).astype(np.int64)
    if valid.size and mean:
        wu, wm, _ = oracle_mod.unique_grads(ids.reshape(-1)[valid], rows.reshape(-1, dim)[valid],
                                            cnt.reshape(-1)[valid] if with_cnt else None)
        assert np.array_equal(u[:k].cpu().numpy(), wu)
        np.testing.assert_allclose(r[:k].cpu().numpy(), wm, rtol=1e-5, atol=1e-6)
