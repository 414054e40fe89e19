"""The allocation-free owner bucketing (hb_bucket_pack_noalloc) gives the same bytes as
hb_bucket_pack.  It exists for hosts that cannot pass a workspace or let the library allocate
(a runtime that owns the allocator, a frozen memory plan); its scratch is a fixed array inside
the library that every call on a device shares, so the check runs twice in a row with
different inputs: the second call must not be disturbed by what the first one left there.

Collected last on purpose (file name), and self-contained: it passes alone in a fresh process
and after the rest of the suite.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _pack(lib, fn_name, ids, rows, cnt, buckets, ws=None):
    n, dim = ids.numel(), rows.size(1)
    out_ids = torch.full_like(ids, -1)
    out_rows = torch.zeros_like(rows)
    out_cnt = torch.full_like(cnt, -1)
    counts = torch.full((buckets,), -1, dtype=torch.int64, device=ids.device)
    stream = torch.cuda.current_stream().cuda_stream
    common = (ids.data_ptr(), rows.data_ptr(), cnt.data_ptr(), n, None, dim * 4, buckets, None, 0, buckets,
              out_ids.data_ptr(), out_rows.data_ptr(), out_cnt.data_ptr(), counts.data_ptr())
    if ws is None:
        rc = getattr(lib, fn_name)(*common, stream)
    else:
        rc = getattr(lib, fn_name)(*common, ws.data_ptr(), ws.numel(), stream)
    assert rc == 0, lib.hb_last_error()
    torch.cuda.synchronize()
    return out_ids, out_rows, out_cnt, counts


def test_noalloc_bucket_pack_matches_workspace_version():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from hades_b200 import _lib

    lib = _lib.load()
    torch.cuda.set_device(0)
    assert lib.hb_bucket_pack_noalloc_max_items() == 1 << 20
    assert lib.hb_bucket_pack_noalloc_max_buckets() == 64
    rng = np.random.default_rng(123)
    # two calls in a row on the shared scratch: a large one, then a smaller one with other
    # bucket counts, whose result must not depend on the leftovers of the first
    for n, dim, buckets in ((1 << 20, 16, 64), (70_001, 64, 8), (5, 4, 3)):
        ids = torch.from_numpy(rng.integers(0, 10**9, n, dtype=np.int64)).cuda()
        rows = torch.from_numpy(rng.standard_normal((n, dim)).astype(np.float32)).cuda()
        cnt = torch.from_numpy(rng.integers(1, 9, n, dtype=np.int64)).cuda()
        ws = torch.empty(lib.hb_partition_workspace_bytes(n, buckets), dtype=torch.uint8, device="cuda")
        want = _pack(lib, "hb_bucket_pack", ids, rows, cnt, buckets, ws)
        got = _pack(lib, "hb_bucket_pack_noalloc", ids, rows, cnt, buckets)
        for g, w in zip(got, want):
            assert torch.equal(g, w)  # integers and row copies: bit-exact, as in the other tests
        own = (ids % buckets).cpu().numpy()
        assert np.array_equal(got[3].cpu().numpy(), np.bincount(own, minlength=buckets))


def test_noalloc_rejects_oversize_requests():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from hades_b200 import _lib

    lib = _lib.load()
    dummy = torch.zeros(8, dtype=torch.int64, device="cuda")
    p = dummy.data_ptr()
    rc = lib.hb_bucket_pack_noalloc(p, None, None, (1 << 20) + 1, None, 0, 8, None, 0, 8, p, None, None, p, None)
    assert rc == 6 and b"exceed the built-in scratch" in lib.hb_last_error()
    rc = lib.hb_bucket_pack_noalloc(p, None, None, 8, None, 0, 65, None, 0, 65, p, None, None, p, None)
    assert rc == 6
