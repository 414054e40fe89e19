"""Failure detection without faulting a GPU: device-side waits have an iteration limit and
report a status code that the host reads; the context stays usable afterwards."""
import os
import socket
import sys
import time
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def test_bounded_wait_times_out_and_context_survives(cuda_lib):
    from hades_b200 import _lib

    lib = _lib.load()
    flag = torch.zeros(1, dtype=torch.int64, device="cuda")
    assert _lib.device_status() == 0
    t0 = time.perf_counter()
    _lib.check(lib.hb_wait_flag(flag.data_ptr(), 1, _lib.stream_ptr()))  # nothing ever sets the flag
    assert _lib.device_status() == 5  # HB_ERR_TIMEOUT, and the word is cleared by the read
    assert time.perf_counter() - t0 < 30
    assert _lib.device_status() == 0
    flag.fill_(3)
    _lib.check(lib.hb_wait_flag(flag.data_ptr(), 2, _lib.stream_ptr()))  # already reached: returns at once
    assert _lib.device_status() == 0
    # the context is still usable
    x = torch.arange(10, device="cuda")
    assert int(x.sum().item()) == 45


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, port):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=2, device_id=torch.device("cuda", rank))
    from hades_b200 import _lib
    from hades_b200.exchange import PeerExchange

    px = PeerExchange(rank, 2, 1024, 16)
    ids = torch.arange(100, dtype=torch.int64, device="cuda")
    rows = torch.ones((100, 16), device="cuda")
    # a healthy exchange first
    p = px.push(ids, rows)
    px.fence()
    got = px.received(p)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert int(got[3].sum().item()) == 100  # 50 rows from each rank
    dist.barrier()
    # rank 1 "fails" between steps: it never pushes nor fences again.  Rank 0 learns it from
    # the status word after its bounded wait, not from a hang.
    if rank == 0:
        px.push(ids, rows)
        px.fence()
        torch.cuda.synchronize()
        assert _lib.device_status() == 5
        assert int(torch.arange(4, device="cuda").sum().item()) == 6  # context usable
    dist.barrier()
    # recovery: rank 1 is back (the host side has agreed on it: the barrier above).  After the
    # reset both ranks start again from exchange number 0 and clean receive areas, although rank 0
    # is one exchange ahead of rank 1.
    px.reset()
    for _ in range(3):
        p = px.push(ids, rows * (rank + 1))
        px.fence()
        got = px.received(p)
        torch.cuda.synchronize()
        assert _lib.device_status() == 0
        counts = got[3].cpu()
        assert counts.tolist() == [50, 50]
        cap = got[0].numel() // 2
        for src in range(2):
            seg_ids = got[0][src * cap: src * cap + 50].cpu()
            assert seg_ids.tolist() == list(range(rank, 100, 2))  # owner = id % 2, in order
            assert bool((got[1][src * cap: src * cap + 50] == float(src + 1)).all())
        px.fence()  # nobody pushes into the area again before everyone has read it
    px.close()
    dist.destroy_process_group()


def test_missing_peer_is_a_status_code_not_a_hang():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    mp.spawn(_worker, args=(_free_port(),), nprocs=2, join=True)
