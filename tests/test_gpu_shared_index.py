"""One cache index shared by two processes of a box, the scenario of the reference's
test/test_cache.py:6-61 (rank 0 creates IndexCache(name, create=True), rank 1 opens it with
create=False; each sees what the other added), here over CUDA IPC on one GPU with gloo barriers
between the phases.  Slots against the oracle index driven by the same calls."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, port, name):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist

    dist.init_process_group("gloo", rank=rank, world_size=2)
    torch.cuda.set_device(0)
    from hades_b200 import EmbCacheLib as E
    from oracle import oracle as om

    rng = np.random.default_rng(5)
    a, b, c = (rng.integers(0, 50_000, 4000, dtype=np.int64) for _ in range(3))
    ora = om.OracleIndex(10_000)
    wa, wl, wb = ora.add(a), ora.lookup(c), ora.add(b)   # the calls both processes make, in order
    wc = ora.lookup(c)
    if rank == 0:
        ix = E.IndexCache(10_000, name, True, False)
        assert np.array_equal(ix.add(torch.from_numpy(a)).numpy(), wa)
        torch.cuda.synchronize()
    dist.barrier()
    if rank == 1:
        ix = E.IndexCache(10_000, name, False, False)     # the creator's lines, mapped
        assert ix.get_capacity() == ora.get_capacity()
        assert np.array_equal(ix.lookup(torch.from_numpy(c)).numpy(), wl)   # sees rank 0's ids (and ages the LRU)
        assert np.array_equal(ix.add(torch.from_numpy(b)).numpy(), wb)      # evicts by the shared LRU counters
        assert np.array_equal(ix.cudalookup(torch.from_numpy(c).cuda(), mode=E.LOOKUP_SORTED).cpu().numpy(),
                              ora.lookup(c, touch=False))
        torch.cuda.synchronize()
    dist.barrier()
    if rank == 0:
        assert np.array_equal(ix.lookup(torch.from_numpy(c)).numpy(), wc)   # sees rank 1's ids
        gi, gl = ix.export_state()
        oi, ol = ora.export()
        assert np.array_equal(gi.cpu().numpy(), oi) and np.array_equal(gl.cpu().numpy(), ol)
    dist.barrier()
    if rank == 1:
        ix.close()  # the opener closes its mapping before the creator frees the lines
        torch.cuda.synchronize()
    dist.barrier()
    if rank == 0:
        ix.close()  # frees the lines and withdraws the handle file
    dist.destroy_process_group()


def test_two_processes_share_one_index():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import torch.multiprocessing as mp

    from oracle import build_oracle

    build_oracle.build_oracle()
    mp.spawn(_worker, args=(_free_port(), f"shared_ix_{os.getpid()}"), nprocs=2, join=True)
    assert not os.path.exists(f"/dev/shm/hades_b200_index_shared_ix_{os.getpid()}")


def test_open_without_creator_raises(cuda_lib):
    from hades_b200 import EmbCacheLib as E

    with pytest.raises(RuntimeError, match="fail to open"):
        E.IndexCache(100, "no_such_index_anywhere", False, False)
