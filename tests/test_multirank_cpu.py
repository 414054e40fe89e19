"""The multi-rank exchange logic among CPU ranks (gloo, world size 2): every rank buckets its
rows by owner (oracle restatement of the pack), `exchange_packed` delivers them, and each rank
ends up with exactly the rows it owns, sender by sender in order."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_inputs(rank, n=5000, dim=8):
    rng = np.random.default_rng(100 + rank)
    ids = rng.integers(0, 1_000_000, n, dtype=np.int64)
    rows = rng.standard_normal((n, dim)).astype(np.float32)
    cnt = rng.integers(1, 9, n, dtype=np.int64)
    return ids, rows, cnt


def _worker(rank, world, port, empty_rank):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from hades_b200.sparse_optim import exchange_packed
    from oracle import oracle as om

    n = 0 if rank == empty_rank else 5000
    ids, rows, cnt = _rank_inputs(rank, n)
    p_ids, p_rows, p_cnt, counts = om.bucket_pack(ids, rows, cnt, world)
    r_ids, r_rows, r_cnt = exchange_packed(torch.from_numpy(p_ids), torch.from_numpy(p_rows),
                                           torch.from_numpy(p_cnt), torch.from_numpy(counts))
    # expectation: for each sender in rank order, its rows owned by me, in its input order
    want_ids, want_rows, want_cnt = [], [], []
    for src in range(world):
        s_ids, s_rows, s_cnt = _rank_inputs(src, 0 if src == empty_rank else 5000)
        mine = s_ids % world == rank
        want_ids.append(s_ids[mine])
        want_rows.append(s_rows[mine])
        want_cnt.append(s_cnt[mine])
    assert np.array_equal(r_ids.numpy(), np.concatenate(want_ids))
    assert np.array_equal(r_rows.numpy(), np.concatenate(want_rows))
    assert np.array_equal(r_cnt.numpy(), np.concatenate(want_cnt))
    assert (r_ids.numpy() % world == rank).all()
    # the exchange in reverse (refill after a flush): every owner answers each id it received
    # with a row; the answers come back in the order the ids were sent
    again = exchange_packed(torch.from_numpy(p_ids), torch.from_numpy(p_rows), torch.from_numpy(p_cnt),
                            torch.from_numpy(counts), return_splits=True, counts_host=counts.tolist())
    assert np.array_equal(again[0].numpy(), r_ids.numpy())
    sent, received = again[3]
    assert sent == counts.tolist() and sum(received) == r_ids.numel()
    answer = (again[0].double() * 3 + rank).reshape(-1, 1).repeat(1, 2)      # a function of (id, owner)
    back = torch.empty((sum(sent), 2), dtype=torch.float64)
    dist.all_to_all_single(back, answer, sent, received)
    want_back = np.stack([p_ids * 3.0 + p_ids % world] * 2, axis=1)
    assert np.array_equal(back.numpy(), want_back[:sum(sent)])
    # presampled hotness: heats and batch counts are summed over the ranks
    from hades_b200 import hotness as H

    mine = [torch.tensor([rank, 5]), torch.tensor([5, 6 + rank])] + ([torch.tensor([9])] if rank == 0 else [])
    heat = H.presampling(mine, 10)
    want = torch.zeros(10)
    want[0] = want[1] = want[6] = want[7] = want[9] = 1.0   # 5 batches in all
    want[5] = 4.0
    assert torch.allclose(heat, want / 5.0)
    dist.barrier()
    dist.destroy_process_group()


def _run(empty_rank):
    from oracle import build_oracle

    build_oracle.build_oracle()
    mp.spawn(_worker, args=(2, _free_port(), empty_rank), nprocs=2, join=True)


def test_exchange_two_ranks_gloo():
    _run(empty_rank=-1)


def test_exchange_with_an_empty_sender():
    _run(empty_rank=1)
