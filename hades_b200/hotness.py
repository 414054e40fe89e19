"""Presampled hotness and what the reference derives from it: the per-node class table of the
forward split, the per-node flush period of the cold cache, and the ids a cache starts with.

    heat = presampling(id_batches, num_nodes, group)        # accesses per sampled batch
    table = class_table(heat, hot_threshold, local_mask)    # 0 local / 1 remote hot / 2 remote cold
    thr = flush_thresholds(heat)                            # cold_cache.flush_thresholds
    fill = hottest_ids(heat, table == 2, entries)           # ids the cold cache is filled with

Plain torch on whatever device the inputs live on; nothing here is on the per-step path.
"""
from __future__ import annotations

import torch

from .cold_cache import flush_thresholds  # noqa: F401  (server.py:87-88, re-exported)


def presampling(id_batches, num_nodes: int, group=None, device=None) -> torch.Tensor:
    """The reference's ``presampling`` (example/train_dist_transductive_graphsage.py:18-52): every
    batch adds one to the heat of the nodes it touches (``heat[input_nodes] += 1``: a node that
    occurs twice in a batch still counts once), heats and batch counts are summed over the ranks,
    and the result is accesses per batch.  id_batches: an iterable of int64 id tensors."""
    heat = torch.zeros(num_nodes, dtype=torch.float32, device=device)
    times = 0
    for ids in id_batches:
        heat[ids.to(heat.device)] += 1
        times += 1
    total = torch.tensor([float(times)], dtype=torch.float32, device=heat.device)
    if group is not None or (torch.distributed.is_available() and torch.distributed.is_initialized()):
        torch.distributed.all_reduce(heat, group=group)
        torch.distributed.all_reduce(total, group=group)
    return heat / total.clamp(min=1.0)


def class_table(hotness: torch.Tensor, hot_threshold: float, local_mask: torch.Tensor | None = None) -> torch.Tensor:
    """``_total_mask`` of the reference (python/EmbCache/dist_emb.py:108-120): int8 per node,
    0 = local, 1 = remote hot (hotness >= hot_threshold), 2 = remote cold.  local_mask None:
    no node is local (every GPU holds a shard of one table, none holds a graph partition)."""
    hot = hotness >= hot_threshold
    table = torch.where(hot, torch.ones((), dtype=torch.int8, device=hotness.device),
                        torch.full((), 2, dtype=torch.int8, device=hotness.device))
    if local_mask is not None:
        table = torch.where(local_mask.to(hotness.device), torch.zeros((), dtype=torch.int8, device=hotness.device),
                            table)
    return table


def hottest_ids(hotness: torch.Tensor, eligible: torch.Tensor, count: int) -> torch.Tensor:
    """The `count` hottest eligible ids, hottest first, ties by ascending id (the order in which
    ``LocalSparseAdamStateCache.create_cache`` ranks its candidates, python/EmbCache/cache.py:
    157-160, made deterministic)."""
    ids = torch.nonzero(eligible).flatten()
    order = torch.argsort(hotness[ids], descending=True, stable=True)
    return ids[order][: int(count)]
