"""The embedding layer and its sparse optimiser as a model sees them: the surface of the
reference's ``DistEmb`` / ``DistEmbeddingTensor`` (python/EmbCache/dist_emb.py:11-292) and
``DistembSparseGradOptimizer`` (python/EmbCache/sparse_optim.py:160-470) over an
``EmbeddingPath``.

    emb_layer = DistEmb(path)
    emb_optimizer = DistembSparseGradOptimizer([emb_layer.sparse_emb])
    ...
    h = emb_layer(input_nodes)          # [n, dim] leaf tensor that requires grad
    loss = model(blocks, h) ...
    emb_optimizer.zero_grad(); loss.backward(); emb_optimizer.step()

As in the reference the layer records ``(ids, rows)`` per call in ``trace``
(dist_emb.py:272-285) and the optimiser reads ``rows.grad`` from it (sparse_optim.py:225-226);
``zero_grad`` only arms the clearing of the trace at the next ``step`` (sparse_optim.py:350-354,
468-470), so a ``step`` without ``zero_grad`` applies the old gradients again, as it does there.
What differs: all of it runs on this GPU's current stream (no cache-server process, no sockets);
``step`` hands the concatenated trace to ``EmbeddingPath.backward`` (aggregation, split, cold
accumulate, exchange, update, periodic flush) and returns its counters.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import EmbCacheLib as E
from .pipeline import EmbeddingPath


class DistEmbeddingTensor:
    def __init__(self, path: EmbeddingPath, name: str = "emb"):
        self.path = path
        self.name = name
        self.num_embeddings, self.embedding_dim = path.num_nodes, path.dim
        self.enable_cache = True
        self.trace: list[tuple] = []
        self._captured_batch = 0
        self._replays = 0

    def capture(self, batch: int) -> None:
        """Replay the forward fetch and the backward path from CUDA graphs for calls with exactly
        ``batch`` ids (other sizes keep running eagerly).  Call after a few eager steps.  The rows
        a replayed call returns live in the graph's output buffer: the next such call overwrites
        them."""
        dev = self.path.device
        ids = torch.zeros(batch, dtype=torch.int64, device=dev)
        grads = torch.zeros((batch, self.embedding_dim), dtype=torch.float32, device=dev)
        out = torch.empty((batch, self.embedding_dim), dtype=self.path.row_dtype, device=dev)
        self.path.capture_split(ids, grads, out)
        self._captured_batch = batch

    def authoritative_rows(self, ids: torch.Tensor) -> torch.Tensor:
        """Current table rows (no cache), the reference's ``self.tensor[ids]``
        (dist_emb.py:168-169): from the owners' shards when the table is sharded."""
        p = self.path
        if p.shared is not None:
            return p.shared.gather(ids)
        out = torch.empty((ids.numel(), self.embedding_dim), dtype=p.table.dtype, device=ids.device)
        E.cudaFetch2(p.table, ids, out)
        return out

    def __call__(self, ids: torch.Tensor, device=None, is_training: bool = True) -> torch.Tensor:
        dev = self.path.device
        ids = ids.to(dev, non_blocking=True)
        if not is_training:
            rows = self.authoritative_rows(ids)
            return rows if device is None else rows.to(device)
        if self._captured_batch and ids.numel() == self._captured_batch:
            rows, locs, _ = self.path.forward_replay(ids)
            self._replays += 1
            serial = self._replays
        else:
            rows, locs, _ = self.path.forward(ids)
            serial = 0
        emb = rows.detach().requires_grad_(True)
        if torch.is_grad_enabled():
            self.trace.append((ids, emb, locs, serial))
        return emb

    def reset_trace(self) -> None:
        self.trace = []


class DistEmb(nn.Module):
    """``nn.Module`` face of the layer (dist_emb.py:11-51)."""

    def __init__(self, path: EmbeddingPath, name: str = "emb_layer"):
        super().__init__()
        self.emb_dim = path.dim
        self.sparse_emb = DistEmbeddingTensor(path, name)

    def forward(self, idx: torch.Tensor) -> torch.Tensor:
        return self.sparse_emb(idx, None, self.training)


class DistembSparseGradOptimizer:
    """``step`` / ``zero_grad`` of the reference's sparse optimiser base class over the paths of
    ``params`` (a list of ``DistEmbeddingTensor``).  The update rule and its state live in the
    path's optimiser (``SparseAdam`` / ``SparseAdagrad`` on the owner shard)."""

    def __init__(self, params, lr: float | None = None):
        self._params = list(params)
        self._clean_grad = False
        if lr is not None:
            for emb in self._params:
                emb.path.opt._lr = float(lr)
        self.last_stats = {}

    def zero_grad(self) -> None:
        self._clean_grad = True

    @torch.no_grad()
    def step(self) -> None:
        for emb in self._params:
            trace = [t for t in emb.trace if t[1].grad is not None]
            if not trace:
                continue
            if len(trace) == 1 and trace[0][3] and trace[0][3] == emb._replays:
                # the one call of this step went through the captured forward and nothing has
                # replayed it since: its ids and slots are still in the graph's buffers
                st = emb.path.backward_replay(trace[0][1].grad)
            else:
                # (every forward call has aged the LRU counters of its own lookup; the backward
                # pass sorts the concatenated ids itself unless they are the last call's batch)
                ids = torch.cat([t[0] for t in trace]) if len(trace) > 1 else trace[0][0]
                grads = torch.cat([t[1].grad for t in trace]) if len(trace) > 1 else trace[0][1].grad
                st = emb.path.backward(ids, grads.contiguous())
            self.last_stats[emb.name] = st
        if self._clean_grad:
            for emb in self._params:
                emb.reset_trace()
            self._clean_grad = False
