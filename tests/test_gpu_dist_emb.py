"""The layer / optimiser surface a model uses (DistEmb, DistembSparseGradOptimizer) against the
same steps driven through EmbeddingPath directly; split CUDA graphs against eager launches; save
and resume."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _cfg(name, dim=64, flush_every=3):
    from hades_b200 import synth

    base = synth.scaled(synth.CONFIG1, 0.05, name)
    return synth.CacheFetchConfig(base.name, base.config, base.table_rows, dim, base.cache_entries, base.batch,
                                  base.zipf_s, flush_every=flush_every)


def _batches(cfg, n, stream):
    from hades_b200 import synth

    sampler = synth.ZipfSampler(cfg.table_rows, cfg.zipf_s)
    rng = synth.rng_for(1, 0, stream)
    return [torch.from_numpy(sampler.ids(rng, cfg.batch)).cuda() for _ in range(n)]


def _same_state(a, b):
    assert torch.equal(a.table, b.table)
    assert torch.equal(a.opt.state_mem, b.opt.state_mem) and torch.equal(a.opt.state_step, b.opt.state_step)
    assert torch.equal(a.cold.remote.grad, b.cold.remote.grad) and torch.equal(a.cold.remote.cnt, b.cold.remote.cnt)
    assert torch.equal(a.cold.emb, b.cold.emb)
    for x, y in zip(a.cold.index.export_state(), b.cold.index.export_state()):
        assert torch.equal(x, y)


@pytest.mark.parametrize("captured", [False, True])
def test_module_and_optimizer_equal_direct_path(cuda_lib, captured):
    from hades_b200 import pipeline
    from hades_b200.dist_emb import DistEmb, DistembSparseGradOptimizer

    cfg = _cfg("distemb_a")
    cfg_b = _cfg("distemb_b")
    pa, pb = pipeline.build_path(cfg), pipeline.build_path(cfg_b)
    layer = DistEmb(pa)
    opt = DistembSparseGradOptimizer([layer.sparse_emb])
    head = torch.nn.Linear(cfg.dim, 8).cuda()
    batches = _batches(cfg, 8, 21)
    for k, ids in enumerate(batches):
        if captured and k == 2:
            torch.cuda.synchronize()
            layer.sparse_emb.capture(cfg.batch)
        h = layer(ids)
        assert h.requires_grad and h.is_leaf
        loss = head(h).square().sum() * 1e-3
        opt.zero_grad()
        loss.backward()
        g = h.grad.clone()
        opt.step()
        assert layer.sparse_emb.trace == []
        # the same step through the path itself
        rows, locs, found, st = pb.step(ids, g)
        assert torch.equal(rows, h.detach())
        assert st.flushed == opt.last_stats[layer.sparse_emb.name].flushed
    assert pa.step_no == pb.step_no == 8
    _same_state(pa, pb)


def test_two_calls_before_step_and_eval_rows(cuda_lib):
    from hades_b200 import pipeline
    from hades_b200.dist_emb import DistEmb, DistembSparseGradOptimizer

    pa, pb = pipeline.build_path(_cfg("distemb_c", 32)), pipeline.build_path(_cfg("distemb_d", 32))
    layer = DistEmb(pa)
    opt = DistembSparseGradOptimizer([layer.sparse_emb], lr=0.01)
    ids1, ids2 = _batches(_cfg("x", 32), 2, 22)
    h1, h2 = layer(ids1), layer(ids2[:1000])
    (h1.sum() * 1e-3 + h2.square().sum()).backward()
    opt.zero_grad()
    opt.step()
    ids = torch.cat([ids1, ids2[:1000]])
    pb.forward(ids1)
    pb.forward(ids2[:1000])
    pb.backward(ids, torch.cat([h1.grad, h2.grad]))
    _same_state(pa, pb)
    layer.eval()
    with torch.no_grad():
        rows = layer(ids2)
    assert torch.equal(rows, pa.table[ids2]) and layer.sparse_emb.trace == []


def test_save_and_resume_is_bit_exact(cuda_lib):
    from hades_b200 import pipeline, synth

    cfg = _cfg("resume_a", 32, flush_every=2)
    pa = pipeline.build_path(cfg)
    batches = _batches(cfg, 9, 23)
    rng = synth.rng_for(1, 0, 24)
    grads = torch.from_numpy(synth.normal_rows(rng, cfg.batch, cfg.dim, cfg.grad_sigma)).cuda()
    for ids in batches[:5]:
        pa.step(ids, grads)
    sd = {k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in pa.state_dict().items()
          if k not in ("staging", "optimizer")}
    full = pa.state_dict()
    sd["staging"] = {k: v.cpu() for k, v in full["staging"].items()}
    sd["optimizer"] = {k: v.cpu() for k, v in full["optimizer"].items()}
    outs_a = [pa.step(ids, grads)[0].clone() for ids in batches[5:]]
    pb = pipeline.build_path(_cfg("resume_b", 32, flush_every=2))
    pb.load_state_dict(sd)
    assert pb.step_no == 5
    outs_b = [pb.step(ids, grads)[0].clone() for ids in batches[5:]]
    for x, y in zip(outs_a, outs_b):
        assert torch.equal(x, y)
    _same_state(pa, pb)
