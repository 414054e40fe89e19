"""The aggregation restatement (oracle, CPU) and the CUDA kernel (GPU) against outputs of the
reference's own ``only_unique_grads`` / ``unique_grads`` run on CPU tensors
(tests/golden/make_golden_py.py): ids and counts bit-exact, fp32 sums within 1e-5 relative to the
sum of magnitudes.  With ``cnt`` the reference divides by 1 + sum(cnt)."""
import numpy as np
import pytest

from .conftest import GOLDEN

RTOL = 1e-5


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN / "aggregation_golden.npz")


def _scale(idx, grad):
    u, inv = np.unique(idx, return_inverse=True)
    s = np.zeros((u.size, grad.shape[1]), np.float64)
    np.add.at(s, inv, np.abs(grad).astype(np.float64))
    return s


def _cases(golden):
    for k in range(int(golden["num_cases"])):
        yield k, golden[f"c{k}_idx"], golden[f"c{k}_grad"], golden[f"c{k}_cnt"]


def test_oracle_matches_reference_python(oracle_mod, golden):
    for k, idx, grad, cnt in _cases(golden):
        u, s, c = oracle_mod.only_unique_grads(idx, grad)
        assert np.array_equal(u, golden[f"c{k}_sum_ids"]) and np.array_equal(c, golden[f"c{k}_sum_counts"])
        bound = RTOL * np.maximum(_scale(idx, grad), 1e-30)
        assert (np.abs(s.astype(np.float64) - golden[f"c{k}_sum_vals"]) <= bound).all()
        mu, mv, mc = oracle_mod.unique_grads(idx, grad)
        assert np.array_equal(mu, golden[f"c{k}_mean_ids"])
        assert (np.abs(mv.astype(np.float64) - golden[f"c{k}_mean_vals"]) <= bound / mc[:, None]).all()
        cu, cvv, cc = oracle_mod.unique_grads(idx, grad, cnt)
        assert np.array_equal(cu, golden[f"c{k}_cntmean_ids"])
        assert (np.abs(cvv.astype(np.float64) - golden[f"c{k}_cntmean_vals"]) <= bound / cc[:, None]).all()
        # the divisor really is 1 + sum(cnt)
        want_c = np.ones(cu.size, np.int64)
        np.add.at(want_c, np.unique(idx, return_inverse=True)[1], cnt)
        assert np.array_equal(cc, want_c)


@pytest.mark.gpu
def test_cuda_matches_reference_python(cuda_lib, golden):
    import torch

    from hades_b200 import sparse_optim

    for k, idx, grad, cnt in _cases(golden):
        ti, tg, tc = torch.from_numpy(idx).cuda(), torch.from_numpy(grad).cuda(), torch.from_numpy(cnt).cuda()
        bound = RTOL * np.maximum(_scale(idx, grad), 1e-30)
        u, s, c = sparse_optim.only_unique_grads(ti, tg, id_bits=20)
        assert np.array_equal(u.cpu().numpy(), golden[f"c{k}_sum_ids"])
        assert np.array_equal(c.cpu().numpy(), golden[f"c{k}_sum_counts"])
        assert (np.abs(s.cpu().numpy().astype(np.float64) - golden[f"c{k}_sum_vals"]) <= bound).all()
        counts = golden[f"c{k}_sum_counts"]
        mu, mv = sparse_optim.unique_grads(ti, tg, id_bits=20)
        assert np.array_equal(mu.cpu().numpy(), golden[f"c{k}_mean_ids"])
        assert (np.abs(mv.cpu().numpy().astype(np.float64) - golden[f"c{k}_mean_vals"]) <= bound / counts[:, None]).all()
        cu, cvv = sparse_optim.unique_grads(ti, tg, tc, id_bits=20)
        assert np.array_equal(cu.cpu().numpy(), golden[f"c{k}_cntmean_ids"])
        assert (np.abs(cvv.cpu().numpy().astype(np.float64) - golden[f"c{k}_cntmean_vals"]) <= bound).all()
