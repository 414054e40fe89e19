"""Pin the oracle's restatement of the cache-server arithmetic and of SparseAdam.update to the
outputs of the reference's own Python (tests/golden/make_golden_server.py ran
python/EmbCache/server.py:346-574 and sparse_optim.py:590-685 on CPU tensors)."""
import numpy as np
import pytest

from . import server_replay
from .conftest import GOLDEN


@pytest.fixture(scope="module")
def server_golden():
    return np.load(GOLDEN / "server_golden.npz")


@pytest.fixture(scope="module")
def adam_golden():
    return np.load(GOLDEN / "adam_golden.npz")


def test_oracle_server_literal_reference(oracle_mod, server_golden):
    """compat_no_clear=True is the reference as written (gradient rows never cleared,
    server.py:414,489,537): every buffer and everything sent is bit-exact in both scenarios."""
    for name in ("once", "again"):
        be = server_replay.OracleBackend(oracle_mod, server_golden, name, compat_no_clear=True)
        server_replay.replay(server_golden, name, be, rows_exact=True, buffers_exact=True)


def test_oracle_server_intended_clear(oracle_mod, server_golden):
    """The read-and-zero behaviour (what the CUDA library implements): where no slot is staged
    into again after its flush the sent rows equal the reference's; in the other scenario
    everything but the gradient rows does."""
    be = server_replay.OracleBackend(oracle_mod, server_golden, "once", compat_no_clear=False)
    server_replay.replay(server_golden, "once", be, rows_exact=True, buffers_exact=False)
    be = server_replay.OracleBackend(oracle_mod, server_golden, "again", compat_no_clear=False)
    server_replay.replay(server_golden, "again", be, rows_exact=False, buffers_exact=False)


def adam_rounds(g, k):
    rows, dim, unique, rounds = (int(x) for x in g[f"a{k}_meta"])
    for r in range(rounds):
        cnt = g[f"a{k}_r{r}_cnt"]
        yield r, bool(unique), g[f"a{k}_r{r}_idx"], g[f"a{k}_r{r}_grad"], (cnt if cnt.size else None)


# fp32 arithmetic in another order (numpy / CUDA against torch CPU): relative to operand scale
ADAM_RTOL = 1e-5


def check_adam_state(g, k, r, step, mem, power, emb):
    assert np.array_equal(step, g[f"a{k}_r{r}_step"]), (k, r)
    np.testing.assert_allclose(mem, g[f"a{k}_r{r}_mem"], rtol=ADAM_RTOL, atol=ADAM_RTOL * 1e-3)
    np.testing.assert_allclose(power, g[f"a{k}_r{r}_power"], rtol=ADAM_RTOL, atol=ADAM_RTOL * 1e-6)
    # the first steps move a weight by about lr (0.01) whatever the gradient's size, and where the
    # duplicates of an id nearly cancel the rounding of their mean is amplified by 1 / |mean|
    np.testing.assert_allclose(emb, g[f"a{k}_r{r}_emb"], rtol=1e-4, atol=0.01 * 1e-3)


def test_oracle_adam_matches_reference(oracle_mod, adam_golden):
    g = adam_golden
    for k in range(int(g["num_cases"])):
        rows, dim = int(g[f"a{k}_meta"][0]), int(g[f"a{k}_meta"][1])
        step, mem, power = np.zeros(rows, np.float32), np.zeros((rows, dim), np.float32), np.zeros((rows, dim), np.float32)
        emb = g[f"a{k}_emb0"].copy()
        for r, unique, idx, grad, cnt in adam_rounds(g, k):
            if unique:
                oracle_mod.sparse_adam_update(idx, grad, step, mem, power, emb, 0.01, cnt=cnt)
            else:
                u, mean, _ = oracle_mod.unique_grads(idx, grad, cnt)
                oracle_mod.sparse_adam_update(u, mean, step, mem, power, emb, 0.01)
            check_adam_state(g, k, r, step, mem, power, emb)
