"""Pin the CPU oracle (oracle/hades_oracle.c) to the reference: against golden vectors
generated from the reference's own compiled CPU index (tests/golden/make_golden.py), against
the known answers of IndexCache(30), and - where oracle/_ref is available - against the
compiled reference itself on fresh random workloads."""
import numpy as np
import pytest

from .conftest import GOLDEN


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN / "index_golden.npz")


def test_known_answers(oracle_mod, golden):
    # IndexCache(30) -> 4 lines; ways fill from 7 downwards, two LRU evictions, one refusal
    ix = oracle_mod.OracleIndex(30)
    assert ix.get_capacity() == 32 and ix.get_space() == 4 * 96
    a1 = ix.add(np.arange(10))
    assert a1.tolist() == [7, 15, 23, 31, 6, 14, 22, 30, 5, 13]
    assert a1.tolist() == golden["ka_add1"].tolist()
    lk = ix.lookup(np.array([0, 1, 4, 5, 8, 9, 11, 40]))
    assert lk.tolist() == [7, 15, 6, 14, 5, 13, -1, -1] == golden["ka_lookup"].tolist()
    a2 = ix.add(np.arange(0, 41, 4))
    assert a2.tolist() == [7, 6, 5, 4, 3, 2, 1, 0, 7, 6, -1] == golden["ka_add2"].tolist()


def replay(index, golden, i, check):
    ops = golden[f"s{i}_ops"]
    for s, op in enumerate(ops):
        ids = golden[f"s{i}_op{s}_ids"]
        if op == "add":
            check(index.add(ids), golden[f"s{i}_op{s}_out"], (i, s, op))
        elif op == "lookup":
            check(index.lookup(ids), golden[f"s{i}_op{s}_out"], (i, s, op))
        else:
            index.reset(ids)
        assert index.get_valid_entries_num() == int(golden[f"s{i}_op{s}_valid"]), (i, s, op)
    valid = index.get_valid_entries_num()
    gi, gl = index.getall(valid)
    check(gi, golden[f"s{i}_final_ids"], (i, "getall ids"))
    check(gl, golden[f"s{i}_final_locs"], (i, "getall locs"))


def _eq(a, b, where):
    assert np.array_equal(np.asarray(a), np.asarray(b)), where


def test_oracle_matches_golden(oracle_mod, golden):
    for i in range(int(golden["num_scenarios"])):
        ix = oracle_mod.OracleIndex(int(golden[f"s{i}_cache_size"]))
        assert ix.get_capacity() == int(golden[f"s{i}_capacity"])
        assert ix.get_space() == int(golden[f"s{i}_space"])
        replay(ix, golden, i, _eq)


def test_oracle_matches_compiled_reference(oracle_mod):
    if not oracle_mod.RefIndex.available():
        pytest.skip("oracle/_ref/libhades_ref.so not built")
    oracle_mod.RefIndex.set_threads(1)
    rng = np.random.default_rng(7)
    for cache_size, id_range in ((40, 100), (5000, 20000), (4096, 4096 * 3)):
        ref = oracle_mod.RefIndex(cache_size)
        ora = oracle_mod.OracleIndex(cache_size)
        assert ref.get_size() == ora.get_size() and ref.get_space() == ora.get_space()
        for step in range(40):
            ids = rng.integers(0, id_range, int(rng.integers(1, 3000)), dtype=np.int64)
            kind = step % 4
            if kind in (0, 3):
                _eq(ref.add(ids), ora.add(ids), (cache_size, step, "add"))
            elif kind == 1:
                _eq(ref.lookup(ids), ora.lookup(ids), (cache_size, step, "lookup"))
            else:
                ref.reset(ids)
                ora.reset(ids)
            assert ref.get_valid_entries_num() == ora.get_valid_entries_num()
        v = ref.get_valid_entries_num()
        ri, rl = ref.getall(v)
        oi, ol = ora.getall(v)
        _eq(ri, oi, "getall ids")
        _eq(rl, ol, "getall locs")


def test_touch_equals_lookup_side_effect(oracle_mod):
    rng = np.random.default_rng(3)
    a = oracle_mod.OracleIndex(256)
    b = oracle_mod.OracleIndex(256)
    ids = rng.integers(0, 1000, 600, dtype=np.int64)
    a.add(ids)
    b.add(ids)
    q = rng.integers(0, 1000, 2000, dtype=np.int64)
    la = a.lookup(q, touch=True)
    lb = b.lookup(q, touch=False)
    b.touch(lb)
    assert np.array_equal(la, lb)
    assert np.array_equal(a.export()[1], b.export()[1])


def test_row_movers_c_vs_numpy(oracle_mod):
    import ctypes as C

    lib = oracle_mod.lib()
    rng = np.random.default_rng(5)
    src = rng.standard_normal((500, 12)).astype(np.float32)
    si = rng.permutation(500)[:100].astype(np.int64)
    di = rng.permutation(300)[:100].astype(np.int64)
    dst_c = np.zeros((300, 12), np.float32)
    dst_n = dst_c.copy()
    lib.oracle_rows_gather(src.ctypes.data_as(C.c_void_p), si.ctypes.data_as(C.c_void_p),
                           dst_c.ctypes.data_as(C.c_void_p), di.ctypes.data_as(C.c_void_p),
                           C.c_int64(100), C.c_int64(48), C.c_int(8))
    oracle_mod.rows_gather(src, si, dst_n, di)
    assert np.array_equal(dst_c, dst_n)
