"""The C-ABI library loads without a GPU and exports every symbol that include/*.h declares;
the ctypes prototype table covers the same set."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    names = set()
    for h in (ROOT / "include").glob("*.h"):
        text = re.sub(r"/\*.*?\*/", "", h.read_text(), flags=re.S)
        names |= set(re.findall(r"\b(hb_[a-z0-9_]+)\s*\(", text))
    return names


@pytest.fixture(scope="module")
def built_lib():
    from hades_b200 import _build

    return _build.build()


def test_header_symbols_exported(built_lib):
    lib = ctypes.CDLL(str(built_lib))
    names = declared_symbols()
    assert len(names) > 30
    missing = [n for n in sorted(names) if not hasattr(lib, n)]
    assert not missing, f"declared in include/*.h but not exported: {missing}"


def test_prototype_table_matches_header(built_lib):
    from hades_b200 import _lib

    assert set(_lib.PROTOTYPES) == declared_symbols()
    _lib.load()  # binds every prototype; raises if one is absent


def test_no_gpu_calls_return_status_not_crash(built_lib):
    from hades_b200 import _lib

    lib = _lib.load()
    assert lib.hb_version() >= 100
    # argument validation happens before any CUDA work
    rc = lib.hb_rows_gather(None, None, None, None, 5, 16, 8, 0, None)
    assert rc == 1 and b"null" in lib.hb_last_error()
    rc = lib.hb_rows_gather(None, None, None, None, 0, 16, 3, 0, None)
    assert rc == 1
    assert lib.hb_index_size(None) == -1


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from hades_b200 import _lib

    monkeypatch.setattr(_lib, "_LIB", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _lib.load()


def test_reference_side_bridge_compiles():
    """hades_b200/bridge/hades_b200_bridge.cc (the translation unit a maintainer of the reference
    adds beside src/pybind.cc) compiles against the torch headers and include/hades_b200.h."""
    import shutil
    import subprocess
    import sysconfig
    from pathlib import Path

    import torch

    root = Path(__file__).resolve().parent.parent
    tdir = Path(torch.__file__).parent
    gxx = "/usr/bin/g++" if Path("/usr/bin/g++").exists() else shutil.which("g++")
    cmd = [gxx, "-std=c++17", "-fsyntax-only", str(root / "hades_b200" / "bridge" / "hades_b200_bridge.cc"),
           "-I", str(root / "include"), "-I", str(tdir / "include"),
           "-I", str(tdir / "include/torch/csrc/api/include"), "-I", sysconfig.get_paths()["include"],
           "-I", "/usr/local/cuda/include"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
