"""TEST INFRASTRUCTURE -- builds the checkers, not the product.

* ``oracle/_oracle.so``  from ``oracle/hades_oracle.c`` (gcc, plain C restatement);
* ``oracle/_ref/libhades_ref.so`` from ``oracle/ref_shim.cpp`` + the reference's own
  ``src/cache/cache.h`` compiled where it lies (g++ on the shim directly; the
  reference's build system is not run).  Only attempted when the reference checkout
  is present; the prebuilt file travels otherwise.
"""
from __future__ import annotations

import os
import subprocess
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
ORACLE_SO = HERE / "_oracle.so"
REF_DIR = HERE / "_ref"
REF_SO = REF_DIR / "libhades_ref.so"
REFERENCE_ROOT = Path(os.environ.get("HADES_REFERENCE_ROOT", "/root/reference"))


def _stale(out: Path, *srcs: Path) -> bool:
    return not out.exists() or any(s.exists() and s.stat().st_mtime > out.stat().st_mtime for s in srcs)


def build_oracle(force: bool = False) -> Path:
    src = HERE / "hades_oracle.c"
    if force or _stale(ORACLE_SO, src):
        subprocess.run(["gcc", "-O2", "-std=c11", "-shared", "-fPIC", "-o", str(ORACLE_SO), str(src)],
                       check=True)
    return ORACLE_SO


def build_ref(force: bool = False) -> Path | None:
    """Compile the reference's CPU index through the shim.  Returns None when the
    reference sources are absent and no prebuilt library exists."""
    header = REFERENCE_ROOT / "src" / "cache" / "cache.h"
    shim = HERE / "ref_shim.cpp"
    if not header.exists():
        return REF_SO if REF_SO.exists() else None
    if not force and not _stale(REF_SO, shim, header):
        return REF_SO
    import pybind11
    import torch

    tdir = Path(torch.__file__).parent
    gxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    REF_DIR.mkdir(exist_ok=True)
    cmd = [gxx, "-O2", "-std=c++17", "-shared", "-fPIC", "-fopenmp", str(shim),
           "-I", str(REFERENCE_ROOT / "src"),
           "-I", str(tdir / "include"), "-I", str(tdir / "include/torch/csrc/api/include"),
           "-I", sysconfig.get_paths()["include"], "-I", pybind11.get_include(),
           "-I", "/usr/local/cuda/include",
           "-L", str(tdir / "lib"), "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_python",
           "-L", "/usr/local/cuda/lib64", "-lcudart",
           f"-Wl,-rpath,{tdir / 'lib'}", "-o", str(REF_SO)]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    return REF_SO


if __name__ == "__main__":
    print(build_oracle())
    print(build_ref())
