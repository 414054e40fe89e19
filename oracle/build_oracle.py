"""TEST INFRASTRUCTURE -- builds the checkers, not the product.

* ``oracle/_oracle.so``  from ``oracle/hades_oracle.c`` (gcc, plain C restatement);
* ``oracle/_ref/libhades_ref.so`` from ``oracle/ref_shim.cpp`` + the reference's own
  ``src/cache/cache.h`` compiled where it lies (g++ on the shim directly; the
  reference's build system is not run).  Only attempted when the reference checkout
  is present; the prebuilt file travels otherwise;
* ``oracle/_ref/libhades_ref_cuda.so`` from ``oracle/ref_cuda_shim.cpp`` + the reference's
  own CUDA operators (``src/cuda/uva_fetch.cu``, ``uva_set.cu``, ``split.cu``,
  ``binary_search.cu``), each compiled where it lies with nvcc for sm_100a against the torch
  headers of this environment.  ``split.cu`` needs ``thrust/execution_policy.h``
  force-included under CUDA 12.9 (it names ``thrust::device`` without including it).

The location of the reference checkout is given by the environment variable
``HADES_REFERENCE_ROOT`` or the ``reference`` argument, else a checkout named ``reference``
beside this repository is used; without any of them nothing is compiled from the reference and
prebuilt libraries under ``oracle/_ref/`` are used when present.
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
REF_CUDA_SO = REF_DIR / "libhades_ref_cuda.so"
REF_CUDA_SOURCES = ("uva_fetch.cu", "uva_set.cu", "split.cu", "binary_search.cu")


def reference_root(arg: str | os.PathLike | None = None) -> Path | None:
    """The reference checkout: the argument, else $HADES_REFERENCE_ROOT, else a directory
    named ``reference`` beside this repository, else None."""
    root = arg if arg is not None else os.environ.get("HADES_REFERENCE_ROOT")
    if root:
        return Path(root)
    sibling = HERE.parent.parent / "reference"
    return sibling if (sibling / "src" / "cache" / "cache.h").exists() else None


def _stale(out: Path, *srcs: Path) -> bool:
    return not out.exists() or any(s.exists() and s.stat().st_mtime > out.stat().st_mtime for s in srcs)


def build_oracle(force: bool = False) -> Path:
    src = HERE / "hades_oracle.c"
    if force or _stale(ORACLE_SO, src):
        subprocess.run(["gcc", "-O2", "-std=c11", "-shared", "-fPIC", "-o", str(ORACLE_SO), str(src)],
                       check=True)
    return ORACLE_SO


def build_ref(force: bool = False, reference: str | os.PathLike | None = None) -> Path | None:
    """Compile the reference's CPU index through the shim.  Returns None when the
    reference sources are absent and no prebuilt library exists."""
    REFERENCE_ROOT = reference_root(reference)
    header = REFERENCE_ROOT / "src" / "cache" / "cache.h" if REFERENCE_ROOT else None
    shim = HERE / "ref_shim.cpp"
    if header is None or not header.exists():
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


def build_ref_cuda(force: bool = False, reference: str | os.PathLike | None = None) -> Path | None:
    """Compile the reference's CUDA operators (nvcc on its own .cu files, sm_100a) and link
    them with the shim.  Returns None when the reference sources are absent and no prebuilt
    library exists.  Takes a few minutes (torch headers through nvcc)."""
    import concurrent.futures as cf
    import shutil

    root = reference_root(reference)
    src_dir = root / "src" / "cuda" if root else None
    shim = HERE / "ref_cuda_shim.cpp"
    if src_dir is None or not (src_dir / "ops.h").exists():
        return REF_CUDA_SO if REF_CUDA_SO.exists() else None
    srcs = [src_dir / s for s in REF_CUDA_SOURCES]
    if not force and not _stale(REF_CUDA_SO, shim, *srcs):
        return REF_CUDA_SO
    import torch

    tdir = Path(torch.__file__).parent
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    gxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    obj_dir = REF_DIR / "obj"
    obj_dir.mkdir(parents=True, exist_ok=True)
    inc = ["-I", str(root / "src"), "-I", str(tdir / "include"),
           "-I", str(tdir / "include/torch/csrc/api/include"), "-I", sysconfig.get_paths()["include"]]
    common = [nvcc, "-ccbin", gxx, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17",
              "--extended-lambda", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
              "-include", "thrust/execution_policy.h", *inc]

    def compile_one(src: Path) -> Path:
        obj = obj_dir / (src.stem + ".o")
        if force or _stale(obj, src):
            subprocess.run([*common, "-x", "cu", "-c", str(src), "-o", str(obj)], check=True,
                           capture_output=True, text=True)
        return obj

    with cf.ThreadPoolExecutor(max_workers=5) as ex:
        objs = list(ex.map(compile_one, [*srcs, shim]))
    cmd = [nvcc, "-ccbin", gxx, "-shared", "-o", str(REF_CUDA_SO), *map(str, objs),
           "-L", str(tdir / "lib"), "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda",
           "-Xlinker", f"-rpath={tdir / 'lib'}", "-lcudart"]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    return REF_CUDA_SO


if __name__ == "__main__":
    import sys

    ref = sys.argv[1] if len(sys.argv) > 1 else None
    print(build_oracle())
    print(build_ref(reference=ref))
    print(build_ref_cuda(reference=ref))
