"""Builds libmgr_b200.so in-tree with nvcc for sm_100a.

The library is the only compiled artefact of the package: a C-ABI shared object (include/mgr_b200.h)
loaded by ctypes. It replaces the reference's `CUDAExtension('rmsnorm_cuda_ops', ...)` build
(setup.py:23-42): one architecture (sm_100a), no Triton, no multi-backend dispatch, no CPU fallback,
and no `--use_fast_math` (the kernels are memory-bound; IEEE sqrt/divide cost nothing).

`build_binding()` then compiles pytorch_binding/binding.cpp into the torch extension
mgrrmsnorm_b200/pybind/rmsnorm_cuda_ops*.so by running the repository's setup.py (torch's BuildExtension,
ninja), the route `pip install -e .` takes as well.

Usage:  python -m mgrrmsnorm_b200.build [--force] [--verbose] [--binding]
"""
from __future__ import annotations

import argparse
import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
INCLUDE = PKG_DIR.parent / "include"
LIB_DIR = PKG_DIR / "lib"
OBJ_DIR = LIB_DIR / "obj"
LIB_PATH = LIB_DIR / "libmgr_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found: libmgr_b200.so can only be built with the CUDA toolkit (sm_100a)")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _fingerprint(src: Path) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    h.update(src.read_bytes())
    for hdr in sorted(list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))):
        h.update(hdr.read_bytes())
    return h.hexdigest()


def _compile_one(nvcc: str, src: Path, force: bool, verbose: bool) -> tuple[Path, str]:
    obj = OBJ_DIR / (src.stem + ".o")
    stamp = OBJ_DIR / (src.stem + ".sha")
    fp = _fingerprint(src)
    if not force and obj.exists() and stamp.exists() and stamp.read_text() == fp:
        return obj, ""
    cmd = [nvcc, *NVCC_FLAGS, "-I", str(INCLUDE), "-c", str(src), "-o", str(obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stdout}\n{proc.stderr}")
    stamp.write_text(fp)
    (OBJ_DIR / (src.stem + ".ptxas.log")).write_text(proc.stderr)
    return obj, proc.stderr if verbose else ""


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compiles every csrc/*.cu for sm_100a and links lib/libmgr_b200.so. Returns the library path."""
    nvcc = _nvcc()
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    srcs = sources()
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        results = list(pool.map(lambda s: _compile_one(nvcc, s, force, verbose), srcs))
    objs = [r[0] for r in results]
    for _, log in results:
        if log:
            print(log)
    newest = max(o.stat().st_mtime for o in objs)
    if force or not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < newest:
        cmd = [nvcc, "-shared", "-o", str(LIB_PATH), *map(str, objs)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    return LIB_PATH


ROOT = PKG_DIR.parent
BINDING_SRC = ROOT / "pytorch_binding" / "binding.cpp"
BINDING_DIR = PKG_DIR / "pybind"


def binding_path() -> Path | None:
    hits = sorted(BINDING_DIR.glob("rmsnorm_cuda_ops*.so"))
    return hits[0] if hits else None


def build_binding(force: bool = False) -> Path:
    """Compiles the torch extension (after the kernel library it links against). Returns its path."""
    build()
    h = hashlib.sha256()
    for f in (BINDING_SRC, ROOT / "setup.py", *sorted(INCLUDE.glob("*.h"))):
        h.update(f.read_bytes())
    fp = h.hexdigest()
    stamp = BINDING_DIR / "rmsnorm_cuda_ops.sha"
    have = binding_path()
    if not force and have is not None and stamp.exists() and stamp.read_text() == fp:
        return have
    proc = subprocess.run([sys.executable, "setup.py", "-q", "build_ext", "--inplace"], cwd=str(ROOT), capture_output=True, text=True)
    if proc.returncode != 0 or binding_path() is None:
        raise RuntimeError(f"building pytorch_binding/binding.cpp failed:\n{proc.stdout[-4000:]}\n{proc.stderr[-4000:]}")
    stamp.write_text(fp)
    return binding_path()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true", help="recompile even if sources are unchanged")
    ap.add_argument("--verbose", action="store_true", help="print ptxas register/shared-memory reports")
    ap.add_argument("--binding", action="store_true", help="also build the torch extension from pytorch_binding/binding.cpp")
    args = ap.parse_args(argv)
    print(build(force=args.force, verbose=args.verbose))
    if args.binding:
        print(build_binding(force=args.force))
    return 0


if __name__ == "__main__":
    sys.exit(main())
