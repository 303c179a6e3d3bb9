"""In-tree build of the native libraries.

* `ds41rt_b200/_lib/libds41_kernels.so` - every CUDA kernel (csrc/kernels/*.cu), compiled by nvcc
  for sm_100a only (`-gencode arch=compute_100a,code=sm_100a`).
* `ds41rt_b200/_lib/libds41_core.so`    - the host runtime (csrc/core/*.cc), compiled by g++.

Both export a plain C ABI consumed through ctypes, so no torch headers are involved and a full
rebuild takes well under a minute.  Objects are cached by source hash.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
LIBDIR = Path(__file__).resolve().parent / "_lib"
OBJDIR = LIBDIR / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-I", str(CSRC / "include"),
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-pthread", "-I", str(CSRC / "include")]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _digest(path: Path, extra: str) -> str:
    h = hashlib.sha256()
    h.update(path.read_bytes())
    h.update(extra.encode())
    for hdr in sorted((CSRC / "include").glob("*")):
        h.update(hdr.read_bytes())
    return h.hexdigest()[:16]


def _compile(cmd, src: Path, obj: Path, verbose: bool):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"compile failed: {src}\n{' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    if verbose and r.stderr.strip():
        sys.stderr.write(r.stderr)
    return obj


def _build_lib(name: str, sources, compiler_cmd, link_cmd, verbose: bool) -> Path:
    OBJDIR.mkdir(parents=True, exist_ok=True)
    jobs = []
    objs = []
    for src in sources:
        tag = _digest(src, " ".join(compiler_cmd))
        obj = OBJDIR / f"{src.stem}.{tag}.o"
        objs.append(obj)
        if not obj.exists():
            for old in OBJDIR.glob(f"{src.stem}.*.o"):
                old.unlink()
            jobs.append((compiler_cmd + ["-c", str(src), "-o", str(obj)], src, obj))
    out = LIBDIR / name
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(lambda j: _compile(j[0], j[1], j[2], verbose), jobs))
    if jobs or not out.exists():
        cmd = link_cmd + ["-o", str(out)] + [str(o) for o in objs]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed: {name}\n{r.stdout}\n{r.stderr}")
    return out


def build_kernels(verbose: bool = False) -> Path:
    nvcc = _nvcc()
    sources = sorted((CSRC / "kernels").glob("*.cu"))
    flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if verbose else [])
    return _build_lib("libds41_kernels.so", sources, [nvcc] + flags,
                      [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"], verbose)


def build_core(verbose: bool = False) -> Path:
    cxx = shutil.which("g++") or "g++"
    sources = sorted((CSRC / "core").glob("*.cc"))
    return _build_lib("libds41_core.so", sources, [cxx] + CXX_FLAGS, [cxx, "-shared", "-pthread"], verbose)


def build_selftest() -> Path:
    """csrc/tests/core_selftest.cc -> _lib/ds41_core_selftest, linked against the host runtime library beside it."""
    cxx = shutil.which("g++") or "g++"
    core = build_core()
    out = LIBDIR / "ds41_core_selftest"
    src = CSRC / "tests" / "core_selftest.cc"
    if not out.exists() or out.stat().st_mtime < max(src.stat().st_mtime, core.stat().st_mtime):
        subprocess.run([cxx, "-std=c++17", "-O1", "-Wall", str(src), "-L", str(LIBDIR), "-lds41_core",
                        "-Wl,-rpath,$ORIGIN", "-o", str(out)], check=True)
    return out


def build_all(verbose: bool = False):
    return build_core(verbose), build_kernels(verbose)


if __name__ == "__main__":
    for p in build_all(verbose="-v" in sys.argv):
        print(p)
