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
# the same flags without the checkout's own path, for identities that must agree between two checkouts of one tree
NVCC_FLAGS_PORTABLE = NVCC_FLAGS[:-1] + ["csrc/include"]
CXX_FLAGS_PORTABLE = CXX_FLAGS[:-1] + ["csrc/include"]


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
        obj = OBJDIR / f"{src.name}.{tag}.o"                 # full file name: engram.cu and engram.cc are two sources
        objs.append(obj)
        if not obj.exists():
            for old in OBJDIR.glob(f"{src.name}.*.o"):
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


def _kernel_recipe(verbose: bool = False):
    nvcc = _nvcc()
    flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if verbose else [])
    return sorted((CSRC / "kernels").glob("*.cu")), [nvcc] + flags


def _core_recipe():
    cxx = shutil.which("g++") or "g++"
    return sorted((CSRC / "core").glob("*.cc")), [cxx] + CXX_FLAGS


def build_kernels(verbose: bool = False) -> Path:
    sources, cmd = _kernel_recipe(verbose)
    return _build_lib("libds41_kernels.so", sources, cmd,
                      [cmd[0], "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"], verbose)


def build_core(verbose: bool = False) -> Path:
    sources, cmd = _core_recipe()
    return _build_lib("libds41_core.so", sources, cmd, [cmd[0], "-shared", "-pthread"], verbose)


def library_status() -> dict:
    """Whether each built library matches the sources beside it, without compiling anything: a library is `current`
    when it exists, an object named by the digest of (source, headers, compile command) exists for every source, and
    the library is not older than any of them.  `stale` lists the sources whose object is missing (edited since the
    build, or built with other flags or another compiler)."""
    out = {}
    for name, recipe in (("libds41_kernels.so", _kernel_recipe), ("libds41_core.so", _core_recipe)):
        lib = LIBDIR / name
        try:
            sources, cmd = recipe()
        except RuntimeError as e:                            # no compiler here: the digests cannot be formed
            out[name] = {"exists": lib.exists(), "current": None, "reason": str(e)}
            continue
        objs = {src.name: OBJDIR / f"{src.name}.{_digest(src, ' '.join(cmd))}.o" for src in sources}
        stale = sorted(n for n, o in objs.items() if not o.exists())
        newest = max((o.stat().st_mtime for o in objs.values() if o.exists()), default=0.0)
        current = lib.exists() and not stale and lib.stat().st_mtime >= newest
        out[name] = {"exists": lib.exists(), "current": current, "sources": len(sources), "stale": stale}
    return out


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
