"""Build the reference's own CUDA kernels, unmodified, into baseline/_ref/libds41rt_ref_kernels.so.

    python baseline/build_ref.py --source <reference tree>

The reference's native library is plain CMake + nvcc (native/CMakeLists.txt:10-60, 251-289; every ahead-of-time option
stays at its OFF default, the grammar adapter is switched off because its pinned sources are not in the tree).  The
configure step and every `cuda/kernels/*.cu` object build for compute capability 10.0; the one host source
(native/src/ds41rt_native.cc:1573-1578) does not compile against CUDA 12.9, so the kernel objects are linked on their
own with `ref_shim.c`, which supplies the single host symbol they import.  The result exports the reference's stock C
entry points (native/include/ds41rt_v41_*.h); `ds41rt_b200.utils.reference_arm` drives them through ctypes.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
KERNELS = ["v41_sparse_attention", "v41_index_topk", "v41_router", "v41_hc", "v41_sampling_gpu", "v41_index_scores",
           "v41_candidate_blocks", "v41_attention_ops", "v41_kv", "v41_compressor", "v41_dspark", "v41_dspark_attention",
           "v41_dspark_cache", "v41_route_reduce", "v41_expert_pack"]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--source", default=os.environ.get("DS41_REFERENCE_TREE", ""), help="root of the reference tree")
    ap.add_argument("--arch", default="100")
    ap.add_argument("--keep", action="store_true", help="keep the build directory")
    args = ap.parse_args(argv)
    native = os.path.join(args.source, "native")
    if not os.path.isfile(os.path.join(native, "CMakeLists.txt")):
        print("no native/CMakeLists.txt under --source", file=sys.stderr)
        return 2
    build = tempfile.mkdtemp(prefix="ds41_ref_build_")
    try:
        subprocess.run(["cmake", "-S", native, "-B", build, "-G", "Ninja", "-DDS41RT_ENABLE_CUDA=ON",
                        "-DDS41RT_ENABLE_XGRAMMAR=OFF", f"-DDS41RT_CUDA_ARCHITECTURES={args.arch}"], check=True)
        objs = [f"CMakeFiles/ds41rt_native.dir/cuda/kernels/{k}.cu.o" for k in KERNELS]
        subprocess.run(["ninja", "-C", build] + objs, check=True)
        os.makedirs(OUT, exist_ok=True)
        lib = os.path.join(OUT, "libds41rt_ref_kernels.so")
        cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
        subprocess.run(["g++", "-shared", "-fPIC", "-o", lib, "-x", "c", os.path.join(HERE, "ref_shim.c"), "-x", "none"]
                       + [os.path.join(build, o) for o in objs]
                       + [f"-L{cuda}/lib64", "-lcudart", "-lcublas", "-ldl", "-lpthread", "-Wl,--no-undefined"], check=True)
        print(lib)
        return 0
    finally:
        if not args.keep:
            shutil.rmtree(build, ignore_errors=True)


if __name__ == "__main__":
    raise SystemExit(main())
