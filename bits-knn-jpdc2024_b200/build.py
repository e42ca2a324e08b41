"""Builds libbitsknn.so (the C-ABI library) with nvcc for sm_100a, in-tree.

    python bits-knn-jpdc2024_b200/build.py [--force] [--verbose]

The library lands in bits-knn-jpdc2024_b200/lib/ and is what the tests, the benchmark, the
C++ host layer and any foreign-language binding load.  Objects are rebuilt only when a
source or header is newer.
"""
import argparse
import os
import pathlib
import shutil
import subprocess
import sys

PKG = pathlib.Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "lib"
OBJ_DIR = LIB_DIR / "obj"
LIB = LIB_DIR / "libbitsknn.so"

SOURCES = ["abi.cu", "select.cu", "ablation.cu", "merge.cu", "sharded.cu", "l2.cu", "l2_tc.cu", "fused.cu", "fused_tiled.cu", "fused_tc.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall", "--expt-relaxed-constexpr",
    "-I", str(ROOT / "include"), "-I", str(CSRC),
]


def nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not pathlib.Path(exe).exists():
        raise RuntimeError("nvcc not found: the CUDA library cannot be built")
    return exe


def host_compiler_flags():
    # the image exports CXX=/opt/gcc/bin/g++ (a wrapper); the system g++ is the safe host compiler
    sys_gxx = "/usr/bin/g++"
    return ["-ccbin", sys_gxx] if pathlib.Path(sys_gxx).exists() else []


def newest_header_mtime():
    headers = list(CSRC.glob("*.cuh")) + list((ROOT / "include").glob("*.h"))
    return max(h.stat().st_mtime for h in headers)


def build(force=False, verbose=False):
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    hdr = newest_header_mtime()
    objects = []
    procs = []
    for name in SOURCES:
        src = CSRC / name
        if not src.exists():
            continue
        obj = OBJ_DIR / (src.stem + ".o")
        objects.append(obj)
        if not force and obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, hdr):
            continue
        cmd = [nvcc(), *NVCC_FLAGS, *host_compiler_flags(), "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
            print(" ".join(cmd), flush=True)
        procs.append((name, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for name, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode != 0:
            failed = True
            print(f"--- nvcc failed on {name}\n{out}", file=sys.stderr)
        elif verbose and out:
            print(f"--- {name}\n{out}")
    if failed:
        raise RuntimeError("nvcc failed")
    if procs or not LIB.exists():
        cmd = [nvcc(), "-shared", *host_compiler_flags(), "-o", str(LIB), *map(str, objects), "-lcudart", "-ldl"]
        subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    args = ap.parse_args()
    print(build(force=args.force, verbose=args.verbose))
