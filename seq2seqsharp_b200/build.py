"""Builds libtsb200.so (sm_100a only) from seq2seqsharp_b200/csrc with nvcc, in-tree.

Usage: python -m seq2seqsharp_b200.build [--force] [--verbose] [--checked]
"""
import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libtsb200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr",
] + os.environ.get("TSB200_NVCC_FLAGS", "").split()   # e.g. -DTSB200_TRACE: kernels stamp %globaltimer for development


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _stamp():
    h = hashlib.sha256()
    for root in (CSRC, os.path.join(HERE, "..", "include")):
        for f in sorted(os.listdir(root)):
            if f.endswith((".cu", ".cuh", ".h")):
                with open(os.path.join(root, f), "rb") as fh:
                    h.update(f.encode())
                    h.update(fh.read())
    h.update(" ".join(FLAGS).encode())
    return h.hexdigest()


VARIANTS = {
    "": [],
    # device-side index / capacity checks that record a code and skip the access (see kernels.cuh), for bring-up and bug hunts
    "checked": ["-DTSB200_CHECKED"],
}


def lib_path(variant=""):
    return LIB if not variant else os.path.join(HERE, "libtsb200_%s.so" % variant)


def build(force=False, verbose=False, variant=""):
    """variant "": the product library; "checked": libtsb200_checked.so with -DTSB200_CHECKED (objects in build/checked)."""
    vflags = VARIANTS[variant]
    OBJ = os.path.join(HERE, "build", variant) if variant else globals()["OBJ"]
    LIB = lib_path(variant)
    os.makedirs(OBJ, exist_ok=True)
    stamp_file = os.path.join(OBJ, "stamp")
    stamp = _stamp() + " ".join(vflags)
    if not force and os.path.exists(LIB) and os.path.exists(stamp_file) and open(stamp_file).read() == stamp:
        return LIB
    extra = (["-Xptxas", "-v"] if verbose else []) + vflags

    def compile_one(src):
        obj = os.path.join(OBJ, src[:-3] + ".o")
        cmd = [NVCC, *FLAGS, *extra, "-c", os.path.join(CSRC, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, r.stdout, r.stderr))
        if verbose:
            sys.stderr.write(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(compile_one, _sources()))
    cmd = [NVCC, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static", "-ldl"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n%s\n%s" % (r.stdout, r.stderr))
    with open(stamp_file, "w") as fh:
        fh.write(stamp)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, variant="checked" if "--checked" in sys.argv else ""))
