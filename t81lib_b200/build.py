"""Build ``libt81_b200.so`` in-tree with nvcc for sm_100a.

    python -m t81lib_b200.build [--force] [--verbose]

The shared library lands in ``t81lib_b200/lib/`` next to the package so that it
travels with the source tree.  Only sm_100a code is generated.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys

_PKG = os.path.dirname(os.path.abspath(__file__))
_CSRC = os.path.join(_PKG, "csrc")
_LIBDIR = os.path.join(_PKG, "lib")
LIB_PATH = os.path.join(_LIBDIR, "libt81_b200.so")

SOURCES = ["capi.cu", "quantize_pack.cu", "gemm_limb.cu", "gemv_trit.cu", "gemv_trit_lut.cu", "gemm_trit_simt.cu", "gemm_trit_tc.cu", "elementwise.cu", "tq_codec.cu", "qat.cu", "pack_t2.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--fmad=true", "-prec-div=true", "-prec-sqrt=true",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def _flags() -> list:
    """The nvcc flags, plus whatever T81B200_NVCC_EXTRA adds (instrumented builds, e.g. -DT81B200_GEMV_TRACE)."""
    return NVCC_FLAGS + os.environ.get("T81B200_NVCC_EXTRA", "").split()


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; libt81_b200.so cannot be built")


_STAMP = os.path.join(_LIBDIR, "BUILD_HASH")


def source_hash() -> str:
    """Hash of every source the library is built from (file times do not survive copies)."""
    import hashlib
    h = hashlib.sha256()
    deps = sorted(os.path.join(_CSRC, f) for f in os.listdir(_CSRC) if os.path.isfile(os.path.join(_CSRC, f)))
    deps.append(os.path.join(os.path.dirname(_PKG), "include", "t81_b200.h"))
    for d in deps:
        h.update(os.path.basename(d).encode())
        with open(d, "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(_flags()).encode())
    return h.hexdigest()


def _stale() -> bool:
    if not os.path.exists(LIB_PATH) or not os.path.exists(_STAMP):
        return True
    with open(_STAMP) as fh:
        return fh.read().strip() != source_hash()


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every CUDA source into one shared library; returns its path."""
    if not force and not _stale():
        return LIB_PATH
    os.makedirs(_LIBDIR, exist_ok=True)
    # one builder at a time: the ranks of a multi-GPU job import the package at the same moment
    import fcntl
    with open(os.path.join(_LIBDIR, ".build.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not force and not _stale():
            return LIB_PATH
        return _build_locked(verbose)


def _build_locked(verbose: bool) -> str:
    objdir = os.path.join(_LIBDIR, "obj")
    os.makedirs(objdir, exist_ok=True)
    nvcc = _nvcc()
    procs = []
    for src in SOURCES:
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        cmd = [nvcc, *_flags(), "-c", os.path.join(_CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    objs = []
    for src, obj, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{out}")
        if verbose:
            print(out)
        objs.append(obj)
    link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB_PATH, *objs, "-lcudart"]
    res = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}")
    with open(_STAMP, "w") as fh:
        fh.write(source_hash())
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
