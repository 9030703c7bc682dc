"""Build libkvip_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

Run as ``python -m kvip_b200.build``; `__graft_entry__.build()` calls `build_library()`.
"""
import hashlib
import os
import shutil
import subprocess
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
CSRC = PACKAGE / "csrc"
LIBRARY = PACKAGE / "libkvip_b200.so"
SOURCES = ("api.cu", "li_score.cu", "topk.cu", "topk_pivot.cu", "topk_split.cu", "cold_predicate.cu", "resolve.cu", "exchange.cu", "cache_ops.cu", "lidu.cu", "speculate.cu", "peer_exchange.cu")
NVCC_FLAGS = (
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--use_fast_math=false",
)


def _nvcc():
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: the CUDA toolkit is required to build libkvip_b200.so")
    return nvcc


def _digest(paths):
    h = hashlib.sha256()
    for path in sorted(paths):
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build_library(force=False, verbose=False):
    """Compile every .cu under csrc/ and link the shared library. Returns its path."""
    sources = [CSRC / name for name in SOURCES if (CSRC / name).exists()]
    headers = list(CSRC.glob("*.cuh")) + [PACKAGE.parent / "include" / "kvip_b200.h"]
    stamp = PACKAGE / "csrc" / ".build_stamp"
    digest = _digest(sources + headers)
    if not force and LIBRARY.exists() and stamp.exists() and stamp.read_text() == digest:
        return LIBRARY
    nvcc = _nvcc()
    build_dir = PACKAGE / "csrc" / "build"
    build_dir.mkdir(exist_ok=True)
    objects = []
    procs = []
    for source in sources:
        obj = build_dir / (source.stem + ".o")
        cmd = [nvcc, *[f for f in NVCC_FLAGS if f != "--use_fast_math=false"], "-c", str(source), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((source, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objects.append(str(obj))
    for source, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode:
            raise RuntimeError(f"nvcc failed on {source.name}:\n{out}")
        if verbose and out:
            print(out)
    link = [nvcc, "-shared", "-o", str(LIBRARY), *objects, "-lcudart"]
    result = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if result.returncode:
        raise RuntimeError(f"link failed:\n{result.stdout}")
    stamp.write_text(digest)
    return LIBRARY


if __name__ == "__main__":
    import sys

    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
