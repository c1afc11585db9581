"""In-tree build of the native library: ``python -m vllm_ascend_b200.build``.

Every ``csrc/*.cu`` / ``csrc/*.cpp`` is compiled for sm_100a only and linked
into ``vllm_ascend_b200/_C.so`` (plain C ABI, loaded with ctypes by
``vllm_ascend_b200._native``).  Objects are cached by source hash so a rebuild
only recompiles what changed.  Build knobs follow the reference's env-driven
setup (setup.py:74-132): ``MAX_JOBS``, ``CMAKE_BUILD_TYPE``.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(HERE, "csrc", "build")
LIB_PATH = os.path.join(HERE, "_C.so")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _common_flags() -> list[str]:
    debug = os.environ.get("CMAKE_BUILD_TYPE", "Release").lower() == "debug"
    flags = ["-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
             "--expt-relaxed-constexpr", "-I", CSRC]
    flags += ["-O0", "-g"] if debug else ["-O3"]      # index checks in the kernels are always on
    if os.environ.get("B200_PTXAS_VERBOSE"):
        flags += ["-Xptxas", "-v"]
    return flags


def _sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC)
                  if f.endswith((".cu", ".cpp")))


def _headers_digest() -> str:
    h = hashlib.sha256()
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cuh", ".h", ".hpp")):
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(fh.read())
    h.update(" ".join(_common_flags()).encode())
    return h.hexdigest()


def _compile_one(src: str, hdr_digest: str, verbose: bool) -> tuple[str, bool]:
    with open(src, "rb") as fh:
        digest = hashlib.sha256(fh.read() + hdr_digest.encode()).hexdigest()[:16]
    base = os.path.splitext(os.path.basename(src))[0]
    obj = os.path.join(OBJ_DIR, f"{base}.{digest}.o")
    if os.path.exists(obj):
        return obj, False
    for old in os.listdir(OBJ_DIR):
        if old.startswith(base + ".") and old.endswith(".o"):
            os.remove(os.path.join(OBJ_DIR, old))
    cmd = [NVCC, *ARCH_FLAGS, *_common_flags(), "-x", "cu", "-c", src, "-o", obj]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
    if res.stderr.strip() and (verbose or os.environ.get("B200_PTXAS_VERBOSE")):
        print(res.stderr, file=sys.stderr)
    return obj, True


def build(verbose: bool = False, force: bool = False) -> str:
    """Compile and link the native library; returns its path."""
    os.makedirs(OBJ_DIR, exist_ok=True)
    if force:
        for f in os.listdir(OBJ_DIR):
            os.remove(os.path.join(OBJ_DIR, f))
    hdr = _headers_digest()
    srcs = _sources()
    jobs = int(os.environ.get("MAX_JOBS", os.cpu_count() or 4))
    with ThreadPoolExecutor(max_workers=jobs) as ex:
        results = list(ex.map(lambda s: _compile_one(s, hdr, verbose), srcs))
    objs = [o for o, _ in results]
    changed = any(c for _, c in results)
    if changed or not os.path.exists(LIB_PATH):
        cmd = [NVCC, *ARCH_FLAGS, "-shared", "-o", LIB_PATH + ".tmp", *objs,
               "-cudart", "static", "-Xlinker", "--no-undefined", "-lpthread", "-ldl", "-lrt"]
        if verbose:
            print(" ".join(cmd), flush=True)
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
        os.replace(LIB_PATH + ".tmp", LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, force="--force" in sys.argv)
    print(path)
