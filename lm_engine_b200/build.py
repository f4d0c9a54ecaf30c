"""In-tree build of the native libraries.

``liblme_cuda.so``  all sm_100a kernels (one nvcc translation unit, C ABI, loaded with ctypes)
``liblme_host.so``  host-side C++ (dataset index builders, alpha-numeric tokenizer)

nvcc cross-compiles without a GPU, so this runs on a CPU-only machine; the shared objects are written next to the
package (``lm_engine_b200/_C``) and are what the Python wrappers in ``lm_engine_b200.ops`` load.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys

_ROOT = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_ROOT, "csrc")
OUT = os.path.join(_ROOT, "_C")

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--use_fast_math",
    "-Xcompiler",
    "-fPIC",
    "-shared",
]
# --use_fast_math would change exp/div accuracy of the fp32 math; the kernels call the fast intrinsics explicitly
NVCC_FLAGS.remove("--use_fast_math")

CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-shared"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _tree_hash(paths: list[str]) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.encode())
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _sources(sub: str, exts: tuple[str, ...]) -> list[str]:
    out = []
    for d, _, files in os.walk(os.path.join(CSRC, sub) if sub else CSRC):
        for f in files:
            if f.endswith(exts):
                out.append(os.path.join(d, f))
    return out


def _needs_build(target: str, stamp: str) -> bool:
    sfile = target + ".sha"
    if not os.path.exists(target) or not os.path.exists(sfile):
        return True
    return open(sfile).read().strip() != stamp


def build_cuda(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OUT, exist_ok=True)
    target = os.path.join(OUT, "liblme_cuda.so")
    # every kernel file plus every header and source directly under csrc/ (lme_api.h, lme_noalloc.h, lme_cuda.cu)
    deps = _sources("kernels", (".cu", ".cuh")) + [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC))
                                                   if f.endswith((".h", ".cu", ".cuh"))]
    stamp = _tree_hash(deps)
    if force or _needs_build(target, stamp):
        cmd = [_nvcc(), *NVCC_FLAGS, "-o", target, os.path.join(CSRC, "lme_cuda.cu")]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + r.stdout + r.stderr)
        if verbose:
            print(r.stderr)
        open(target + ".sha", "w").write(stamp)
    return target


def build_host(force: bool = False) -> str:
    os.makedirs(OUT, exist_ok=True)
    target = os.path.join(OUT, "liblme_host.so")
    deps = _sources("host", (".cpp", ".h"))
    if not deps:
        return target
    stamp = _tree_hash(deps)
    if force or _needs_build(target, stamp):
        cxx = os.environ.get("CXX", "g++")
        cmd = [cxx, *CXX_FLAGS, "-o", target, *[d for d in deps if d.endswith(".cpp")]]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("g++ failed:\n" + r.stdout + r.stderr)
        open(target + ".sha", "w").write(stamp)
    return target


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_cuda(force=force, verbose=verbose)
    build_host(force=force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print("built:", sorted(f for f in os.listdir(OUT) if f.endswith(".so")))
