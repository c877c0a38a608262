"""Builds the native parts of hivemind_b200 in-tree.

Two artefacts are produced next to their sources:

* ``hivemind_b200/ops/libhm_kernels.so`` — every sm_100a CUDA kernel of the package behind a C ABI
  (``extern "C"`` launchers that take raw device pointers and a stream). It is loaded with ``ctypes``.
* ``hivemind_b200/native/hmp2pd`` — the C++ transport daemon that plays the part of the reference's
  external Go ``p2pd`` (hivemind/p2p/p2p_daemon.py:205-262 spawns it).

``python -m hivemind_b200.ops._build`` rebuilds both; ``build_kernels()`` / ``build_daemon()`` rebuild only when a
source is newer than the artefact.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path
from typing import List, Optional

OPS_DIR = Path(__file__).resolve().parent
CSRC_DIR = OPS_DIR / "csrc"
KERNELS_SO = OPS_DIR / "libhm_kernels.so"
NATIVE_DIR = OPS_DIR.parent / "native"
DAEMON_BIN = NATIVE_DIR / "hmp2pd"

NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
PRECISE_SOURCES = ("multi_tensor", "codec", "butterfly_round", "powersgd")


def _find_nvcc() -> Optional[str]:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    return None


def _stale(target: Path, sources: List[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(s.stat().st_mtime > t for s in sources)


def _run(cmd: List[str], verbose: bool) -> None:
    if verbose:
        print(" ".join(cmd), flush=True)
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose and (proc.stdout or proc.stderr):
        print(proc.stdout, proc.stderr, sep="\n", flush=True)
    if proc.returncode != 0:
        raise RuntimeError(f"build failed ({proc.returncode}): {' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")


def build_kernels(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` for sm_100a into one shared library (objects are compiled in parallel)."""
    sources = sorted(CSRC_DIR.glob("*.cu"))
    headers = sorted(CSRC_DIR.glob("*.cuh")) + sorted(CSRC_DIR.glob("*.h"))
    if not force and not _stale(KERNELS_SO, sources + headers):
        return KERNELS_SO
    nvcc = _find_nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found; cannot build libhm_kernels.so")
    build_dir = OPS_DIR / "build"
    build_dir.mkdir(exist_ok=True)
    common = [nvcc, *NVCC_ARCH, "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-I", str(CSRC_DIR)]
    if ptxas_info:
        common += ["-Xptxas", "-v"]
    procs = []
    objects = []
    for src in sources:
        obj = build_dir / (src.stem + ".o")
        objects.append(obj)
        if not force and not _stale(obj, [src] + headers):
            continue
        # optimizer updates and codecs keep IEEE division, square roots and denormals (they are compared with, and
        # interoperate with, plain PyTorch math); the tensor-core and activation kernels take the fast intrinsics
        fast_math = [] if src.stem in PRECISE_SOURCES else ["--use_fast_math"]
        cmd = common + fast_math + ["-c", str(src), "-o", str(obj)]
        if verbose:
            print(" ".join(cmd), flush=True)
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for cmd, proc in procs:
        out, _ = proc.communicate()
        if verbose or ptxas_info:
            print(out, flush=True)
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed: {' '.join(cmd)}\n{out}")
    _run([nvcc, *NVCC_ARCH, "-shared", "-o", str(KERNELS_SO), *map(str, objects), "-lcuda"], verbose)
    return KERNELS_SO


def build_daemon(force: bool = False, verbose: bool = False) -> Path:
    """Compile the C++ transport daemon."""
    cxx = shutil.which("g++") or "g++"
    daemon_src = sorted(NATIVE_DIR.glob("hmp2pd*.cpp"))
    headers = sorted(NATIVE_DIR.glob("*.h"))
    if daemon_src and (force or _stale(DAEMON_BIN, daemon_src + headers)):
        _run([cxx, "-O2", "-std=c++17", "-pthread", "-o", str(DAEMON_BIN), *map(str, daemon_src)], verbose)
    return DAEMON_BIN


def build_all(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> None:
    build_kernels(force=force, verbose=verbose, ptxas_info=ptxas_info)
    build_daemon(force=force, verbose=verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv)
