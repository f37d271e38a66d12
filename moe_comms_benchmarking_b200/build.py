"""Ahead-of-time build of the CUDA library for sm_100a.

The reference has no native code of its own: its kernels are Triton functions compiled at
run time (nvls/torch_symm_triton/*.py), with a per-rank JIT cache to manage
(run.sbatch:62).  Here every kernel is a hand-written ``.cu`` file compiled once, in tree,
into ``lib/libmcb.so`` with plain ``nvcc``; there is no JIT and no cache.

    python -m moe_comms_benchmarking_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import argparse
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_DIR = PKG_DIR / "lib"
OBJ_DIR = LIB_DIR / "obj"
LIB_PATH = LIB_DIR / "libmcb.so"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-Wall", "-Xptxas", "-v"]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build libmcb.so")
    return exe


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _digest() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()


def is_current() -> bool:
    stamp = LIB_DIR / "build.stamp"
    return LIB_PATH.exists() and stamp.exists() and stamp.read_text().strip() == _digest()


def _compile(src: Path, verbose: bool) -> tuple[Path, str]:
    obj = OBJ_DIR / (src.stem + ".o")
    cmd = [_nvcc(), *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    log = res.stdout + res.stderr
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{log}")
    if verbose:
        print(f"[build] {src.name}\n{log}", flush=True)
    return obj, log


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` for sm_100a and link ``lib/libmcb.so``.

    Returns the library path.  A content hash of the sources and flags makes repeated calls
    cheap.  The ptxas resource report of every kernel is kept in ``lib/ptxas.log``.
    """
    if not force and is_current():
        return LIB_PATH
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    # Several ranks of one job may get here at once: one builds, the others wait on the lock and
    # then find the library current.  The library is linked under a temporary name and renamed into
    # place, so a process that loads it never sees a half-written file.
    with open(LIB_DIR / ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and is_current():
                return LIB_PATH
            srcs = sources()
            if not srcs:
                raise RuntimeError(f"no .cu sources under {CSRC}")
            with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
                results = list(pool.map(lambda s: _compile(s, verbose), srcs))
            objs = [str(o) for o, _ in results]
            (LIB_DIR / "ptxas.log").write_text(
                "\n".join(f"=== {s.name} ===\n{log}" for s, (_, log) in zip(srcs, results)))
            tmp = LIB_DIR / f".libmcb.{os.getpid()}.so"
            cmd = [_nvcc(), *ARCH_FLAGS, "-shared", "-o", str(tmp), *objs]
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                raise RuntimeError(f"link failed:\n{res.stdout}{res.stderr}")
            os.replace(tmp, LIB_PATH)
            (LIB_DIR / "build.stamp").write_text(_digest())
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return LIB_PATH


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    args = ap.parse_args(argv)
    path = build(force=args.force, verbose=args.verbose)
    print(f"built {path}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
