"""In-tree build of the native library (nvcc, sm_100a only).

``python -m moonep_b200._build`` compiles every source under ``csrc/`` into
``moonep_b200/_lib/libmoonep_b200.so``.  Objects are cached by source mtime; files are
compiled in parallel.  nvcc cross-compiles without a GPU.

Counterpart of the reference's ``setup.py`` (setup.py:24-77 there: one ``CUDAExtension`` of
host-only code with torch's default architectures); here every kernel is device code built for
``sm_100a`` explicitly and the result stays in the source tree.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
LIBDIR = Path(__file__).resolve().parent / "_lib"
OBJDIR = ROOT / "build" / "obj"
LIB = LIBDIR / "libmoonep_b200.so"

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Wno-deprecated-gpu-targets",
          "--expt-relaxed-constexpr", "-diag-suppress", "550"]


def sources():
    return sorted(list((CSRC / "host").glob("*.cc")) + list((CSRC / "device").glob("*.cu")))


def headers():
    return (list(CSRC.glob("*.h")) + list((CSRC / "host").glob("*.h")) + list((CSRC / "device").glob("*.cuh"))
            + list((CSRC / "device").glob("*.h")))


def nvcc_path() -> str | None:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else None


def _compile(src: Path, obj: Path, verbose: bool):
    cmd = [nvcc_path(), *ARCH, *COMMON, "-c", str(src), "-o", str(obj)]
    if os.environ.get("MOONEP_POLL_SLEEP_NS"):
        cmd.insert(1, "-DMEP_POLL_SLEEP_NS=" + str(int(os.environ["MOONEP_POLL_SLEEP_NS"])))
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    return r.stderr


def is_stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    return any(p.stat().st_mtime > t for p in sources() + headers())


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile what is out of date and link.  Safe to call from several processes at once (one
    rank per GPU importing the package): the work is serialised with a file lock, the library is
    linked under a temporary name and renamed into place, and a process that finds the library
    fresh once it holds the lock does nothing."""
    if nvcc_path() is None:
        raise RuntimeError("nvcc not found; cannot build libmoonep_b200.so")
    LIBDIR.mkdir(parents=True, exist_ok=True)
    OBJDIR.mkdir(parents=True, exist_ok=True)
    import fcntl
    with open(LIBDIR / ".build.lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not force and not is_stale():
            return LIB
        return _build_locked(force, verbose)


def _build_locked(force: bool, verbose: bool) -> Path:
    hdr_t = max(p.stat().st_mtime for p in headers())
    jobs, objs = [], []
    for src in sources():
        obj = OBJDIR / (src.stem + ".o")
        objs.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_t):
            jobs.append((src, obj))
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for out in ex.map(lambda j: _compile(j[0], j[1], verbose), jobs):
            if verbose and out:
                print(out, file=sys.stderr)
    if jobs or not LIB.exists() or is_stale():
        tmp = LIB.with_suffix(".so.tmp")
        cmd = [nvcc_path(), *ARCH, "-shared", "--cudart", "shared", "-o", str(tmp), *map(str, objs)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(p)
