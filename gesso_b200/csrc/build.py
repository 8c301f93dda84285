"""Builds the sm_100a kernel library from the ``.cu`` files beside this module.

Every source is compiled by ``nvcc`` for ``sm_100a`` into an object file and the
objects are linked into one shared library, ``_build/libgesso_b200.so``, inside
this folder (so the library travels with the tree).  A fingerprint of the
sources and flags is kept beside it; the library is rebuilt only when that
changes.  Compilation prints a line per file and a heartbeat line while it
waits, because a first call in a fresh checkout compiles everything.

There is no fallback: if ``nvcc`` is missing or a file fails to compile, the
caller gets a :class:`~gesso_b200.errors.GessoError` with the compiler output.
"""
from __future__ import annotations

import concurrent.futures as cf
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from typing import List

from ..errors import ErrorCode, GessoError

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libgesso_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler",
              "-fvisibility=hidden", "--expt-relaxed-constexpr"]
# more flags for every file (macro definitions for tuning, say), part of the fingerprint
NVCC_FLAGS += os.environ.get("GESSO_NVCC_FLAGS", "").split()


_SLOW_FIRST = ("attention_generic", "gemm_skinny_")


def _say(msg: str) -> None:
    print(f"[gesso_b200 build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("GESSO_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 shutil.which("nvcc")):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise GessoError(ErrorCode.COMPILE, "nvcc not found (set CUDA_HOME or GESSO_NVCC); "
                     "the kernel library cannot be built and there is no fallback")


def sources() -> List[str]:
    return sorted(f for f in os.listdir(_HERE) if f.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(_HERE) if f.endswith((".cuh", ".h")))


def _fingerprint(nvcc: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    try:
        h.update(subprocess.run([nvcc, "--version"], capture_output=True, text=True).stdout.encode())
    except OSError:
        pass
    for name in sources() + _headers():
        h.update(name.encode())
        with open(os.path.join(_HERE, name), "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def build_dir() -> str:
    """In-tree ``_build`` folder; a per-user temporary folder if the tree is read-only."""
    d = os.environ.get("GESSO_BUILD_DIR") or os.path.join(_HERE, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.unlink(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"gesso_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _compile_one(nvcc: str, src: str, obj: str, extra: List[str]) -> str:
    cmd = [nvcc] + ARCH_FLAGS + NVCC_FLAGS + extra + ["-I", _HERE, "-c", os.path.join(_HERE, src), "-o", obj]
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0:
        raise GessoError(ErrorCode.COMPILE, f"nvcc failed on {src}:\n{p.stdout}\n{p.stderr}")
    return p.stderr


def build(verbose: bool = True, ptxas_info: bool = False) -> str:
    """Compile what is stale and return the path of the shared library."""
    nvcc = find_nvcc()
    out_dir = build_dir()
    lib = os.path.join(out_dir, LIB_NAME)
    stamp = os.path.join(out_dir, "fingerprint.txt")
    want = _fingerprint(nvcc)
    lock_path = os.path.join(out_dir, ".lock")
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if os.path.isfile(lib) and os.path.isfile(stamp) and open(stamp).read().strip() == want \
                    and not ptxas_info:
                return lib
            srcs = sources()
            if verbose:
                _say(f"compiling {len(srcs)} CUDA files for sm_100a into {out_dir} (first call only)")
            t0 = time.time()
            extra = ["-Xptxas", "-v"] if ptxas_info else []
            objs = [os.path.join(out_dir, s[:-3] + ".o") for s in srcs]
            logs = {}
            with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs), os.cpu_count() or 2)) as pool:
                # the files with the most template instantiations take longest and start first
                order = sorted(zip(srcs, objs), key=lambda so: (not so[0].startswith(_SLOW_FIRST), so[0]))
                futs = {pool.submit(_compile_one, nvcc, s, o, extra): s for s, o in order}
                pending = set(futs)
                while pending:
                    done, pending = cf.wait(pending, timeout=10.0, return_when=cf.FIRST_COMPLETED)
                    for f in done:
                        logs[futs[f]] = f.result()
                        if verbose:
                            _say(f"  {futs[f]} done ({time.time() - t0:.0f}s)")
                    if pending and not done and verbose:
                        _say(f"  still compiling {len(pending)} file(s) ... {time.time() - t0:.0f}s")
            tmp_lib = lib + f".tmp{os.getpid()}"
            p = subprocess.run([nvcc] + ARCH_FLAGS + ["-shared", "-o", tmp_lib] + objs,
                               capture_output=True, text=True)
            if p.returncode != 0:
                raise GessoError(ErrorCode.COMPILE, f"link failed:\n{p.stdout}\n{p.stderr}")
            os.replace(tmp_lib, lib)
            with open(stamp, "w") as f:
                f.write(want)
            if verbose:
                _say(f"built {lib} in {time.time() - t0:.0f}s")
            if ptxas_info:
                for s in srcs:
                    sys.stderr.write(f"==== {s}\n{logs[s]}\n")
            return lib
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


if __name__ == "__main__":
    build(verbose=True, ptxas_info="--ptxas" in sys.argv)
