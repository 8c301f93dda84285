"""Builds and loads the host runtime library (``host/*.cpp``: the cache manager's bookkeeping and the
packing of a step's metadata), plain C++ behind a C ABI.

It is compiled with the system C++ compiler into ``_build/libgesso_host.so`` at the first use (a
second or two) and rebuilt when a source changes.  It needs neither a GPU nor ``nvcc``, so the
bookkeeping can be tested anywhere.  There is no Python fallback: without a C++ compiler the caller gets
a :class:`~gesso_b200.errors.GessoError`.
"""
from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
from ctypes import POINTER, c_int, c_int64, c_void_p

from ..errors import ErrorCode, GessoError
from .build import build_dir

_HERE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "host")
LIB_NAME = "libgesso_host.so"
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-Wall"]

_lib = None


def _sources():
    return sorted(f for f in os.listdir(_HERE) if f.endswith(".cpp"))


def find_cxx() -> str:
    for cand in (os.environ.get("GESSO_CXX"), os.environ.get("CXX"), "g++", "c++", "clang++"):
        if cand:
            path = cand if os.path.isabs(cand) else shutil.which(cand)
            if path and os.access(path, os.X_OK):
                return path
    raise GessoError(ErrorCode.COMPILE, "no C++ compiler found (set GESSO_CXX); the host runtime cannot be built "
                     "and there is no fallback")


def build() -> str:
    cxx = find_cxx()
    out_dir = build_dir()
    lib = os.path.join(out_dir, LIB_NAME)
    stamp = os.path.join(out_dir, "host_fingerprint.txt")
    h = hashlib.sha256(" ".join([cxx] + CXX_FLAGS).encode())
    for name in _sources():
        with open(os.path.join(_HERE, name), "rb") as f:
            h.update(name.encode())
            h.update(f.read())
    want = h.hexdigest()
    with open(os.path.join(out_dir, ".host_lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if os.path.isfile(lib) and os.path.isfile(stamp) and open(stamp).read().strip() == want:
                return lib
            print(f"[gesso_b200 build] compiling the host runtime ({len(_sources())} C++ file(s)) into {out_dir}",
                  file=sys.stderr, flush=True)
            tmp = lib + f".tmp{os.getpid()}"
            cmd = [cxx] + CXX_FLAGS + [os.path.join(_HERE, s) for s in _sources()] + ["-o", tmp]
            p = subprocess.run(cmd, capture_output=True, text=True)
            if p.returncode != 0:
                raise GessoError(ErrorCode.COMPILE, f"{cxx} failed on the host runtime:\n{p.stdout}\n{p.stderr}")
            os.replace(tmp, lib)
            with open(stamp, "w") as f:
                f.write(want)
            return lib
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


_IP = POINTER(c_int)
_LP = POINTER(c_int64)
_SIGNATURES = {
    "gesso_pool_new": ([c_int], c_void_p),
    "gesso_pool_delete": ([c_void_p], None),
    "gesso_pool_alloc": ([c_void_p], c_int),
    "gesso_pool_free": ([c_void_p, c_int], c_int),
    "gesso_pool_free_count": ([c_void_p], c_int),
    "gesso_pool_is_held": ([c_void_p, c_int], c_int),
    "gesso_cm_new": ([c_int, _IP, c_int, _IP, c_int, c_int], c_void_p),
    "gesso_cm_delete": ([c_void_p], None),
    "gesso_cm_admit": ([c_void_p, c_int64], c_int),
    "gesso_cm_release": ([c_void_p, c_int64], c_int),
    "gesso_cm_info": ([c_void_p, c_int64, _IP], c_int),
    "gesso_cm_take_fresh": ([c_void_p, c_int64], c_int),
    "gesso_cm_pages_needed": ([c_void_p, c_int64, c_int, _IP], c_int),
    "gesso_cm_reserve": ([c_void_p, c_int64, c_int], c_int),
    "gesso_cm_commit": ([c_void_p, c_int64, c_int], c_int),
    "gesso_cm_commit_many": ([c_void_p, _LP, c_int, c_int], c_int),
    "gesso_cm_row": ([c_void_p, c_int64, c_int, _IP], _IP),
    "gesso_cm_counts": ([c_void_p, _IP], None),
    "gesso_cm_live": ([c_void_p, _LP, c_int], c_int),
    "gesso_cm_last_short": ([c_void_p, _IP], None),
    "gesso_cm_check": ([c_void_p], c_int),
    "gesso_cm_reserve_step": ([c_void_p, _LP, _IP, c_int, _IP, _IP, _IP, _IP], c_int),
    "gesso_cm_commit_step": ([c_void_p, _LP, _IP, c_int], c_int),
    "gesso_step_prepare": ([c_void_p, _LP, _IP, c_int, _IP, _IP, _IP, _IP, c_int, _IP, c_int, c_int, c_int, c_int,
                            _IP, c_void_p, c_int, _IP, _IP], c_int),
}


def library():
    """The loaded host runtime (built first if need be)."""
    global _lib
    if _lib is None:
        lib = ctypes.CDLL(build())
        for name, (args, res) in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = res
        _lib = lib
    return _lib
