"""Build and load the C-ABI CUDA library (`libcastle_b200.so`, built in-tree).

There is no fallback: if the library is missing or fails to load, every
operator of this package raises.
"""
from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libcastle_b200.so"
SOURCES = ["api.cu", "decode.cu", "selftest.cu", "convert.cu", "fwd.cu", "bwd.cu", "bwd128.cu"]

BF16, F16, F32 = 0, 1, 2


class CastleTensor(ctypes.Structure):
    _fields_ = [("ptr", ctypes.c_void_p), ("stride_b", ctypes.c_int64), ("stride_h", ctypes.c_int64),
                ("stride_n", ctypes.c_int64)]


class CastleProblem(ctypes.Structure):
    _fields_ = [("batch", ctypes.c_int32), ("heads", ctypes.c_int32), ("seq_len", ctypes.c_int32),
                ("dim_head", ctypes.c_int32), ("dtype", ctypes.c_int32), ("scale", ctypes.c_float)]


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; cannot build libcastle_b200.so")


def _sources():
    return [CSRC / s for s in SOURCES if (CSRC / s).exists()]


NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-shared",
              "-Xcompiler", "-fPIC"]
STAMP_PATH = PKG_DIR / "libcastle_b200.so.stamp"


def _deps():
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list((PKG_DIR.parent / "include").glob("*.h")))


def _source_hash() -> str:
    """Digest of every source the library is built from plus the compiler flags.  Compared with
    the stamp written next to the library, so a stale build is noticed whatever the file times say
    (a copied tree does not keep them)."""
    import hashlib
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    for d in _deps():
        h.update(d.name.encode())
        h.update(d.read_bytes())
    return h.hexdigest()


def needs_build():
    if not LIB_PATH.exists() or not STAMP_PATH.exists():
        return True
    return STAMP_PATH.read_text().strip() != _source_hash()


def _locked(fn):
    """Run `fn` holding the build lock (one builder per tree; ranks that start together queue here)."""
    import fcntl
    with open(PKG_DIR / ".build.lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            return fn()
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def _build_unlocked(verbose: bool = False):
    tmp = LIB_PATH.with_name(f".libcastle_b200.{os.getpid()}.tmp.so")
    cmd = [_nvcc()] + NVCC_FLAGS + ["-Xptxas", "-v" if verbose else "-warn-spills", "-o", str(tmp)] + \
          [str(s) for s in _sources()]
    digest = _source_hash()
    try:
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
        os.replace(tmp, LIB_PATH)          # readers see the old library or the complete new one, never half of it
        STAMP_PATH.write_text(digest + "\n")
    finally:
        if tmp.exists():
            tmp.unlink()
    if verbose:
        print(res.stderr)
    return LIB_PATH


def build(force: bool = False, verbose: bool = False):
    """Compile every kernel for sm_100a into one shared library next to this file."""
    def go():
        if not force and not needs_build():
            return LIB_PATH
        return _build_unlocked(verbose)
    return _locked(go)


_lib = None

P = ctypes.POINTER
_T, _PR = P(CastleTensor), P(CastleProblem)
_vp, _i32, _sz = ctypes.c_void_p, ctypes.c_int32, ctypes.c_size_t

_SIGNATURES = {
    "castle_abi_version": (ctypes.c_int, []),
    "castle_last_error": (ctypes.c_char_p, []),
    "castle_fwd_workspace_bytes": (_sz, [_PR]),
    "castle_fwd": (ctypes.c_int, [_PR] + [_T] * 7 + [_vp, _T, _i32, _vp, _vp, _sz, _vp, _vp]),
    "castle_fwd_prefill": (ctypes.c_int, [_PR] + [_T] * 7 + [_vp] + [_T] * 4 + [_vp, _vp, _sz, _vp, _vp]),
    "castle_convert_16bit": (ctypes.c_int, [_i32, _vp, _vp, ctypes.c_int64, _vp, _vp]),
    "castle_bwd_workspace_bytes": (_sz, [_PR]),
    "castle_bwd": (ctypes.c_int, [_PR] + [_T] * 8 + [_vp, _vp] + [_T] * 6 + [_vp, _sz, _vp, _vp]),
    "castle_decode_workspace_bytes": (_sz, [_PR, _i32]),
    "castle_decode_step": (ctypes.c_int, [_PR, _i32, _i32] + [_T] * 11 + [_vp, _sz, _vp, _vp]),
    "castle_decode_step_static": (ctypes.c_int, [_PR, _i32, _i32] + [_T] * 11 + [_vp, _vp]),
    "castle_set_kernel_events": (ctypes.c_int, [_i32, _vp, _vp]),
    "castle_selftest_mma_rate": (ctypes.c_int, [_i32, _i32, _i32, _vp, _vp, _vp]),
    "castle_selftest_mma": (ctypes.c_int, [_i32, _vp, _vp, _vp, _vp, _vp]),
    "castle_selftest_wait_timeout": (ctypes.c_int, [_i32, _vp, _vp, _vp]),
}


def load():
    """Return the ctypes handle of the library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    override = os.environ.get("CASTLE_B200_LIB")   # a developer's own build of the same sources (other -D flags)
    if override:
        return _bind(ctypes.CDLL(override))

    def ensure():
        # compile on demand when the library is missing or was built from other sources; there is
        # no other code path to fall back to
        if needs_build():
            try:
                _build_unlocked()
            except Exception as e:
                raise RuntimeError(f"{LIB_PATH} is missing or stale and could not be rebuilt ({e}); run "
                                   "`python -c 'import __graft_entry__ as g; g.build()'` where nvcc is "
                                   "available - this package has no fallback path") from e
    _locked(ensure)
    return _bind(ctypes.CDLL(str(LIB_PATH)))


def _bind(lib):
    global _lib
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    if lib.castle_abi_version() != 1:
        raise RuntimeError("libcastle_b200.so ABI version mismatch")
    _lib = lib
    return lib


def last_error() -> str:
    return load().castle_last_error().decode()


def check(rc: int, what: str):
    if rc != 0:
        raise RuntimeError(f"{what} failed (rc={rc}): {last_error()}")
