"""Builds and loads the sm_100a INT8 kernel library (``libhy3d_int8.so``).

Mirrors the loader surface of the reference's ``csrc/build.py`` (``load_int8_kernels`` :77-94,
``load_tc_gemm`` :97-114, ``load_sparse_tc`` :117-134, CLI :137-156) with two differences:

* one architecture only: ``-gencode arch=compute_100a,code=sm_100a``;
* the product is a plain C-ABI shared library compiled by ``nvcc`` directly and opened with
  ``ctypes`` -- no torch headers are involved, so a cold build takes seconds and the ``.so``
  sits in-tree next to its sources.

The three ``load_*`` functions return small namespace objects exposing the reference's
extension function names (see ``_binding.py``); all of them share the single library.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import threading
from concurrent.futures import ThreadPoolExecutor

_CSRC = os.path.dirname(os.path.abspath(__file__))
_REPO_INCLUDE = os.path.normpath(os.path.join(_CSRC, "..", "..", "include"))
_BUILD_DIR = os.path.join(_CSRC, "_build")
LIB_NAME = "libhy3d_int8.so"
LIB_PATH = os.path.join(_CSRC, LIB_NAME)

# hy3d_int8.cu is the only translation unit; it #includes the kernel files listed in HEADERS.
SOURCES = ["hy3d_int8.cu"]
HEADERS = ["common.cuh", "quantize.cu", "prune_pack.cu", "gemm_dense.cu", "gemm_sparse.cu",
           "linear_fused.cu", "groupnorm.cu", "capi.cu", "static_scratch.cu", "probes.cu", os.path.join(_REPO_INCLUDE, "hy3d_int8.h")]

_lock = threading.Lock()
_lib = None


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; set NVCC or put it on PATH")
    return cand


def cuda_flags() -> list[str]:
    """nvcc flags for every translation unit.  No --use_fast_math: the quantiser's rounding
    and the epilogue's erf must stay IEEE."""
    return [
        "-O3", "-std=c++17", "-lineinfo",
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-Xcompiler", "-fPIC",
        "-I", _REPO_INCLUDE,
    ]


def _source_digest() -> str:
    """Hash of the sources and of the flags that affect code generation.  Nothing in it
    depends on where the tree lives, so a library built in one checkout is accepted as
    up to date in a copy of that checkout elsewhere."""
    h = hashlib.sha256()
    for name in SOURCES + HEADERS:
        path = name if os.path.isabs(name) else os.path.join(_CSRC, name)
        with open(path, "rb") as f:
            h.update(os.path.basename(name).encode())
            h.update(f.read())
    h.update(" ".join(fl for fl in cuda_flags() if fl != _REPO_INCLUDE).encode())
    return h.hexdigest()


def _up_to_date(stamp: str, digest: str) -> bool:
    if not (os.path.exists(LIB_PATH) and os.path.exists(stamp)):
        return False
    with open(stamp) as f:
        return f.read().strip() == digest


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if its sources changed; returns the path of the .so.  Several
    processes may call this at once (one per GPU under torchrun): a file lock lets one of them
    build while the others wait and then find the library up to date."""
    stamp = os.path.join(_BUILD_DIR, "digest.txt")
    digest = _source_digest()
    if not force and _up_to_date(stamp, digest):
        return LIB_PATH
    os.makedirs(_BUILD_DIR, exist_ok=True)
    import fcntl
    with open(os.path.join(_BUILD_DIR, "build.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and _up_to_date(stamp, digest):
                return LIB_PATH
            return _build_locked(stamp, digest, verbose)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def _build_locked(stamp: str, digest: str, verbose: bool) -> str:
    nvcc = _nvcc()
    # The digest of the sources is baked into the library (hy3d_source_digest()), so a loaded
    # .so can be told apart from one built from other sources.
    flags = cuda_flags() + [f'-DHY3D_SOURCE_DIGEST="{digest}"'] + (["-Xptxas", "-v"] if verbose else [])

    def compile_one(src: str) -> str:
        obj = os.path.join(_BUILD_DIR, src.replace(".cu", ".o"))
        cmd = [nvcc, *flags, "-c", os.path.join(_CSRC, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stderr}")
        return obj

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        objs = list(pool.map(compile_one, SOURCES))
    tmp = LIB_PATH + f".tmp{os.getpid()}"
    cmd = [nvcc, "-shared", "-o", tmp, *objs, "-gencode", "arch=compute_100a,code=sm_100a",
           "-Xcompiler", "-fPIC"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stderr}")
    os.replace(tmp, LIB_PATH)
    with open(stamp, "w") as f:
        f.write(digest)
    return LIB_PATH


def load_library(build_if_missing: bool = True) -> ctypes.CDLL:
    """Open libhy3d_int8.so (building it first when the sources are newer)."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = LIB_PATH
        if build_if_missing:
            try:
                _nvcc()
                have_nvcc = True
            except RuntimeError:
                have_nvcc = False
            if have_nvcc:
                path = build()          # compile and link errors propagate
            elif not os.path.exists(LIB_PATH):
                raise RuntimeError(f"{LIB_NAME} is missing and there is no nvcc to build it")
        if not os.path.exists(path):
            raise RuntimeError(f"{LIB_NAME} is missing; run `python csrc/build.py`")
        lib = ctypes.CDLL(path)
        # A library that travelled with the tree must come from these sources: a stale one
        # could be driven with argument lists it does not have.
        lib.hy3d_source_digest.restype = ctypes.c_char_p
        lib.hy3d_source_digest.argtypes = []
        built_from = lib.hy3d_source_digest().decode()
        if built_from != _source_digest():
            raise RuntimeError(f"{LIB_NAME} was built from other sources (digest {built_from[:12]}...); "
                               "rebuild it with `python csrc/build.py`")
        _lib = lib
        return _lib


def load_int8_kernels():
    """Quantise / dequantise helpers (reference: csrc/build.py:77-94)."""
    from . import _binding
    return _binding.Int8KernelsModule(load_library())


def load_tc_gemm():
    """Dense W8A8 tensor-core GEMM (reference: csrc/build.py:97-114)."""
    from . import _binding
    return _binding.TcGemmModule(load_library())


def load_sparse_tc():
    """2:4 sparse W8A8 tensor-core GEMM (reference: csrc/build.py:117-134)."""
    from . import _binding
    return _binding.SparseTcModule(load_library())


if __name__ == "__main__":
    target = sys.argv[1] if len(sys.argv) > 1 else "all"
    if target not in ("all", "kernels", "tc", "sparse_tc"):
        print("usage: python build.py [all|kernels|tc|sparse_tc]")
        sys.exit(1)
    # Every target lives in the same library.
    print("Building", LIB_NAME, "for sm_100a ...")
    print("  ->", build(force="--force" in sys.argv, verbose="-v" in sys.argv))
