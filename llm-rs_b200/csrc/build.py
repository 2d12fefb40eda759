"""Compiles the kernel library for sm_100a with nvcc, and the host library (cache
bookkeeping and step packing, plain C++ under ``csrc/host/``) with the C++ compiler, and
loads them.

The library is plain CUDA behind C entry points (no framework headers), so a fresh
checkout compiles in well under a minute. It is built next to the sources in
``csrc/_build/`` (or in a per-user temporary folder when the checkout is read-only) at
the first call that needs a kernel, and rebuilt when a source or a flag changes. While
nvcc runs, a line is printed to stderr every few seconds.
"""
from __future__ import annotations

import ctypes
import fcntl
import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile
import time
from typing import List, Optional

CSRC_DIR = os.path.dirname(os.path.abspath(__file__))
# Two build variants, chosen by the environment at import (each has its own library beside the normal one):
#   LLMRS_DEBUG_KERNELS=1  the kernels check the indices they are about to use (page ids, positions, token
#                          ids); a bad one is recorded in a word that ``ops.debug_take()`` reads and its
#                          access is skipped: no trap, no fault. For hunting a wrong table or position
#                          where a memory checker cannot be run.
#   LLMRS_HOST_SANITIZE=1  the C++ host library built with AddressSanitizer and UndefinedBehaviorSanitizer
#                          (run Python with the sanitizer's runtime preloaded; tests/test_host_sanitized.py).
DEBUG_KERNELS = os.environ.get("LLMRS_DEBUG_KERNELS", "0") == "1"
HOST_SANITIZE = os.environ.get("LLMRS_HOST_SANITIZE", "0") == "1"
_VARIANT = "_debug" if DEBUG_KERNELS else ""
LIB_NAME = f"libllmrs_b200{_VARIANT}.so"
STAMP_NAME = f"stamp{_VARIANT}.json"
# Fast math stays off: norms, softmax and rotation are checked against float32 references.
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"] + (["-DLLMRS_DEBUG_CHECKS"] if DEBUG_KERNELS else [])
ABI_VERSION = 4
HOST_DIR = os.path.join(CSRC_DIR, "host")
HOST_LIB_NAME = "libllmrs_b200_host_san.so" if HOST_SANITIZE else "libllmrs_b200_host.so"
HOST_STAMP_NAME = "host_san_stamp.json" if HOST_SANITIZE else "host_stamp.json"
HOST_FLAGS = ["-std=c++17", "-fPIC", "-Wall"] + (
    ["-O1", "-g", "-fno-omit-frame-pointer", "-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"]
    if HOST_SANITIZE else ["-O2"])
HOST_ABI_VERSION = 3

_lib: Optional[ctypes.CDLL] = None
_host_lib: Optional[ctypes.CDLL] = None


class KernelBuildError(RuntimeError):
    pass


def _log(msg: str) -> None:
    print(f"[llm_rs_b200 build] {msg}", file=sys.stderr, flush=True)


def sources() -> List[str]:
    return sorted(f for f in os.listdir(CSRC_DIR) if f.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(CSRC_DIR) if f.endswith((".cuh", ".h")))


def _fingerprint() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for name in sources() + _headers():
        h.update(name.encode())
        with open(os.path.join(CSRC_DIR, name), "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def find_nvcc() -> Optional[str]:
    for base in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if base:
            cand = os.path.join(base, "bin", "nvcc")
            if os.path.isfile(cand) and os.access(cand, os.X_OK):
                return cand
    return shutil.which("nvcc")


def _build_dirs() -> List[str]:
    dirs = [os.path.join(CSRC_DIR, "_build")]
    tmp = os.path.join(tempfile.gettempdir(), f"llm_rs_b200_build_{os.getuid()}")
    dirs.append(tmp)
    return dirs


def _is_current(build_dir: str, fp: str, stamp_name: str = STAMP_NAME, lib_name: str = LIB_NAME) -> bool:
    stamp = os.path.join(build_dir, stamp_name)
    lib = os.path.join(build_dir, lib_name)
    if not (os.path.isfile(stamp) and os.path.isfile(lib)):
        return False
    try:
        with open(stamp) as f:
            return json.load(f).get("fingerprint") == fp
    except (OSError, ValueError):
        return False


def _writable_dir() -> str:
    for d in _build_dirs():
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".probe_{os.getpid()}")
            with open(probe, "w"):
                pass
            os.unlink(probe)
            return d
        except OSError:
            continue
    raise KernelBuildError(f"no writable folder for the kernel library among {_build_dirs()}")


def _compile(build_dir: str, fp: str) -> None:
    nvcc = find_nvcc()
    if nvcc is None:
        raise KernelBuildError(
            "the CUDA kernel library is not built and nvcc was not found (looked in $CUDA_HOME, "
            "/usr/local/cuda and PATH); this engine has no fallback without its kernels")
    srcs = sources()
    _log(f"compiling {len(srcs)} CUDA sources for sm_100a with {nvcc} into {build_dir}")
    t0 = time.time()
    procs = []
    for name in srcs:
        obj = os.path.join(build_dir, name[:-3] + _VARIANT + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", CSRC_DIR, "-c", os.path.join(CSRC_DIR, name), "-o", obj]
        procs.append((name, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    pending = list(procs)
    last = time.time()
    while pending:
        for item in list(pending):
            name, _, p = item
            if p.poll() is not None:
                out = p.stdout.read()
                pending.remove(item)
                if p.returncode != 0:
                    for _, _, q in pending:
                        q.kill()
                    raise KernelBuildError(f"nvcc failed on {name}:\n{out}")
                _log(f"compiled {name} ({time.time() - t0:.0f} s)")
        if pending and time.time() - last > 5:
            _log(f"still compiling: {', '.join(n for n, _, _ in pending)} ({time.time() - t0:.0f} s)")
            last = time.time()
        time.sleep(0.1)
    lib_tmp = os.path.join(build_dir, f".{LIB_NAME}.{os.getpid()}")
    cmd = [nvcc, "-shared", "-o", lib_tmp, *[o for _, o, _ in procs], "-lcudart"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise KernelBuildError(f"linking the kernel library failed:\n{r.stdout}")
    os.replace(lib_tmp, os.path.join(build_dir, LIB_NAME))
    with open(os.path.join(build_dir, STAMP_NAME), "w") as f:
        json.dump({"fingerprint": fp, "flags": NVCC_FLAGS, "sources": srcs}, f)
    _log(f"built {LIB_NAME} in {time.time() - t0:.0f} s")


def build(force: bool = False) -> str:
    """Make sure the library is built for the current sources; return its path."""
    fp = _fingerprint()
    if not force:
        for d in _build_dirs():
            if _is_current(d, fp):
                return os.path.join(d, LIB_NAME)
    d = _writable_dir()
    with open(os.path.join(d, ".lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if force or not _is_current(d, fp):
                _compile(d, fp)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return os.path.join(d, LIB_NAME)


def library() -> ctypes.CDLL:
    """The loaded kernel library (built first if needed). Raises if it cannot be had."""
    global _lib
    if _lib is None:
        path = build()
        lib = ctypes.CDLL(path)
        lib.llmrs_abi_version.restype = ctypes.c_int
        lib.llmrs_last_error.restype = ctypes.c_char_p
        if lib.llmrs_abi_version() != ABI_VERSION:
            raise KernelBuildError(f"{path} has ABI {lib.llmrs_abi_version()}, expected {ABI_VERSION}")
        _lib = lib
    return _lib


# -- the host library ------------------------------------------------------------------
def host_sources() -> List[str]:
    return sorted(f for f in os.listdir(HOST_DIR) if f.endswith(".cpp"))


def _host_fingerprint() -> str:
    h = hashlib.sha256()
    h.update(" ".join(HOST_FLAGS).encode())
    for name in sorted(os.listdir(HOST_DIR)):
        if name.endswith((".cpp", ".hpp", ".h")):
            h.update(name.encode())
            with open(os.path.join(HOST_DIR, name), "rb") as f:
                h.update(f.read())
    return h.hexdigest()


def find_cxx() -> Optional[List[str]]:
    """The command that compiles C++: $CXX, g++, c++ or clang++ (nvcc needs one of them too)."""
    for cand in (os.environ.get("CXX"), "g++", "c++", "clang++"):
        if cand and shutil.which(cand):
            return [shutil.which(cand)]
    return None


def _compile_host(build_dir: str, fp: str) -> None:
    cxx = find_cxx()
    if cxx is None:
        raise KernelBuildError("the host library is not built and no C++ compiler was found ($CXX, g++, c++, clang++)")
    srcs = [os.path.join(HOST_DIR, n) for n in host_sources()]
    lib_tmp = os.path.join(build_dir, f".{HOST_LIB_NAME}.{os.getpid()}")
    cmd = [*cxx, *HOST_FLAGS, "-shared", "-I", HOST_DIR, *srcs, "-o", lib_tmp]
    t0 = time.time()
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise KernelBuildError(f"compiling the host library failed:\n{r.stdout}")
    os.replace(lib_tmp, os.path.join(build_dir, HOST_LIB_NAME))
    with open(os.path.join(build_dir, HOST_STAMP_NAME), "w") as f:
        json.dump({"fingerprint": fp, "flags": HOST_FLAGS, "sources": host_sources()}, f)
    _log(f"built {HOST_LIB_NAME} in {time.time() - t0:.0f} s")


def build_host(force: bool = False) -> str:
    """Make sure the host library is built for the current sources; return its path."""
    fp = _host_fingerprint()
    if not force:
        for d in _build_dirs():
            if _is_current(d, fp, HOST_STAMP_NAME, HOST_LIB_NAME):
                return os.path.join(d, HOST_LIB_NAME)
    d = _writable_dir()
    with open(os.path.join(d, ".host_lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if force or not _is_current(d, fp, HOST_STAMP_NAME, HOST_LIB_NAME):
                _compile_host(d, fp)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return os.path.join(d, HOST_LIB_NAME)


# -- the engine's C entry points ---------------------------------------------------------
CAPI_DIR = os.path.join(CSRC_DIR, "capi")
CAPI_LIB_NAME = "libllmrs_b200_engine.so"


def _capi_flags() -> List[str]:
    """The interpreter a plain C program gets: the library of the Python that builds this, with its module paths."""
    import sysconfig
    pylib = sysconfig.get_config_var("INSTSONAME") or sysconfig.get_config_var("LDLIBRARY") or "libpython3.so"
    libdir = sysconfig.get_config_var("LIBDIR") or ""
    if libdir and os.path.exists(os.path.join(libdir, pylib)):
        pylib = os.path.join(libdir, pylib)
    paths = ":".join(p for p in sys.path if p and os.path.isdir(p))
    return [*HOST_FLAGS, f'-DLLMRS_PY_LIB="{pylib}"', f'-DLLMRS_PY_PATHS="{paths}"']


def _capi_fingerprint() -> str:
    h = hashlib.sha256()
    h.update(" ".join(_capi_flags()).encode())
    for name in sorted(os.listdir(CAPI_DIR)):
        if name.endswith((".cpp", ".h")):
            h.update(name.encode())
            with open(os.path.join(CAPI_DIR, name), "rb") as f:
                h.update(f.read())
    return h.hexdigest()


def build_engine_api(force: bool = False) -> str:
    """Make sure the library with the engine's C entry points (``capi/llm_engine.h``) is built; return its path."""
    fp = _capi_fingerprint()
    if not force:
        for d in _build_dirs():
            if _is_current(d, fp, "capi_stamp.json", CAPI_LIB_NAME):
                return os.path.join(d, CAPI_LIB_NAME)
    d = _writable_dir()
    with open(os.path.join(d, ".capi_lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if force or not _is_current(d, fp, "capi_stamp.json", CAPI_LIB_NAME):
                cxx = find_cxx()
                if cxx is None:
                    raise KernelBuildError("no C++ compiler was found ($CXX, g++, c++, clang++)")
                tmp = os.path.join(d, f".{CAPI_LIB_NAME}.{os.getpid()}")
                cmd = [*cxx, *_capi_flags(), "-shared", "-I", CAPI_DIR, os.path.join(CAPI_DIR, "llm_engine.cpp"),
                       "-o", tmp, "-ldl"]
                t0 = time.time()
                r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
                if r.returncode != 0:
                    raise KernelBuildError(f"compiling the engine's C entry points failed:\n{r.stdout}")
                os.replace(tmp, os.path.join(d, CAPI_LIB_NAME))
                with open(os.path.join(d, "capi_stamp.json"), "w") as f:
                    json.dump({"fingerprint": fp}, f)
                _log(f"built {CAPI_LIB_NAME} in {time.time() - t0:.0f} s")
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return os.path.join(d, CAPI_LIB_NAME)


def host_library() -> ctypes.CDLL:
    """The loaded host library (built first if needed)."""
    global _host_lib
    if _host_lib is None:
        path = build_host()
        lib = ctypes.CDLL(path)
        lib.llmrs_host_abi_version.restype = ctypes.c_int
        lib.llmrs_host_last_error.restype = ctypes.c_char_p
        if lib.llmrs_host_abi_version() != HOST_ABI_VERSION:
            raise KernelBuildError(f"{path} has ABI {lib.llmrs_host_abi_version()}, expected {HOST_ABI_VERSION}")
        _host_lib = lib
    return _host_lib
