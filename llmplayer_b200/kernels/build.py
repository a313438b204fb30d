"""Compiling the CUDA sources into shared libraries, one per source file.

The reference compiles its kernel sources at run time with NVRTC for whatever
device it finds (java21 gpu/CudaContext.java:163-239). Here each ``.cu`` under
``csrc/`` becomes ``csrc/_build/<name>.so`` with nvcc for sm_100a, at the first
use of an operation that lives in it (or all at once through ``build_all``);
a library is rebuilt when its source, a header or the flags change.
"""
from __future__ import annotations

import fcntl
import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from typing import Dict, Iterable, List

from ..errors import ExtensionMissing

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")

# library name -> source file; headers are dependencies of all of them
LIBRARIES: Dict[str, str] = {
    "elementwise": "elementwise.cu",
    "gemm_plain": "gemm_plain.cu",
    "attention_plain": "attention_plain.cu",
    "sampling": "sampling.cu",
    "gemm_tcgen05": "gemm_tcgen05.cu",
    "attention_mma": "attention_mma.cu",
    "attention_tcgen05": "attention_tcgen05.cu",
    "host_loop": "host_loop.cu",
}
HEADERS = ("common.cuh", "attention_noalloc.h", "tcgen05_utils.cuh", "attention_decode.cuh")

NVCC_FLAGS: List[str] = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC",
]


def _log(msg: str) -> None:
    print(f"[llmplayer_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    candidates = []
    for var in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(var):
            candidates.append(os.path.join(os.environ[var], "bin", "nvcc"))
    candidates.append("/usr/local/cuda/bin/nvcc")
    which = shutil.which("nvcc")
    if which:
        candidates.append(which)
    for cand in candidates:
        if os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise ExtensionMissing("nvcc was not found (looked in $CUDA_HOME/bin, /usr/local/cuda/bin and PATH); "
                           "the CUDA kernels cannot be compiled")


_build_dir_lock = threading.Lock()
_build_dir_cache: Dict[str, str] = {}


def build_dir() -> str:
    """Where libraries are kept: $LLMPLAYER_B200_BUILD_DIR, else csrc/_build in the
    package, else (package not writable) a per-user folder under the temp dir."""
    key = os.environ.get("LLMPLAYER_B200_BUILD_DIR", "")
    with _build_dir_lock:
        if key not in _build_dir_cache:
            _build_dir_cache[key] = _choose_build_dir()
        return _build_dir_cache[key]


def _choose_build_dir() -> str:
    override = os.environ.get("LLMPLAYER_B200_BUILD_DIR")
    if override:
        os.makedirs(override, exist_ok=True)
        return override
    in_tree = os.path.join(CSRC, "_build")
    try:
        os.makedirs(in_tree, exist_ok=True)
        probe = os.path.join(in_tree, f".probe{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return in_tree
    except OSError:
        fallback = os.path.join(tempfile.gettempdir(), f"llmplayer_b200_build_{os.getuid()}")
        os.makedirs(fallback, exist_ok=True)
        return fallback


def _fingerprint(name: str) -> str:
    h = hashlib.sha256()
    for rel in (LIBRARIES[name],) + tuple(HEADERS):
        with open(os.path.join(CSRC, rel), "rb") as fh:
            h.update(rel.encode())
            h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def library_path(name: str) -> str:
    return os.path.join(build_dir(), f"{name}.so")


def is_current(name: str) -> bool:
    so = library_path(name)
    stamp = so + ".json"
    if not (os.path.exists(so) and os.path.exists(stamp)):
        return False
    try:
        with open(stamp) as fh:
            return json.load(fh).get("fingerprint") == _fingerprint(name)
    except (OSError, ValueError):
        return False


def _run_nvcc(cmd: List[str], what: str) -> None:
    start = time.time()
    done = threading.Event()

    def heartbeat():
        while not done.wait(10.0):
            _log(f"still compiling {what} ({time.time() - start:.0f} s)")

    beat = threading.Thread(target=heartbeat, daemon=True)
    beat.start()
    try:
        proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    finally:
        done.set()
    if proc.returncode != 0:
        raise ExtensionMissing(f"nvcc failed for {what}:\n{' '.join(cmd)}\n{proc.stdout}")
    _log(f"compiled {what} in {time.time() - start:.1f} s")


def ensure_built(name: str) -> str:
    """Path of the up-to-date library ``name``, compiling it if need be."""
    if name not in LIBRARIES:
        raise ExtensionMissing(f"no CUDA library named {name!r}")
    if is_current(name):
        return library_path(name)
    out_dir = build_dir()
    lock_path = os.path.join(out_dir, f"{name}.lock")
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if is_current(name):          # another process built it meanwhile
                return library_path(name)
            nvcc = find_nvcc()
            so = library_path(name)
            tmp = f"{so}.{os.getpid()}.tmp"
            src = os.path.join(CSRC, LIBRARIES[name])
            _log(f"compiling {LIBRARIES[name]} for sm_100a (first use)")
            _run_nvcc([nvcc] + NVCC_FLAGS + ["-I", CSRC, "-o", tmp, src], LIBRARIES[name])
            os.replace(tmp, so)
            with open(so + ".json", "w") as fh:
                json.dump({"fingerprint": _fingerprint(name), "source": LIBRARIES[name]}, fh)
            return so
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def build_all(names: Iterable[str] = None, jobs: int = 4) -> Dict[str, str]:
    """Compile every library (several at a time); returns name -> path."""
    names = list(names or LIBRARIES)
    results: Dict[str, str] = {}
    errors: List[BaseException] = []
    gate = threading.Semaphore(max(1, jobs))

    def work(n: str) -> None:
        with gate:
            try:
                results[n] = ensure_built(n)
            except BaseException as exc:  # collected and re-raised below
                errors.append(exc)

    threads = [threading.Thread(target=work, args=(n,)) for n in names]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    if errors:
        raise errors[0]
    return results
