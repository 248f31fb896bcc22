"""Builds the CUDA sources under ``csrc/`` into shared libraries and loads them.

Every library is compiled by ``nvcc`` for sm_100a alone and loaded with
``ctypes``; no Python extension headers are involved, so a build takes
seconds.  Built files live in ``csrc/_build`` beside the sources (falling back
to a temporary folder when the tree is read-only) and carry a hash of the
sources and flags in their name, so an edit never loads a stale library.

Libraries are built on first use: a float32 run builds only what the float32
path calls.  A line is printed to stderr while a build runs.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

CSRC = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "csrc"))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-shared",
]

# library name -> sources (headers are hashed with every library)
LIBRARIES: dict[str, list[str]] = {
    "core": ["core.cu"],
    "linear_f32": ["linear_f32.cu"],
    "attn_simt": ["attn_simt.cu"],
    "attn_mma": ["attn_mma.cu"],
    "skinny_gemm": ["skinny_gemm.cu"],
    "attn_noalloc": ["attn_decode_noalloc.cu"],
    "gemm_tc": ["gemm_tc.cu"],
    "gemm_tc2": ["gemm_tc2.cu"],
    "attn_tc": ["attn_tc.cu"],
    "gemm_stream": ["gemm_stream.cu"],
    "sampling": ["sampling.cu"],
}
HEADERS = ["common.cuh", "attn_mma.cuh", "attn_decode_noalloc.h", "tcgen05.cuh"]

_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class KernelBuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for cand in (os.environ.get("BROLM_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise KernelBuildError("nvcc was not found (looked at $BROLM_NVCC, PATH and /usr/local/cuda/bin); "
                           "the CUDA kernels of brolm_b200 cannot be built and there is no other path")


_build_dir_cache: dict[str, str] = {}
_dir_lock = threading.Lock()


def _build_dir() -> str:
    """The folder for built libraries, decided once per wanted path (the write
    probe must not race with itself when several libraries build at a time)."""
    want = os.environ.get("BROLM_BUILD_DIR") or os.path.join(CSRC, "_build")
    with _dir_lock:
        got = _build_dir_cache.get(want)
        if got is not None:
            return got
        try:
            os.makedirs(want, exist_ok=True)
            fd, probe = tempfile.mkstemp(prefix=".w", dir=want)
            os.close(fd)
            os.remove(probe)
            got = want
        except OSError:
            got = os.path.join(tempfile.gettempdir(), f"brolm_b200_build_{os.getuid()}")
            os.makedirs(got, exist_ok=True)
        _build_dir_cache[want] = got
        return got


def _digest(name: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for rel in HEADERS + LIBRARIES[name]:
        with open(os.path.join(CSRC, rel), "rb") as fh:
            h.update(rel.encode())
            h.update(fh.read())
    return h.hexdigest()[:16]


def library_path(name: str) -> str:
    return os.path.join(_build_dir(), f"libbrolm_{name}_{_digest(name)}.so")


def build_library(name: str, verbose: bool = True) -> str:
    """Compile one library if its file is not there yet; return its path."""
    if name not in LIBRARIES:
        raise KernelBuildError(f"unknown kernel library '{name}'")
    out = library_path(name)
    if os.path.exists(out):
        return out
    nvcc = _nvcc()
    tmp = f"{out}.{os.getpid()}.tmp"
    cmd = [nvcc] + NVCC_FLAGS + ["-I", CSRC, "-o", tmp] + [os.path.join(CSRC, s) for s in LIBRARIES[name]]
    if verbose:
        print(f"[brolm_b200] building kernel library '{name}' for sm_100a ...", file=sys.stderr, flush=True)
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    out_text: list[str] = []
    reader = threading.Thread(target=lambda: out_text.append(proc.stdout.read()), daemon=True)
    reader.start()
    while True:
        try:
            proc.wait(timeout=10)
            break
        except subprocess.TimeoutExpired:
            if verbose:
                print(f"[brolm_b200]   still compiling '{name}' ({time.time() - t0:.0f} s)", file=sys.stderr,
                      flush=True)
    reader.join()
    if proc.returncode != 0:
        try:
            os.remove(tmp)
        except OSError:
            pass
        raise KernelBuildError(f"nvcc failed for '{name}':\n{' '.join(cmd)}\n{''.join(out_text)}")
    os.replace(tmp, out)
    if verbose:
        print(f"[brolm_b200]   built '{name}' in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return out


def build_all(verbose: bool = True) -> list[str]:
    """Compile every library (several at a time)."""
    names = list(LIBRARIES)
    results: dict[str, object] = {}

    def work(n: str) -> None:
        try:
            results[n] = build_library(n, verbose)
        except Exception as e:  # noqa: BLE001 - reported below
            results[n] = e

    threads = [threading.Thread(target=work, args=(n,)) for n in names]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    for n in names:
        if isinstance(results[n], Exception):
            raise results[n]
    paths = [str(results[n]) for n in names]
    _prune(paths)
    return paths


def _prune(keep: list[str]) -> None:
    """Remove libraries of earlier source versions from the build folder."""
    folder = _build_dir()
    wanted = {os.path.basename(p) for p in keep}
    for f in os.listdir(folder):
        if f.startswith("libbrolm_") and f.endswith(".so") and f not in wanted:
            try:
                os.remove(os.path.join(folder, f))
            except OSError:
                pass


def library_loaded(name: str) -> bool:
    """Whether this process has already loaded (and so used) the library."""
    return name in _loaded


def load_library(name: str) -> ctypes.CDLL:
    """Build if needed, then load; fails loudly, there is no fallback."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = build_library(name)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelBuildError(f"cannot load kernel library '{path}': {e}") from e
            _loaded[name] = lib
        return lib
