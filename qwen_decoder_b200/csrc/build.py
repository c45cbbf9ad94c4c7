"""Compiling and loading the CUDA libraries.

Each ``.cu`` file under ``csrc/`` becomes one shared library of ``extern "C"``
launchers, compiled for sm_100a with nvcc and loaded with ctypes.  A library is
built the first time an operation needs it (so a run compiles what its model and
dtype use, nothing else) and kept under ``csrc/_build/`` (or, if the package
folder is read-only, a per-user folder under the temporary directory), keyed by a
hash of its sources and flags.  There is no fallback: if nvcc or the built library
is missing, the operation raises.
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
from typing import Dict, List

CSRC = os.path.dirname(os.path.abspath(__file__))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
]

# library name -> source file (headers every library may include are hashed into all keys)
LIBRARIES: Dict[str, str] = {
    "elementwise": "elementwise.cu",
    "gemm_generic": "gemm_generic.cu",
    "gemm_skinny": "gemm_skinny.cu",
    "gemm_stream": "gemm_stream.cu",
    "gemm_tc5": "gemm_tc5.cu",
    "attention_generic": "attention_generic.cu",
    "attention_flash": "attention_flash.cu",
    "attention_decode_rope": "attention_decode_rope.cu",
    "attention_tc5": "attention_tc5.cu",
    "sampling": "sampling.cu",
    "decode_attention_noalloc": "decode_attention_noalloc.cu",
    "prompt_exec": "prompt_exec.cu",
}
HEADERS = ["common.cuh", "entry_points.h"]
# further files a library's source includes (hashed into its key)
EXTRA_DEPS: Dict[str, List[str]] = {
    "decode_attention_noalloc": ["attention_flash.cu", "decode_attention_noalloc.h"],
}

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()
_dir_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def _log(msg: str) -> None:
    print(f"[qwen_decoder_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("QD_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
                 shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (looked at $QD_NVCC, $CUDA_HOME/bin, PATH, /usr/local/cuda/bin); "
                     "the CUDA kernels cannot be built and there is no fallback")


_nvcc_version_cache: List[str] = []


def _nvcc_version(nvcc: str) -> str:
    if not _nvcc_version_cache:
        out = subprocess.run([nvcc, "--version"], capture_output=True, text=True).stdout
        _nvcc_version_cache.append(out.strip().splitlines()[-1] if out.strip() else "unknown")
    return _nvcc_version_cache[0]


_build_dir_cache: List[str] = []


def _build_dir() -> str:
    with _dir_lock:
        if _build_dir_cache:
            return _build_dir_cache[0]
        cand = os.environ.get("QD_BUILD_DIR") or os.path.join(CSRC, "_build")
        try:
            os.makedirs(cand, exist_ok=True)
            fd, probe = tempfile.mkstemp(prefix=".w", dir=cand)
            os.close(fd)
            os.unlink(probe)
            d = cand
        except OSError:
            d = os.path.join(tempfile.gettempdir(), f"qwen_decoder_b200-build-{os.getuid()}")
            os.makedirs(d, exist_ok=True)
        _build_dir_cache.append(d)
        return d


def _key(name: str, nvcc: str) -> str:
    h = hashlib.sha256()
    for f in [LIBRARIES[name]] + HEADERS + EXTRA_DEPS.get(name, []):
        with open(os.path.join(CSRC, f), "rb") as fh:
            h.update(f.encode() + b"\0" + fh.read() + b"\0")
    h.update(" ".join(NVCC_FLAGS).encode())
    h.update(_nvcc_version(nvcc).encode())
    return h.hexdigest()[:16]


def library_path(name: str) -> str:
    nvcc = find_nvcc()
    return os.path.join(_build_dir(), f"libqd_{name}-{_key(name, nvcc)}.so")


def build_library(name: str, verbose: bool = True, extra_flags=()) -> str:
    """Compile library ``name`` if its file is not there yet; return the path."""
    if name not in LIBRARIES:
        raise BuildError(f"unknown kernel library {name!r}")
    nvcc = find_nvcc()
    path = library_path(name)
    if os.path.isfile(path):
        return path
    src = os.path.join(CSRC, LIBRARIES[name])
    tmp = f"{path}.tmp{os.getpid()}"
    cmd = [nvcc] + NVCC_FLAGS + list(extra_flags) + ["-I", CSRC, "-o", tmp, src]
    if verbose:
        _log(f"compiling {LIBRARIES[name]} for sm_100a (first use) ...")
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    out_chunks: List[str] = []
    reader = threading.Thread(target=lambda: out_chunks.append(proc.stdout.read()), daemon=True)
    reader.start()
    while True:
        try:
            proc.wait(timeout=10)
            break
        except subprocess.TimeoutExpired:
            if verbose:
                _log(f"  still compiling {LIBRARIES[name]} ({time.time() - t0:.0f} s)")
    reader.join()
    out = "".join(out_chunks)
    if proc.returncode != 0:
        try:
            os.unlink(tmp)
        except OSError:
            pass
        raise BuildError(f"nvcc failed on {LIBRARIES[name]} (exit {proc.returncode}):\n{out}")
    os.replace(tmp, path)
    # builds of older sources of this library are of no use any more (a process that still has one mapped keeps it)
    prefix = f"libqd_{name}-"
    for f in os.listdir(os.path.dirname(path)):
        if f.startswith(prefix) and f.endswith(".so") and f != os.path.basename(path):
            try:
                os.unlink(os.path.join(os.path.dirname(path), f))
            except OSError:
                pass
    if verbose:
        _log(f"  built {os.path.basename(path)} in {time.time() - t0:.1f} s")
    return path


def library(name: str) -> ctypes.CDLL:
    """The loaded library ``name`` (built first if needed)."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = build_library(name)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise BuildError(f"cannot load {path}: {e}") from None
            _loaded[name] = lib
        return lib


def build_all(verbose: bool = True, jobs: int = 0) -> Dict[str, str]:
    """Compile every library (in parallel); returns name -> path."""
    from concurrent.futures import ThreadPoolExecutor
    names = list(LIBRARIES)
    jobs = jobs or min(len(names), os.cpu_count() or 1)
    with ThreadPoolExecutor(max_workers=jobs) as ex:
        paths = list(ex.map(lambda n: build_library(n, verbose), names))
    return dict(zip(names, paths))


if __name__ == "__main__":
    for n, p in build_all().items():
        print(n, p)


def loaded(name: str) -> bool:
    """Whether the library ``name`` has been loaded in this process (no build, no load)."""
    return name in _loaded

