"""Compile the CUDA sources for sm_100a with nvcc, on first use, into shared libraries.

Each source (plus its -D definitions) is one *unit*; its library is named after a hash of
the source text, of the headers beside it and of the flags, so that a changed source is rebuilt
and an unchanged one is loaded as it is.  Libraries go to ``kernels/_build`` inside the
package, or to a per-user folder under the temporary directory when the package is
read-only.  Only what is asked for is compiled: a model compiles the attention unit of
its own head size, not every size.  While nvcc runs, a line is printed now and then.
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
from concurrent.futures import ThreadPoolExecutor

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-lineinfo", "-std=c++17", "--shared", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden"]

_lock = threading.Lock()
_loaded: dict = {}
#: called with every library right after it is loaded (the bindings register their status words)
on_load: list = []


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[tinyserve_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("TINYSERVE_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 shutil.which("nvcc")):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc was not found (looked at $TINYSERVE_NVCC, $CUDA_HOME/bin, "
                     "/usr/local/cuda/bin and PATH); the CUDA kernels cannot be built")


_build_dir = None


def build_dir() -> str:
    """Where libraries go: ``kernels/_build`` inside the package (or $TINYSERVE_BUILD_DIR), or a
    per-user folder under the temporary directory when that cannot be written.  Decided once per
    process."""
    global _build_dir
    with _lock:
        if _build_dir is not None:
            return _build_dir
        env = os.environ.get("TINYSERVE_BUILD_DIR")
        here = env or os.path.join(os.path.dirname(os.path.abspath(__file__)), "_build")
        try:
            os.makedirs(here, exist_ok=True)
            probe = os.path.join(here, f".w{os.getpid()}.{threading.get_ident()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            _build_dir = here
        except OSError:
            alt = os.path.join(tempfile.gettempdir(), f"tinyserve_b200_build_{os.getuid()}")
            os.makedirs(alt, exist_ok=True)
            _build_dir = alt
        return _build_dir


def unit_path(source: str, defines: dict) -> tuple:
    src = os.path.join(CSRC, source)
    h = hashlib.sha1()
    headers = sorted(f for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))
    for path in [src] + [os.path.join(CSRC, f) for f in headers]:
        with open(path, "rb") as fh:
            h.update(fh.read())
    flags = [f"-D{k}={v}" for k, v in sorted(defines.items())]
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + flags).encode())
    stem = os.path.splitext(source)[0] + "".join(f"_{k.lower()}{v}" for k, v in sorted(defines.items()))
    return os.path.join(build_dir(), f"lib{stem}_{h.hexdigest()[:12]}.so"), src, flags


def compile_unit(source: str, defines: dict | None = None) -> str:
    """Build one unit if its library is not there yet; returns the library's path."""
    defines = dict(defines or {})
    if os.environ.get("TINYSERVE_TIMELINE", "0") == "1":
        defines["TS_TIMELINE"] = 1         # the build that records when every block starts and waits
    out, src, flags = unit_path(source, defines)
    if os.path.isfile(out):
        return out
    nvcc = find_nvcc()
    tmp = f"{out}.{os.getpid()}.{threading.get_ident()}.tmp"
    cmd = [nvcc] + ARCH_FLAGS + NVCC_FLAGS + flags + ["-I", CSRC, "-o", tmp, src]
    label = os.path.basename(out)
    _say(f"compiling {label} for sm_100a ...")
    start = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def heartbeat():
        while not done.wait(10.0):
            _say(f"  still compiling {label} ({time.time() - start:.0f} s)")

    beat = threading.Thread(target=heartbeat, daemon=True)
    beat.start()
    try:
        log, _ = proc.communicate()
    finally:
        done.set()
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise BuildError(f"nvcc failed on {source}:\n{log}")
    os.replace(tmp, out)
    _say(f"built {label} in {time.time() - start:.1f} s")
    return out


def load_unit(source: str, defines: dict | None = None) -> ctypes.CDLL:
    key = (source, tuple(sorted((defines or {}).items())))
    with _lock:
        if key in _loaded:
            return _loaded[key]
    path = compile_unit(source, defines)
    lib = ctypes.CDLL(path)
    lib.ts_last_error.restype = ctypes.c_char_p
    for hook in on_load:
        hook(lib)
    with _lock:
        _loaded[key] = lib
    return lib


def loaded_units() -> list:
    with _lock:
        return list(_loaded.values())


def compile_many(units) -> list:
    """Build several (source, defines) units side by side."""
    units = list(units)
    with ThreadPoolExecutor(max_workers=min(len(units), os.cpu_count() or 1) or 1) as pool:
        return list(pool.map(lambda u: compile_unit(*u), units))
