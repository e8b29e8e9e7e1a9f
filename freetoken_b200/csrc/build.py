"""Compiling and loading the CUDA libraries.

Every ``.cu`` file of this folder becomes one shared library with plain
``extern "C"`` launchers, compiled by ``nvcc`` for sm_100a the first time it is
needed and loaded with :mod:`ctypes`.  A library is looked up by a hash of its
sources and flags, so an edited kernel is rebuilt and a stale binary is never
used.  Nothing here falls back to another implementation: without ``nvcc`` or
with a failed build, :class:`BuildError` is raised.

The reference JIT-compiles its CUDA through ``tvm_ffi.cpp.load_inline`` with
``-std=c++20 -O3 --expt-relaxed-constexpr`` and looks up prebuilt binaries in a
kernel-cache wheel first (python/freetoken/kernel/utils.py:20-42,148-169,232-284).
"""

from __future__ import annotations

import ctypes
import hashlib
import os
import re
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, Iterable, List, Optional

HERE = os.path.dirname(os.path.abspath(__file__))

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
              "-shared"]

# library name -> source file; headers every library depends on
LIBRARIES: Dict[str, str] = {
    "elementwise": "elementwise.cu",
    "gemm_simt": "gemm_simt.cu",
    "attention_simt": "attention_simt.cu",
    "moe_route": "moe_route.cu",
    "sampling": "sampling.cu",
    "skinny_gemm": "skinny_gemm.cu",
    "attention_decode": "attention_decode.cu",
    "attention_decode_tma": "attention_decode_tma.cu",
    "attention_prefill": "attention_prefill.cu",
    "attention_prefill_tc": "attention_prefill_tc.cu",
    "moe_gemm_tc": "moe_gemm_tc.cu",
}
HEADERS: List[str] = ["common.cuh", "mma_utils.cuh", "tcgen05.cuh", "status_codes.h", "sampling_static.h"]
EXTRA_LINK: Dict[str, List[str]] = {}


class BuildError(RuntimeError):
    """A CUDA library could not be built or loaded."""


def register_library(name: str, source: str, link: Optional[List[str]] = None) -> None:
    LIBRARIES[name] = source
    if link:
        EXTRA_LINK[name] = link


def _say(msg: str) -> None:
    print(f"[freetoken_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> Optional[str]:
    for root in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if root:
            cand = os.path.join(root, "bin", "nvcc")
            if os.path.exists(cand):
                return cand
    return shutil.which("nvcc")


def build_dir() -> str:
    """``csrc/_build`` inside the package when it can be written, else a
    per-user folder under the system's temporary directory."""
    override = os.environ.get("FREETOKEN_B200_BUILD_DIR")
    candidates = [override] if override else []
    candidates.append(os.path.join(HERE, "_build"))
    candidates.append(os.path.join(tempfile.gettempdir(), f"freetoken_b200_build_{os.getuid()}"))
    for path in candidates:
        try:
            os.makedirs(path, exist_ok=True)
            probe = os.path.join(path, f".probe_{os.getpid()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return path
        except OSError:
            continue
    raise BuildError("no writable folder for compiled CUDA libraries")


def _digest(name: str) -> str:
    h = hashlib.sha256()
    for rel in [LIBRARIES[name]] + HEADERS:
        with open(os.path.join(HERE, rel), "rb") as f:
            h.update(f.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + EXTRA_LINK.get(name, [])).encode())
    return h.hexdigest()[:16]


def library_path(name: str, folder: Optional[str] = None) -> str:
    return os.path.join(folder or build_dir(), f"libft_{name}_{_digest(name)}.so")


def _compile(name: str, out: str, verbose_ptxas: bool = False) -> None:
    nvcc = find_nvcc()
    if nvcc is None:
        raise BuildError(
            f"CUDA library '{name}' is not built and nvcc was not found "
            "(looked in $CUDA_HOME, /usr/local/cuda and PATH)")
    src = os.path.join(HERE, LIBRARIES[name])
    tmp = f"{out}.{os.getpid()}.{threading.get_ident()}.tmp"
    cmd = [nvcc] + ARCH_FLAGS + NVCC_FLAGS + ["-I", HERE]
    if verbose_ptxas:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", tmp, src] + EXTRA_LINK.get(name, [])
    _say(f"compiling {LIBRARIES[name]} for sm_100a ...")
    start = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    output: List[str] = []
    reader = threading.Thread(target=lambda: output.append(proc.stdout.read()), daemon=True)
    reader.start()
    beat = 0
    while proc.poll() is None:
        time.sleep(0.2)
        if time.time() - start > 10 * (beat + 1):
            beat += 1
            _say(f"still compiling {LIBRARIES[name]} ({int(time.time() - start)} s)")
    reader.join()
    text = "".join(output)
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise BuildError(f"nvcc failed for {LIBRARIES[name]}:\n{text}")
    os.replace(tmp, out)
    if verbose_ptxas:
        _say(text)
    drop_stale(os.path.dirname(out), name, out)
    _say(f"built {os.path.basename(out)} in {time.time() - start:.1f} s")


def drop_stale(folder: str, name: str, keep: str) -> List[str]:
    """Remove older binaries of library ``name`` from ``folder`` (all but ``keep``);
    a library whose name merely starts with ``name`` is someone else's."""
    stale = re.compile(rf"libft_{re.escape(name)}_[0-9a-f]{{16}}\.so$")
    removed = []
    for f in os.listdir(folder):
        if stale.match(f) and os.path.join(folder, f) != keep:
            try:
                os.remove(os.path.join(folder, f))
                removed.append(f)
            except OSError:
                pass
    return removed


_loaded: Dict[str, ctypes.CDLL] = {}
_locks: Dict[str, threading.Lock] = {}
_global_lock = threading.Lock()


def ensure_built(names: Optional[Iterable[str]] = None, verbose_ptxas: bool = False) -> List[str]:
    """Compile whichever of ``names`` (default: all) has no current binary, in
    parallel.  Returns the library paths."""
    names = list(names) if names is not None else list(LIBRARIES)
    folder = build_dir()
    todo = [n for n in names if verbose_ptxas or not os.path.exists(library_path(n, folder))]
    if todo:
        with ThreadPoolExecutor(max_workers=min(len(todo), os.cpu_count() or 4)) as pool:
            list(pool.map(lambda n: _compile(n, library_path(n, folder), verbose_ptxas), todo))
    return [library_path(n, folder) for n in names]


def load(name: str) -> ctypes.CDLL:
    """The loaded library ``name``, compiled first if need be."""
    lib = _loaded.get(name)
    if lib is not None:
        return lib
    with _global_lock:
        lock = _locks.setdefault(name, threading.Lock())
    with lock:
        lib = _loaded.get(name)
        if lib is not None:
            return lib
        if name not in LIBRARIES:
            raise BuildError(f"unknown CUDA library '{name}'")
        path = library_path(name)
        if not os.path.exists(path):
            _compile(name, path)
        try:
            lib = ctypes.CDLL(path)
        except OSError as exc:
            raise BuildError(f"cannot load {path}: {exc}") from exc
        _loaded[name] = lib
        return lib
