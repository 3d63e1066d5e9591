"""Compile and load the CUDA kernels (sm_100a) as plain shared libraries.

Every ``csrc/<name>.cu`` becomes ``csrc/_build/lib<name>-<hash>.so`` with
``extern "C"`` launchers that take raw device pointers and a stream; Python
calls them through ``ctypes``.  A library is compiled at its first use (so a
run compiles only what its model needs), with a line printed now and then
while the compiler runs.  There is no fallback: if ``nvcc`` is missing or the
compile fails the call raises.
"""
from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from typing import Dict, List, Optional

CSRC_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    "-shared",
]

# the kernel libraries of this package, in csrc/
LIBRARIES = ["rowwise", "gemm_simt", "gemm_skinny", "gemm_stream", "gemm_tc", "shortconv", "qkrope", "attention", "attention_decode", "attention_mma", "attention_tc", "attention_noalloc", "sampling"]


class KernelBuildError(RuntimeError):
    pass


_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.RLock()


def _find_nvcc() -> str:
    cands = []
    for env in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(env):
            cands.append(os.path.join(os.environ[env], "bin", "nvcc"))
    cands.append("/usr/local/cuda/bin/nvcc")
    w = shutil.which("nvcc")
    if w:
        cands.append(w)
    for c in cands:
        if os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise KernelBuildError("nvcc not found (looked in $CUDA_HOME/bin, /usr/local/cuda/bin and PATH); "
                           "the CUDA kernels of kappai_b200 cannot be built and there is no fallback")


def _headers() -> List[str]:
    return sorted(os.path.join(CSRC_DIR, f) for f in os.listdir(CSRC_DIR) if f.endswith((".cuh", ".h")))


def _included_sources(src: str) -> List[str]:
    """``.cu`` files that ``src`` includes by name (a library built on another's kernels)."""
    import re
    with open(src, "r", encoding="utf-8") as f:
        names = re.findall(r'^\s*#include\s+"([^"]+\.cu)"', f.read(), flags=re.M)
    return [os.path.join(CSRC_DIR, n) for n in names if os.path.isfile(os.path.join(CSRC_DIR, n))]


def _digest(src: str, extra_flags: List[str]) -> str:
    h = hashlib.sha256()
    for p in [src] + _included_sources(src) + _headers():
        with open(p, "rb") as f:
            h.update(os.path.basename(p).encode())
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS + extra_flags).encode())
    return h.hexdigest()[:16]


_build_dir: Optional[str] = None


def build_dir() -> str:
    """``$KAPPAI_B200_BUILD_DIR`` if set, else in-tree ``csrc/_build`` when it
    can be written, else a per-user folder under the temp dir."""
    global _build_dir
    if _build_dir is None:
        with _lock:
            if _build_dir is None:
                _build_dir = _pick_build_dir()
    return _build_dir


def _pick_build_dir() -> str:
    env = os.environ.get("KAPPAI_B200_BUILD_DIR")
    cands = [env] if env else []
    cands.append(os.path.join(CSRC_DIR, "_build"))
    cands.append(os.path.join(tempfile.gettempdir(), f"kappai_b200_build_{os.getuid()}"))
    for d in cands:
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".w{os.getpid()}_{threading.get_ident()}")
            with open(probe, "w"):
                pass
            os.unlink(probe)
            return d
        except OSError:
            continue
    raise KernelBuildError("no writable folder for built kernels (set KAPPAI_B200_BUILD_DIR)")


def _stem(name: str, variant: str) -> str:
    return f"lib{name}.{variant}" if variant else f"lib{name}"


def library_path(name: str, extra_flags: Optional[List[str]] = None, variant: str = "") -> str:
    src = os.path.join(CSRC_DIR, name + ".cu")
    if not os.path.isfile(src):
        raise KernelBuildError(f"no kernel source {src}")
    return os.path.join(build_dir(), f"{_stem(name, variant)}-{_digest(src, extra_flags or [])}.so")


def compile_library(name: str, extra_flags: Optional[List[str]] = None, verbose: bool = True,
                    variant: str = "") -> str:
    """Compile ``csrc/<name>.cu`` if its built library is missing; return the path.
    ``variant`` names a second build of the same source with ``extra_flags``
    (its own file beside the ordinary one)."""
    extra_flags = extra_flags or []
    out = library_path(name, extra_flags, variant)
    if os.path.isfile(out):
        return out
    nvcc = _find_nvcc()
    src = os.path.join(CSRC_DIR, name + ".cu")
    lock_path = out + ".lock"
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if os.path.isfile(out):
                return out
            tmp = f"{out}.tmp{os.getpid()}"
            cmd = [nvcc] + NVCC_FLAGS + extra_flags + ["-I", CSRC_DIR, "-o", tmp, src]
            t0 = time.time()
            if verbose:
                print(f"[kappai_b200] compiling {name}.cu for sm_100a ...", file=sys.stderr, flush=True)
            env = dict(os.environ)
            env.setdefault("TMPDIR", tempfile.gettempdir())
            proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env)
            beat = t0
            while True:
                try:
                    outp, _ = proc.communicate(timeout=5)
                    break
                except subprocess.TimeoutExpired:
                    if verbose and time.time() - beat >= 10:
                        beat = time.time()
                        print(f"[kappai_b200]   still compiling {name}.cu ({beat - t0:.0f} s)",
                              file=sys.stderr, flush=True)
            if proc.returncode != 0:
                try:
                    os.unlink(tmp)
                except OSError:
                    pass
                raise KernelBuildError(f"nvcc failed on {name}.cu (exit {proc.returncode}):\n"
                                       + outp.decode("utf-8", "replace"))
            os.replace(tmp, out)
            # libraries of earlier versions of this source are of no use any more (a process that still has
            # one loaded keeps its mapping)
            prefix = _stem(name, variant) + "-"
            for f in os.listdir(os.path.dirname(out)):
                if f.startswith(prefix) and f.endswith(".so") and f != os.path.basename(out):
                    try:
                        os.unlink(os.path.join(os.path.dirname(out), f))
                    except OSError:
                        pass
            if verbose:
                print(f"[kappai_b200] built {os.path.basename(out)} in {time.time() - t0:.1f} s",
                      file=sys.stderr, flush=True)
            return out
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
            try:
                os.unlink(lock_path)
            except OSError:
                pass


TIMELINE = [False]      # ops.timeline.enable(): every library loaded from now on is its build with the trace marks


def load_library(name: str, variant: str = "", extra_flags: Optional[List[str]] = None) -> ctypes.CDLL:
    """The loaded library ``name``; compiled first if need be."""
    key = f"{name}.{variant}" if variant else name
    lib = _loaded.get(key)
    if lib is not None:
        return lib
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            if TIMELINE[0] and not variant and name in LIBRARIES:
                path = compile_library(name, [f"-DKP_TRACE={LIBRARIES.index(name) + 1}"], variant="timeline")
            else:
                path = compile_library(name, extra_flags, variant=variant)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelBuildError(f"cannot load {path}: {e}") from None
            _loaded[key] = lib
    return lib


def is_loaded(name: str) -> bool:
    return name in _loaded


def loaded_libraries() -> dict:
    """Name (``name`` or ``name.variant``) -> loaded library."""
    return dict(_loaded)


def build_all(verbose: bool = True, jobs: int = 4) -> List[str]:
    """Compile every kernel library (used by the build check)."""
    from concurrent.futures import ThreadPoolExecutor

    with ThreadPoolExecutor(max_workers=jobs) as ex:
        return list(ex.map(lambda n: compile_library(n, verbose=verbose), LIBRARIES))
