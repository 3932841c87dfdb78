"""Compiling and loading the CUDA kernel libraries.

Each library is a few ``.cu`` files under ``infurnace_b200/csrc`` compiled by ``nvcc`` for
sm_100a into one shared object with plain C entry points, loaded with ``ctypes``.  The
object's file name carries a hash of its sources and flags, so an edited source is
rebuilt and a stale object is never loaded.  Objects live in ``infurnace_b200/_build``
(or, if that folder cannot be written, in a per-user folder under the system's temporary
directory).  A library is compiled at its first use; while the compiler runs, a line is
printed every few seconds.
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
from typing import Dict, List, Optional, Sequence

from ..errors import KernelError

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-lineinfo", "-std=c++17", "-shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
              "--threads", "4"]      # the sources of a library are compiled side by side

# library name -> (sources, extra flags); sources are file names under csrc, or absolute paths (register_library)
LIBRARIES: Dict[str, tuple] = {
    "core": (["elementwise.cu", "linear_simt.cu", "attention_simt.cu", "linear_skinny.cu", "linear_gemv.cu"], []),
    "linear_tcgen05": (["linear_tcgen05.cu"], []),
    # the few-rows product with its scratch inside the library, for callers that must not allocate
    "linear_skinny_static": (["linear_skinny_static.cu"], []),
    "attention_tc": (["attention_tc.cu"], []),            # head size 128
    # compiled once per head size: defines={"HEAD_DIM": d}
    "attention_mma": (["attention_mma.cu"], []),
}

# what the build check compiles beside "core": the head size of the Qwen3 checkpoints and those of
# the tiny test models; any other multiple of 16 up to 256 is compiled when a model first needs it
DEFAULT_VARIANTS = [("attention_mma", {"HEAD_DIM": d}) for d in (128, 16, 32, 48)]

def register_library(name: str, sources: Sequence[str], flags: Sequence[str] = (), *, replace: bool = False) -> None:
    """Make a library of CUDA sources from outside the package known to :func:`load_library`, so that a
    part defined elsewhere brings its own kernels: ``sources`` are paths of ``.cu`` files (relative paths
    are taken from the caller's working directory), which may include the package's headers (``common.cuh``)
    by name.  The part then calls ``load_library(name)``, declares the argument types of its entry points on the
    returned ``ctypes.CDLL`` and launches on ``torch.cuda.current_stream().cuda_stream``."""
    if name in LIBRARIES and not replace:
        raise KernelError(f"a kernel library named {name!r} is already registered")
    paths = [os.path.abspath(s) for s in sources]
    for p in paths:
        if not os.path.exists(p):
            raise KernelError(f"kernel source {p} does not exist")
    LIBRARIES[name] = (paths, list(flags))
    for key in [k for k in _loaded if k.startswith(name + "[")]:
        del _loaded[key]


_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()
_dir_lock = threading.Lock()


def _say(progress, msg):
    if progress is not None:
        progress(msg)
    else:
        print(f"[infurnace_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("INFURNACE_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")):
        if cand and os.path.exists(cand):
            return cand
    raise KernelError("nvcc was not found (PATH, CUDA_HOME, /usr/local/cuda): the CUDA kernels cannot be compiled")


_build_dir: Optional[str] = None


def build_dir() -> str:
    global _build_dir
    with _dir_lock:
        if _build_dir is None:
            d = os.path.join(os.path.dirname(CSRC), "_build")
            try:
                os.makedirs(d, exist_ok=True)
                fd, probe = tempfile.mkstemp(dir=d)
                os.close(fd)
                os.remove(probe)
            except OSError:
                d = os.path.join(tempfile.gettempdir(), f"infurnace_b200-build-{os.getuid()}")
                os.makedirs(d, exist_ok=True)
            _build_dir = d
        return _build_dir


def _source_path(name: str, beside: Optional[str] = None) -> Optional[str]:
    """Where a source or a quoted include is: an absolute path, a file beside the including file, or under csrc."""
    for cand in ([name] if os.path.isabs(name) else
                 ([os.path.join(os.path.dirname(beside), name)] if beside else []) + [os.path.join(CSRC, name)]):
        if os.path.exists(cand):
            return cand
    return None


def _closure(sources: Sequence[str]) -> List[str]:
    """The paths of the sources and of every file that they include with quotes, directly or not."""
    import re
    seen, todo = [], [(s, None) for s in sources]
    while todo:
        name, beside = todo.pop(0)
        path = _source_path(name, beside)
        if path is None or path in seen:
            continue
        seen.append(path)
        with open(path, "r", encoding="utf-8") as f:
            todo.extend((inc, path) for inc in re.findall(r'^\s*#\s*include\s*"([^"]+)"', f.read(), flags=re.M))
    return seen


def _hash(sources: Sequence[str], flags: Sequence[str]) -> str:
    h = hashlib.sha256()
    for path in _closure(sources):
        with open(path, "rb") as f:
            h.update(os.path.basename(path).encode() + b"\0" + f.read())
    h.update(" ".join(list(ARCH_FLAGS) + list(BASE_FLAGS) + list(flags)).encode())
    return h.hexdigest()[:16]


def library_path(name: str, defines: Optional[Dict[str, object]] = None) -> str:
    sources, flags = LIBRARIES[name]
    flags = list(flags) + [f"-D{k}={v}" for k, v in sorted((defines or {}).items())]
    tag = "".join(f"_{k.lower()}{v}" for k, v in sorted((defines or {}).items()))
    return os.path.join(build_dir(), f"libifb_{name}{tag}-{_hash(sources, flags)}.so")


def compile_library(name: str, defines: Optional[Dict[str, object]] = None, progress=None) -> str:
    """Compile if the object for the current sources is absent.  Returns its path."""
    path = library_path(name, defines)
    if os.path.exists(path):
        return path
    sources, flags = LIBRARIES[name]
    flags = list(flags) + [f"-D{k}={v}" for k, v in sorted((defines or {}).items())]
    tmp = f"{path}.{os.getpid()}.tmp"
    cmd = [find_nvcc(), *ARCH_FLAGS, *BASE_FLAGS, *flags, "-I", CSRC, "-o", tmp,
           *[_source_path(s) or os.path.join(CSRC, s) for s in sources]]
    label = os.path.basename(path)
    _say(progress, f"compiling {label} ({len(sources)} source files) with nvcc ...")
    t0 = time.monotonic()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    out: List[str] = []
    reader = threading.Thread(target=lambda: out.append(proc.stdout.read()), daemon=True)
    reader.start()
    while True:
        try:
            proc.wait(timeout=10)
            break
        except subprocess.TimeoutExpired:
            _say(progress, f"still compiling {label} ({time.monotonic() - t0:.0f} s)")
    reader.join()
    if proc.returncode != 0:
        try:
            os.remove(tmp)
        except OSError:
            pass
        raise KernelError(f"nvcc failed on {label}:\n{''.join(out)[-4000:]}")
    os.replace(tmp, path)
    _say(progress, f"compiled {label} in {time.monotonic() - t0:.1f} s")
    return path


def load_library(name: str, defines: Optional[Dict[str, object]] = None, progress=None) -> ctypes.CDLL:
    key = name + repr(sorted((defines or {}).items()))       # "name[...]"
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            path = compile_library(name, defines, progress)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelError(f"cannot load {path}: {e}") from None
            _loaded[key] = lib
        return lib


def build_all(progress=None) -> List[str]:
    """Compile every library (used by the build check; needs no GPU)."""
    from concurrent.futures import ThreadPoolExecutor
    jobs = [("core", None), ("linear_tcgen05", None), ("linear_skinny_static", None), ("attention_tc", None)] + DEFAULT_VARIANTS
    with ThreadPoolExecutor(max_workers=4) as pool:
        built = list(pool.map(lambda j: compile_library(j[0], j[1], progress), jobs))
    # objects of older sources are never loaded (their names carry another hash); take them out of the folder
    keep = {os.path.basename(p) for p in built}
    for name in os.listdir(build_dir()):
        if name.startswith("libifb_") and name.endswith(".so") and name not in keep:
            try:
                os.remove(os.path.join(build_dir(), name))
            except OSError:
                pass
    return built
