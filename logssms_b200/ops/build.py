"""Compiling and loading the CUDA kernel libraries.

Each `csrc/<name>.cu` becomes one shared library, compiled for sm_100a with nvcc
the first time something asks for it and kept under `csrc/_build/` (or a
per-user temporary folder when the package folder cannot be written).  The
library's file name carries a hash of its sources and flags, so an edit never
loads a stale binary.  There is no fallback: without nvcc or without the source
the call raises.

A library is named by the bare name of a source in the package's `csrc/`, or by
the path of a `.cu` file anywhere else: a part that lives outside the package
lists the path of its own kernels in its `kernels` attribute and they are built
and loaded the same way (with the package's `include/` and the file's own
folder on the include path).
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
INCLUDE = os.path.join(CSRC, "include")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-shared",
]


def package_libraries() -> tuple[str, ...]:
    """Names of all kernel sources of the package itself."""
    return tuple(sorted(f[:-3] for f in os.listdir(CSRC) if f.endswith(".cu")))


def all_libraries() -> tuple[str, ...]:
    """Every library anything registered may ask for: the package's own sources and what the parts in the
    registries name in their `kernels` (a part outside the package may name `.cu` files of its own)."""
    from .. import registry
    names = list(package_libraries())
    for reg in (registry.MIXERS, registry.FEED_FORWARDS, registry.NORMS, registry.POSITION_ENCODINGS, registry.BLOCKS):
        for key in reg.names():
            names.extend(getattr(reg.get(key), "kernels", ()))
    return tuple(dict.fromkeys(names))


def source_path(name: str) -> str:
    """The `.cu` file behind a library name: `name` itself if it is a path, else `csrc/<name>.cu`."""
    src = name if (os.sep in name or name.endswith(".cu")) else os.path.join(CSRC, f"{name}.cu")
    if not os.path.isfile(src):
        raise KernelBuildError(f"kernel source {src} is missing")
    return os.path.abspath(src)


def _stem(name: str) -> str:
    return os.path.splitext(os.path.basename(name))[0]


_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.RLock()


class KernelBuildError(RuntimeError):
    pass


def _log(msg: str) -> None:
    print(f"[logssms_b200] {msg}", file=sys.stderr, flush=True)


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise KernelBuildError("nvcc not found: the CUDA kernels of logssms_b200 cannot be built "
                           "(looked at $NVCC, PATH and /usr/local/cuda/bin/nvcc)")


_build_dir_cache: str | None = None


def _build_dir() -> str:
    global _build_dir_cache
    if _build_dir_cache is None:
        with _lock:
            if _build_dir_cache is None:
                _build_dir_cache = _find_build_dir()
    return _build_dir_cache


def _find_build_dir() -> str:
    override = os.environ.get("LOGSSMS_B200_BUILD_DIR")
    candidates = [override] if override else []
    candidates.append(os.path.join(CSRC, "_build"))
    candidates.append(os.path.join(tempfile.gettempdir(), f"logssms_b200_build_{os.getuid()}"))
    for d in candidates:
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".probe{os.getpid()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return d
        except OSError:
            continue
    raise KernelBuildError(f"no writable folder for built kernels among {candidates}")


def _digest(name: str) -> str:
    h = hashlib.sha1()
    h.update(" ".join(NVCC_FLAGS).encode())
    src = source_path(name)
    paths = [src]
    for root, _, files in sorted(os.walk(INCLUDE)):
        paths += [os.path.join(root, f) for f in sorted(files)]
    for p in paths:
        with open(p, "rb") as f:
            h.update((p[len(CSRC):] if p.startswith(CSRC) else p).encode())
            h.update(f.read())
    return h.hexdigest()[:12]


def library_path(name: str) -> str:
    return os.path.join(_build_dir(), f"lb200_{_stem(name)}-{_digest(name)}.so")


def build(name: str, verbose: bool = True) -> str:
    """Compile the library's source if its library is not there yet; return the path."""
    src = source_path(name)
    out = library_path(name)
    if os.path.isfile(out):
        return out
    tmp = f"{out}.{os.getpid()}.{threading.get_ident()}.tmp"
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", INCLUDE, "-I", os.path.dirname(src), "-o", tmp, src]
    name = _stem(name)
    if verbose:
        _log(f"compiling {name}.cu for sm_100a ...")
    start = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                            env={**os.environ, "TMPDIR": os.path.dirname(out)})
    while True:
        try:
            output, _ = proc.communicate(timeout=15)
            break
        except subprocess.TimeoutExpired:
            if verbose:
                _log(f"  still compiling {name}.cu ({time.time() - start:.0f} s)")
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise KernelBuildError(f"nvcc failed on {name}.cu:\n{output}")
    os.replace(tmp, out)
    # builds of earlier versions of this source are of no use any more
    prefix = f"lb200_{name}-"
    for f in os.listdir(os.path.dirname(out)):
        if f.startswith(prefix) and f.endswith(".so") and f != os.path.basename(out):
            try:
                os.remove(os.path.join(os.path.dirname(out), f))
            except OSError:
                pass
    if verbose:
        _log(f"built {os.path.basename(out)} in {time.time() - start:.1f} s")
    return out


def build_many(names, verbose: bool = True) -> None:
    """Compile several libraries side by side (used at engine start and by `__graft_entry__.build`)."""
    names = [n for n in dict.fromkeys(names) if n not in _loaded]
    todo = [n for n in names if not os.path.isfile(library_path(n))]
    if not todo:
        return
    with ThreadPoolExecutor(max_workers=min(8, len(todo))) as pool:
        list(pool.map(lambda n: build(n, verbose), todo))


def load(name: str) -> ctypes.CDLL:
    """The loaded library of a kernel source (a name in `csrc/`, or a path), building it first if needed."""
    lib = _loaded.get(name)
    if lib is not None:
        return lib
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            lib = ctypes.CDLL(build(name))
            _loaded[name] = lib
    return lib
