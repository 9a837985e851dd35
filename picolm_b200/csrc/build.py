"""Compiles the CUDA sources of this folder for sm_100a with nvcc and loads them
through ctypes.  Nothing is compiled at import: a kernel library is built the
first time an op from it is called (or all at once by `build_all`), and only
when its `.so` is missing or older than its sources.

The libraries have a plain C ABI (raw device pointers and a stream handle), so
they do not include the PyTorch headers and compile in seconds.  They are kept
in `_build/` beside the sources; if that folder cannot be written (a read-only
install), in a per-user folder under the system's temporary directory.
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
from typing import Dict, Iterable, List, Optional, Sequence

CSRC = os.path.dirname(os.path.abspath(__file__))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC",
]

# library name -> sources (relative to this folder)
LIBRARIES: Dict[str, List[str]] = {
    "elementwise": ["elementwise.cu"],
    "gemm_simt": ["gemm_simt.cu"],
    "gemm_tc": ["gemm_tc.cu"],
    "gemm_tc_skinny": ["gemm_tc_skinny.cu"],
    "gemm_tc_wide": ["gemm_tc_wide.cu"],
    "decode_chain": ["decode_chain.cu"],
    "attention_simt": ["attention_simt.cu"],
    "attention_mma": ["attention_mma.cu"],          # one variant per head size: "attention_mma@hd64" with -DPLM_HD=64
    "attention_tc": ["attention_tc.cu"],            # likewise, head sizes 64 and 128
    "sampling": ["sampling.cu"],
}
HEADERS = ["common.cuh", "tc_common.cuh", "gemm_tc_static.h"]

# Libraries that are specialised at compile time.  At run time only the variant a
# model needs is built (`attention_variant`); the build check builds these.
VARIANTS: Dict[str, Dict[str, List[str]]] = {
    "attention_mma": {f"hd{hd}": [f"-DPLM_HD={hd}"] for hd in (64, 128)},
    "attention_tc": {f"hd{hd}": [f"-DPLM_HD={hd}"] for hd in (64, 128)},
}


# Variants of libraries that also exist plain: (name, flags).  The build check builds them too.
MORE_BUILDS: List = [("gemm_tc_wide@stream", ["-DPLM_WIDE_STREAM"])]


def attention_variant(head_dim: int, family: str = "attention_mma"):
    """(library name, extra flags) of a tensor-core attention library for a head size."""
    return f"{family}@hd{head_dim}", [f"-DPLM_HD={head_dim}"]

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[picolm_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    cands = []
    for var in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(var):
            cands.append(os.path.join(os.environ[var], "bin", "nvcc"))
    which = shutil.which("nvcc")
    if which:
        cands.append(which)
    cands.append("/usr/local/cuda/bin/nvcc")
    for c in cands:
        if os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise BuildError("nvcc was not found (looked at $CUDA_HOME/bin, $PATH and /usr/local/cuda/bin); "
                     "the CUDA kernels of picolm_b200 cannot be built")


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f"probe-{os.getpid()}.tmp")
        with open(probe, "w"):
            pass
        try:
            os.remove(probe)
        except OSError:
            pass                                             # it could be created: that is what counts
        return True
    except OSError as e:
        print(f"[picolm_b200] {path} cannot be written ({e}); trying the next folder", file=sys.stderr, flush=True)
        return False


_build_dir: Optional[str] = None


def build_dir() -> str:
    global _build_dir
    if _build_dir is None:
        cands = []
        if os.environ.get("PICOLM_B200_BUILD_DIR"):
            cands.append(os.environ["PICOLM_B200_BUILD_DIR"])
        cands.append(os.path.join(CSRC, "_build"))
        cands.append(os.path.join(tempfile.gettempdir(), f"picolm_b200-build-{os.getuid()}"))
        for c in cands:
            if _writable_dir(c):
                _build_dir = c
                break
        else:
            raise BuildError("no writable folder for the compiled kernels: tried " + ", ".join(cands))
    return _build_dir


def _stamp(sources: Sequence[str], extra_flags: Sequence[str]) -> str:
    h = hashlib.sha256()
    for rel in list(sources) + HEADERS:
        with open(os.path.join(CSRC, rel), "rb") as f:
            h.update(rel.encode())
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS + list(extra_flags)).encode())
    return h.hexdigest()[:16]


def library_path(name: str, extra_flags: Sequence[str] = ()) -> str:
    sources = LIBRARIES[name.split("@")[0]]
    return os.path.join(build_dir(), f"libplm_{name.replace('@', '_')}-{_stamp(sources, extra_flags)}.so")


def compile_library(name: str, extra_flags: Sequence[str] = (), verbose: bool = False) -> str:
    """Build one library if it is stale; returns the path of its `.so`.
    `name` may carry a variant after '@' (e.g. "attention@hd64"), built from the
    same sources with `extra_flags`."""
    base = name.split("@")[0]
    if base not in LIBRARIES:
        raise BuildError(f"unknown kernel library {name!r}")
    out = library_path(name, extra_flags)
    if os.path.exists(out):
        return out
    nvcc = find_nvcc()
    srcs = [os.path.join(CSRC, s) for s in LIBRARIES[base]]
    tmp = f"{out}.{os.getpid()}.tmp"
    cmd = [nvcc] + NVCC_FLAGS + list(extra_flags) + ["-I", CSRC, "-o", tmp] + srcs
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    _say(f"compiling {name} for sm_100a (first use) ...")
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, cwd=build_dir())
    done = threading.Event()

    def heartbeat():
        while not done.wait(10.0):
            _say(f"  still compiling {name} ({time.time() - t0:.0f} s)")

    hb = threading.Thread(target=heartbeat, daemon=True)
    hb.start()
    log, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise BuildError(f"nvcc failed on {name}:\n{' '.join(cmd)}\n{log}")
    os.replace(tmp, out)
    prefix = f"libplm_{name.replace('@', '_')}-"
    for old in os.listdir(build_dir()):                  # builds of older sources
        if old.startswith(prefix) and old.endswith(".so") and os.path.join(build_dir(), old) != out:
            try:
                os.remove(os.path.join(build_dir(), old))
            except OSError:
                pass
    _say(f"compiled {name} in {time.time() - t0:.1f} s -> {out}")
    if verbose and log:
        print(log, file=sys.stderr)
    return out


def load_library(name: str, extra_flags: Sequence[str] = ()) -> ctypes.CDLL:
    """The ctypes handle of a kernel library, compiled first if need be."""
    key = name + "|" + " ".join(extra_flags)
    lib = _loaded.get(key)
    if lib is not None:
        return lib
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            path = compile_library(name, extra_flags)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise BuildError(f"the compiled kernel library {path} cannot be loaded: {e}") from None
            _loaded[key] = lib
    return lib


def build_all(names: Optional[Iterable[str]] = None, jobs: int = 4, verbose: bool = False) -> List[str]:
    """Compile every library (in parallel); used by the build check."""
    from concurrent.futures import ThreadPoolExecutor
    if names is None:
        names = [n for n in LIBRARIES if n not in VARIANTS]
        for base, variants in VARIANTS.items():
            names += [f"{base}@{v}" for v in variants]
        names += [n for n, _ in MORE_BUILDS]
    names = list(names)
    more = dict(MORE_BUILDS)

    def one(n):
        base, _, variant = n.partition("@")
        flags = more[n] if n in more else VARIANTS[base][variant] if variant else ()
        return compile_library(n, flags, verbose=verbose)

    with ThreadPoolExecutor(max_workers=jobs) as pool:
        return list(pool.map(one, names))
