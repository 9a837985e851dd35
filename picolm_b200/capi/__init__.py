"""The C API of the library: `plm.h`, and `libplm.so` built from `plm.c` (a few hundred lines of C that
forward every call to `host.py` inside an interpreter; see the header for why).  `build_library()` compiles
it with the system's C compiler against the running interpreter's libpython; a C program links with
`-lplm` from `library_dir()` and includes `plm.h` from `include_dir()`."""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def include_dir() -> str:
    return HERE


def library_dir() -> str:
    from ..csrc.build import build_dir
    return build_dir()


def library_path() -> str:
    return os.path.join(library_dir(), "libplm.so")


def python_link_flags():
    """What a program that links libplm.so needs for libpython (the directory and the library's name)."""
    libdir = sysconfig.get_config_var("LIBDIR") or "/usr/lib"
    version = sysconfig.get_config_var("LDVERSION") or f"{sys.version_info.major}.{sys.version_info.minor}"
    return [f"-L{libdir}", f"-lpython{version}", f"-Wl,-rpath,{libdir}"]


def build_library(verbose: bool = False) -> str:
    """Compile libplm.so if it is missing or older than its sources; returns its path."""
    out = library_path()
    srcs = [os.path.join(HERE, "plm.c"), os.path.join(HERE, "plm.h")]
    h = hashlib.sha256()
    for src in srcs:
        with open(src, "rb") as f:
            h.update(f.read())
    h.update(sys.executable.encode() + ROOT.encode())
    stamp = out + ".stamp"
    want = h.hexdigest()
    if os.path.exists(out) and os.path.exists(stamp) and open(stamp).read() == want:
        return out
    cc = os.environ.get("CC") or ("/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else "cc")
    cmd = [cc, "-O2", "-std=c11", "-D_GNU_SOURCE", "-shared", "-fPIC", "-Wall", srcs[0], f"-I{HERE}",
           f"-I{sysconfig.get_paths()['include']}", f'-DPLM_DEFAULT_PYTHON="{sys.executable}"',
           f'-DPLM_DEFAULT_ROOT="{ROOT}"', "-o", out + ".tmp"] + python_link_flags() + ["-lpthread"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"building libplm.so failed:\n{' '.join(cmd)}\n{r.stdout}{r.stderr}")
    if verbose and (r.stdout or r.stderr):
        print(r.stdout + r.stderr, file=sys.stderr)
    os.replace(out + ".tmp", out)
    with open(stamp, "w") as f:
        f.write(want)
    return out
