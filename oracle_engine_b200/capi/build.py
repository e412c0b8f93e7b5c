"""Builds `liboe.so`, the C API of this library (`oe.h`), with the host compiler.

    python -m oracle_engine_b200.capi.build        # prints the library's path and the flags to link against it

The library lies under `_build/` beside its source, under a fixed name so that C and C++ programs
can link against it; it is rebuilt when the source, the header or the flags change (a digest is kept
beside it).  It links against the Python library of the interpreter that builds it.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

from ..utils.log import log

HERE = Path(__file__).resolve().parent
SOURCES = ("oe_capi.cpp", "oe.h")
CXX_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=default", "-Wall"]


class BuildError(RuntimeError):
    pass


def _python_flags() -> tuple[list[str], list[str]]:
    """(compile flags, link flags) for embedding this interpreter."""
    include = sysconfig.get_paths()["include"]
    libdir = sysconfig.get_config_var("LIBDIR") or ""
    version = sysconfig.get_config_var("LDVERSION") or f"{sys.version_info.major}.{sys.version_info.minor}"
    if not Path(include, "Python.h").is_file():
        raise BuildError(f"Python.h not found under {include}: the C API needs the interpreter's headers")
    link = [f"-lpython{version}", "-ldl"]
    if libdir:
        link = [f"-L{libdir}", f"-Wl,-rpath,{libdir}"] + link
    return [f"-I{include}"], link


def _digest(flags: list[str]) -> str:
    h = hashlib.sha1()
    for name in SOURCES:
        h.update((HERE / name).read_bytes())
    h.update(" ".join(flags).encode())
    return h.hexdigest()


def library_path() -> Path:
    return HERE / "_build" / "liboe.so"


def link_flags() -> list[str]:
    """What a C or C++ program adds to its compiler's command line."""
    d = library_path().parent
    return [f"-I{HERE}", f"-L{d}", f"-Wl,-rpath,{d}", "-loe"]


def build(verbose: bool = True) -> Path:
    cxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
    if not cxx:
        raise BuildError("no C++ compiler found ($CXX, g++, c++)")
    cflags, lflags = _python_flags()
    flags = CXX_FLAGS + cflags + lflags
    out, stamp = library_path(), library_path().with_suffix(".digest")
    digest = _digest(flags)
    if out.is_file() and stamp.is_file() and stamp.read_text() == digest:
        return out
    out.parent.mkdir(exist_ok=True)
    tmp = out.with_suffix(f".tmp{os.getpid()}.so")
    cmd = [cxx] + CXX_FLAGS + cflags + ["-o", str(tmp), str(HERE / "oe_capi.cpp")] + lflags
    if verbose:
        log.info("build", "compiling oe_capi.cpp ...")
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise BuildError(f"the C++ compiler failed on oe_capi.cpp (exit {proc.returncode}):\n{' '.join(cmd)}\n{proc.stdout}")
    os.replace(tmp, out)
    stamp.write_text(digest)
    if verbose:
        log.info("build", f"built {out}")
    return out


if __name__ == "__main__":
    print(build())
    print(" ".join(link_flags()))
