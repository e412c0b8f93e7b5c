"""Compiles the CUDA sources of this folder for sm_100a with nvcc and loads them (ctypes).

Each `.cu` file becomes one shared library, built the first time one of its kernels is
needed and kept under `_build/` beside the sources (or, if that folder cannot be
written, under the system's temporary folder), named by a hash of the sources and flags
so that an edited source is rebuilt.  Only the libraries a model uses are built: the
32-bit path never compiles the tensor-core kernels, and the other way round.

There is no fallback: if nvcc is missing or a source does not compile, the error is
raised to the caller.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import tempfile
import threading
import time
from pathlib import Path

from ..utils.log import log

CSRC = Path(__file__).resolve().parent
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=default"]

# library name -> (source file, extra link flags)
LIBRARIES = {
    "elementwise": ("elementwise.cu", []),
    "gemm_simple": ("gemm_simple.cu", []),
    "attention": ("attention.cu", []),
    "sampling": ("sampling.cu", []),
    "gemm_tc": ("gemm_tcgen05.cu", []),
    "gemm_pair": ("gemm_tcgen05_pair.cu", []),
    "gemm_skinny": ("gemm_skinny.cu", []),
    "attention_tc": ("attention_mma.cu", []),
    "attention_tc5": ("attention_tcgen05.cu", []),
}

_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).is_file():
            return cand
    raise BuildError("nvcc not found (looked at $NVCC, PATH and /usr/local/cuda/bin); "
                     "the CUDA kernels of oracle_engine_b200 cannot be built")


_dir_lock = threading.Lock()
_dir_cache: list[Path] = []


def _build_dir() -> Path:
    with _dir_lock:
        if _dir_cache:
            return _dir_cache[0]
        d = CSRC / "_build"
        try:
            d.mkdir(exist_ok=True)
            probe = d / f".w{os.getpid()}"
            probe.write_bytes(b"")
            probe.unlink()
        except OSError:
            d = Path(tempfile.gettempdir()) / f"oracle_engine_b200_build_{os.getuid()}"
            d.mkdir(parents=True, exist_ok=True)
        _dir_cache.append(d)
        return d


def _digest(source: Path, flags: list[str]) -> str:
    h = hashlib.sha1()
    for p in [source] + sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + flags).encode())
    return h.hexdigest()[:16]


def _define_flags(defines) -> tuple[str, list[str]]:
    """(tag for the file name, nvcc flags) of a dict of -D macros."""
    if not defines:
        return "", []
    items = sorted(defines.items())
    return "_" + "_".join(f"{k.lower()}{v}" for k, v in items), [f"-D{k}={v}" for k, v in items]


def library_path(name: str, defines=None) -> Path:
    src, flags = LIBRARIES[name]
    tag, dflags = _define_flags(defines)
    return _build_dir() / f"liboe_{name}{tag}_{_digest(CSRC / src, flags + dflags)}.so"


def build(name: str, verbose: bool = True, defines=None) -> Path:
    """Builds library `name` (specialised by the -D macros of `defines`) if its .so is not
    there yet; returns the path."""
    src, flags = LIBRARIES[name]
    tag, dflags = _define_flags(defines)
    flags = flags + dflags
    out = library_path(name, defines)
    if out.is_file():
        return out
    cmd = [_nvcc()] + ARCH_FLAGS + NVCC_FLAGS + flags + ["-I", str(CSRC), "-o", None, str(CSRC / src)]
    tmp = out.with_suffix(f".tmp{os.getpid()}.so")
    cmd[cmd.index(None)] = str(tmp)
    t0 = time.time()
    what = src + (f" ({', '.join(dflags)})" if dflags else "")
    if verbose:
        log.info("build", f"compiling {what} for sm_100a ...")
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    while True:
        try:
            output, _ = proc.communicate(timeout=10)
            break
        except subprocess.TimeoutExpired:
            if verbose:
                log.info("build", f"... still compiling {what} ({time.time() - t0:.0f} s)")
    if proc.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise BuildError(f"nvcc failed on {src} (exit {proc.returncode}):\n{' '.join(cmd)}\n{output}")
    os.replace(tmp, out)
    # drop stale builds of the same library
    for old in out.parent.glob(f"liboe_{name}{tag}_*.so"):
        if old != out and len(old.name) == len(out.name):
            old.unlink(missing_ok=True)
    if verbose:
        log.info("build", f"built {out.name} in {time.time() - t0:.1f} s")
    return out


def load(name: str, defines=None) -> ctypes.CDLL:
    """The loaded library `name`, built first if needed."""
    key = name + _define_flags(defines)[0]
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            lib = ctypes.CDLL(str(build(name, defines=defines)))
            _loaded[key] = lib
        return lib


# head sizes the build check compiles the specialised attention for (others are built on demand)
DEFAULT_HEAD_DIMS = (16, 32, 48, 64, 128)


def build_all(names=None, verbose: bool = True) -> list[Path]:
    """Builds every library (in parallel processes of nvcc); used by the build check."""
    names = list(names or [n for n, (src, _) in LIBRARIES.items() if (CSRC / src).is_file()])
    jobs = []
    for n in names:
        if n == "attention_tc":
            jobs.extend((n, {"OE_HD": hd}) for hd in DEFAULT_HEAD_DIMS)
        elif n == "attention_tc5":
            jobs.extend((n, {"OE_HD": hd}) for hd in (64, 128))
        else:
            jobs.append((n, None))
    results: dict[object, object] = {}

    def work(job):
        try:
            results[id(job)] = build(job[0], verbose, job[1])
        except Exception as e:           # noqa: BLE001 - reported below
            results[id(job)] = e

    names = jobs
    threads = [threading.Thread(target=work, args=(n,)) for n in names]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    errors = [f"{j[0]}: {results[id(j)]}" for j in jobs if isinstance(results[id(j)], Exception)]
    if errors:
        raise BuildError("\n".join(errors))
    return [results[id(j)] for j in jobs]
