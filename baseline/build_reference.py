#!/usr/bin/env python3
"""Compiles the reference engine's own benchmark program, unmodified, into baseline/_ref/.

    python baseline/build_reference.py /path/to/oracle-engine        (or the path in $ORACLE_REFERENCE_SRC)

The reference is a C++17 CPU program without a Python package, so there is nothing for pip
to install; its Makefile builds `oracle_bench` from benchmark/bench_engine.cpp and the
engine sources with `-std=c++17 -O3 -DNDEBUG -mavx2 -mfma -march=native -fopenmp`.  This
script runs the same compile line on a copy of the sources (the source tree may be
read-only), without `-march=native` because the binary is built on one machine and run on
another.  `bench.py --impl reference` runs the binary; baseline/_ref/ is not committed.
"""
from __future__ import annotations

import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
ENGINE_SRC = ["core/engine.cpp", "core/model.cpp", "core/tokenizer.cpp", "core/sampler.cpp", "core/ops.cpp",
              "core/gguf_parser.cpp", "core/platform.cpp", "core/machine_profile.cpp", "bug/logger.cpp"]
ARCH = ["-mavx2", "-mfma"]
OMP = ["-fopenmp"]


def build(source: Path) -> Path:
    cxx = shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        raise RuntimeError("no C++ compiler found")
    if not (source / "benchmark" / "bench_engine.cpp").is_file():
        raise RuntimeError(f"{source} does not hold the reference's sources")
    OUT.mkdir(parents=True, exist_ok=True)
    version = subprocess.run([cxx, "--version"], capture_output=True, text=True).stdout.splitlines()[0]
    with tempfile.TemporaryDirectory() as tmp:
        tree = Path(tmp) / "src"
        shutil.copytree(source, tree, ignore=shutil.ignore_patterns("*.png", "*.svg", ".git"))
        cmd = [cxx, "-std=c++17", "-O3", "-DNDEBUG", *ARCH, *OMP, "-I.",
               f'-DBENCH_COMPILER="{version}"', f'-DBENCH_CXX_FLAGS="{" ".join(ARCH + OMP)}"',
               "benchmark/bench_engine.cpp", *ENGINE_SRC, "-o", str(OUT / "oracle_bench"), "-ldl", "-lpthread"]
        subprocess.run(cmd, cwd=tree, check=True)
    (OUT / "BUILD.txt").write_text(f"oracle_bench built from {source} with: {version}; flags {' '.join(ARCH + OMP)} -O3\n")
    return OUT / "oracle_bench"


if __name__ == "__main__":
    import os
    where = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("ORACLE_REFERENCE_SRC")
    if not where:
        sys.exit(__doc__)
    print(build(Path(where)))
