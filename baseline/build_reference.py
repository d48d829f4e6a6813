"""Build the unmodified reference (llnl/Aluminum) into ``baseline/_ref`` for the reference arm.

The reference needs an MPI at configure time and as its control plane at run time; none is
installed, so ``baseline/mpi_shim`` (a single-node MPI stand-in over Unix sockets) is built first
and handed to CMake's FindMPI through its documented hint variables.  Then the reference's own
CMake project is configured with its NCCL backend, built and installed, and the small C driver
``baseline/ref_driver.cpp`` (the reference's public API behind a C interface for ctypes) is
compiled against the installed headers and library.

    python baseline/build_reference.py [--reference /path/to/Aluminum] [--cpu-only]

Layout produced (all git-ignored):
    baseline/_ref/mpi/{include/mpi.h, lib/libmpi.so}
    baseline/_ref/build/         CMake build tree of the reference
    baseline/_ref/install/       include/Al.hpp, include/aluminum/*, lib*/libAl.so
    baseline/_ref/lib/libref_driver.so
    baseline/_ref/BUILD_INFO.json
``--cpu-only`` builds the reference without CUDA (MPI backend only) into ``baseline/_ref/cpu`` -
used by the CPU test of the MPI stand-in.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_OUT = HERE / "_ref"
CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))


def run(cmd, **kw):
    r = subprocess.run([str(c) for c in cmd], capture_output=True, text=True, **kw)
    if r.returncode != 0:
        sys.stderr.write(r.stdout[-6000:] + r.stderr[-6000:])
        raise RuntimeError("command failed: " + " ".join(str(c) for c in cmd))
    return r.stdout


def build_shim() -> Path:
    inc = REF_OUT / "mpi" / "include"
    lib = REF_OUT / "mpi" / "lib"
    inc.mkdir(parents=True, exist_ok=True)
    lib.mkdir(parents=True, exist_ok=True)
    shutil.copy2(HERE / "mpi_shim" / "mpi.h", inc / "mpi.h")
    run(["g++", "-std=c++17", "-O2", "-g1", "-fPIC", "-shared", "-pthread", "-Wall", "-Wextra",
         f"-I{inc}", HERE / "mpi_shim" / "mpi_shim.cpp", "-o", lib / "libmpi.so"])
    return REF_OUT / "mpi"


def find_lib_dir(prefix: Path) -> Path:
    for name in ("lib", "lib64"):
        if (prefix / name / "libAl.so").exists():
            return prefix / name
    raise RuntimeError(f"libAl.so not found under {prefix}")


def build_reference(src: Path, mpi: Path, cpu_only: bool) -> Path:
    tag = "cpu" if cpu_only else ""
    build = REF_OUT / tag / "build" if tag else REF_OUT / "build"
    prefix = REF_OUT / tag / "install" if tag else REF_OUT / "install"
    build.mkdir(parents=True, exist_ok=True)
    cfg = ["cmake", "-S", src, "-B", build, "-G", "Ninja",
           f"-DCMAKE_INSTALL_PREFIX={prefix}", "-DCMAKE_BUILD_TYPE=Release",
           "-DALUMINUM_ENABLE_HWLOC=OFF", "-DALUMINUM_ENABLE_TESTS=OFF", "-DALUMINUM_ENABLE_BENCHMARKS=OFF",
           f"-DMPI_CXX_HEADER_DIR={mpi / 'include'}", "-DMPI_CXX_LIB_NAMES=mpi",
           f"-DMPI_mpi_LIBRARY={mpi / 'lib' / 'libmpi.so'}", "-DMPI_CXX_SKIP_MPICXX=ON"]
    if not cpu_only:
        cfg += ["-DALUMINUM_ENABLE_CUDA=ON", "-DALUMINUM_ENABLE_NCCL=ON",
                f"-DCMAKE_CUDA_COMPILER={CUDA_HOME / 'bin' / 'nvcc'}", "-DCMAKE_CUDA_ARCHITECTURES=100a"]
    run(cfg)
    run(["cmake", "--build", build, "-j", str(os.cpu_count() or 4)])
    run(["cmake", "--install", build])
    return prefix


def build_driver(prefix: Path, mpi: Path) -> Path:
    out = REF_OUT / "lib"
    out.mkdir(parents=True, exist_ok=True)
    libdir = find_lib_dir(prefix)
    so = out / "libref_driver.so"
    run(["g++", "-std=c++17", "-O2", "-g1", "-fPIC", "-shared", "-pthread",
         f"-I{prefix / 'include'}", f"-I{mpi / 'include'}", f"-I{CUDA_HOME / 'include'}",
         HERE / "ref_driver.cpp", "-o", so,
         f"-L{libdir}", "-lAl", f"-L{mpi / 'lib'}", "-lmpi", f"-L{CUDA_HOME / 'lib64'}", "-lcudart", "-lnccl",
         "-Wl,-rpath,$ORIGIN/../install/lib:$ORIGIN/../install/lib64:$ORIGIN/../mpi/lib"])
    return so


def driver_is_stale() -> bool:
    so = REF_OUT / "lib" / "libref_driver.so"
    return (not so.exists()) or so.stat().st_mtime < (HERE / "ref_driver.cpp").stat().st_mtime


def rebuild_driver_only() -> Path:
    """Recompile libref_driver.so against an already installed reference (no reference sources needed)."""
    prefix = REF_OUT / "install"
    mpi = REF_OUT / "mpi"
    if not (prefix / "include" / "Al.hpp").exists() or not (mpi / "lib" / "libmpi.so").exists():
        raise RuntimeError("the reference is not installed under baseline/_ref: run baseline/build_reference.py")
    return build_driver(prefix, mpi)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("AL_REFERENCE_SRC", "/root/reference"))
    ap.add_argument("--cpu-only", action="store_true")
    a = ap.parse_args()
    src = Path(a.reference)
    if not (src / "CMakeLists.txt").exists():
        print(f"reference sources not found at {src}", file=sys.stderr)
        return 2
    mpi = build_shim()
    prefix = build_reference(src, mpi, a.cpu_only)
    info = {"reference": str(src), "prefix": str(prefix.relative_to(HERE.parent)), "cpu_only": a.cpu_only,
            "mpi": "baseline/mpi_shim (single-node stand-in)"}
    if not a.cpu_only:
        info["driver"] = str(build_driver(prefix, mpi).relative_to(HERE.parent))
    (REF_OUT / ("BUILD_INFO_cpu.json" if a.cpu_only else "BUILD_INFO.json")).write_text(json.dumps(info, indent=1))
    print(json.dumps(info))
    return 0


if __name__ == "__main__":
    sys.exit(main())
