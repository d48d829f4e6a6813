"""The MPI stand-in of the reference arm, checked without a GPU.

The unmodified reference library is configured with its own CMake project against
``baseline/mpi_shim`` (no CUDA: MPI backend only) and a small program drives a dozen of its
operations, blocking and non-blocking, on 1, 2 and 4 processes; every result is compared with a
locally computed value.  Skipped where the reference sources or CMake are absent.
"""
import os
import shutil
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
REF_SRC = Path(os.environ.get("AL_REFERENCE_SRC", "/root/reference"))


@pytest.fixture(scope="module")
def shim_check():
    if not (REF_SRC / "CMakeLists.txt").exists() or shutil.which("cmake") is None or shutil.which("ninja") is None:
        pytest.skip("reference sources, cmake or ninja not available")
    r = subprocess.run([sys.executable, str(ROOT / "baseline" / "build_reference.py"), "--cpu-only",
                        "--reference", str(REF_SRC)], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    cpu = ROOT / "baseline" / "_ref" / "cpu"
    mpi = ROOT / "baseline" / "_ref" / "mpi"
    exe = cpu / "check_ref_mpi"
    libdir = cpu / "install" / ("lib" if (cpu / "install" / "lib" / "libAl.so").exists() else "lib64")
    c = subprocess.run(["g++", "-std=c++17", "-O1", "-pthread", f"-I{cpu / 'install' / 'include'}", f"-I{mpi / 'include'}",
                        str(ROOT / "baseline" / "mpi_shim" / "check_ref_mpi.cpp"), "-o", str(exe), f"-L{libdir}", "-lAl",
                        f"-L{mpi / 'lib'}", "-lmpi", f"-Wl,-rpath,{libdir}:{mpi / 'lib'}"],
                       capture_output=True, text=True, timeout=600)
    assert c.returncode == 0, c.stderr[-3000:]
    return exe


@pytest.mark.parametrize("nranks", [1, 2, 4])
def test_reference_mpi_backend_runs_on_the_shim(shim_check, nranks):
    procs = []
    for r in range(nranks):
        env = {**os.environ, "RANK": str(r), "WORLD_SIZE": str(nranks), "MPISHIM_JOB": f"pytest-{os.getpid()}-{nranks}",
               "MPISHIM_TIMEOUT_S": "60"}
        procs.append(subprocess.Popen([str(shim_check)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=120)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n<timed out>"
        outs.append((p.returncode, out))
    for rc, out in outs:
        assert rc == 0 and "ok" in out, "\n".join(o for _, o in outs)
