"""In-tree build of the native library and tools.

Compiles every ``src/*.cpp`` with g++ and every ``kernels/*.cu`` with nvcc for
``sm_100a`` into ``build/obj``, links ``aluminum_b200/lib/libal_b200.so`` and the
command-line tools under ``aluminum_b200/bin``.  Objects are rebuilt only when
their source, any header or the flags changed.  The same sources can be built
with the CMake project at the repository root; this script exists so that the
Python package can build itself without CMake.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
PKG = ROOT / "aluminum_b200"
OBJ = ROOT / "build" / "obj"
LIB = PKG / "lib" / "libal_b200.so"
BIN = PKG / "bin"

CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
NVCC = str(CUDA_HOME / "bin" / "nvcc")
CXX = os.environ.get("CXX", "g++")

GENCODE = ["-gencode", "arch=compute_100a,code=sm_100a"]
CXXFLAGS = ["-std=c++17", "-O2", "-g1", "-fPIC", "-Wall", "-Wextra", "-pthread",
            f"-I{ROOT / 'include'}", f"-I{CUDA_HOME / 'include'}"]
NVCCFLAGS = GENCODE + ["-lineinfo", "-O3", "-std=c++17", "--extended-lambda", "-Xcompiler", "-fPIC",
                       f"-I{ROOT / 'include'}", f"-I{ROOT / 'kernels'}"]

# tool name -> sources (relative to the repository root)
TOOLS = {
    "alrun": ["util/alrun.cpp"],
    "al_info": ["util/al_info.cpp"],
    "test_ops": ["cpp_tests/test_ops.cpp"],
    "test_units": ["cpp_tests/test_units.cpp"],
    "test_rma": ["cpp_tests/test_rma.cpp"],
    "test_exchange": ["cpp_tests/test_exchange.cpp"],
    "test_stream_mem_ops": ["cpp_tests/test_stream_mem_ops.cpp"],
    "test_ht_failure": ["cpp_tests/test_ht_failure.cpp"],
    "benchmark_ops": ["benchmark/benchmark_ops.cpp"],
    "bandwidth": ["benchmark/bandwidth.cpp"],
    "benchmark_waits": ["benchmark/benchmark_waits.cpp"],
    "benchmark_events": ["benchmark/benchmark_events.cpp"],
    "stress_progress": ["benchmark/stress_progress.cpp"],
    "barrier_skew": ["benchmark/barrier_skew.cpp"],
    "hello_world": ["examples/hello_world.cpp"],
    "allreduce": ["examples/allreduce.cpp"],
    "pingpong": ["examples/pingpong.cpp"],
    "recover": ["examples/recover.cpp"],
}


def _headers_digest() -> str:
    h = hashlib.sha1()
    for d in (ROOT / "include", ROOT / "kernels", ROOT / "src", ROOT / "cpp_tests", ROOT / "benchmark", ROOT / "examples"):
        if not d.exists():
            continue
        for f in sorted(d.rglob("*")):
            if f.suffix in (".hpp", ".h", ".cuh"):
                h.update(str(f).encode())
                h.update(str(f.stat().st_mtime_ns).encode())
    return h.hexdigest()


def _needs(obj: Path, src: Path, stamp: str) -> bool:
    tag = obj.with_suffix(obj.suffix + ".stamp")
    if not obj.exists() or not tag.exists():
        return True
    want = f"{stamp}:{src.stat().st_mtime_ns}"
    return tag.read_text() != want


def _mark(obj: Path, src: Path, stamp: str) -> None:
    obj.with_suffix(obj.suffix + ".stamp").write_text(f"{stamp}:{src.stat().st_mtime_ns}")


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    if r.stderr.strip() and os.environ.get("AL_BUILD_VERBOSE"):
        sys.stderr.write(r.stderr)


def _compile(src: Path, stamp: str) -> Path:
    obj = OBJ / (src.relative_to(ROOT).as_posix().replace("/", "__") + ".o")
    if _needs(obj, src, stamp):
        if src.suffix == ".cu":
            _run([NVCC] + NVCCFLAGS + ["-c", str(src), "-o", str(obj)])
        else:
            _run([CXX] + CXXFLAGS + ["-c", str(src), "-o", str(obj)])
        _mark(obj, src, stamp)
    return obj


def library_sources() -> list[Path]:
    return sorted((ROOT / "src").glob("*.cpp")) + sorted((ROOT / "kernels").glob("*.cu"))


def build(tools: bool = True, jobs: int | None = None, verbose: bool = False) -> Path:
    """Build the shared library (and the tools); returns the library path."""
    if shutil.which(NVCC) is None:
        raise RuntimeError(f"nvcc not found at {NVCC}")
    OBJ.mkdir(parents=True, exist_ok=True)
    LIB.parent.mkdir(parents=True, exist_ok=True)
    BIN.mkdir(parents=True, exist_ok=True)
    stamp = _headers_digest() + hashlib.sha1(" ".join(CXXFLAGS + NVCCFLAGS).encode()).hexdigest()
    jobs = jobs or max(1, (os.cpu_count() or 4))
    srcs = library_sources()
    with ThreadPoolExecutor(jobs) as ex:
        objs = list(ex.map(lambda s: _compile(s, stamp), srcs))
    newest = max(o.stat().st_mtime_ns for o in objs)
    if not LIB.exists() or LIB.stat().st_mtime_ns < newest:
        _run([NVCC] + GENCODE + ["-shared", "-o", str(LIB)] + [str(o) for o in objs] +
             ["-lpthread", "-ldl", "-lrt"])
        if verbose:
            print(f"linked {LIB}")
    if tools:
        todo = {n: [ROOT / s for s in ss] for n, ss in TOOLS.items() if all((ROOT / s).exists() for s in ss)}

        def one(item):
            name, sources = item
            out = BIN / name
            tobjs = [_compile(s, stamp) for s in sources]
            if (not out.exists() or out.stat().st_mtime_ns < max(o.stat().st_mtime_ns for o in tobjs)
                    or out.stat().st_mtime_ns < LIB.stat().st_mtime_ns):
                _run([NVCC] + GENCODE + ["-o", str(out)] + [str(o) for o in tobjs] +
                     [f"-L{LIB.parent}", "-lal_b200", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../lib",
                      "-lpthread", "-ldl", "-lrt"])
            return out

        with ThreadPoolExecutor(jobs) as ex:
            list(ex.map(one, todo.items()))
    return LIB


def _sanitizer_compiler(kind: str) -> str:
    """First of $CXX, g++, clang++ that can link a program with the sanitizer's runtime."""
    import tempfile
    with tempfile.TemporaryDirectory() as td:
        src = Path(td) / "t.cpp"
        src.write_text("int main() { return 0; }\n")
        for cand in (CXX, "/usr/bin/g++", "g++", "clang++"):
            exe = shutil.which(cand)
            if exe is None:
                continue
            r = subprocess.run([exe, f"-fsanitize={kind}", str(src), "-o", str(Path(td) / "t")],
                               capture_output=True, text=True)
            if r.returncode == 0:
                return exe
    raise RuntimeError(f"no compiler on this machine links with -fsanitize={kind}")


def build_sanitized(kind: str = "thread", tools: tuple[str, ...] = ("test_units", "test_ops"),
                    jobs: int | None = None) -> dict[str, Path]:
    """Build some tools with every host source compiled under a sanitizer.

    The host runtime is compiled again with ``-fsanitize=<kind>`` into
    ``build/obj_<kind>`` and linked statically into each tool together with the
    ordinary kernel objects (device code is not instrumented).  Returns the
    paths of the instrumented tools, ``build/<kind>/<tool>``.
    """
    build(tools=False, jobs=jobs)
    cxx = _sanitizer_compiler(kind)
    odir = ROOT / "build" / f"obj_{kind}"
    bdir = ROOT / "build" / kind
    odir.mkdir(parents=True, exist_ok=True)
    bdir.mkdir(parents=True, exist_ok=True)
    # -g1 keeps function names and line numbers in the reports at a tenth of the size of -g.
    flags = [f for f in CXXFLAGS if f != "-O2"] + ["-O1", "-g1", f"-fsanitize={kind}", f"-I{ROOT / 'cpp_tests'}"]
    stamp = _headers_digest() + hashlib.sha1(" ".join(flags).encode()).hexdigest()
    jobs = jobs or max(1, (os.cpu_count() or 4))

    def cc(src: Path) -> Path:
        obj = odir / (src.relative_to(ROOT).as_posix().replace("/", "__") + ".o")
        if _needs(obj, src, stamp):
            _run([cxx] + flags + ["-c", str(src), "-o", str(obj)])
            _mark(obj, src, stamp)
        return obj

    host = sorted((ROOT / "src").glob("*.cpp"))
    tool_srcs = [ROOT / s for t in tools for s in TOOLS[t]]
    with ThreadPoolExecutor(jobs) as ex:
        objs = list(ex.map(cc, host + tool_srcs))
    host_objs, tool_objs = objs[:len(host)], objs[len(host):]
    kernels = [OBJ / (k.relative_to(ROOT).as_posix().replace("/", "__") + ".o")
               for k in sorted((ROOT / "kernels").glob("*.cu"))]
    out: dict[str, Path] = {}
    i = 0
    for t in tools:
        n = len(TOOLS[t])
        exe = bdir / t
        _run([cxx, f"-fsanitize={kind}", "-pthread", "-o", str(exe)] + [str(o) for o in tool_objs[i:i + n]] +
             [str(o) for o in host_objs] + [str(k) for k in kernels] +
             [f"-L{CUDA_HOME / 'lib64'}", "-lcudart_static", "-ldl", "-lrt"])
        out[t] = exe
        i += n
    return out


def clean_sanitized(kind: str) -> None:
    """Remove what build_sanitized(kind) wrote (the instrumented objects and tools are large)."""
    for d in (ROOT / "build" / f"obj_{kind}", ROOT / "build" / kind):
        shutil.rmtree(d, ignore_errors=True)


if __name__ == "__main__":
    p = build(verbose=True)
    print(p)
