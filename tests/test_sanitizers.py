"""The host runtime under ThreadSanitizer and AddressSanitizer: queues, progress engine, host backend.

The tools are rebuilt with every host source instrumented (device objects are
linked as they are) and must finish without a single sanitizer report.  Ranks
are separate processes, so what is checked is each rank's user thread against
its progress thread and the test's own helper threads.
"""
import subprocess

import pytest

OPS = ["allreduce", "reduce_scatter", "allgatherv", "alltoallv", "bcast", "sendrecv", "multisendrecv"]


@pytest.fixture(scope="module")
def tsan_tools(built_lib):
    from aluminum_b200 import _build
    try:
        yield _build.build_sanitized("thread")
    except RuntimeError as e:
        if "no compiler" in str(e):
            pytest.skip(str(e))
        raise
    finally:
        _build.clean_sanitized("thread")  # instrumented builds are large; leave nothing behind


def _clean(out: str) -> bool:
    return "ThreadSanitizer" not in out


def test_units_are_race_free(tsan_tools):
    r = subprocess.run([str(tsan_tools["test_units"])], capture_output=True, text=True, timeout=600)
    out = r.stdout + r.stderr
    assert r.returncode == 0 and "all unit tests passed" in out, out[-3000:]
    assert _clean(out), out[-3000:]


@pytest.mark.parametrize("op", OPS)
def test_host_backend_is_race_free(tsan_tools, bin_dir, op):
    r = subprocess.run([str(bin_dir / "alrun"), "-n", "3", "--timeout", "300", str(tsan_tools["test_ops"]),
                        "--backend", "host", "--op", op, "--max-size", "16384"],
                       capture_output=True, text=True, timeout=600)
    out = r.stdout + r.stderr
    assert r.returncode == 0 and ": ok" in out, out[-3000:]
    assert _clean(out), out[-3000:]


@pytest.mark.parametrize("op", ["allreduce", "alltoall", "sendrecv"])
def test_thread_multiple_is_race_free(tsan_tools, bin_dir, op):
    """Three user threads per rank plus the progress thread, non-blocking, under ThreadSanitizer."""
    r = subprocess.run([str(bin_dir / "alrun"), "-n", "2", "--timeout", "300", str(tsan_tools["test_ops"]),
                        "--backend", "host", "--op", op, "--threads", "3", "--nonblocking", "--max-size", "4096"],
                       capture_output=True, text=True, timeout=600)
    out = r.stdout + r.stderr
    assert r.returncode == 0 and ": ok" in out, out[-3000:]
    assert _clean(out), out[-3000:]


@pytest.mark.parametrize("op", ["allreduce", "reduce", "alltoallv", "bcast", "multisendrecv"])
def test_socket_path_is_race_free(tsan_tools, bin_dir, op):
    """Ranks on different (modelled) nodes: the TCP data plane under ThreadSanitizer, two user threads."""
    r = subprocess.run([str(bin_dir / "alrun"), "-n", "4", "--nodes", "2", "--timeout", "300", str(tsan_tools["test_ops"]),
                        "--backend", "host", "--op", op, "--threads", "2", "--nonblocking", "--max-size", "300000"],
                       capture_output=True, text=True, timeout=600)
    out = r.stdout + r.stderr
    assert r.returncode == 0 and ": ok" in out, out[-3000:]
    assert _clean(out), out[-3000:]


@pytest.fixture(scope="module")
def asan_tools(built_lib):
    from aluminum_b200 import _build
    try:
        yield _build.build_sanitized("address")
    except RuntimeError as e:
        if "no compiler" in str(e):
            pytest.skip(str(e))
        raise
    finally:
        _build.clean_sanitized("address")


def test_units_are_memory_clean(asan_tools):
    r = subprocess.run([str(asan_tools["test_units"])], capture_output=True, text=True, timeout=600)
    out = r.stdout + r.stderr
    assert r.returncode == 0 and "all unit tests passed" in out and "AddressSanitizer" not in out, out[-3000:]


@pytest.mark.parametrize("op", ["allreduce", "alltoallv", "gatherv", "multisendrecv"])
def test_host_backend_is_memory_clean(asan_tools, bin_dir, op):
    """Out-of-bounds accesses, use after free and leaks at exit all fail the run."""
    r = subprocess.run([str(bin_dir / "alrun"), "-n", "3", "--timeout", "300", str(asan_tools["test_ops"]),
                        "--backend", "host", "--op", op, "--max-size", "16384"],
                       capture_output=True, text=True, timeout=600)
    out = r.stdout + r.stderr
    assert r.returncode == 0 and ": ok" in out and "Sanitizer" not in out, out[-3000:]
    r = subprocess.run([str(bin_dir / "alrun"), "-n", "4", "--nodes", "2", "--timeout", "300", str(asan_tools["test_ops"]),
                        "--backend", "host", "--op", op, "--max-size", "300000", "--odd-sizes", "--inplace"],
                       capture_output=True, text=True, timeout=600)
    out = r.stdout + r.stderr
    assert r.returncode == 0 and ": ok" in out and "Sanitizer" not in out, out[-3000:]
