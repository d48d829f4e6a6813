"""The CMake project configures and produces a package configuration (find_package(AluminumB200) support)
with the options the build offers.  Configure only - compiling the CUDA sources is covered by the in-tree
build every other test uses."""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def test_cmake_configures_and_writes_a_package_config(tmp_path):
    if shutil.which("cmake") is None or shutil.which("ninja") is None or not Path("/usr/local/cuda/bin/nvcc").exists():
        pytest.skip("cmake, ninja or nvcc not available")
    b = tmp_path / "b"
    r = subprocess.run(["cmake", "-S", str(ROOT), "-B", str(b), "-G", "Ninja", "-DALUMINUM_ENABLE_TESTS=OFF",
                        "-DALUMINUM_ENABLE_BENCHMARKS=OFF", "-DALUMINUM_ENABLE_EXAMPLES=OFF", "-DALUMINUM_ENABLE_DEBUG=ON",
                        "-DCMAKE_CUDA_COMPILER=/usr/local/cuda/bin/nvcc", f"-DCMAKE_INSTALL_PREFIX={tmp_path / 'inst'}"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    cfg = (b / "AluminumB200Config.cmake").read_text()
    assert "AluminumB200Targets.cmake" in cfg and "find_dependency(CUDAToolkit" in cfg
    assert "ALUMINUM_B200_ENABLE_DEBUG_DEFAULT ON" in cfg and 'ALUMINUM_B200_CUDA_ARCH "sm_100a"' in cfg
    ver = (b / "AluminumB200ConfigVersion.cmake").read_text()
    assert "0.1.0" in ver
    cache = (b / "CMakeCache.txt").read_text()
    for opt in ("ALUMINUM_ENABLE_DEBUG", "ALUMINUM_ENABLE_TRACE", "ALUMINUM_ENABLE_TESTS", "ALUMINUM_ENABLE_BENCHMARKS",
                "ALUMINUM_ENABLE_EXAMPLES"):
        assert opt in cache
