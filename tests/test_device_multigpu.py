"""Multi-process device backend (one process per GPU).  Needs at least two GPUs; on a
single-GPU box these tests skip and the emulated tests cover the same kernels."""
import os
import subprocess

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.mark.parametrize("op", ["allreduce", "reduce", "reduce_scatter", "reduce_scatterv", "allgather", "allgatherv",
                                "alltoall", "alltoallv", "bcast", "gather", "scatterv", "barrier", "send", "sendrecv",
                                "multisendrecv"])
def test_ops_device_backend(bin_dir, op):
    n = _ngpu()
    if n < 2:
        pytest.skip("needs >= 2 GPUs")
    env = {**os.environ, "NCCL_NVLS_ENABLE": "0"}
    for extra in ([], ["--inplace", "--nonblocking"]):
        r = subprocess.run([str(bin_dir / "alrun"), "-n", str(n), "--timeout", "180", str(bin_dir / "test_ops"),
                            "--backend", "device", "--op", op, "--max-size", str(1 << 20), "--odd-sizes", "--zero"] + extra,
                           capture_output=True, text=True, timeout=240, env=env)
        assert r.returncode == 0, r.stdout + r.stderr


def test_rma_ring_exchange_and_bandwidth(bin_dir):
    n = min(_ngpu(), 4)
    if n < 2:
        pytest.skip("needs >= 2 GPUs")
    for cmd in (["test_rma", "--max-size", "65536"], ["test_exchange", "--backend", "device", "--peers", "1"],
                ["bandwidth", "--bytes", "8388608", "--iters", "3"], ["pingpong", "device"]):
        r = subprocess.run([str(bin_dir / "alrun"), "-n", str(n if cmd[0] != "pingpong" else 2), "--timeout", "120",
                            str(bin_dir / cmd[0])] + cmd[1:], capture_output=True, text=True, timeout=180)
        assert r.returncode == 0, " ".join(cmd) + r.stdout + r.stderr


def test_rma_halo_exchange_on_a_2d_grid(bin_dir):
    n = min(_ngpu(), 4)
    if n < 2:
        pytest.skip("needs >= 2 GPUs")
    r = subprocess.run([str(bin_dir / "alrun"), "-n", str(n), "--timeout", "120", str(bin_dir / "test_rma"),
                        "--mode", "halo", "--max-size", "65536"], capture_output=True, text=True, timeout=180)
    assert r.returncode == 0 and "rma halo" in r.stdout and "FAIL" not in r.stdout, r.stdout + r.stderr


def test_torch_distributed_backend_on_gpus(bin_dir):
    import sys
    from pathlib import Path
    n = min(_ngpu(), 4)
    if n < 2:
        pytest.skip("needs >= 2 GPUs")
    worker = Path(__file__).resolve().parent / "workers" / "torch_backend_worker.py"
    r = subprocess.run([str(bin_dir / "alrun"), "-n", str(n), "--timeout", "240", sys.executable, str(worker), "cuda"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.count("torch backend ok") == n, r.stdout + r.stderr


def test_data_paths_over_real_ranks(bin_dir):
    """Packets, staged, pipelined and window paths, registration through CUDA IPC, multimem on symmetric
    buffers, the NVLS tail rule, Get, from_ranks and the path-mismatch error, on every GPU of the machine."""
    import sys
    from pathlib import Path
    n = _ngpu()
    if n < 2:
        pytest.skip("needs >= 2 GPUs")
    worker = Path(__file__).resolve().parent / "workers" / "device_paths_worker.py"
    env = {**os.environ, "AL_TEST_LARGE": os.environ.get("AL_TEST_LARGE", "1")}
    r = subprocess.run([str(bin_dir / "alrun"), "-n", str(n), "--timeout", "420", sys.executable, str(worker)],
                       capture_output=True, text=True, timeout=480, env=env)
    assert r.returncode == 0 and r.stdout.count("device paths ok") == n, r.stdout[-4000:] + r.stderr[-4000:]


def test_parallel_components_over_real_ranks(bin_dir):
    """Tensor + sequence parallel training, Ulysses / expert exchanges, a two-stage pipeline with backward and
    ring attention on real GPUs, each against the single-device computation."""
    import sys
    from pathlib import Path
    n = min(_ngpu(), 4)
    if n < 2:
        pytest.skip("needs >= 2 GPUs")
    worker = Path(__file__).resolve().parent / "workers" / "parallel_worker.py"
    r = subprocess.run([str(bin_dir / "alrun"), "-n", str(n), "--timeout", "300", sys.executable, str(worker)],
                       capture_output=True, text=True, timeout=360)
    assert r.returncode == 0 and r.stdout.count("parallel components ok") == n, r.stdout[-4000:] + r.stderr[-4000:]


def test_data_parallel_matches_single_process(bin_dir):
    import sys
    from pathlib import Path
    n = min(_ngpu(), 4)
    if n < 2:
        pytest.skip("needs >= 2 GPUs")
    worker = Path(__file__).resolve().parent / "workers" / "ddp_worker.py"
    r = subprocess.run([str(bin_dir / "alrun"), "-n", str(n), "--timeout", "240", sys.executable, str(worker)],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.count("ok") == n, r.stdout + r.stderr
