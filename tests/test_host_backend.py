"""CPU tests (no GPU): C++ unit tests, the op-vs-serial-oracle driver on the host backend over
several rank counts, the world-size-2 plumbing configuration, launcher environments, tracing and
host-side failure detection."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
W = ROOT / "tests" / "workers"


def run(cmd, env=None, timeout=300):
    e = {**os.environ, **(env or {})}
    return subprocess.run([str(c) for c in cmd], capture_output=True, text=True, timeout=timeout, env=e)


def test_cpp_unit_tests(bin_dir):
    r = run([bin_dir / "test_units"])
    assert r.returncode == 0, r.stdout + r.stderr


def test_al_info(bin_dir):
    r = run([bin_dir / "al_info"])
    assert r.returncode == 0 and "Aluminum-B200" in r.stdout and "dev_stage_bytes" in r.stdout


OPS = ["allreduce", "reduce", "reduce_scatter", "reduce_scatterv", "allgather", "allgatherv", "gather", "gatherv",
       "scatter", "scatterv", "alltoall", "alltoallv", "bcast", "barrier", "send", "sendrecv", "multisendrecv"]


@pytest.mark.parametrize("op", OPS)
@pytest.mark.parametrize("ranks", [2, 3])
def test_ops_host(bin_dir, op, ranks):
    for extra in ([], ["--inplace", "--nonblocking", "--root", "1"]):
        r = run([bin_dir / "alrun", "-n", ranks, "--timeout", "120", bin_dir / "test_ops", "--backend", "host", "--op", op,
                 "--max-size", "4096", "--odd-sizes", "--zero", "--quiet"] + extra)
        assert r.returncode == 0, f"{op} {extra}: {r.stdout}{r.stderr}"


@pytest.mark.parametrize("dtype,rop", [("double", "prod"), ("int", "band"), ("uchar", "max"), ("llong", "min"),
                                       ("half", "sum"), ("bfloat16", "sum"), ("int", "lxor"), ("float", "avg"),
                                       ("short", "bor")])
def test_ops_host_types(bin_dir, dtype, rop):
    r = run([bin_dir / "alrun", "-n", "4", "--timeout", "120", bin_dir / "test_ops", "--backend", "host", "--op", "allreduce",
             "--datatype", dtype, "--reduction-op", rop, "--max-size", "2048", "--odd-sizes", "--quiet"])
    assert r.returncode == 0, r.stdout + r.stderr


def test_multichunk_small_staging(bin_dir):
    env = {"AL_HOST_STAGE_BYTES": "4096", "AL_HOST_MAILBOX_BYTES": "256"}
    for op in ("allreduce", "alltoallv", "reduce_scatterv", "multisendrecv", "gatherv"):
        r = run([bin_dir / "alrun", "-n", "4", "--timeout", "120", bin_dir / "test_ops", "--backend", "host", "--op", op,
                 "--min-size", "1024", "--max-size", "32768", "--odd-sizes", "--nonblocking", "--quiet"], env=env)
        assert r.returncode == 0, op + r.stdout + r.stderr


def test_config1_world2_python(bin_dir):
    r = run([bin_dir / "alrun", "-n", "2", "--timeout", "200", sys.executable, W / "host_config1.py"])
    assert r.returncode == 0 and r.stdout.count("ok") == 2, r.stdout + r.stderr


def test_torchrun_style_environment(bin_dir):
    """RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT are understood without the library's own launcher."""
    procs = []
    for rank in range(2):
        env = {**os.environ, "RANK": str(rank), "WORLD_SIZE": "2", "LOCAL_RANK": str(rank), "MASTER_ADDR": "127.0.0.1",
               "MASTER_PORT": str(29000 + os.getpid() % 2000)}
        for k in ("AL_RANK", "AL_WORLD_SIZE", "AL_JOB_KEY"):
            env.pop(k, None)
        procs.append(subprocess.Popen([str(bin_dir / "test_ops"), "--backend", "host", "--op", "allreduce", "--max-size", "512"],
                                      env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=120)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs


def test_rank_that_never_joins_is_detected(bin_dir):
    env = {"AL_HOST_WAIT_TIMEOUT_S": "60"}
    r = run([bin_dir / "alrun", "-n", "2", "--timeout", "60", sys.executable, W / "host_fault.py"], env=env, timeout=120)
    assert "rank 0 detected the failure" in r.stdout, r.stdout + r.stderr


def test_bootstrap_times_out_when_a_rank_is_missing(bin_dir):
    env = {"AL_RANK": "0", "AL_WORLD_SIZE": "2", "AL_JOB_KEY": f"lonely-{os.getpid()}", "AL_BOOTSTRAP_TIMEOUT_S": "1"}
    r = run([bin_dir / "test_ops", "--backend", "host", "--op", "barrier"], env=env, timeout=60)
    assert r.returncode != 0 and "timed out" in r.stderr


def test_trace_file_is_written(bin_dir, tmp_path):
    env = {"AL_TRACE": "1", "AL_TRACE_DIR": str(tmp_path)}
    r = run([bin_dir / "alrun", "-n", "2", bin_dir / "test_ops", "--backend", "host", "--op", "bcast", "--size", "64",
             "--nonblocking"], env=env)
    assert r.returncode == 0, r.stdout + r.stderr
    files = list(tmp_path.glob("*.trace.txt"))
    assert len(files) == 2
    text = files[0].read_text()
    assert "HostBackend float nonblocking-bcast" in text and "PE START HostBcast" in text and "PE DONE HostBcast" in text


def test_debug_checks_reject_bad_arguments(bin_dir):
    code = ("import sys; sys.path.insert(0, %r); import numpy as np, aluminum_b200 as al; c = al.HostComm();\n"
            "x = np.ones(4, dtype=np.float32)\n"
            "try:\n    c.bcast(x, root=5)\n    print('no error')\nexcept al.AlError as e:\n    print('rejected')\n") % str(ROOT)
    r = run([sys.executable, "-c", code], env={"AL_DEBUG": "1"})
    assert "rejected" in r.stdout, r.stdout + r.stderr


def test_examples_and_exchange_on_cpu_ranks(bin_dir):
    r = run([bin_dir / "alrun", "-n", "3", bin_dir / "hello_world"])
    assert r.returncode == 0 and r.stdout.count("sum of ranks = 3") == 3, r.stdout + r.stderr
    r = run([bin_dir / "alrun", "-n", "2", bin_dir / "allreduce"])
    assert r.returncode == 0 and r.stdout.count("value 3 (expected 3)") == 2, r.stdout + r.stderr
    r = run([bin_dir / "alrun", "-n", "2", bin_dir / "pingpong"])
    assert r.returncode == 0 and "per round trip" in r.stdout
    r = run([bin_dir / "alrun", "-n", "4", bin_dir / "test_exchange", "--peers", "2", "--size", "5000"])
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout + r.stderr
    r = run([bin_dir / "alrun", "-n", "2", bin_dir / "benchmark_ops", "--backend", "host", "--op", "allreduce",
             "--max-bytes", "4096", "--num-iters", "5"])
    assert r.returncode == 0 and "host float allreduce" in r.stdout


def test_python_host_api(bin_dir):
    r = run([bin_dir / "alrun", "-n", "3", "--timeout", "120", sys.executable, W / "host_python_api.py"])
    assert r.returncode == 0 and r.stdout.count("ok") == 3, r.stdout + r.stderr


def test_info_and_tuning_from_python(built_lib):
    import aluminum_b200 as al
    assert "Aluminum-B200" in al.info() and "max_ctas" in al.info()
    old = al.get_tuning("max_ctas")
    al.set_tuning("max_ctas", 48)
    assert al.get_tuning("max_ctas") == 48
    al.set_tuning("max_ctas", old)
    with pytest.raises(al.AlError):
        al.set_tuning("no_such_entry", 1)


def test_crossover_table_per_rank_count(built_lib, bin_dir):
    """The algorithm crossovers are a table with one row per communicator size: a plain name sets every row,
    "name@p" the row of p ranks; environment variables follow the same scheme (AL_X, AL_X_P2 / _P4 / _P8)."""
    import aluminum_b200 as al
    names = ["ll_max_bytes", "ar_ll_max_bytes", "ar_ll2_max_bytes", "ar_oneshot_max_bytes", "ar_nvls_min_bytes",
             "ar_pipeline_min_bytes", "nvls_pipeline_min_bytes", "pipeline_min_bytes", "window_min_bytes", "rs_nvls_min_bytes"]
    info = al.info()
    for n in names:
        assert n in info, n
        for p in (2, 4, 8):
            assert al.get_tuning(f"{n}@{p}") >= 0
    old = [al.get_tuning(f"ar_ll_max_bytes@{p}") for p in (2, 4, 8)]
    assert old[0] >= old[1] >= old[2] > 0          # one-phase packets pay p-1 times the vector: the limit shrinks with p
    al.set_tuning("ar_ll_max_bytes@4", 12345)
    assert [al.get_tuning(f"ar_ll_max_bytes@{p}") for p in (2, 4, 8)] == [old[0], 12345, old[2]]
    assert al.get_tuning("ar_ll_max_bytes@3") == 12345   # three ranks share the row of four
    al.set_tuning("ar_ll_max_bytes", 777)
    assert [al.get_tuning(f"ar_ll_max_bytes@{p}") for p in (2, 4, 8)] == [777, 777, 777]
    for p, v in zip((2, 4, 8), old):
        al.set_tuning(f"ar_ll_max_bytes@{p}", v)
    for n in ("p2p_ll_max_bytes", "nvls_chunk_bytes", "max_ctas_pipelined", "window_ctas"):
        assert al.get_tuning(n) > 0
    r = run([bin_dir / "al_info"], env={"AL_AR_LL2_MAX": "4096", "AL_AR_LL2_MAX_P8": "8192", "AL_P2P_LL_MAX": "1024"})
    assert r.returncode == 0, r.stderr
    row = [l for l in r.stdout.splitlines() if "ar_ll2_max_bytes" in l][0].split()
    assert row[1:] == ["4096", "4096", "8192"], row
    assert "p2p_ll_max_bytes = 1024" in r.stdout


def test_injected_missing_signal_times_out_and_recovers(bin_dir):
    env = {"AL_HOST_WAIT_TIMEOUT_S": "1", "AL_FAULT_RANK": "1", "AL_FAULT_OP": "2", "AL_FAULT_KIND": "1"}
    r = run([bin_dir / "alrun", "-n", "3", "--timeout", "120", sys.executable, W / "host_inject.py", "skip"], env=env)
    assert r.returncode == 0 and r.stdout.count("recovered") == 3, r.stdout + r.stderr


def test_injected_delay_is_tolerated(bin_dir):
    env = {"AL_FAULT_RANK": "1", "AL_FAULT_OP": "2", "AL_FAULT_KIND": "2", "AL_FAULT_DELAY_MS": "300"}
    r = run([bin_dir / "alrun", "-n", "3", "--timeout", "120", sys.executable, W / "host_inject.py", "delay"], env=env)
    assert r.returncode == 0 and r.stdout.count("delayed op ok") == 3, r.stdout + r.stderr


def test_abort_ends_pending_requests(bin_dir):
    r = run([bin_dir / "alrun", "-n", "2", "--timeout", "120", sys.executable, W / "host_inject.py", "abort"])
    assert r.returncode == 0 and r.stdout.count("abort ok") == 2, r.stdout + r.stderr


def test_random_delays_between_ranks_do_not_change_results(bin_dir):
    env = {"AL_FAULT_JITTER_US": "300"}
    r = run([bin_dir / "alrun", "-n", "4", "--timeout", "200", sys.executable, W / "host_inject.py", "jitter"], env=env)
    assert r.returncode == 0 and r.stdout.count("jitter ok") == 4, r.stdout + r.stderr


@pytest.mark.parametrize("op", ["allreduce", "reduce_scatter", "alltoallv", "bcast", "sendrecv", "multisendrecv"])
def test_thread_multiple(bin_dir, op):
    """Three user threads per rank, each on its own communicator, all inside the library at once."""
    for extra in ([], ["--nonblocking"]):
        r = run([bin_dir / "alrun", "-n", "4", "--timeout", "120", bin_dir / "test_ops", "--backend", "host", "--op", op,
                 "--threads", "3", "--max-size", "8192", "--odd-sizes"] + extra)
        assert r.returncode == 0 and "threads=3: ok" in r.stdout, r.stdout + r.stderr


@pytest.mark.parametrize("op", ["allreduce", "gather", "scatterv", "send"])
def test_permuted_ranks(bin_dir, op):
    r = run([bin_dir / "alrun", "-n", "4", "--timeout", "120", bin_dir / "test_ops", "--backend", "host", "--op", op,
             "--permute", "2,0,3,1", "--root", "3", "--max-size", "8192"])
    assert r.returncode == 0 and "permuted" in r.stdout and ": ok" in r.stdout, r.stdout + r.stderr
    r = run([bin_dir / "alrun", "-n", "3", "--timeout", "60", bin_dir / "test_ops", "--backend", "host", "--op", op,
             "--permute", "2,0,0"])
    assert r.returncode != 0 and "not a permutation" in r.stderr, r.stdout + r.stderr


def test_serialized_mode_runs_blocking_calls_on_the_progress_thread(bin_dir, tmp_path):
    env = {"AL_HOST_SERIALIZE": "1", "AL_TRACE": "1", "AL_TRACE_DIR": str(tmp_path)}
    r = run([bin_dir / "alrun", "-n", "3", "--timeout", "120", bin_dir / "test_ops", "--backend", "host", "--op", "allreduce",
             "--max-size", "4096"], env=env)
    assert r.returncode == 0 and ": ok" in r.stdout, r.stdout + r.stderr
    text = next(iter(tmp_path.glob("*.trace.txt"))).read_text()
    assert "PE START HostAllreduce" in text  # a blocking call went through the engine


def test_many_short_lived_communicators(bin_dir, tmp_path):
    """More communicators than the progress engine has slots, one after another, each with a
    non-blocking operation: destroyed communicators give their slot back."""
    script = tmp_path / "many.py"
    script.write_text(
        "import sys, numpy as np\n"
        f"sys.path.insert(0, {str(ROOT)!r})\n"
        "import aluminum_b200 as al\n"
        "w = al.HostComm()\n"
        "for i in range(150):\n"
        "    c = w.split(0, w.rank)\n"
        "    x = np.ones(8, dtype=np.float32)\n"
        "    c.allreduce(x, nonblocking=True).wait()\n"
        "    assert x[0] == c.size\n"
        "    c.close()\n"
        "print('many ok')\n")
    r = run([bin_dir / "alrun", "-n", "2", "--timeout", "120", sys.executable, script])
    assert r.returncode == 0 and r.stdout.count("many ok") == 2, r.stdout + r.stderr


@pytest.mark.parametrize("launch", [["-n", "4"], ["-n", "4", "--nodes", "2"]])
def test_progress_engine_stress_on_cpu_ranks(bin_dir, launch):
    """64 non-blocking allreduces of 4-256 KB on 8 communicators started before the first Wait."""
    r = run([bin_dir / "alrun", *launch, "--timeout", "200", bin_dir / "stress_progress", "--backend", "host", "--rounds", "5"])
    assert r.returncode == 0 and "ops_per_s=" in r.stdout, r.stdout + r.stderr


@pytest.mark.parametrize("launch", [["-n", "2"], ["-n", "3"], ["-n", "4", "--nodes", "2"]])
def test_torch_distributed_backend_on_cpu_ranks(bin_dir, launch):
    """torch.distributed collectives, a sub-group and DistributedDataParallel on the "aluminum" backend."""
    n = int(launch[1])
    r = run([bin_dir / "alrun"] + launch + ["--timeout", "120", sys.executable, W / "torch_backend_worker.py"], timeout=240)
    assert r.returncode == 0 and r.stdout.count("torch backend ok") == n, r.stdout + r.stderr


def test_compare_settings_tool(bin_dir, tmp_path):
    """The tuning comparison drives benchmark_ops under two settings and tabulates both."""
    out = tmp_path / "cmp.md"
    r = run([sys.executable, ROOT / "benchmark" / "compare_settings.py", "--ranks", "2", "--backend", "host", "--ops", "allreduce",
             "--min-bytes", "1024", "--max-bytes", "4096", "--num-iters", "3", "--num-warmup", "1",
             "--setting", "default", "--setting", "small-stage:AL_HOST_STAGE_BYTES=4096", "--out", out], timeout=240)
    assert r.returncode == 0, r.stdout + r.stderr
    text = out.read_text()
    assert "| bytes | default | small-stage | fastest |" in text and "| 4 KiB |" in text, text


@pytest.mark.parametrize("launch", [["-n", "3"], ["-n", "4", "--nodes", "2"], ["-n", "6", "--nodes", "2"]])
def test_survivors_rebuild_a_communicator_and_continue(bin_dir, launch):
    """A rank leaves; the others fail fast (also those waiting in another level of a two-level operation,
    which hear of it through the shared workspace / closed connections), agree on who is left, build a
    communicator of the survivors and keep training with equal replicas."""
    n = int(launch[1])
    r = run([bin_dir / "alrun"] + launch + ["--timeout", "90", sys.executable, W / "host_recover.py"],
            env={"AL_HOST_WAIT_TIMEOUT_S": "30"}, timeout=180)
    assert r.stdout.count("recovered with") == n - 1, r.stdout + r.stderr


def test_cpp_recover_example(bin_dir):
    """examples/recover.cpp: Al::AliveRanks + HostCommunicator::from_ranks after a rank left."""
    for launch, n in ((["-n", "4"], 4), (["-n", "6", "--nodes", "2"], 6)):
        r = run([bin_dir / "alrun"] + launch + ["--timeout", "60", bin_dir / "recover"], env={"AL_HOST_WAIT_TIMEOUT_S": "30"}, timeout=120)
        assert r.stdout.count("carried on with %d of %d" % (n - 1, n)) == n - 1, r.stdout + r.stderr


@pytest.mark.parametrize("launch", [["-n", "3"], ["-n", "4", "--nodes", "2"]])
def test_data_parallel_training_outlives_a_rank(bin_dir, launch):
    """HostDataParallel.rebuild on the survivors' communicator: training goes on, replicas stay equal."""
    n = int(launch[1])
    r = run([bin_dir / "alrun"] + launch + ["--timeout", "90", sys.executable, W / "host_ddp_recover.py"],
            env={"AL_HOST_WAIT_TIMEOUT_S": "30"}, timeout=180)
    assert r.stdout.count(f"trained on with {n - 1} ranks, steps 6") == n - 1, r.stdout + r.stderr

