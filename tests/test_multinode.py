"""Worlds that span several nodes, modelled on one machine: `alrun --nodes K` gives consecutive
blocks of ranks different node names and selects the TCP transport, so ranks of different blocks
cannot share memory or pass descriptors and every byte between them crosses a socket."""
import subprocess
import sys
from pathlib import Path

import pytest

W = Path(__file__).resolve().parent / "workers"

ALL_OPS = ["allreduce", "reduce", "reduce_scatter", "reduce_scatterv", "allgather", "allgatherv", "alltoall",
           "alltoallv", "bcast", "gather", "gatherv", "scatter", "scatterv", "barrier", "send", "sendrecv",
           "multisendrecv"]


def run(cmd, env=None, timeout=300):
    import os
    e = dict(os.environ)
    e.update(env or {})
    return subprocess.run([str(c) for c in cmd], capture_output=True, text=True, timeout=timeout, env=e)


@pytest.mark.parametrize("op", ALL_OPS)
def test_every_operation_across_nodes(bin_dir, op):
    for extra in ([], ["--inplace", "--nonblocking"]):
        r = run([bin_dir / "alrun", "-n", "4", "--nodes", "2", "--timeout", "120", bin_dir / "test_ops", "--backend", "host",
                 "--op", op, "--max-size", "262144", "--odd-sizes", "--zero", "--root", "2"] + extra)
        assert r.returncode == 0 and ": ok" in r.stdout, r.stdout + r.stderr


@pytest.mark.parametrize("ranks,nodes,dtype,rop", [(3, 3, "half", "sum"), (5, 2, "int", "max"), (8, 2, "float", "avg"),
                                                   (6, 3, "bfloat16", "sum"), (4, 4, "ullong", "bxor"),
                                                   (5, 5, "double", "prod")])
def test_reductions_across_nodes(bin_dir, ranks, nodes, dtype, rop):
    for op in ("allreduce", "reduce", "reduce_scatterv"):
        r = run([bin_dir / "alrun", "-n", str(ranks), "--nodes", str(nodes), "--timeout", "120", bin_dir / "test_ops",
                 "--backend", "host", "--op", op, "--datatype", dtype, "--reduction-op", rop, "--max-size", "300000",
                 "--odd-sizes", "--root", "1"])
        assert r.returncode == 0 and ": ok" in r.stdout, r.stdout + r.stderr


def test_large_messages_across_nodes(bin_dir):
    """Sizes beyond the socket buffers: partial writes and reads on every connection."""
    for op in ("allreduce", "bcast", "alltoall", "sendrecv"):
        r = run([bin_dir / "alrun", "-n", "4", "--nodes", "2", "--timeout", "200", bin_dir / "test_ops", "--backend", "host",
                 "--op", op, "--min-size", "4194304", "--max-size", "8388608", "--odd-sizes"])
        assert r.returncode == 0 and ": ok" in r.stdout, r.stdout + r.stderr


def test_threads_and_permuted_ranks_across_nodes(bin_dir):
    r = run([bin_dir / "alrun", "-n", "4", "--nodes", "2", "--timeout", "120", bin_dir / "test_ops", "--backend", "host",
             "--op", "alltoallv", "--threads", "3", "--nonblocking", "--permute", "3,1,0,2", "--max-size", "65536"])
    assert r.returncode == 0 and "threads=3: ok" in r.stdout, r.stdout + r.stderr


def test_node_local_and_cross_node_communicators(bin_dir):
    r = run([bin_dir / "alrun", "-n", "6", "--nodes", "2", "--timeout", "120", sys.executable, W / "host_multinode.py", "hier"])
    assert r.returncode == 0 and r.stdout.count("hierarchical ok") == 6, r.stdout + r.stderr


def test_dead_rank_is_reported_by_its_connections(bin_dir):
    r = run([bin_dir / "alrun", "-n", "4", "--nodes", "2", "--timeout", "120", sys.executable, W / "host_multinode.py", "dead"],
            env={"AL_HOST_WAIT_TIMEOUT_S": "5"})
    assert r.stdout.count("detected the dead rank") == 3, r.stdout + r.stderr


def test_mismatched_sizes_are_reported(bin_dir):
    r = run([bin_dir / "alrun", "-n", "2", "--nodes", "2", "--timeout", "60", sys.executable, W / "host_multinode.py",
             "mismatch"], env={"AL_HOST_WAIT_TIMEOUT_S": "3"})
    assert "mismatch reported" in r.stdout, r.stdout + r.stderr


def test_examples_across_nodes(bin_dir):
    r = run([bin_dir / "alrun", "-n", "3", "--nodes", "3", bin_dir / "hello_world"])
    assert r.returncode == 0 and r.stdout.count("sum of ranks = 3") == 3, r.stdout + r.stderr
    r = run([bin_dir / "alrun", "-n", "2", "--nodes", "2", bin_dir / "pingpong"])
    assert r.returncode == 0 and "per round trip" in r.stdout, r.stdout + r.stderr
    r = run([bin_dir / "alrun", "-n", "4", "--nodes", "2", bin_dir / "test_exchange", "--peers", "2", "--size", "5000"])
    assert r.returncode == 0 and ": ok" in r.stdout, r.stdout + r.stderr


def test_rendezvous_times_out_without_rank_zero(bin_dir):
    env = {"AL_RANK": "1", "AL_WORLD_SIZE": "2", "AL_TRANSPORT": "tcp", "MASTER_ADDR": "127.0.0.1", "AL_MASTER_PORT": "1",
           "AL_JOB_KEY": "nobody-home", "AL_BOOTSTRAP_TIMEOUT_S": "1"}
    r = run([bin_dir / "test_ops", "--backend", "host", "--op", "barrier"], env=env, timeout=60)
    assert r.returncode != 0 and "could not reach the rendezvous" in r.stderr, r.stdout + r.stderr


@pytest.mark.parametrize("launch", [["-n", "3"], ["-n", "4", "--nodes", "2"]])
def test_data_parallel_training_on_cpu_ranks(bin_dir, launch):
    """Bucketed, overlapped gradient averaging on the progress thread reproduces full-batch training."""
    r = run([bin_dir / "alrun", *launch, "--timeout", "200", sys.executable, W / "host_ddp_worker.py"])
    assert r.returncode == 0 and r.stdout.count("data parallel on CPU ok") == int(launch[1]), r.stdout + r.stderr


def test_two_level_path_is_taken_for_small_messages(bin_dir, tmp_path):
    """Several ranks per node: small allreduce / bcast and barriers are composed of node-level
    (shared memory) and leader-level (socket) operations; large ones use the flat socket path."""
    env = {"AL_TRACE": "1", "AL_TRACE_DIR": str(tmp_path)}
    for op in ("allreduce", "bcast", "barrier"):
        for extra in ([], ["--inplace", "--nonblocking"]):
            r = run([bin_dir / "alrun", "-n", "6", "--nodes", "2", "--timeout", "120", bin_dir / "test_ops", "--backend",
                     "host", "--op", op, "--max-size", "65536", "--odd-sizes", "--zero", "--root", "4"] + extra, env=env)
            assert r.returncode == 0 and ": ok" in r.stdout, r.stdout + r.stderr
    text = "".join(f.read_text() for f in tmp_path.glob("*.trace.txt"))
    # small messages and (over the rails) large allreduce: composites; large bcast: flat sockets
    for name in ("HierAllreduce", "HierBcast", "HierBarrier", "NetBcast"):
        assert name in text, name
    r = run([bin_dir / "alrun", "-n", "6", "--nodes", "3", "--timeout", "120", bin_dir / "test_ops", "--backend", "host",
             "--op", "allreduce", "--max-size", "4096", "--threads", "2", "--nonblocking"], env={"AL_HOST_TWO_LEVEL": "0"})
    assert r.returncode == 0 and ": ok" in r.stdout, r.stdout + r.stderr
    # uneven nodes (3 + 2 members): no rails, large allreduce falls back to the flat path; tiny staging: many chunks
    for launch, env2 in ((["-n", "5", "--nodes", "2"], {}), (["-n", "6", "--nodes", "2"], {"AL_HOST_STAGE_BYTES": "65536"})):
        r = run([bin_dir / "alrun", *launch, "--timeout", "120", bin_dir / "test_ops", "--backend", "host", "--op",
                 "allreduce", "--max-size", "1048576", "--odd-sizes", "--inplace"], env=env2)
        assert r.returncode == 0 and ": ok" in r.stdout, r.stdout + r.stderr
