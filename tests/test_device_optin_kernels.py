"""The opt-in kernels on ONE GPU with emulated ranks: the bulk-copy pipeline
(kernels/bulk_pipeline.cu; tuning entry ``bulk_pipeline`` / ``AL_DEV_BULK_PIPELINE=1``) and the direct
allgather / alltoall into symmetric receive buffers (kernels/direct.cu; ``direct_symmetric`` /
``AL_DEV_DIRECT=1``, with ``direct_bulk`` / ``AL_DEV_DIRECT_BULK=1`` for its copy-engine flavour).

They are off by default and so is this file: it runs only with ``AL_TEST_UNVERIFIED=1`` in the
environment.  Results are compared with plain PyTorch references, exactly as for the generic kernel
in test_device_emulated.py.
"""
import os

import pytest
import torch

pytestmark = [
    pytest.mark.gpu,
    pytest.mark.skipif(os.environ.get("AL_TEST_UNVERIFIED") != "1",
                       reason="opt-in kernel: set AL_TEST_UNVERIFIED=1 to test them"),
]


@pytest.fixture(scope="module")
def al():
    import aluminum_b200 as al
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    al.init()
    old = {k: al.get_tuning(k) for k in ("pipeline_min_bytes", "bulk_pipeline", "direct_symmetric", "direct_bulk")}
    al.set_tuning("pipeline_min_bytes", 16384)
    al.set_tuning("bulk_pipeline", 1)
    yield al
    for k, v in old.items():
        al.set_tuning(k, v)


def rand(n, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randint(-16, 17, (n,), generator=g, device="cuda").float() / 8


@pytest.mark.parametrize("p", [2, 4, 8])
def test_allgather_alltoall_reduce_scatter(al, p):
    comm = al.DeviceComm(emulate=p)
    comm.set_timeout_ms(2000)
    n = 1_500_004  # per-rank slice: a multiple of 16 bytes, of nothing larger
    for it in range(2):
        before = comm.stats()["bulk_pipeline"]
        ss = [rand(n, 300 + r + it) for r in range(p)]
        outs = [torch.zeros(n * p, device="cuda") for _ in range(p)]
        comm.allgather(ss, outs)
        xs = [rand(n * p, 310 + r + it) for r in range(p)]
        rs = [torch.zeros(n, device="cuda") for _ in range(p)]
        comm.reduce_scatter(xs, rs)
        a2 = [torch.zeros(n * p, device="cuda") for _ in range(p)]
        comm.alltoall(xs, a2)
        small = [torch.full((3,), float(r), device="cuda") for r in range(p)]
        comm.allreduce(small)  # the generic kernel right after: both halves must be free again
        torch.cuda.synchronize()
        assert comm.status()["code"] == 0, comm.status()
        assert comm.stats()["bulk_pipeline"] == before + 3
        full = torch.cat(ss)
        want = torch.stack(xs).sum(0)
        for r in range(p):
            assert torch.equal(outs[r], full)
            torch.testing.assert_close(rs[r], want[r * n:(r + 1) * n])
            assert torch.equal(a2[r], torch.cat([xs[q][r * n:(r + 1) * n] for q in range(p)]))
            assert torch.all(small[r] == sum(range(p)))
    comm.close()


def test_bf16_reduce_scatter_and_fallback_for_odd_sizes(al):
    p = 4
    comm = al.DeviceComm(emulate=p)
    comm.set_timeout_ms(2000)
    n = 400_000
    xs = [rand(n * p, 330 + r).to(torch.bfloat16) for r in range(p)]
    rs = [torch.zeros(n, device="cuda", dtype=torch.bfloat16) for _ in range(p)]
    comm.reduce_scatter(xs, rs)
    torch.cuda.synchronize()
    want = torch.stack([x.float() for x in xs]).sum(0)
    for r in range(p):
        torch.testing.assert_close(rs[r].float(), want[r * n:(r + 1) * n], rtol=1e-2, atol=1e-2)
    assert comm.stats()["bulk_pipeline"] == 1
    # a slice that is not a multiple of 16 bytes runs on the generic kernel
    m = 1_500_007
    ss = [rand(m, 340 + r) for r in range(p)]
    outs = [torch.zeros(m * p, device="cuda") for _ in range(p)]
    comm.allgather(ss, outs)
    torch.cuda.synchronize()
    assert comm.stats()["bulk_pipeline"] == 1
    for r in range(p):
        assert torch.equal(outs[r], torch.cat(ss))
    comm.close()


@pytest.mark.parametrize("bulk", [0, 1])
@pytest.mark.parametrize("p", [2, 8])
def test_direct_allgather_alltoall_into_symmetric_buffers(al, p, bulk):
    al.set_tuning("direct_symmetric", 1)
    al.set_tuning("direct_bulk", bulk)
    try:
        comm = al.DeviceComm(emulate=p)
        comm.set_timeout_ms(2000)
        for n in (4, 1000, 1_500_004):  # per-rank slice in floats: multiples of 16 bytes
            outs = comm.symm_empty((n * p,), torch.float32)
            for it in range(2):
                before = comm.stats()["direct"]
                for o in outs:
                    o.fill_(-1.0)
                ss = [rand(n, 400 + r + it) for r in range(p)]
                comm.allgather(ss, outs)
                torch.cuda.synchronize()
                assert comm.status()["code"] == 0, comm.status()
                assert comm.stats()["direct"] == before + 1
                for r in range(p):
                    assert torch.equal(outs[r], torch.cat(ss))
                xs = [rand(n * p, 410 + r + it) for r in range(p)]
                comm.alltoall(xs, outs)
                small = [torch.full((3,), float(r), device="cuda") for r in range(p)]
                comm.allreduce(small)  # a staged operation right after
                torch.cuda.synchronize()
                assert comm.stats()["direct"] == before + 2
                for r in range(p):
                    assert torch.equal(outs[r], torch.cat([xs[q][r * n:(r + 1) * n] for q in range(p)]))
                    assert torch.all(small[r] == sum(range(p)))
            # in-place allgather: every rank's contribution already sits at its place
            for r in range(p):
                outs[r].zero_()
                outs[r][r * n:(r + 1) * n] = float(r + 1)
            comm.allgather([outs[r][r * n:(r + 1) * n] for r in range(p)], outs)
            torch.cuda.synchronize()
            want = torch.cat([torch.full((n,), float(r + 1), device="cuda") for r in range(p)])
            for r in range(p):
                assert torch.equal(outs[r], want)
            # a private receive buffer takes the staged path
            before = comm.stats()["direct"]
            priv = [torch.zeros(n * p, device="cuda") for _ in range(p)]
            comm.allgather([rand(n, 420 + r) for r in range(p)], priv)
            torch.cuda.synchronize()
            assert comm.stats()["direct"] == before
            comm.symm_free(outs)
        comm.close()
    finally:
        al.set_tuning("direct_symmetric", 0)
        al.set_tuning("direct_bulk", 0)
