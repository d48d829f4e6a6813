"""The opt-in bulk-copy pipeline on ONE GPU with emulated ranks (kernels/bulk_pipeline.cu; tuning entry
``bulk_pipeline`` / ``AL_DEV_BULK_PIPELINE=1``): large uniform reduce_scatter / allgather / alltoall whose
data is moved by the bulk copy engine (cp.async.bulk) instead of SM store loops.  Off by default, switched
on for this file.  Results are compared with plain PyTorch references, exactly as for the generic kernel in
test_device_emulated.py.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def al():
    import aluminum_b200 as al
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    al.init()
    old = {k: al.get_tuning(k) for k in ("pipeline_min_bytes", "bulk_pipeline")}
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
    n = 4_000_000  # 8 MB per rank slice: more than one pipeline chunk
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
