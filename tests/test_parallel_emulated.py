"""Parallelism helpers (tensor / sequence / Ulysses / expert / context-ring) on emulated ranks of one
GPU, each checked against the same computation done on a single device."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
P = 4


@pytest.fixture(scope="module")
def comm():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import aluminum_b200 as al
    al.init()
    c = al.DeviceComm(emulate=P)
    yield c
    c.close()


def test_tensor_parallel_linear(comm):
    from aluminum_b200.parallel.tensor import column_parallel_linear, row_parallel_linear
    torch.manual_seed(0)
    x = torch.randn(6, 32, device="cuda")
    w = torch.randn(64, 32, device="cuda")
    want = x @ w.t()
    ys = column_parallel_linear(comm, [x.clone() for _ in range(P)], list(w.chunk(P, dim=0)))
    for y in ys:
        torch.testing.assert_close(y, want, rtol=1e-4, atol=1e-4)
    ys = row_parallel_linear(comm, list(x.chunk(P, dim=1)), list(w.chunk(P, dim=1)))
    for y in ys:
        torch.testing.assert_close(y, want, rtol=1e-4, atol=1e-4)


def test_sequence_parallel(comm):
    from aluminum_b200.parallel.sequence import gather_sequence, scatter_sequence
    full = torch.randn(16, 8, device="cuda")
    shards = [s.contiguous() for s in full.chunk(P, dim=0)]
    for g in gather_sequence(comm, shards):
        assert torch.equal(g, full)
    for g in gather_sequence(comm, shards, out_dtype=torch.bfloat16):   # cast fused into the gather
        torch.testing.assert_close(g, full.to(torch.bfloat16))
    partials = [torch.randn(16, 8, device="cuda") for _ in range(P)]
    total = torch.stack(partials).sum(0)
    for r, s in enumerate(scatter_sequence(comm, partials)):
        torch.testing.assert_close(s, total.chunk(P, dim=0)[r], rtol=1e-5, atol=1e-5)


def test_ulysses_roundtrip(comm):
    from aluminum_b200.parallel.ulysses import head_to_seq, seq_to_head
    s, h, d = 8, 8, 4
    full = torch.randn(s * P, h, d, device="cuda")
    shards = [t.contiguous() for t in full.chunk(P, dim=0)]
    heads = seq_to_head(comm, shards)
    for r in range(P):
        assert torch.equal(heads[r], full[:, r * (h // P):(r + 1) * (h // P)])
    back = head_to_seq(comm, heads)
    for r in range(P):
        assert torch.equal(back[r], shards[r])


def test_expert_dispatch_combine(comm):
    from aluminum_b200.parallel.expert import combine, dispatch
    torch.manual_seed(1)
    toks = [torch.randn(10 + r, 16, device="cuda") for r in range(P)]
    dests = [torch.randint(0, P, (t.shape[0],), device="cuda") for t in toks]
    got, state = dispatch(comm, toks, dests)
    for d in range(P):
        want = torch.cat([toks[r][torch.argsort(dests[r], stable=True)][torch.sort(dests[r], stable=True).values == d]
                          for r in range(P)])
        assert torch.equal(got[d], want)
    back = combine(comm, [g * 2 for g in got], state)
    for r in range(P):
        torch.testing.assert_close(back[r], toks[r] * 2)


def test_ring_attention(comm):
    from aluminum_b200.parallel.context import ring_attention
    torch.manual_seed(2)
    s, h, d = 6, 2, 8
    q, k, v = (torch.randn(s * P, h, d, device="cuda") for _ in range(3))
    scores = torch.einsum("qhd,khd->qhk", q, k) / math.sqrt(d)
    want = torch.einsum("qhk,khd->qhd", torch.softmax(scores, dim=-1), v)
    outs = ring_attention(comm, [t.contiguous() for t in q.chunk(P)], [t.contiguous() for t in k.chunk(P)],
                          [t.contiguous() for t in v.chunk(P)])
    for r in range(P):
        torch.testing.assert_close(outs[r], want.chunk(P)[r], rtol=1e-4, atol=1e-4)
