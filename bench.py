"""Headline benchmark: data-parallel ResNet-50 training throughput (images/s), plus a collective sweep.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Config (the reference's consumer workload): ResNet-50, batch 256 per GPU, synthetic
3x224x224 fp32 inputs ~ N(0,1) with random labels in 1000 classes, bf16 autocast,
random-initialised weights, gradients in 25 MB fp32 buckets whose allreduce is fused
with the 1/world scale and overlapped with backward, SGD with momentum 0.9.

Rank 0 prints one JSON line.  `value` is measured with the batch resident on the
device and CUDA events around exactly K steps (max over ranks); `e2e.value` goes
through the public `Trainer.run` API with a host->device copy of every step's
inputs from pinned memory and a device->host read of every step's loss.  With two or
more GPUs the line also carries `collectives`: allreduce / reduce_scatter / allgather /
alltoall on fp32 vectors of 1 KiB, 64 KiB, 16 MiB and 1 GiB (20 warm-up + 100 timed
calls each, a host barrier before and a CUDA event pair around every call, per-rank
median, max over ranks) as latency and bus bandwidth.

--impl ours        this library (default).
--impl reference   the unmodified llnl/Aluminum built into baseline/_ref (NCCL backend on a
                   single-node MPI stand-in, see baseline/build_reference.py): same model,
                   same buckets, Al::NonblockingAllreduce<NCCLBackend> + Al::Wait per bucket,
                   torch.optim.SGD; none of this package is imported on that path.
--impl ddp-nccl    PyTorch DistributedDataParallel over NCCL, kept as a local comparison.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

COLL_SIZES = (1024, 65536, 16 << 20, 1 << 30)
COLL_KINDS = ("allreduce", "reduce_scatter", "allgather", "alltoall")


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "ddp-nccl"])
    ap.add_argument("--batch", type=int, default=256, help="per-GPU batch")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-collectives", action="store_true")
    ap.add_argument("--coll-max-bytes", type=int, default=1 << 30, help="largest vector of the collective sweep")
    ap.add_argument("--timeline", type=str, default="", help="(ours) after the timed runs, write a per-bucket timeline of a "
                    "few extra steps to this file: when each gradient bucket was ready, when its average was available")
    return ap.parse_args()


class ClockSampler:
    """nvidia-smi sampling of SM clocks and throttle reasons during the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.idx)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def synthetic_batch(batch: int, seed: int, pinned: bool):
    import torch
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(batch, 3, 224, 224, generator=g, dtype=torch.float32)
    y = torch.randint(0, 1000, (batch,), generator=g, dtype=torch.int64)
    if pinned:
        x, y = x.pin_memory(), y.pin_memory()
    return x, y


def collectives_block(time_fn, world: int, rank_max, max_bytes: int, warmup: int = 20, iters: int = 100) -> dict:
    """``time_fn(kind, total_bytes, warmup, iters) -> [ms per call]`` on this rank; ``rank_max(v)`` = max over ranks.
    A size is the byte length S of the full fp32 vector (allreduce: the vector; reduce_scatter: the input;
    allgather: the output; alltoall: either buffer).  Bus bandwidth: allreduce S/t*2(p-1)/p, the others S/t*(p-1)/p."""
    out = {"protocol": f"{warmup} warm-up + {iters} timed calls per size; host barrier before and CUDA event pair "
                       "around every call; per-rank median, max over ranks; fp32 sum; private (unregistered) buffers"}
    for kind in COLL_KINDS:
        rows = {}
        for s in COLL_SIZES:
            if s > max_bytes:
                continue
            ms = time_fn(kind, s, warmup, iters)
            med = rank_max(statistics.median(ms))
            factor = 2.0 * (world - 1) / world if kind == "allreduce" else (world - 1) / world
            rows[str(s)] = {"us": round(med * 1e3, 2), "bus_gbs": round(s / (med * 1e-3) * factor / 1e9, 1)}
        out[kind] = rows
    return out


class CollBuffers:
    """Two fp32 device vectors of the largest sweep size, with random contents."""

    def __init__(self, max_bytes: int, seed: int):
        import torch
        g = torch.Generator(device="cuda").manual_seed(seed)
        self.send = torch.rand(max_bytes // 4, device="cuda", generator=g, dtype=torch.float32) * 2 - 1
        self.recv = torch.empty(max_bytes // 4, device="cuda", dtype=torch.float32)

    def args(self, kind: str, total_bytes: int, world: int):
        """(send view, recv view, element count the operation takes)."""
        n = total_bytes // 4
        per = max(1, n // world)
        if kind == "allreduce":
            return self.send[:n], self.recv[:n], n
        if kind == "reduce_scatter":
            return self.send[:per * world], self.recv[:per], per
        if kind == "allgather":
            return self.send[:per], self.recv[:per * world], per
        return self.send[:per * world], self.recv[:per * world], per


# ------------------------------------------------------------------------------------------------------
# arms
# ------------------------------------------------------------------------------------------------------
class OursArm:
    name = "ours"

    def __init__(self, a, rank, world, local):
        import torch
        import aluminum_b200 as al
        from aluminum_b200.models import resnet50
        from aluminum_b200.parallel import DataParallel, Trainer
        self.torch, self.al, self.world = torch, al, world
        al.init()
        model = resnet50().cuda().to(memory_format=torch.channels_last)
        self.comm = al.DeviceComm() if world > 1 else None
        self.dp = DataParallel(model, self.comm, bucket_bytes=25 * 1024 * 1024, lr=0.1, momentum=0.9)
        self.trainer = Trainer(self.dp, torch.nn.CrossEntropyLoss())
        from aluminum_b200 import _lib
        self.native = [str(_lib.lib_path())]

    def device_step(self, x, y):
        return self.trainer.step_device(x, y)

    def barrier(self):
        if self.comm is not None:
            self.comm.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, v: float) -> float:
        if self.comm is None:
            return v
        t = self.torch.tensor([v], device="cuda", dtype=self.torch.float32)
        self.comm.allreduce(t, op="max")
        return float(t.item())

    def launches(self) -> int:
        return self.dp.launches

    def run(self, batches):
        return self.trainer.run(batches)

    def io_bytes(self):
        return self.trainer.h2d_bytes, self.trainer.d2h_bytes

    def time_collective(self, bufs, kind, total_bytes, warmup, iters):
        s, r, n = bufs.args(kind, total_bytes, self.world)
        return self.comm.time_collective(kind, s, r, n, warmup, iters)

    def close(self):
        if self.comm is not None:
            self.comm.close()
        self.al.finalize()


class ReferenceArm:
    name = "reference"

    def __init__(self, a, rank, world, local):
        import torch
        import torchvision
        from baseline import ref_bench
        self.torch, self.world = torch, world
        self.al = ref_bench.RefAl(local)
        self.comm = self.al.comm(torch.cuda.current_stream())
        if self.comm.size != world:
            raise RuntimeError(f"reference world size {self.comm.size} != {world}")
        model = torchvision.models.resnet50().cuda().to(memory_format=torch.channels_last)
        self.trainer = ref_bench.RefTrainer(model, self.comm, lr=0.1, momentum=0.9)
        self.native = [str(ref_bench.DRIVER)]

    def device_step(self, x, y):
        return self.trainer.step_device(x, y)

    def barrier(self):
        self.torch.cuda.synchronize()
        self.comm.host_barrier()

    def max_over_ranks(self, v: float) -> float:
        return self.comm.host_max(v)

    def launches(self) -> int:
        return 0

    def run(self, batches):
        return self.trainer.run(batches)

    def io_bytes(self):
        return self.trainer.h2d_bytes, self.trainer.d2h_bytes

    def time_collective(self, bufs, kind, total_bytes, warmup, iters):
        s, r, n = bufs.args(kind, total_bytes, self.world)
        return self.comm.time_collective(kind, s, r, n, warmup, iters)

    def close(self):
        self.torch.cuda.synchronize()
        self.comm.close()
        self.al.finalize()


class DdpNcclArm:
    name = "ddp-nccl"

    def __init__(self, a, rank, world, local):
        import torch
        import torch.distributed as dist
        from aluminum_b200.models import resnet50
        self.torch, self.dist, self.world = torch, dist, world
        model = resnet50().cuda().to(memory_format=torch.channels_last)
        if world > 1:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
            self.ddp = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local], bucket_cap_mb=25,
                                                                 gradient_as_bucket_view=True)
        else:
            self.ddp = model
        self.opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9)
        self.loss_fn = torch.nn.CrossEntropyLoss()
        self.native = []

    def device_step(self, x, y):
        torch = self.torch
        x = x.contiguous(memory_format=torch.channels_last)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = self.loss_fn(self.ddp(x).float(), y)
        self.opt.zero_grad(set_to_none=True)
        loss.backward()
        self.opt.step()
        return loss.detach()

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, v: float) -> float:
        if self.world == 1:
            return v
        t = self.torch.tensor([v], device="cuda")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def launches(self) -> int:
        return 0

    run = None
    time_collective = None

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def main():
    a = parse()
    if a.impl == "reference":
        from baseline import ref_bench
        why = ref_bench.unavailable_reason()
        if why:
            print(json.dumps({"impl": "reference", "unavailable": why}))
            return 0

    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != a.gpus and rank == 0:
        print(f"warning: --gpus {a.gpus} but WORLD_SIZE={world}", file=sys.stderr)
    torch.cuda.set_device(local)
    torch.backends.cudnn.benchmark = True
    torch.manual_seed(1234)

    arm = {"ours": OursArm, "reference": ReferenceArm, "ddp-nccl": DdpNcclArm}[a.impl](a, rank, world, local)
    xh, yh = synthetic_batch(a.batch, 100 + rank, pinned=True)
    xd, yd = xh.cuda(non_blocking=True), yh.cuda(non_blocking=True)
    warmup = max(a.warmup, 3)

    # ---------------- device-resident measurement -------------------------------------------
    for _ in range(warmup):
        arm.device_step(xd, yd)
    arm.barrier()
    launches0 = arm.launches()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    arm.barrier()
    e0.record()
    for _ in range(a.steps):
        arm.device_step(xd, yd)
    e1.record()
    arm.barrier()
    ms = arm.max_over_ranks(e0.elapsed_time(e1))
    clocks = sampler.stop() if rank == 0 else {}
    launches = arm.launches() - launches0
    value = a.batch * world * a.steps / (ms / 1e3)

    # ---------------- end-to-end measurement (public API, pinned host -> device each step) ----
    e2e = None
    if arm.run is not None and not a.no_e2e:
        def host_batches(n):
            for _ in range(n):
                yield xh, yh
        for _ in arm.run(host_batches(3)):
            pass
        arm.barrier()
        h0, d0 = arm.io_bytes()
        t0 = time.perf_counter()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        last = None
        for last in arm.run(host_batches(a.steps)):
            pass
        g1.record()
        arm.barrier()
        wall_ms = (time.perf_counter() - t0) * 1e3
        ms_e = arm.max_over_ranks(max(g0.elapsed_time(g1), wall_ms))
        h1, d1 = arm.io_bytes()
        e2e = {"value": a.batch * world * a.steps / (ms_e / 1e3), "unit": "images/s", "ms_per_step": ms_e / a.steps,
               "h2d_bytes_per_step": (h1 - h0) // a.steps, "d2h_bytes_per_step": (d1 - d0) // a.steps,
               "last_loss": last}

    # ---------------- collective sweep (first half of the metric) --------------------------------
    collectives = None
    if world > 1 and arm.time_collective is not None and not a.no_collectives:
        del xd, yd
        torch.cuda.empty_cache()
        try:  # the training figures above stand on their own: a failure here is reported, not fatal
            bufs = CollBuffers(min(a.coll_max_bytes, max(COLL_SIZES)), 7 + rank)
            torch.cuda.synchronize()
            collectives = collectives_block(lambda k, s, w, i: arm.time_collective(bufs, k, s, w, i), world,
                                            arm.max_over_ranks, a.coll_max_bytes)
        except Exception as e:  # noqa: BLE001
            collectives = {"error": f"{type(e).__name__}: {e}"[:300]}

    if a.timeline and a.impl == "ours" and world > 1:
        dp = arm.dp
        dp.timeline = True
        xd2, yd2 = xh.cuda(non_blocking=True), yh.cuda(non_blocking=True)
        recs = []
        for i in range(6):
            dp.mark_step_start()
            arm.device_step(xd2, yd2)
            r = dp.collect_timeline()
            if i >= 2 and r is not None:
                recs.append(r)
        dp.timeline = False
        tails = [arm.max_over_ranks(r["exposed_tail_ms"]) for r in recs]
        if rank == 0:
            with open(a.timeline, "w") as f:
                json.dump({"n_gpus": world, "exposed_tail_ms_max_over_ranks": tails, "rank0_steps": recs}, f, indent=1)

    if rank == 0:
        out = {"metric": "ResNet-50 data-parallel training throughput", "value": value, "unit": "images/s",
               "n_gpus": world, "steps": a.steps, "warmup": warmup, "ms_per_step": ms / a.steps,
               "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
               "data": "synthetic N(0,1) images, random labels, random-init weights", "impl": a.impl,
               "config": {"model": "resnet50", "global_batch": a.batch * world, "per_gpu_batch": a.batch,
                          "seq_len": None, "image": "3x224x224 fp32", "parallelism": f"dp{world}",
                          "bucket_mb": 25, "optimizer": "sgd momentum 0.9",
                          "l2": "inputs (154 MB per step) and activations exceed the 126 MB L2; no explicit flush"},
               "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "native_libraries": arm.native}
        if collectives is not None:
            out["collectives"] = collectives
        print(json.dumps(out))
    arm.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
