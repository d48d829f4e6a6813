"""Headline benchmark: data-parallel ResNet-50 training throughput (images/s).

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
inputs from pinned memory and a device->host read of every step's loss.

--impl reference   the unmodified reference cannot be installed here (it is a CMake
                   project that requires MPI, which this image lacks) -> prints "unavailable".
--impl ddp-nccl    PyTorch DistributedDataParallel over NCCL on the same model and
                   data: the "path that only calls NCCL", kept as a local comparison.
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


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "ddp-nccl"])
    ap.add_argument("--batch", type=int, default=256, help="per-GPU batch")
    ap.add_argument("--no-e2e", action="store_true")
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


def main():
    a = parse()
    if a.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "llnl/Aluminum is a CMake C++ library that hard-requires MPI (none installed, no network); "
                          "pip install of the reference tree fails: neither setup.py nor pyproject.toml"}))
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

    from aluminum_b200.models import resnet50
    model = resnet50().cuda().to(memory_format=torch.channels_last)
    loss_fn = torch.nn.CrossEntropyLoss()
    xh, yh = synthetic_batch(a.batch, 100 + rank, pinned=True)
    xd, yd = xh.cuda(non_blocking=True), yh.cuda(non_blocking=True)

    if a.impl == "ours":
        import aluminum_b200 as al
        from aluminum_b200.parallel import DataParallel, Trainer
        al.init()
        comm = al.DeviceComm() if world > 1 else None
        dp = DataParallel(model, comm, bucket_bytes=25 * 1024 * 1024, lr=0.1, momentum=0.9)
        trainer = Trainer(dp, loss_fn)

        def device_step():
            return trainer.step_device(xd, yd)

        def barrier():
            if comm is not None:
                comm.barrier()
            torch.cuda.synchronize()

        def max_over_ranks(v: float) -> float:
            if comm is None:
                return v
            t = torch.tensor([v], device="cuda", dtype=torch.float32)
            comm.allreduce(t, op="max")
            return float(t.item())
    else:
        import torch.distributed as dist
        if world > 1:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
            ddp = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local], bucket_cap_mb=25,
                                                            gradient_as_bucket_view=True)
        else:
            ddp = model
        opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9)

        def device_step():
            x = xd.contiguous(memory_format=torch.channels_last)
            with torch.autocast("cuda", dtype=torch.bfloat16):
                loss = loss_fn(ddp(x).float(), yd)
            opt.zero_grad(set_to_none=True)
            loss.backward()
            opt.step()
            return loss.detach()

        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        def max_over_ranks(v: float) -> float:
            if world == 1:
                return v
            t = torch.tensor([v], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())

    # ---------------- device-resident measurement -------------------------------------------
    for _ in range(max(a.warmup, 3)):
        device_step()
    barrier()
    launches0 = dp.launches if a.impl == "ours" else 0
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(a.steps):
        device_step()
    e1.record()
    barrier()
    ms = max_over_ranks(e0.elapsed_time(e1))
    clocks = sampler.stop() if rank == 0 else {}
    launches = (dp.launches - launches0) if a.impl == "ours" else 0
    value = a.batch * world * a.steps / (ms / 1e3)

    # ---------------- end-to-end measurement (public API, pinned host -> device each step) ----
    e2e = None
    if a.impl == "ours" and not a.no_e2e:
        def host_batches(n):
            for _ in range(n):
                yield xh, yh
        for _ in trainer.run(host_batches(3)):
            pass
        barrier()
        h0, d0 = trainer.h2d_bytes, trainer.d2h_bytes
        t0 = time.perf_counter()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        last = None
        for last in trainer.run(host_batches(a.steps)):
            pass
        g1.record()
        barrier()
        wall_ms = (time.perf_counter() - t0) * 1e3
        ms_e = max_over_ranks(max(g0.elapsed_time(g1), wall_ms))
        e2e = {"value": a.batch * world * a.steps / (ms_e / 1e3), "unit": "images/s", "ms_per_step": ms_e / a.steps,
               "h2d_bytes_per_step": (trainer.h2d_bytes - h0) // a.steps,
               "d2h_bytes_per_step": (trainer.d2h_bytes - d0) // a.steps, "last_loss": last}

    if rank == 0:
        out = {"metric": "ResNet-50 data-parallel training throughput", "value": value, "unit": "images/s",
               "n_gpus": world, "steps": a.steps, "warmup": max(a.warmup, 3), "ms_per_step": ms / a.steps,
               "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
               "data": "synthetic N(0,1) images, random labels, random-init weights", "impl": a.impl,
               "config": {"model": "resnet50", "global_batch": a.batch * world, "per_gpu_batch": a.batch,
                          "seq_len": None, "image": "3x224x224 fp32", "parallelism": f"dp{world}",
                          "bucket_mb": 25, "optimizer": "sgd momentum 0.9",
                          "l2": "inputs (154 MB per step) and activations exceed the 126 MB L2; no explicit flush"},
               "clocks": clocks, "e2e": e2e, "gpu_launches": launches}
        print(json.dumps(out))
    if a.impl == "ours":
        import aluminum_b200 as al
        if comm is not None:
            comm.close()
        al.finalize()
    elif world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
