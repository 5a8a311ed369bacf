#!/usr/bin/env python
"""Headline benchmark: GPT-3-6.7B-shaped decoder training step on 1/2/4/8 B200 (2-D tensor
parallelism, mesh 1x1 / 1x2 / 2x2 / 2x4), synthetic uniform-random token ids, random-init
weights, bf16 with fp32 AdamW master weights, global batch 32 x 2048 tokens at every N
(strong scaling; micro-batches accumulate gradients).

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 3 --warmup 3

Rank 0 prints one JSON line.  ``value`` is the model TFLOP/s of the whole job, timed on the
device (CUDA events, max over ranks) with the token ids already resident on the GPU; ``e2e`` is
the same metric through ``Trainer.train_step`` with the per-step host-to-device copy of the ids
from pinned memory and the device-to-host read of the loss inside the timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="meshslice_b200", choices=["meshslice_b200", "reference", "collective"])
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--d-model", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--ffn", type=int, default=16384)
    ap.add_argument("--vocab", type=int, default=50257)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--global-batch", type=int, default=32)
    ap.add_argument("--micro-batch", type=int, default=0, help="sequences per mesh row per micro-batch (0: auto)")
    ap.add_argument("--mesh", default="", help="RxC (default 1x1, 1x2, 2x2, 2x4 by GPU count)")
    ap.add_argument("--ksplit", type=int, nargs=4, default=[4, 4, 4, 4])
    ap.add_argument("--no-e2e", action="store_true")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_ids=None):
        """``gpu_ids``: nvidia-smi identifiers (UUIDs or indices) of the GPUs of this job; the
        other GPUs of a shared box idle at low clocks and would drag the median down."""
        self.proc = None
        self.gpu_ids = list(gpu_ids or [])
        self.path = f"/tmp/bench_clocks_{os.getpid()}.csv"

    def start(self):
        try:
            self.f = open(self.path, "w")
            sel = ["-i", ",".join(self.gpu_ids)] if self.gpu_ids else []
            self.proc = subprocess.Popen(["nvidia-smi", *sel, f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            p = [x.strip() for x in line.split(",")]
            if len(p) < 9:
                continue
            try:
                sm.append(float(p[1]))
                mx.append(float(p[2]))
            except ValueError:
                continue
            for n, v in zip(names, p[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if sm:
            out = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                   "samples": len(sm)}
        try:
            os.remove(self.path)
        except OSError:
            pass
        return out


def main():
    args = parse()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "reference is a JAX/TPU script collection without setup.py/pyproject (pip install "
                          "refused: not installable) and jax is not installed nor in the offline wheelhouse"}))
        return 0

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if rank == 0:
            print(f"bench.py: --gpus {args.gpus} but WORLD_SIZE={world}; launch with torchrun", file=sys.stderr)
        return 2
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    from meshslice_b200 import _native
    from meshslice_b200.models.gpt import GPTConfig
    from meshslice_b200.trainer import TrainConfig, Trainer, choose_mesh

    mesh_shape = tuple(int(v) for v in args.mesh.split("x")) if args.mesh else choose_mesh(world)
    R, C = mesh_shape
    cfg = GPTConfig(n_layers=args.layers, d_model=args.d_model, n_heads=args.heads, ffn=args.ffn, vocab=args.vocab,
                    seq=args.seq, ksplits=tuple(args.ksplit), causal=True)
    rows_batch = args.global_batch // R
    mb = args.micro_batch or min(rows_batch, 4 * C)
    tcfg = TrainConfig(global_batch=args.global_batch, micro_batch=mb,
                       backend="collective" if args.impl == "collective" else "fused")
    trainer = Trainer(cfg, tcfg, mesh_shape=mesh_shape)

    # synthetic data: uniform-random ids, one pinned host buffer per step slot (cycled)
    g = torch.Generator().manual_seed(1234)
    n_slots = 4
    host = [torch.randint(0, cfg.vocab, (args.global_batch, cfg.seq + 1), generator=g)[
        trainer.r * rows_batch:(trainer.r + 1) * rows_batch].contiguous().pin_memory() for _ in range(n_slots)]
    dev = [h.to(trainer.device) for h in host]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(n_steps, e2e):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        last = None
        for i in range(n_steps):
            if e2e:
                last = trainer.train_step(host[i % n_slots], read_loss=True)
            else:
                last = trainer.train_step(dev[i % n_slots], read_loss=False)
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=trainer.device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item() / n_steps, last

    for i in range(args.warmup):
        trainer.train_step(dev[i % n_slots], read_loss=False)
    trainer.check()

    def _uuid(i):
        u = str(torch.cuda.get_device_properties(i).uuid)
        return u if u.startswith("GPU-") else "GPU-" + u
    try:       # the job's ranks use the first `world` visible devices of this node
        ids = [_uuid(i) for i in range(min(world, torch.cuda.device_count()))]
    except Exception:
        ids = [str(i) for i in range(world)]
    sampler = ClockSampler(ids)
    C_ = _native.load()
    if rank == 0:
        sampler.start()
    l0 = C_.launch_count()
    ms, last = timed(args.steps, e2e=False)
    launches = C_.launch_count() - l0
    clocks = sampler.stop() if rank == 0 else {}
    trainer.check()
    loss_val = float(last.item())
    e2e = None
    if not args.no_e2e:
        ms_e, loss_e = timed(args.steps, e2e=True)
        trainer.check()
        e2e = {"value": trainer.tflops(ms_e), "unit": "TFLOP/s", "ms_per_step": ms_e,
               "h2d_bytes_per_step": int(host[0].numel() * 8 * world), "d2h_bytes_per_step": 4 * world,
               "loss": loss_e}
    if rank == 0:
        tf = trainer.tflops(ms)
        out = {"metric": "gpt3_6.7b_train_model_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": world,
               "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
               "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
               "impl": args.impl, "tflops_per_gpu": tf / world,
               "tokens_per_s": trainer.n_tokens / (ms * 1e-3), "loss": loss_val,
               "config": {"model": f"gpt3-{args.layers}L-d{args.d_model}-h{args.heads}-ffn{args.ffn}-v{args.vocab}",
                          "global_batch": args.global_batch, "seq_len": args.seq,
                          "parallelism": f"2d-tp mesh {R}x{C}", "micro_batch_per_row": mb,
                          "optimizer": "AdamW fp32 master lr1e-4 b(0.9,0.95)", "ksplit": list(args.ksplit),
                          "l2_policy": "inputs larger than L2 (activations and weights are GBs per step)"},
               "clocks": clocks, "gpu_launches": int(launches)}
        if e2e is not None:
            out["e2e"] = e2e
        try:   # library / eager paths taken instead of the package's own kernels (0 unless a fallback was allowed)
            from meshslice_b200.ops import functional as _F
            out["fallbacks"] = int(getattr(getattr(trainer, "engine", None), "fallbacks", 0) or 0) + \
                int(sum(_F.FALLBACKS.values()))
        except Exception:
            pass
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
