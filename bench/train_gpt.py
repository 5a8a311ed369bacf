#!/usr/bin/env python
"""GPT training entry point: synthetic token ids, AdamW, per-step JSONL metrics, periodic
per-coordinate checkpoints with resume.

    python bench/train_gpt.py --layers 4 --steps 20                                  # one GPU
    torchrun --nproc-per-node 8 bench/train_gpt.py --mesh 2x4 --layers 32 --steps 10 \
        --tuned-json tuned.json --log train.jsonl --ckpt-dir ckpt --ckpt-every 5
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--mesh", default="")
    p.add_argument("--layers", type=int, default=32)
    p.add_argument("--d_model", type=int, default=4096)
    p.add_argument("--nheads", type=int, default=32)
    p.add_argument("--ffn", type=int, default=16384)
    p.add_argument("--vocab", type=int, default=50257)
    p.add_argument("--seqlen", type=int, default=2048)
    p.add_argument("--batchsize", type=int, default=32)
    p.add_argument("--micro-batch", type=int, default=0)
    p.add_argument("--steps", type=int, default=10)
    p.add_argument("--lr", type=float, default=1e-4)
    p.add_argument("--ksplit", type=int, nargs=4, default=[4, 4, 4, 4])
    p.add_argument("--alg", default="meshflow", choices=["meshflow", "collective"])
    p.add_argument("--tuned-json", default="", help="autotuner output: per-layer dataflow and slice count")
    p.add_argument("--log", default="")
    p.add_argument("--ckpt-dir", default="")
    p.add_argument("--ckpt-every", type=int, default=0)
    p.add_argument("--resume-step", type=int, default=-1)
    p.add_argument("--peer-timeout", type=float, default=60.0,
                   help="seconds a rank waits for its peers' heartbeat before a step")
    p.add_argument("--trace", default="", help="write a Chrome trace of the last step here (rank 0)")
    a = p.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    from meshslice_b200.checkpoint import load_checkpoint, save_checkpoint
    from meshslice_b200.models.gpt import GPTConfig
    from meshslice_b200.trainer import TrainConfig, Trainer, choose_mesh
    from meshslice_b200.utils.logging import RunLogger
    from meshslice_b200.utils.timing import DeviceTimer, annotate, trace

    R, C = [int(v) for v in a.mesh.split("x")] if a.mesh else choose_mesh(world)
    dataflows, ksplits = ("os", "os", "os", "ls"), tuple(a.ksplit)
    if a.tuned_json:
        tuned = json.load(open(a.tuned_json))
        if tuned.get("mesh") and not a.mesh:
            R, C = tuned["mesh"]
        if len(tuned.get("layers", [])) == 4:
            dataflows = tuple(l["dataflow"] for l in tuned["layers"])
            ksplits = tuple(int(l["ksplit"] or 1) for l in tuned["layers"])
    cfg = GPTConfig(n_layers=a.layers, d_model=a.d_model, n_heads=a.nheads, ffn=a.ffn, vocab=a.vocab, seq=a.seqlen,
                    dataflows=dataflows, ksplits=ksplits)
    rows_batch = a.batchsize // R
    mb = a.micro_batch or min(rows_batch, 4 * C)
    tr = Trainer(cfg, TrainConfig(global_batch=a.batchsize, micro_batch=mb, lr=a.lr,
                                  backend="fused" if a.alg == "meshflow" else "collective"), mesh_shape=(R, C))
    log = RunLogger(a.log or None, rank)
    log.log("config", mesh=f"{R}x{C}", layers=a.layers, d_model=a.d_model, params=cfg.n_params(),
            global_batch=a.batchsize, micro_batch=mb, dataflows=str(dataflows), ksplits=str(ksplits))
    start = 0
    if a.ckpt_dir and a.resume_step >= 0:
        load_checkpoint(a.ckpt_dir, a.resume_step, tr.model, tr.opt)
        start = a.resume_step
        log.log("resume", step=start)
    hb = None
    if world > 1:
        # between steps every rank publishes its step counter in the job's store and looks at its
        # peers' entries, so a rank that left or raised is reported before the next fused launch
        from torch.distributed.distributed_c10d import _get_default_store
        from meshslice_b200.utils.health import Heartbeat, guarded_step
        hb = Heartbeat(_get_default_store(), rank, world)
    for step in range(start, a.steps):
        # the batch of step k depends on k only, so a resumed run continues the same data stream
        g = torch.Generator().manual_seed(1234 + step)
        ids = torch.randint(0, cfg.vocab, (a.batchsize, cfg.seq + 1), generator=g)
        ids = tr.rows_of_global_batch(ids).contiguous().pin_memory()
        last = step == a.steps - 1
        with trace(a.trace if (last and rank == 0) else None), annotate("train_step"), DeviceTimer() as t:
            if hb is not None:
                loss = guarded_step(hb, step + 1, lambda: tr.train_step(ids), timeout_s=a.peer_timeout)
            else:
                loss = tr.train_step(ids)
        tr.check(all_ranks=True)      # a kernel error of any rank raises on every rank
        log.log("step", step=step + 1, loss=loss, ms=t.ms, tokens_per_s=tr.n_tokens / (t.ms * 1e-3),
                tflops_per_gpu=tr.tflops(t.ms) / world,
                grad_norm=float(tr.opt.last_grad_norm) if tr.opt.last_grad_norm is not None else -1.0)
        if a.ckpt_dir and a.ckpt_every and (step + 1) % a.ckpt_every == 0:
            save_checkpoint(a.ckpt_dir, step + 1, tr.model, tr.opt, rank0=rank == 0,
                            extra={"data_seed": 1234, "next_step": step + 1},
                            barrier=dist.barrier if world > 1 else None)
            log.log("checkpoint", step=step + 1)
    log.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
