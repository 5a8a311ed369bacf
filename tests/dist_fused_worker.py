"""Worker of the multi-GPU tests: run under torchrun, one rank per GPU.  MODE selects the part:

  gemm    fused OS / LS / RS kernels (and the SUMMA / Wang / Cannon schedules of OS) against the dense
          fp32 product of the global operands; every product runs twice and must be bit-identical
  ops     LayerNorm forward / backward and vocabulary-parallel cross-entropy with the in-kernel row
          exchange against a single-device fp32 formulation of the global tensors
  p2p     stand-alone peer-to-peer all-gather / reduce-scatter / send-recv against torch
  train   a few optimizer steps of a small GPT; rank 0 writes the loss curve to $OUT as JSON
"""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    mode = os.environ.get("MODE", "gemm")
    R, C = [int(v) for v in os.environ.get("MESH", f"1x{world}").split("x")]
    fails = []
    try:
        _run(mode, R, C, rank, world, fails)
    except Exception as e:     # a kernel status error or a plan error: say which rank and what
        import traceback
        fails.append(f"{type(e).__name__}: {e}")
        print(f"rank {rank} EXCEPTION {type(e).__name__}: {e}\n{traceback.format_exc(limit=6)}", flush=True)
        # the other ranks may be inside kernels that wait for this one: they give up at their own
        # bounded waits; nothing more can be agreed on
        os._exit(1)
    t = torch.tensor([len(fails)], device="cuda")
    if world > 1:
        dist.all_reduce(t)
    if fails:
        print(f"rank {rank} FAIL: {fails}", flush=True)
    if rank == 0:
        print("FUSED_MULTI_GPU_OK" if t.item() == 0 else "FUSED_MULTI_GPU_FAILED", flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    sys.exit(0 if t.item() == 0 else 1)


def _run(mode, R, C, rank, world, fails):
    if mode == "train":
        train(R, C, rank, world)
    else:
        from meshslice_b200.parallel.engine import FusedEngine
        from meshslice_b200.parallel.mesh import DistMesh
        mesh = DistMesh(R, C)
        big = os.environ.get("BIG", "0") == "1"
        ws = (512 << 20) if big else (64 << 20)
        eng = FusedEngine(mesh, ws, ws, ws, timeout_ns=int(os.environ.get("TIMEOUT_NS", "2000000000")), exchange_rows=8192,
                          extra_heap_bytes=(32 << 20) * (2 + max(R, C)) if mode == "p2p" else 0)
        {"gemm": gemm, "ops": ops, "p2p": p2p}[mode](mesh, eng, fails, big)


def _close(fails, name, out, ref, K):
    err = (out.float() - ref).abs().max().item()
    rel = ((out.float() - ref).norm() / ref.norm()).item()
    if not (err < 0.03 * K ** 0.5 + 0.05 and rel < 1.5e-2):
        fails.append(f"{name}: err {err} rel {rel}")


def gemm(mesh, eng, fails, big):
    R, C, r, c = mesh.R, mesh.C, mesh.r, mesh.c
    dev = torch.device("cuda")
    slices = int(os.environ.get("SLICES", "2"))
    g = torch.Generator(device="cpu").manual_seed(7)
    u = 2 if big else 1          # BIG: shapes of the size class of a transformer layer on 8 GPUs

    def twice(name, fn):
        a = fn().clone()
        eng.check()
        b = fn()
        eng.check()
        if not torch.equal(a, b):
            fails.append(f"{name}: two runs differ in {(a != b).sum().item()} elements")
        return b

    for rep in range(2):
        # OS
        M, Kd, N = 512 * R * u, 2048 * u, 512 * C * u
        X = torch.randn(M, Kd, generator=g).bfloat16().to(dev)
        W = torch.randn(Kd, N, generator=g).bfloat16().to(dev)
        m, kl, kr, n = M // R, Kd // C, Kd // R, N // C
        xl = X[r * m:(r + 1) * m, c * kl:(c + 1) * kl].contiguous()
        wl = W[r * kr:(r + 1) * kr, c * n:(c + 1) * n].contiguous()
        ref = (X.float() @ W.float())[r * m:(r + 1) * m, c * n:(c + 1) * n]
        _close(fails, "os", twice("os", lambda: eng.os(xl, wl, n_slices=slices)), ref, Kd)
        # the same product on the K-panel schedules of the baseline algorithms
        for order in ("summa", "wang") + (("cannon",) if R == C else ()):
            _close(fails, "os_" + order, twice("os_" + order, lambda: eng.os_kpanel(xl, wl, order=order, sub=2)), ref, Kd)
        # LS
        M, Kd, N = 256 * R * u, 256 * C * u, 512 * R * C
        X = torch.randn(M, Kd, generator=g).bfloat16().to(dev)
        W = torch.randn(N, Kd, generator=g).bfloat16().to(dev)
        m, kl, nr, nc = M // R, Kd // C, N // R, N // C
        xl = X[r * m:(r + 1) * m, c * kl:(c + 1) * kl].contiguous()
        wl = W[r * nr:(r + 1) * nr, c * kl:(c + 1) * kl].contiguous()
        ref = (X.float() @ W.float().t())[r * m:(r + 1) * m, c * nc:(c + 1) * nc]
        _close(fails, "ls", twice("ls", lambda: eng.ls(xl, wl, n_slices=slices)), ref, Kd)
        # RS
        Kd, M, N = 320 * R * u, 512 * R * C, 256 * C * u
        X = torch.randn(Kd, M, generator=g).bfloat16().to(dev)
        W = torch.randn(Kd, N, generator=g).bfloat16().to(dev)
        kr, ml, mr, n = Kd // R, M // C, M // R, N // C
        xl = X[r * kr:(r + 1) * kr, c * ml:(c + 1) * ml].contiguous()
        wl = W[r * kr:(r + 1) * kr, c * n:(c + 1) * n].contiguous()
        ref = (X.float().t() @ W.float())[r * mr:(r + 1) * mr, c * n:(c + 1) * n]
        _close(fails, "rs", twice("rs", lambda: eng.rs(xl, wl, n_slices=slices)), ref, Kd)
        # RS accumulating into an fp32 gradient buffer
        acc = torch.ones(mr, n, device=dev, dtype=torch.float32)
        eng.rs(xl, wl, n_slices=slices, out=acc, accumulate=True)
        eng.check()
        _close(fails, "rs_acc_fp32", acc - 1.0, ref, Kd)


def ops(mesh, eng, fails, big):
    """Column-sharded LayerNorm and cross-entropy whose row statistics travel inside the kernels."""
    from meshslice_b200.models.sharded_layers import ShardedLayerNorm
    from meshslice_b200.ops import functional as F
    from meshslice_b200.parallel.mesh import ShardedTensor
    R, C, r, c = mesh.R, mesh.C, mesh.r, mesh.c
    if C == 1:
        return
    dev = torch.device("cuda")
    g = torch.Generator(device="cpu").manual_seed(11)
    rows, D = 1024, 256 * C
    dl = D // C
    for rep in range(3):             # consecutive exchanges alternate between the two slot sets
        x = torch.randn(rows, D, generator=g).bfloat16().to(dev)
        res = torch.randn(rows, D, generator=g).bfloat16().to(dev)
        dy = torch.randn(rows, D, generator=g).bfloat16().to(dev)
        gamma = (1 + 0.1 * torch.randn(D, generator=g)).bfloat16().to(dev)
        beta = (0.1 * torch.randn(D, generator=g)).bfloat16().to(dev)
        ln = ShardedLayerNorm(mesh, D, affine=True, eps=1e-5, device=dev)
        key = (r, c)
        ln.gamma.shards[key].copy_(gamma[c * dl:(c + 1) * dl])
        ln.bias.shards[key].copy_(beta[c * dl:(c + 1) * dl])
        sh = lambda t: ShardedTensor(mesh, {key: t[:, c * dl:(c + 1) * dl].contiguous()})
        y = ln.forward(sh(x), sh(res)).shards[key]
        dx = ln.backward(sh(dy)).shards[key]
        eng.check()
        hf = (x.float() + res.float()).bfloat16().float().requires_grad_(True)
        gf, bf = gamma.float().requires_grad_(True), beta.float().requires_grad_(True)
        yr = torch.nn.functional.layer_norm(hf, (D,), gf, bf, 1e-5)
        yr.backward(dy.float())
        if (y.float() - yr.detach()[:, c * dl:(c + 1) * dl]).abs().max().item() > 0.06:
            fails.append(f"ln fwd rep {rep}: {(y.float() - yr.detach()[:, c * dl:(c + 1) * dl]).abs().max().item()}")
        if (dx.float() - hf.grad[:, c * dl:(c + 1) * dl]).abs().max().item() > 0.06:
            fails.append(f"ln bwd rep {rep}: {(dx.float() - hf.grad[:, c * dl:(c + 1) * dl]).abs().max().item()}")
        dg = ln.dgamma.shards[key]
        if (dg - gf.grad[c * dl:(c + 1) * dl]).abs().max().item() > 0.02 * rows ** 0.5:
            fails.append(f"ln dgamma rep {rep}")
        # cross-entropy over a column-sharded vocabulary (the last slice is partly padding)
        V, vocab = 512 * C, 512 * C - 100
        logits = (3 * torch.randn(rows, V, generator=g)).bfloat16().to(dev)
        tgt = torch.randint(0, vocab, (rows,), generator=g).to(dev)
        vc = V // C
        ll = logits[:, c * vc:(c + 1) * vc].contiguous()
        from meshslice_b200 import _native
        prod, cons = eng.row_exchange.next(rows, _native.load().ce_grid(rows))
        F.ce_partial(ll, tgt, c * vc, vocab, exch=prod)
        row_loss = F.ce_grad_exchanged_(ll, tgt, c * vc, vocab, 1.0 / rows, cons)
        eng.check()
        lf = logits.float()[:, :vocab].requires_grad_(True)
        lr = torch.nn.functional.cross_entropy(lf, tgt, reduction="none")
        lr.mean().backward()
        if (row_loss - lr.detach()).abs().max().item() > 2e-3:
            fails.append(f"ce loss rep {rep}: {(row_loss - lr.detach()).abs().max().item()}")
        gref = torch.zeros(rows, V, device=dev)
        gref[:, :vocab] = lf.grad
        if (ll.float() - gref[:, c * vc:(c + 1) * vc]).abs().max().item() > 2e-5 + 1e-2 / rows:
            fails.append(f"ce grad rep {rep}: {(ll.float() - gref[:, c * vc:(c + 1) * vc]).abs().max().item()}")


def p2p(mesh, eng, fails, big):
    from meshslice_b200.parallel.collectives import P2PCollectives
    coll = P2PCollectives(mesh, eng.heap, 32 << 20)
    dev = torch.device("cuda")
    rank = mesh.r * mesh.C + mesh.c
    for axis in ("col", "row"):
        peers = coll._peers(axis)
        n = len(peers)
        if n == 1:
            continue
        me = peers.index(rank)
        rows, cols = 64 * n, 256 * n
        full = [torch.randn(rows, cols, generator=torch.Generator().manual_seed(100 + q)).bfloat16().to(dev) for q in peers]
        for dim in (0, 1):
            coll.input((rows, cols)).copy_(full[me])
            coll.barrier()
            for push in (True, False):
                out = coll.all_gather(rows, cols, axis, dim, push=push)
                eng.check()
                if not torch.equal(out, torch.cat(full, dim=dim)):
                    fails.append(f"all_gather {axis} dim {dim} push={push}")
                coll.barrier()
            out = coll.reduce_scatter(rows, cols, axis, dim)
            eng.check()
            tot = sum(t.float() for t in full)
            ref = tot.chunk(n, dim=dim)[me]
            if (out.float() - ref).abs().max().item() > 0.05 * n ** 0.5:
                fails.append(f"reduce_scatter {axis} dim {dim}")
            coll.barrier()
        coll.input((rows, cols)).copy_(full[me])
        coll.barrier()
        for push in (True, False):
            out = coll.send_recv(rows, cols, axis, push=push)
            eng.check()
            if not torch.equal(out, full[(me - 1) % n]):
                fails.append(f"send_recv {axis} push={push}")
            coll.barrier()


def train(R, C, rank, world):
    from meshslice_b200.models.gpt import GPTConfig
    from meshslice_b200.trainer import TrainConfig, Trainer
    cfg = GPTConfig(n_layers=2, d_model=2048, n_heads=16, ffn=8192, vocab=8000, seq=256, ksplits=(2, 2, 2, 2),
                    head_ksplit=2)
    gb = 16
    tr = Trainer(cfg, TrainConfig(global_batch=gb, micro_batch=min(gb // R, 8), lr=3e-4), mesh_shape=(R, C))
    losses = []
    for step in range(int(os.environ.get("STEPS", "4"))):
        ids = torch.randint(0, cfg.vocab, (gb, cfg.seq + 1), generator=torch.Generator().manual_seed(500 + step % 2))
        losses.append(tr.train_step(tr.rows_of_global_batch(ids).contiguous().pin_memory()))
        tr.check(all_ranks=True)
    if rank == 0:
        with open(os.environ["OUT"], "w") as f:
            json.dump({"mesh": [R, C], "losses": losses,
                       "fallbacks": getattr(tr.engine, "fallbacks", 0)}, f)


if __name__ == "__main__":
    main()
