"""Worker for the multi-process CPU tests (Gloo): algorithms on a DistMesh, a model step, and
host-side failure detection.  Started by torch.distributed.run."""
import os
import time
import sys
from datetime import timedelta

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    mode = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", timeout=timedelta(seconds=20))
    from meshslice_b200.parallel.mesh import DistMesh, ShardedTensor
    from meshslice_b200.parallel.tensor_parallel import SPMD

    if mode == "algorithms":
        R, C = (2, 2) if world == 4 else (1, world)
        mesh = DistMesh(R, C)
        g = torch.Generator().manual_seed(0)
        X, W = torch.randn(256, 512, generator=g), torch.randn(512, 256, generator=g)
        Y = X @ W
        ok = True
        for alg in ("collective", "meshslice", "wang", "summa") + (("cannon",) if R == C else ()):
            sp = SPMD(mesh, alg, blocksize=8)
            y = mesh.unshard(sp.OS(2)(mesh.shard(X), mesh.shard(W)))
            dx = mesh.unshard(sp.LS(2)(mesh.shard(Y), mesh.shard(W)))
            dw = mesh.unshard(sp.RS(2)(mesh.shard(X), mesh.shard(Y)))
            for got, ref in ((y, Y), (dx, Y @ W.t()), (dw, X.t() @ Y)):
                ok &= bool(torch.allclose(got, ref, rtol=1e-4, atol=1e-3 * ref.abs().max().item()))
        print(f"rank {rank} ALGORITHMS_{'OK' if ok else 'FAILED'}", flush=True)
    elif mode == "model":
        from meshslice_b200.models.gpt import GPTConfig, GPTModel
        R, C = (2, 2) if world == 4 else (1, world)
        mesh = DistMesh(R, C)
        cfg = GPTConfig(n_layers=1, d_model=64, n_heads=4, ffn=256, vocab=300, seq=16, ksplits=(2, 2, 2, 2),
                        head_ksplit=2, vocab_pad=64, dtype=torch.float32)
        model = GPTModel(mesh, cfg)
        ids = torch.randint(0, cfg.vocab, (4, cfg.seq + 1), generator=torch.Generator().manual_seed(1))
        per = 4 // R
        key = (mesh.r, mesh.c)
        tok = ShardedTensor(mesh, {key: ids[mesh.r * per:(mesh.r + 1) * per, :-1].reshape(-1)})
        tgt = ShardedTensor(mesh, {key: ids[mesh.r * per:(mesh.r + 1) * per, 1:].reshape(-1)})
        loss = model.forward_backward(tok, tgt, 4 * cfg.seq).shards[key].clone()
        model.sync_replicated_grads()
        dist.all_reduce(loss, group=mesh.row_groups[mesh.c])
        print(f"rank {rank} MODEL_LOSS {loss.item():.5f}", flush=True)
    elif mode == "peer_leaves":
        # rank 1 leaves between steps; the others learn it from the store before their next step
        from torch.distributed.distributed_c10d import _get_default_store
        from meshslice_b200.utils.health import Heartbeat, PeerLostError, guarded_step
        hb = Heartbeat(_get_default_store(), rank, world)
        x = torch.ones(4)
        for step in range(1, 4):
            if rank == 1 and step == 3:
                hb.leave("simulated failure")
                print("rank 1 LEFT", flush=True)
                os._exit(0)
            try:
                guarded_step(hb, step, lambda: dist.all_reduce(x), timeout_s=5.0)
            except PeerLostError as e:
                print(f"rank {rank} PEER_LOST at step {step}: {e}", flush=True)
                os._exit(0)
        print(f"rank {rank} UNEXPECTED_END", flush=True)
        os._exit(0)
    elif mode == "rank_raises":
        from torch.distributed.distributed_c10d import _get_default_store
        from meshslice_b200.utils.health import Heartbeat, PeerLostError, guarded_step
        hb = Heartbeat(_get_default_store(), rank, world)
        def work():
            if rank == 0:
                raise ValueError("bad shard file")
            return 1
        try:
            guarded_step(hb, 1, work)
        except ValueError:
            print("rank 0 RAISED", flush=True)
            time.sleep(2.0)       # a failing rank takes a moment to tear down; it hosts the store
            os._exit(0)
        except PeerLostError as e:    # rank 0 was already gone when this rank looked before step 1
            print(f"rank {rank} PEER_LOST: {e}", flush=True)
            os._exit(0)
        try:
            guarded_step(hb, 2, lambda: 1, timeout_s=5.0)
        except PeerLostError as e:
            print(f"rank {rank} PEER_LOST: {e}", flush=True)
        os._exit(0)
    elif mode == "status_agreement":
        from meshslice_b200.utils.health import RemoteKernelError, agree_on_status
        agree_on_status(0)                       # nobody failed: no exception anywhere
        try:
            agree_on_status(5 if rank == 1 else 0)   # rank 1's kernel timed out waiting for a chunk
            print(f"rank {rank} MISSED", flush=True)
        except RemoteKernelError as e:
            print(f"rank {rank} AGREED: {e}", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
