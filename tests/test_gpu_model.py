"""GPT training step on one GPU through the native kernels against the CPU oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_training_step_matches_cpu_oracle_and_loss_decreases():
    from meshslice_b200 import _native
    from meshslice_b200.models.gpt import GPTConfig, GPTModel
    from meshslice_b200.parallel.mesh import EmuMesh, ShardedTensor
    from meshslice_b200.trainer import TrainConfig, Trainer

    cfg = GPTConfig(n_layers=2, d_model=256, n_heads=2, ffn=1024, vocab=1000, seq=128, ksplits=(2, 2, 2, 2),
                    vocab_pad=256)
    tr = Trainer(cfg, TrainConfig(global_batch=4, micro_batch=2, lr=1e-3), mesh_shape=(1, 1))
    ids = torch.randint(0, cfg.vocab, (4, cfg.seq + 1), generator=torch.Generator().manual_seed(0))
    # CPU oracle with the same weights (fp32 math on the bf16-rounded parameters)
    import dataclasses
    ocfg = dataclasses.replace(cfg, dtype=torch.float32)
    omesh = EmuMesh(1, 1)
    oracle = GPTModel(omesh, ocfg)
    for (_, p, _, _), (_, q, _, _) in zip(tr.model.parameters(), oracle.parameters()):
        q.shards[(0, 0)].copy_(p.shards[(0, 0)].float().cpu())
    tok = ShardedTensor(omesh, {(0, 0): ids[:, :-1].reshape(-1)})
    tgt = ShardedTensor(omesh, {(0, 0): ids[:, 1:].reshape(-1)})
    ref = oracle.forward_backward(tok, tgt, 4 * cfg.seq).shards[(0, 0)].item()
    losses = [tr.train_step(ids.pin_memory()) for _ in range(4)]
    tr.check()
    assert abs(losses[0] - ref) < 0.05, (losses[0], ref)
    assert losses[-1] < losses[0]
    assert _native.load().launch_count() > 0
