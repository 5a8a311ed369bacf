"""Checkpoint save / load / re-shard round trips and host-side failure cases."""
import dataclasses
import json
import os

import numpy as np
import pytest
import torch

from meshslice_b200.checkpoint import import_jax_blocks, load_checkpoint, reshard_checkpoint, save_checkpoint
from meshslice_b200.models.gpt import GPTConfig, GPTModel
from meshslice_b200.parallel.mesh import EmuMesh

CFG = GPTConfig(n_layers=1, d_model=64, n_heads=4, ffn=256, vocab=200, seq=16, ksplits=(1, 1, 1, 1),
                head_ksplit=1, vocab_pad=64, dtype=torch.float32)


def _full(mesh, st, kind):
    if kind == "sharded":
        return mesh.unshard(st)
    return torch.cat([st.shards[(0, c)] for c in range(mesh.C)], dim=-1)


def test_save_load_roundtrip_and_layout(tmp_path):
    mesh = EmuMesh(2, 2)
    m1 = GPTModel(mesh, CFG)
    d = save_checkpoint(str(tmp_path), 3, m1, extra={"note": "x"})
    meta = json.load(open(os.path.join(d, "meta.json")))
    assert meta["mesh"] == [2, 2] and meta["step"] == 3
    assert meta["params"]["block0.ShardedFFLayer5.weight"]["dataflow"] == "ls"
    assert meta["params"]["block0.ShardedFFLayer5.weight"]["orientation"] == "[out,in]"
    assert meta["params"]["block0.ShardedFFLayer1.weight"]["global_shape"] == [64, 192]
    blob = torch.load(os.path.join(d, "shard_r1_c0.pt"))
    W = _full(mesh, m1.blocks[0].in_proj.weight, "sharded")
    assert torch.equal(blob["block0.ShardedFFLayer1.weight"], W[32:64, 0:96])      # block (r=1, c=0)
    m2 = GPTModel(mesh, dataclasses.replace(CFG, init_std=0.5))
    load_checkpoint(str(tmp_path), 3, m2)
    for (n, p, _, k), (_, q, _, _) in zip(m1.parameters(), m2.parameters()):
        for key in p.shards:
            assert torch.equal(p.shards[key], q.shards[key]), n


def test_reshard_2x2_to_1x4_and_4x1(tmp_path):
    m1 = GPTModel(EmuMesh(2, 2), CFG)
    save_checkpoint(str(tmp_path / "a"), 1, m1)
    for shape in ((1, 4), (4, 1)):
        out = str(tmp_path / f"b{shape[0]}{shape[1]}")
        reshard_checkpoint(str(tmp_path / "a"), 1, shape, out)
        mesh2 = EmuMesh(*shape)
        m2 = GPTModel(mesh2, CFG)
        load_checkpoint(out, 1, m2)
        for (n, p, _, k), (_, q, _, _) in zip(m1.parameters(), m2.parameters()):
            assert torch.equal(_full(m1.mesh, p, k), _full(mesh2, q, k)), n


def test_load_rejects_mesh_mismatch_missing_and_corrupted_shards(tmp_path):
    m1 = GPTModel(EmuMesh(2, 2), CFG)
    d = save_checkpoint(str(tmp_path), 1, m1)
    with pytest.raises(ValueError):
        load_checkpoint(str(tmp_path), 1, GPTModel(EmuMesh(1, 4), CFG))
    with open(os.path.join(d, "shard_r0_c1.pt"), "wb") as f:
        f.write(b"not a checkpoint")
    with pytest.raises(RuntimeError):
        load_checkpoint(str(tmp_path), 1, GPTModel(EmuMesh(2, 2), CFG))
    os.remove(os.path.join(d, "shard_r0_c1.pt"))
    with pytest.raises(FileNotFoundError):
        load_checkpoint(str(tmp_path), 1, GPTModel(EmuMesh(2, 2), CFG))


def test_import_blocks_exported_per_device_coordinate(tmp_path):
    mesh = EmuMesh(2, 2)
    model = GPTModel(mesh, CFG)
    W = torch.arange(64 * 192, dtype=torch.float32).reshape(64, 192) / 1000
    g = torch.arange(64, dtype=torch.float32)
    for r in range(2):
        for c in range(2):
            np.save(tmp_path / f"in_proj.r{r}.c{c}.npy", W[r * 32:(r + 1) * 32, c * 96:(c + 1) * 96].numpy())
    for c in range(2):
        np.save(tmp_path / f"norm1_gamma.c{c}.npy", g[c * 32:(c + 1) * 32].numpy())
    loaded = import_jax_blocks(str(tmp_path), model, {"block0.ShardedFFLayer1.weight": "in_proj",
                                                      "block0.ShardedLayerNorm0.gamma": "norm1_gamma"})
    assert len(loaded) == 2
    assert torch.equal(mesh.unshard(model.blocks[0].in_proj.weight), W)
    assert torch.equal(model.blocks[0].ln1.gamma.shards[(1, 1)], g[32:])


@pytest.mark.parametrize("chain", [[(1, 1), (2, 2), (4, 1), (1, 2)], [(2, 1), (1, 4), (2, 2), (1, 1)]])
def test_reshard_chains_preserve_every_parameter(tmp_path, chain):
    """Re-sharding through a chain of mesh shapes and back gives bit-identical global parameters."""
    first = GPTModel(EmuMesh(*chain[0]), CFG)
    save_checkpoint(str(tmp_path / "s0"), 7, first)
    prev = str(tmp_path / "s0")
    for i, shape in enumerate(chain[1:], 1):
        out = str(tmp_path / f"s{i}")
        reshard_checkpoint(prev, 7, shape, out)
        prev = out
    mesh = EmuMesh(*chain[-1])
    last = GPTModel(mesh, dataclasses.replace(CFG, init_std=0.3))
    meta = load_checkpoint(prev, 7, last)
    assert meta["step"] == 7 and meta["mesh"] == list(chain[-1])
    for (n, p, _, k), (_, q, _, _) in zip(first.parameters(), last.parameters()):
        assert torch.equal(_full(first.mesh, p, k), _full(mesh, q, k)), n


# ---------------------------------------------------------------------------------------------
# optimizer state: save / resume / re-shard
# ---------------------------------------------------------------------------------------------
from meshslice_b200.optim import AdamW, FlatGroup
from meshslice_b200.parallel.mesh import ShardedTensor
from meshslice_b200.trainer import Arena, param_elems


def _flat_model(shape, cfg=CFG, init_std=None):
    """GPT model of an emulated mesh on flat parameter / gradient buffers with AdamW, the way the
    trainer lays one rank out (here all coordinates share the buffers)."""
    R, C = shape
    mesh = EmuMesh(R, C)
    n_sh, n_rep = param_elems(cfg, R, C)
    n_sh, n_rep = n_sh * R * C, n_rep * R * C
    p_sh, g_sh = torch.zeros(n_sh), torch.zeros(n_sh)
    p_rep, g_rep = torch.zeros(n_rep), torch.zeros(n_rep)
    a = [Arena(t) for t in (p_sh, g_sh, p_rep, g_rep)]
    c = cfg if init_std is None else dataclasses.replace(cfg, init_std=init_std)
    model = GPTModel(mesh, c, alloc_sharded=a[0].alloc, alloc_rep=a[2].alloc, grad_sharded=a[1].alloc,
                     grad_rep=a[3].alloc)
    opt = AdamW([FlatGroup(p_sh, g_sh, "sharded"), FlatGroup(p_rep, g_rep, "row_replicated")], lr=1e-2,
                max_grad_norm=None)
    return mesh, model, opt


def _step(mesh, model, opt, step):
    B = 4
    ids = torch.randint(0, CFG.vocab, (B, CFG.seq + 1), generator=torch.Generator().manual_seed(100 + step))
    per = B // mesh.R
    tok = ShardedTensor(mesh, {(r, c): ids[r * per:(r + 1) * per, :-1].reshape(-1) for (r, c) in mesh.coords()})
    tgt = ShardedTensor(mesh, {(r, c): ids[r * per:(r + 1) * per, 1:].reshape(-1) for (r, c) in mesh.coords()})
    loss = model.forward_backward(tok, tgt, B * CFG.seq)
    model.sync_replicated_grads()
    opt.step()
    opt.zero_grad()
    return sum(loss.shards[(r, 0)] for r in range(mesh.R)).item()


def _globals(mesh, model):
    return {n: _full(mesh, p, k).clone() for n, p, _, k in model.parameters()}


def test_resume_with_optimizer_state_reproduces_the_uninterrupted_run_bit_for_bit(tmp_path):
    mesh, model, opt = _flat_model((2, 2))
    losses = [_step(mesh, model, opt, s) for s in range(2)]
    save_checkpoint(str(tmp_path), 2, model, opt)
    losses += [_step(mesh, model, opt, s) for s in range(2, 4)]
    want = _globals(mesh, model)
    # a fresh process: different initial weights, then resume at step 2
    mesh2, model2, opt2 = _flat_model((2, 2), init_std=0.3)
    meta = load_checkpoint(str(tmp_path), 2, model2, opt2)
    assert meta["has_optimizer"] and opt2.step_count == 2
    resumed = [_step(mesh2, model2, opt2, s) for s in range(2, 4)]
    assert resumed == losses[2:]
    got = _globals(mesh2, model2)
    for n in want:
        assert torch.equal(want[n], got[n]), n


def test_reshard_carries_optimizer_state_and_the_next_step_is_the_adamw_update(tmp_path):
    mesh, model, opt = _flat_model((2, 2))
    for s in range(2):
        _step(mesh, model, opt, s)
    save_checkpoint(str(tmp_path / "a"), 2, model, opt)
    loaded = _globals(mesh, model)
    _step(mesh, model, opt, 2)
    want = _globals(mesh, model)
    reshard_checkpoint(str(tmp_path / "a"), 2, (1, 4), str(tmp_path / "b"))
    mesh2, model2, opt2 = _flat_model((1, 4), init_std=0.3)
    meta = load_checkpoint(str(tmp_path / "b"), 2, model2, opt2)
    assert meta["has_optimizer"] and meta["mesh"] == [1, 4] and opt2.step_count == 2
    for n, t in _globals(mesh2, model2).items():
        assert torch.equal(t, loaded[n]), n
    # moments travelled too: the next step on 1x4 is the step the 2x2 run took
    _step(mesh2, model2, opt2, 2)
    got = _globals(mesh2, model2)
    for n in want:
        assert torch.allclose(want[n], got[n], atol=2e-5, rtol=1e-4), n
        assert not torch.equal(got[n], loaded[n]) or n.endswith("bias"), n


def test_loading_parameters_without_optimizer_state_refreshes_the_master_copies(tmp_path):
    mesh, model, _ = _flat_model((2, 2))
    save_checkpoint(str(tmp_path), 5, model)                       # parameters only
    mesh2, model2, opt2 = _flat_model((2, 2), init_std=0.3)
    load_checkpoint(str(tmp_path), 5, model2, opt2)
    assert opt2.step_count == 5
    for g in opt2.groups:
        assert torch.equal(g.master, g.param.float())
        assert not g.m.any() and not g.v.any()
    before = _globals(mesh2, model2)
    _step(mesh2, model2, opt2, 0)
    after = _globals(mesh2, model2)
    # one AdamW step with lr 1e-2 moves a weight by at most about lr: the loaded weights survive
    for n in before:
        assert (after[n] - before[n]).abs().max() <= 1.01e-2 + 1e-6, n


def test_interrupted_save_has_no_meta_json(tmp_path):
    mesh, model, opt = _flat_model((1, 1))
    class Stop(Exception):
        pass
    def barrier():
        raise Stop()
    with pytest.raises(Stop):
        save_checkpoint(str(tmp_path), 1, model, opt, barrier=barrier)
    assert os.path.exists(tmp_path / "step_1" / "shard_r0_c0.pt")
    assert not os.path.exists(tmp_path / "step_1" / "meta.json")
    with pytest.raises(FileNotFoundError):
        load_checkpoint(str(tmp_path), 1, model, opt)
