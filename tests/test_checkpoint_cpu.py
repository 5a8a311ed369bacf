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
