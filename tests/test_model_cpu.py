"""GPT model and the reference-style Transformer block on emulated CPU meshes against a dense
fp32 PyTorch model built from the same (unsharded) weights."""
import math

import pytest
import torch

from meshslice_b200.models.gpt import GPTConfig, GPTModel
from meshslice_b200.models.sharded_layers import ShardedFFLayer, TransformerBlock
from meshslice_b200.parallel.mesh import EmuMesh, ShardedTensor

CFG = GPTConfig(n_layers=2, d_model=128, n_heads=4, ffn=512, vocab=1000, seq=32, ksplits=(2, 2, 2, 2),
                head_ksplit=2, vocab_pad=256, dtype=torch.float32, causal=True)


def _full(mesh, st):
    return mesh.unshard(st)


def _cols(mesh, st):
    return torch.cat([st.shards[(0, c)] for c in range(mesh.C)], dim=-1)


def _dense_loss(model, mesh, cfg, ids):
    """Plain PyTorch forward of the same network with autograd."""
    P = {}
    def leaf(t):
        t = t.clone().float().requires_grad_(True)
        return t
    P["tok"], P["pos"] = leaf(_cols(mesh, model.tok)), leaf(_cols(mesh, model.pos))
    x = P["tok"][ids[:, :-1].reshape(-1)] + P["pos"][torch.arange(ids.shape[0] * cfg.seq) % cfg.seq]
    H, D = cfg.n_heads, cfg.d_model // cfg.n_heads
    Bsz = ids.shape[0]
    def ln(v, layer, tag):
        g, b = leaf(_cols(mesh, layer.gamma)), leaf(_cols(mesh, layer.bias))
        P[tag + ".g"], P[tag + ".b"] = g, b
        return torch.nn.functional.layer_norm(v, (cfg.d_model,), g, b, cfg.eps)
    def lin(v, layer, tag):
        w = leaf(_full(mesh, layer.weight))
        P[tag] = w
        return v @ (w.t() if layer.dataflow == "ls" else w)
    for i, blk in enumerate(model.blocks):
        y = ln(x, blk.ln1, f"{i}.ln1")
        qkv = lin(y, blk.in_proj, f"{i}.in").view(Bsz, cfg.seq, H, 3, D)
        q, k, v = (qkv[:, :, :, j].permute(0, 2, 1, 3) for j in range(3))
        s = q @ k.transpose(-1, -2) / math.sqrt(D)
        s = s.masked_fill(torch.ones(cfg.seq, cfg.seq, dtype=torch.bool).triu(1), float("-inf"))
        a = (torch.softmax(s, -1) @ v).permute(0, 2, 1, 3).reshape(Bsz * cfg.seq, H * D)
        x = x + lin(a, blk.out_proj, f"{i}.out")
        y = ln(x, blk.ln2, f"{i}.ln2")
        m = lin(torch.nn.functional.gelu(lin(y, blk.ff1, f"{i}.ff1"), approximate="tanh"), blk.ff2, f"{i}.ff2")
        x = x + m
    y = ln(x, model.ln_f, "lnf")
    logits = lin(y, model.head, "head")[:, :cfg.vocab]
    loss = torch.nn.functional.cross_entropy(logits, ids[:, 1:].reshape(-1))
    loss.backward()
    return loss, P


@pytest.mark.parametrize("shape", [(1, 1), (2, 2), (2, 4), (4, 1)])
def test_gpt_loss_and_grads_match_dense_model(shape):
    R, C = shape
    mesh = EmuMesh(R, C)
    model = GPTModel(mesh, CFG)
    B = 4
    ids = torch.randint(0, CFG.vocab, (B, CFG.seq + 1), generator=torch.Generator().manual_seed(1))
    per = B // R
    tok = ShardedTensor(mesh, {(r, c): ids[r * per:(r + 1) * per, :-1].reshape(-1) for (r, c) in mesh.coords()})
    tgt = ShardedTensor(mesh, {(r, c): ids[r * per:(r + 1) * per, 1:].reshape(-1) for (r, c) in mesh.coords()})
    loss = model.forward_backward(tok, tgt, B * CFG.seq)
    model.sync_replicated_grads()
    total = sum(loss.shards[(r, 0)] for r in range(R))
    ref, P = _dense_loss(model, mesh, CFG, ids)
    assert abs(total.item() - ref.item()) < 1e-4
    b0 = model.blocks[0]
    for layer, tag in ((b0.in_proj, "0.in"), (b0.out_proj, "0.out"), (b0.ff1, "0.ff1"), (b0.ff2, "0.ff2"),
                       (model.head, "head")):
        got = _full(mesh, layer.grad)
        assert torch.allclose(got, P[tag].grad, atol=2e-5, rtol=1e-3), tag
    assert torch.allclose(_cols(mesh, b0.ln1.dgamma), P["0.ln1.g"].grad, atol=2e-5, rtol=1e-3)
    assert torch.allclose(_cols(mesh, b0.ln2.dbias), P["0.ln2.b"].grad, atol=2e-5, rtol=1e-3)
    assert torch.allclose(_cols(mesh, model.dtok), P["tok"].grad, atol=2e-5, rtol=1e-3)
    assert torch.allclose(_cols(mesh, model.dpos), P["pos"].grad, atol=2e-5, rtol=1e-3)


@pytest.mark.parametrize("dataflow", ["os", "ls", "rs"])
def test_ff_layer_forward_backward_each_dataflow(dataflow):
    """ShardedLayers.py:41-81: forward, dX and dW of every dataflow against dense autograd."""
    mesh = EmuMesh(2, 4)
    T, I, O = 64, 128, 256
    layer = ShardedFFLayer(mesh, "meshslice", dataflow, 2, I, O, blocksize=8, dtype=torch.float32)
    W = _full(mesh, layer.weight).clone().requires_grad_(True)
    g = torch.Generator().manual_seed(3)
    X = torch.randn(T, I, generator=g, requires_grad=True)
    Yd = X @ (W.t() if dataflow == "ls" else W)
    dY = torch.randn(T, O, generator=g)
    Yd.backward(dY)
    xin = mesh.shard(X.detach().t().contiguous() if dataflow == "rs" else X.detach())
    y = layer.forward(xin)
    assert torch.allclose(_full(mesh, y), Yd.detach(), atol=1e-4, rtol=1e-4)
    dx = layer.backward(mesh.shard(dY))
    dxf = _full(mesh, dx)
    assert torch.allclose(dxf.t() if dataflow == "rs" else dxf, X.grad, atol=1e-4, rtol=1e-4)
    assert torch.allclose(_full(mesh, layer.grad), W.grad, atol=1e-4, rtol=1e-4)


def test_reference_transformer_block_forward_backward():
    """The reference block (norm1..norm3, non-causal attention, no affine) vs dense autograd."""
    mesh = EmuMesh(2, 2)
    S, H, D, B = 16, 4, 16, 4
    blk = TransformerBlock(mesh, S, H, D, ["os", "os", "os", "ls"], alg="meshflow", ksplits=(2, 2, 2, 2),
                           dtype=torch.float32, std=0.05)
    g = torch.Generator().manual_seed(0)
    X = torch.randn(B * S, H * D, generator=g, requires_grad=True)
    dY = torch.randn(B * S, H * D, generator=g)
    Ws = {n: _full(mesh, getattr(blk, n).weight) for n in ("in_proj", "out_proj", "ff1", "ff2")}
    def ln(v):
        mu = v.mean(-1, keepdim=True)
        return (v - mu) / torch.sqrt((v * v).mean(-1, keepdim=True) - mu * mu + 1e-6)
    o = ln(X) @ Ws["in_proj"]
    qkv = o.view(B, S, H, 3, D)
    q, k, v = (qkv[:, :, :, j].permute(0, 2, 1, 3) for j in range(3))
    a = (torch.softmax(q @ k.transpose(-1, -2) / math.sqrt(D), -1) @ v).permute(0, 2, 1, 3).reshape(B * S, H * D)
    res = ln(a @ Ws["out_proj"] + X)
    o = torch.nn.functional.gelu(res @ Ws["ff1"], approximate="tanh") @ Ws["ff2"].t()
    Yd = ln(o + res)
    Yd.backward(dY)
    y = blk.forward(mesh.shard(X.detach()))
    assert torch.allclose(_full(mesh, y), Yd.detach(), atol=2e-4, rtol=1e-3)
    dx = blk.backward(mesh.shard(dY))
    assert torch.allclose(_full(mesh, dx), X.grad, atol=2e-4, rtol=1e-3)


def test_initial_weights_do_not_depend_on_the_mesh_shape():
    ref = GPTModel(EmuMesh(1, 1), CFG)
    want = {n: (p.shards[(0, 0)], k) for n, p, _, k in ref.parameters()}
    for shape in ((1, 2), (2, 2), (2, 4), (4, 1)):
        mesh = EmuMesh(*shape)
        for n, p, _, k in GPTModel(mesh, CFG).parameters():
            got = _full(mesh, p) if k == "sharded" else _cols(mesh, p)
            assert torch.equal(got, want[n][0]), (shape, n)


def test_loss_curve_is_the_same_on_every_mesh_shape():
    """Four optimizer steps from the same initial weights on the same batches: the loss of every
    step agrees across 1x1, 1x2, 2x2 and 2x4 (fp32 on the emulated mesh: to rounding)."""
    from meshslice_b200.optim import AdamW, FlatGroup
    from meshslice_b200.trainer import Arena, param_elems
    curves = {}
    for shape in ((1, 1), (1, 2), (2, 2), (2, 4)):
        R, C = shape
        mesh = EmuMesh(R, C)
        n_sh, n_rep = (n * R * C for n in param_elems(CFG, R, C))
        bufs = [torch.zeros(n_sh), torch.zeros(n_sh), torch.zeros(n_rep), torch.zeros(n_rep)]
        a = [Arena(t) for t in bufs]
        model = GPTModel(mesh, CFG, alloc_sharded=a[0].alloc, grad_sharded=a[1].alloc, alloc_rep=a[2].alloc,
                         grad_rep=a[3].alloc)
        opt = AdamW([FlatGroup(bufs[0], bufs[1], "sharded"), FlatGroup(bufs[2], bufs[3], "row_replicated")],
                    lr=1e-3, max_grad_norm=None)
        B, losses = 4, []
        for step in range(4):
            ids = torch.randint(0, CFG.vocab, (B, CFG.seq + 1), generator=torch.Generator().manual_seed(50 + step % 2))
            per = B // R
            tok = ShardedTensor(mesh, {(r, c): ids[r * per:(r + 1) * per, :-1].reshape(-1) for (r, c) in mesh.coords()})
            tgt = ShardedTensor(mesh, {(r, c): ids[r * per:(r + 1) * per, 1:].reshape(-1) for (r, c) in mesh.coords()})
            loss = model.forward_backward(tok, tgt, B * CFG.seq)
            model.sync_replicated_grads()
            opt.step()
            opt.zero_grad()
            losses.append(sum(loss.shards[(r, 0)] for r in range(R)).item())
        curves[shape] = losses
    ref = curves[(1, 1)]
    assert ref[2] < ref[0] and ref[3] < ref[1]      # the two batches repeat: the model learns them
    for shape, c in curves.items():
        assert all(abs(x - y) < 2e-4 for x, y in zip(c, ref)), (shape, c, ref)


@pytest.mark.parametrize("dataflow", ["os", "is", "fsdp"])
def test_1d_layers_forward_backward_match_dense(dataflow):
    """BenchTransformer1D.py:21-38: the 1-D linear layers (Wang ring schedule on a 1 x n mesh, FSDP on
    an n x 1 mesh) against dense autograd."""
    from meshslice_b200.models.sharded_layers_1d import ShardedFFLayer1D
    n, T, I, O = 4, 32, 64, 96
    mesh = EmuMesh(n, 1) if dataflow == "fsdp" else EmuMesh(1, n)
    layer = ShardedFFLayer1D(mesh, dataflow, I, O, dtype=torch.float32)
    W = _full(mesh, layer.weight).clone().requires_grad_(True)
    g = torch.Generator().manual_seed(5)
    X = torch.randn(T, I, generator=g, requires_grad=True)
    Yd = X @ (W if dataflow == "os" else W.t())
    dY = torch.randn(T, O, generator=g)
    Yd.backward(dY)
    y = layer.forward(mesh.shard(X.detach()))
    assert torch.allclose(_full(mesh, y), Yd.detach(), atol=1e-4, rtol=1e-4)
    dx = layer.backward(mesh.shard(dY))
    assert torch.allclose(_full(mesh, dx), X.grad, atol=1e-4, rtol=1e-4)
    assert torch.allclose(_full(mesh, layer.grad), W.grad, atol=1e-4, rtol=1e-4)
    with pytest.raises(ValueError):
        ShardedFFLayer1D(EmuMesh(2, 2), dataflow, I, O, dtype=torch.float32)


@pytest.mark.parametrize("dataflows", [("rs", "os", "os", "ls"), ("os", "rs", "rs", "rs"), ("ls", "ls", "rs", "os")])
def test_gpt_block_runs_every_dataflow_the_tuner_can_pick(dataflows):
    """Right-stationary layers want transposed activations (Autotuner.py:304-337); the block
    re-orients around them, so any per-layer choice of os / ls / rs gives the dense model's loss
    and gradients."""
    import dataclasses
    cfg = dataclasses.replace(CFG, dataflows=dataflows, n_layers=1)
    mesh = EmuMesh(2, 4)
    model = GPTModel(mesh, cfg)
    B = 4
    ids = torch.randint(0, cfg.vocab, (B, cfg.seq + 1), generator=torch.Generator().manual_seed(2))
    per = B // mesh.R
    tok = ShardedTensor(mesh, {(r, c): ids[r * per:(r + 1) * per, :-1].reshape(-1) for (r, c) in mesh.coords()})
    tgt = ShardedTensor(mesh, {(r, c): ids[r * per:(r + 1) * per, 1:].reshape(-1) for (r, c) in mesh.coords()})
    loss = model.forward_backward(tok, tgt, B * cfg.seq)
    total = sum(loss.shards[(r, 0)] for r in range(mesh.R))

    class View:                                    # the dense oracle multiplies by W or W^T by dataflow
        pass
    ref, P = _dense_loss(model, mesh, cfg, ids)
    assert abs(total.item() - ref.item()) < 1e-4
    b0 = model.blocks[0]
    for layer, tag in ((b0.in_proj, "0.in"), (b0.out_proj, "0.out"), (b0.ff1, "0.ff1"), (b0.ff2, "0.ff2")):
        assert torch.allclose(_full(mesh, layer.grad), P[tag].grad, atol=2e-5, rtol=1e-3), tag


def test_mesh_transpose_is_the_global_transpose():
    for shape in ((2, 4), (4, 2), (3, 2), (1, 4)):
        mesh = EmuMesh(*shape)
        X = torch.arange(24 * 48, dtype=torch.float32).reshape(24, 48)
        assert torch.equal(mesh.unshard(mesh.transpose(mesh.shard(X))), X.t())
