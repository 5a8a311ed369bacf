"""tcgen05 flash attention forward / backward against the plain PyTorch fp32 formulation."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(qkv, batch, seq, heads, causal, dout):
    D = 128
    x = qkv.float().clone().requires_grad_(True)
    t = x.view(batch, seq, heads, 3, D)
    q, k, v = (t[:, :, :, i].permute(0, 2, 1, 3) for i in range(3))
    s = q @ k.transpose(-1, -2) / math.sqrt(D)
    if causal:
        s = s.masked_fill(torch.ones(seq, seq, dtype=torch.bool, device=s.device).triu(1), float("-inf"))
    lse = torch.logsumexp(s, -1)
    o = (torch.softmax(s, -1) @ v).permute(0, 2, 1, 3).reshape(batch * seq, heads * D)
    o.backward(dout.float())
    return o.detach(), lse.detach(), x.grad


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", [(1, 128, 1), (2, 256, 2), (2, 512, 3), (1, 2048, 2)])
def test_attention_fwd_bwd(shape, causal):
    from meshslice_b200 import _native
    from meshslice_b200.ops import functional as F
    batch, seq, heads = shape
    g = torch.Generator(device="cuda").manual_seed(seq + heads)
    qkv = torch.randn(batch * seq, heads * 3 * 128, device="cuda", generator=g).bfloat16()
    dout = torch.randn(batch * seq, heads * 128, device="cuda", generator=g).bfloat16()
    out, lse = F.attention_fwd(qkv, batch, seq, heads, causal)
    _native.check_status()
    o_ref, lse_ref, dqkv_ref = _ref(qkv, batch, seq, heads, causal, dout)
    assert (out.float() - o_ref).abs().max().item() < 0.03
    assert (lse - lse_ref).abs().max().item() < 0.02
    dqkv = F.attention_bwd(dout, qkv, out, lse, batch, seq, heads, causal)
    _native.check_status()
    err = (dqkv.float() - dqkv_ref).abs().max().item()
    rel = ((dqkv.float() - dqkv_ref).norm() / dqkv_ref.norm()).item()
    assert err < 0.15 and rel < 2e-2, (err, rel)


def test_attention_large_scores_exercise_rescaling():
    """Scores that grow along the keys force the running maximum (and O) to be rescaled."""
    from meshslice_b200 import _native
    from meshslice_b200.ops import functional as F
    batch, seq, heads = 1, 512, 1
    qkv = torch.randn(batch * seq, 3 * 128, device="cuda").bfloat16()
    ramp = torch.linspace(0.2, 3.0, seq, device="cuda")[:, None]
    qkv[:, 128:256] = (qkv[:, :128].float().mean(0, keepdim=True) * ramp * 4).bfloat16()
    dout = torch.randn(batch * seq, 128, device="cuda").bfloat16()
    out, lse = F.attention_fwd(qkv, batch, seq, heads, False)
    _native.check_status()
    o_ref, lse_ref, _ = _ref(qkv, batch, seq, heads, False, dout)
    assert (out.float() - o_ref).abs().max().item() < 0.05
    assert (lse - lse_ref).abs().max().item() < 0.05


def test_attention_backward_is_bit_identical_from_run_to_run():
    """dQ, dK and dV are accumulated in tensor memory by the CTA that owns them, never added to
    global memory from several CTAs: the same inputs give the same bits."""
    from meshslice_b200 import _native
    from meshslice_b200.ops import functional as F
    batch, seq, heads = 2, 1024, 4
    g = torch.Generator(device="cuda").manual_seed(5)
    qkv = torch.randn(batch * seq, heads * 3 * 128, device="cuda", generator=g).bfloat16()
    dout = torch.randn(batch * seq, heads * 128, device="cuda", generator=g).bfloat16()
    out, lse = F.attention_fwd(qkv, batch, seq, heads, True)
    a = F.attention_bwd(dout, qkv, out, lse, batch, seq, heads, True).clone()
    b = F.attention_bwd(dout, qkv, out, lse, batch, seq, heads, True)
    _native.check_status()
    assert torch.equal(a, b)
