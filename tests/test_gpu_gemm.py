"""tcgen05 GEMM kernel against a plain PyTorch fp32 reference of the same product."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, layout):
    a32, b32 = a.float(), b.float()
    if layout == "nn":
        return a32 @ b32
    if layout == "nt":
        return a32 @ b32.t()
    return a32.t() @ b32


def _operands(M, N, K, layout, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    sa = (M, K) if layout != "tn" else (K, M)
    sb = (K, N) if layout != "nt" else (N, K)
    a = torch.randn(sa, device="cuda", generator=g).bfloat16()
    b = torch.randn(sb, device="cuda", generator=g).bfloat16()
    return a, b


def _check(out, ref, K):
    err = (out.float() - ref).abs().max().item()
    tol = 0.02 * (K ** 0.5) + 1e-2
    assert err < tol, f"max abs err {err} > {tol}"
    rel = (out.float() - ref).norm() / ref.norm()
    assert rel < 1e-2, f"relative error {rel}"


@pytest.mark.parametrize("layout", ["nt", "nn", "tn"])
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 256), (384, 768, 1024), (200, 264, 72),
                                   (1024, 1024, 4096)])
def test_gemm_matches_fp32_reference(layout, shape):
    from meshslice_b200 import _native
    from meshslice_b200.ops.gemm import gemm
    M, N, K = shape
    a, b = _operands(M, N, K, layout)
    out = gemm(a, b, layout)
    _native.check_status()
    _check(out, _ref(a, b, layout), K)


def test_gemm_fp32_out_and_accumulate():
    from meshslice_b200 import _native
    from meshslice_b200.ops.gemm import gemm
    a, b = _operands(256, 512, 320, "nt")
    out = torch.ones(256, 512, device="cuda", dtype=torch.float32)
    gemm(a, b, "nt", out=out, accumulate=True)
    _native.check_status()
    _check(out, _ref(a, b, "nt") + 1.0, 320)
    outb = torch.ones(256, 512, device="cuda", dtype=torch.bfloat16)
    gemm(a, b, "nt", out=outb, accumulate=True)
    _native.check_status()
    _check(outb, _ref(a, b, "nt") + 1.0, 320)


def test_gemm_bias_gelu_epilogue():
    from meshslice_b200 import _native
    from meshslice_b200.ops.gemm import gemm
    a, b = _operands(256, 512, 256, "nn")
    a = a * 0.1
    bias = torch.randn(512, device="cuda", generator=torch.Generator(device="cuda").manual_seed(5)).bfloat16()
    pre = torch.empty(256, 512, device="cuda", dtype=torch.bfloat16)
    out = gemm(a, b, "nn", bias=bias, act="gelu", pre_act=pre)
    _native.check_status()
    h = _ref(a, b, "nn") + bias.float()
    _check(pre, h, 256)
    ref = torch.nn.functional.gelu(h, approximate="tanh")   # the kernel applies GeLU to the fp32 sum
    assert ((out.float() - ref).abs() <= 0.03 + 0.01 * ref.abs()).all()


def test_gemm_many_tiles_persistent_schedule():
    """More tiles than SMs, so every CTA walks several tiles and both TMEM accumulators."""
    from meshslice_b200 import _native
    from meshslice_b200.ops.gemm import gemm
    a, b = _operands(4096, 4096, 512, "nt", seed=3)
    out = gemm(a, b, "nt")
    _native.check_status()
    _check(out, _ref(a, b, "nt"), 512)
