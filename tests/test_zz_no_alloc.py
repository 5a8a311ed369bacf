"""The allocation-free attention-backward entry point, called through its exported C symbol.

Some hosts of this library cannot allocate device memory when they call it (a fixed memory
budget, a plugin that only gets its buffers, another allocator's pool that must stay
untouched).  For them ``msb_attention_bwd_noalloc`` keeps its scratch in a fixed array inside the
library.  The test checks that it returns what the regular entry point returns, twice in a row
(the second call reuses the scratch the first one dirtied), and that oversize problems are
refused.  This file is collected last so that a failure here cannot hide other results.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

CUDA_ERROR_INVALID_VALUE = 1


def _lib():
    from meshslice_b200.build import ext_path
    lib = ctypes.CDLL(str(ext_path()))
    fn = lib.msb_attention_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int] * 4 + [ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p]
    return fn


def test_noalloc_attention_bwd_matches_regular_entry_point_twice():
    from meshslice_b200 import _native
    from meshslice_b200.ops import functional as F
    fn = _lib()
    batch, seq, heads, causal = 2, 256, 2, 1
    stream = torch.cuda.current_stream().cuda_stream
    for trial in range(2):
        g = torch.Generator(device="cuda").manual_seed(100 + trial)
        qkv = torch.randn(batch * seq, heads * 3 * 128, device="cuda", generator=g).bfloat16()
        dout = torch.randn(batch * seq, heads * 128, device="cuda", generator=g).bfloat16()
        out, lse = F.attention_fwd(qkv, batch, seq, heads, bool(causal))
        ref = F.attention_bwd(dout, qkv, out, lse, batch, seq, heads, bool(causal))
        _native.check_status()
        got = torch.empty_like(qkv)
        torch.cuda.synchronize()
        # free bytes as the driver reports them: this sees a cudaMalloc inside the library, which
        # torch's own counters (its caching allocator only) would not.  The first call may still
        # load the kernels' code; the second one must leave the device's free memory untouched.
        free_before = torch.cuda.mem_get_info()[0]
        rc = fn(qkv.data_ptr(), out.data_ptr(), dout.data_ptr(), lse.data_ptr(), got.data_ptr(), batch, seq, heads,
                causal, 1.0 / 128 ** 0.5, stream, None)
        assert rc == 0
        torch.cuda.synchronize()
        if trial == 1:
            assert torch.cuda.mem_get_info()[0] == free_before
        # same kernels, same inputs; the fp32 reductions into dQ may be applied in another order
        assert (got.float() - ref.float()).abs().max().item() < 0.05
        assert ((got.float() - ref.float()).norm() / ref.float().norm()).item() < 1e-2


def test_noalloc_rejects_problems_beyond_its_scratch():
    fn = _lib()
    x = torch.zeros(8, device="cuda")
    p = x.data_ptr()
    stream = torch.cuda.current_stream().cuda_stream
    # 8 * 2048 * 2 rows > 16384
    assert fn(p, p, p, p, p, 8, 2048, 2, 0, 1.0, stream, None) == CUDA_ERROR_INVALID_VALUE
    assert fn(p, p, p, p, p, 1, 100, 1, 0, 1.0, stream, None) == CUDA_ERROR_INVALID_VALUE
