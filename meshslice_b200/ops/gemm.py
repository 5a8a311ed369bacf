"""Local GEMM on the tcgen05 kernel: C = op(A) @ op(B), bf16 inputs, fp32 accumulation.

Layouts follow the reference cost model's naming (CostModel.py:74-98):
  'nn': A [M,K] @ B [K,N]      'nt': A [M,K] @ B[N,K]^T      'tn': A[K,M]^T @ B [K,N]
All operands are row-major; no operand is ever transposed in memory, the tensor-core
descriptors select the major-ness.
"""
from __future__ import annotations

import os

import torch

from .. import _native

_SM_COUNT = {}


def sm_count(device=None) -> int:
    dev = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    if dev not in _SM_COUNT:
        _SM_COUNT[dev] = torch.cuda.get_device_properties(dev).multi_processor_count
    return _SM_COUNT[dev]


def _dims(a, b, layout):
    if layout == "nn":
        M, K = a.shape
        K2, N = b.shape
    elif layout == "nt":
        M, K = a.shape
        N, K2 = b.shape
    elif layout == "tn":
        K, M = a.shape
        K2, N = b.shape
    else:
        raise ValueError(f"unknown layout {layout!r}")
    if K != K2:
        raise ValueError(f"contraction mismatch: {tuple(a.shape)} x {tuple(b.shape)} ({layout})")
    return M, N, K


def gemm_args(a, b, layout, out, *, accumulate=False, bias=None, act=None, pre_act=None, two_cta=None):
    """Argument dict of the native launcher for a plain local GEMM."""
    M, N, K = _dims(a, b, layout)
    for t in (a, b):
        if t.dtype != torch.bfloat16 or t.stride(-1) != 1:
            raise ValueError("GEMM operands must be bf16 with a contiguous last dimension")
    if out.shape != (M, N) or out.stride(-1) != 1:
        raise ValueError("bad output shape")
    d = dict(M=M, N=N, K=K, A=a.data_ptr(), B=b.data_ptr(), lda=a.stride(0), ldb=b.stride(0),
             a_mn_major=1 if layout == "tn" else 0, b_mn_major=0 if layout == "nt" else 1,
             C=out.data_ptr(), ldc=out.stride(0), c_fp32=1 if out.dtype == torch.float32 else 0,
             accumulate=1 if accumulate else 0, status=_native.status().dev, grid=sm_count(a.device),
             stream=_native.stream_ptr(), timeout_ns=1_000_000_000)
    if two_cta is None:
        two_cta = os.environ.get("MSB_TWO_CTA", "1") != "0"
    d["two_cta"] = 1 if two_cta else 0
    for key, env in (("stages", "MSB_G2_STAGES"), ("group", "MSB_G2_GROUP"), ("map3d", "MSB_G2_MAP3D")):
        if env in os.environ:
            d[key] = int(os.environ[env])
    if bias is not None:
        d["bias"] = bias.data_ptr()
    if act is not None:
        if act != "gelu":
            raise ValueError("only act='gelu' is fused")
        d["act"] = 1
        if pre_act is not None:
            d["C_pre"] = pre_act.data_ptr()
    return d


def gemm(a, b, layout="nn", *, out=None, out_dtype=torch.bfloat16, accumulate=False, bias=None,
         act=None, pre_act=None, two_cta=None):
    """C = op(A) @ op(B) on the tensor cores of the current GPU.  ``two_cta`` selects the
    cta_group::2 kernel (default: on, MSB_TWO_CTA=0 turns it off)."""
    M, N, K = _dims(a, b, layout)
    if out is None:
        if accumulate:
            raise ValueError("accumulate=True needs an output tensor")
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    _native.load().gemm_run(gemm_args(a, b, layout, out, accumulate=accumulate, bias=bias, act=act,
                                      pre_act=pre_act, two_cta=two_cta))
    return out
