"""MoE ops: router scoring + top-k, token permutation, grouped expert GEMMs, weighted combine.

CUDA path = hand-written kernels (csrc/kernels/moe_router.cu, moe_permute.cu,
grouped_gemm.cu); CPU path = fp32 PyTorch definitions in ``ops.reference``.

Reference counterparts: ``softmax_topk`` / ``sigmoid_topk`` (xlite/csrc/kernels/softmax_topk.h:268,
sigmoid_topk.h:387), ``permutation`` / ``unpermutation`` (permutation.cpp:201, unpermutation.h:125),
``group_matmul`` (group_matmul.h:57). The reference emits dense ``[T, E]`` weights plus a
bitmap; here routing is compact ``[T, K]`` (ids, weights) and the permutation is a counting
sort on device (per-expert counts -> exclusive scan -> scatter), so the expert GEMM sees
expert-major contiguous segments and nothing is synchronised with the host.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native
from . import functional as F
from . import reference as ref


def router_logits(h: torch.Tensor, w_router: torch.Tensor) -> torch.Tensor:
    """fp32 logits [T, E]. The gate GEMM runs in the storage dtype (tcgen05 on CUDA)."""
    if not h.is_cuda:
        return h.float() @ w_router.float().t()
    return F.linear(h, w_router if w_router.dtype == h.dtype else w_router.to(h.dtype)).float()


def softmax_topk(logits: torch.Tensor, k: int, renorm: bool = True):
    if not logits.is_cuda:
        return ref.softmax_topk(logits, k, renorm)
    return _topk_cuda(logits, None, k, 0, 1, 1, renorm, 1.0)


def sigmoid_topk(logits, bias, k, n_group, topk_group, renorm=True, route_scale=1.0):
    if not logits.is_cuda:
        return ref.sigmoid_topk(logits, bias, k, n_group, topk_group, renorm, route_scale)
    return _topk_cuda(logits, bias, k, 1, n_group, topk_group, renorm, route_scale)


def _topk_cuda(logits, bias, k, mode, n_group, topk_group, renorm, route_scale):
    T, E = logits.shape
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    w = torch.empty(T, k, dtype=torch.float32, device=logits.device)
    ids = torch.empty(T, k, dtype=torch.int32, device=logits.device)
    b = bias.float().contiguous() if bias is not None else None
    _native.call("router_topk", logits, b, w, ids, T, E, k, mode, n_group, topk_group,
                 int(renorm), float(route_scale))
    return w, ids


def interleave16(w13: torch.Tensor) -> torch.Tensor:
    """[E, 2 I, K] rows [gate (I) | up (I)] -> blocks of 32 rows = [16 gate | 16 up] of the same 16
    features (I % 16 == 0): the layout whose grouped GEMM applies SwiGLU in its epilogue."""
    E, N, K = w13.shape
    I = N // 2
    assert I % 16 == 0
    g = w13[:, :I].reshape(E, I // 16, 16, K)
    u = w13[:, I:].reshape(E, I // 16, 16, K)
    return torch.cat([g, u], 2).reshape(E, N, K).contiguous()


def deinterleave16(w13_il: torch.Tensor) -> torch.Tensor:
    """Inverse of `interleave16`."""
    E, N, K = w13_il.shape
    b = w13_il.reshape(E, N // 32, 2, 16, K)
    return torch.cat([b[:, :, 0].reshape(E, N // 2, K), b[:, :, 1].reshape(E, N // 2, K)], 1).contiguous()


def grouped_gemm_swiglu(xs: torch.Tensor, w13_il: torch.Tensor, offsets: torch.Tensor, act: torch.Tensor,
                        clamp: float = 0.0) -> torch.Tensor:
    """act[r] = silu(xs[r] @ gate_e^T) * (xs[r] @ up_e^T) for rows r of expert e's segment, with
    w13_il in the `interleave16` layout: the [rows, 2 I] intermediate is never written."""
    E, N, K = w13_il.shape
    if not xs.is_cuda:
        gu = torch.zeros(xs.shape[0], N, dtype=xs.dtype)
        grouped_gemm(xs, deinterleave16(w13_il), offsets, gu)
        act.copy_(ref.silu_and_mul(gu, None, clamp))
        return act
    _native.call("grouped_gemm_bf16_swiglu", xs, w13_il, offsets, act, xs.shape[0], N, K, E, float(clamp))
    return act


def experts_forward(x, weights, ids, w13, w2, local_start=0, clamp=0.0, out=None,
                    w13_scale=None, w2_scale=None, il16: bool = False):
    """y[t] = sum_k weights[t,k] * Expert_{ids[t,k]}(x[t]) over the experts held locally
    (ids in [local_start, local_start + E_local)); other (token, k) pairs contribute zero.
    `il16`: w13 is in the `interleave16` layout (bf16 only)."""
    if not x.is_cuda:
        if il16:
            w13 = deinterleave16(w13)
        if w13_scale is not None:
            w13 = torch.stack([ref.dequant_fp8_block(w13[e], w13_scale[e]) for e in range(w13.shape[0])]).to(x.dtype)
            w2 = torch.stack([ref.dequant_fp8_block(w2[e], w2_scale[e]) for e in range(w2.shape[0])]).to(x.dtype)
        y = ref.moe_ffn(x, weights, ids, w13, w2, local_start, clamp)
        if out is not None:
            out.copy_(y)
            return out
        return y
    T, H = x.shape
    K = ids.shape[1]
    E_local = w13.shape[0]
    inter = w13.shape[1] // 2
    dev = x.device
    rows_cap = T * K
    # counting-sort permutation of the (token, k) pairs routed to local experts
    counts = torch.zeros(E_local + 1, dtype=torch.int32, device=dev)   # [E_local] + total
    offsets = torch.empty(E_local + 1, dtype=torch.int32, device=dev)
    row_of = torch.empty(T, K, dtype=torch.int32, device=dev)          # permuted row or -1
    xs = torch.empty(rows_cap, H, dtype=x.dtype, device=dev)
    _native.call("moe_permute", x, ids, counts, offsets, row_of, xs, T, H, K, E_local, local_start,
                 rows_cap)
    act = torch.empty(rows_cap, inter, dtype=x.dtype, device=dev)
    if il16:
        assert w13_scale is None
        grouped_gemm_swiglu(xs, w13, offsets, act, clamp)
    else:
        gu = torch.empty(rows_cap, 2 * inter, dtype=x.dtype, device=dev)
        grouped_gemm(xs, w13, offsets, gu, w_scale=w13_scale)
        F.silu_and_mul(gu, out=act, num=offsets[E_local:], clamp=clamp)
    ys = torch.empty(rows_cap, H, dtype=x.dtype, device=dev)
    grouped_gemm(act, w2, offsets, ys, w_scale=w2_scale)
    if out is None:
        out = torch.empty(T, H, dtype=x.dtype, device=dev)
    _native.call("moe_unpermute", ys, weights, row_of, out, T, H, K)
    return out


def grouped_gemm(xs: torch.Tensor, w: torch.Tensor, offsets: torch.Tensor, out: torch.Tensor,
                 w_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r] = xs[r] @ w[e]^T for rows r in [offsets[e], offsets[e+1]).
    w [E, N, K] bf16, or fp8 e4m3 with w_scale [E, N/128, K/128] (block-scaled)."""
    E, N, K = w.shape
    if not xs.is_cuda:
        off = offsets.tolist()
        for e in range(E):
            a, b = off[e], off[e + 1]
            if b > a:
                we = w[e] if w_scale is None else ref.dequant_fp8_block(w[e], w_scale[e])
                out[a:b] = ref.linear(xs[a:b], we.to(xs.dtype) if w_scale is not None else we)
        return out
    if w_scale is None:
        _native.call("grouped_gemm_bf16", xs, w, offsets, out, xs.shape[0], N, K, E)
    else:
        rows = xs.shape[0]
        xq, sx = quant_fp8(xs, num=offsets[E:])
        _native.call("grouped_gemm_fp8", xq, sx, w, w_scale, offsets, out, rows, N, K, E, sx.shape[1])
    return out


def quant_fp8(x: torch.Tensor, num: Optional[torch.Tensor] = None):
    """Per-token, per-128-column e4m3 quantisation. -> (q [T, K] fp8, scales fp32 [K/128, T])."""
    T, K = x.shape
    if not x.is_cuda:
        q, s = ref.quant_fp8_group(x)
        return q, s.t().contiguous()
    q = torch.empty(T, K, dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty(K // 128, max(T, 1), dtype=torch.float32, device=x.device)
    _native.call("quant_fp8_group128", x, q, s, T, K, x.stride(0), K, s.shape[1], num)
    return q, s


def linear_fp8(x: torch.Tensor, wq: torch.Tensor, w_scale: torch.Tensor, out=None) -> torch.Tensor:
    """Block-scaled fp8 linear: x bf16 [M, K] (quantised on the fly), wq e4m3 [N, K] with 128x128
    scales [ceil(N/128), K/128] -> bf16 [M, N]."""
    if not x.is_cuda:
        y = ref.linear_fp8(x, wq, w_scale)
        return y if out is None else out.copy_(y)
    M, K = x.shape
    N = wq.shape[0]
    xq, sx = quant_fp8(x)
    if out is None:
        out = torch.empty(M, N, dtype=x.dtype, device=x.device)
    _native.call("gemm_fp8", xq, sx, wq, w_scale, out, M, N, K, sx.shape[1], out.stride(0))
    return out
