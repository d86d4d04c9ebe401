"""Decode-step GEMMs with the neighbouring layer ops in their epilogues (csrc/kernels/gemm_decode.cu).

RMSNorm does not run as an op of its own on this path. Whoever produces the residual stream leaves
the partial sums of squares of every token row behind (``ss`` fp32 ``[tokens, tiles]``: entry
``[t, i]`` covers features ``128 i .. 128 i + 127`` of token ``t``; a producer that only knows the
whole row writes the flat prefix ``ss.view(-1)[:T]``, one value per token, and the consumer is told
``tiles=1``), the norm weight is folded into the consumer's weight columns (``fold_norm_weight``)
and the consumer GEMM multiplies its output row by ``rsqrt(sum_i ss[t, i] / H + eps)``. Off the GPU each function computes the same thing with the
fp32 definitions, which is also what the GPU tests compare against.

Replaces, at decode sizes, the reference's separate launches around its matmuls: add + norm
(xlite/csrc/model.cpp:1413-1433), rope_and_cache (model.cpp:545-566) and silu_and_mul
(model.cpp:820-830).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native
from . import functional as F
from . import reference as ref

MAX_TOKENS = 128      # rows the fused decode kernels take


def fold_norm_weight(w: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
    """W' = W diag(g): the norm weight of the producer moved into the consumer's weight columns."""
    return (w.float() * g.float()[None, :]).to(w.dtype)


def unfold_norm_weight(w: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
    """Inverse of `fold_norm_weight` (exact when g is a power of two, else to one rounding)."""
    return (w.float() / g.float()[None, :]).to(w.dtype)


def fold_layer_norms(lw) -> None:
    """Fold a dense layer's two RMSNorm weights into the GEMMs that consume the normalised rows
    (attn_norm -> w_qkv, mlp_norm -> w_gate_up) and replace them by ones, so that every path —
    fused or not — computes with the same weights. The original norm weights are kept for saving."""
    lw.attn_norm_g, lw.mlp_norm_g = lw.attn_norm, lw.mlp_norm
    lw.w_qkv = fold_norm_weight(lw.w_qkv, lw.attn_norm)
    lw.w_gate_up = fold_norm_weight(lw.w_gate_up, lw.mlp_norm)
    lw.attn_norm = torch.ones_like(lw.attn_norm)
    lw.mlp_norm = torch.ones_like(lw.mlp_norm)
    lw.norm_folded = True


def unfolded_layer(lw):
    """A shallow copy of a folded layer with the checkpoint's weights restored (for saving)."""
    from types import SimpleNamespace
    u = SimpleNamespace(**vars(lw))
    u.w_qkv = unfold_norm_weight(lw.w_qkv, lw.attn_norm_g)
    u.w_gate_up = unfold_norm_weight(lw.w_gate_up, lw.mlp_norm_g)
    u.attn_norm, u.mlp_norm = lw.attn_norm_g, lw.mlp_norm_g
    u.norm_folded = False
    return u


def new_sumsq(hidden: int, device) -> torch.Tensor:
    """Buffer for the sums of squares of up to MAX_TOKENS rows of `hidden` features."""
    return torch.zeros(MAX_TOKENS, hidden // 128, dtype=torch.float32, device=device)


def token_scale(ss: torch.Tensor, rows: int, norm_h: int, eps: float, tiles: Optional[int] = None) -> torch.Tensor:
    """fp32 [rows]: rsqrt(sum over tiles of ss / norm_h + eps). tiles=1: the flat one-value-per-token
    form written by `row_sumsq` / `add_residual_sumsq`."""
    if tiles == 1:
        tot = ss.reshape(-1)[:rows].float()
    else:
        tot = ss[:rows].float().sum(1)
    return torch.rsqrt(tot / norm_h + eps)


def row_sumsq(x: torch.Tensor, ss: torch.Tensor) -> torch.Tensor:
    """Whole-row sums of squares of x [T, H] into the first T floats of `ss` (pass `tiles=1` to
    the consumer). Used where the residual stream does not come out of a fused producer: after the
    embedding and after a library collective."""
    T = x.shape[0]
    if x.device.type == "meta":
        return ss
    if x.is_cuda:
        _native.call("norm", 0, x, None, None, None, None, ss, None, 1.0, T, x.shape[1], 1, x.stride(0), 0, 0,
                     0.0)
    else:
        ss.view(-1)[:T] = ref.sumsq(x)[:, 0]
    return ss


def add_residual_sumsq(a: torch.Tensor, x: torch.Tensor, ss: torch.Tensor) -> torch.Tensor:
    """x += a in place and ss.view(-1)[:T] = whole-row sums of squares of the new x (tiles=1): the
    stand-alone form of what `linear_residual` does in a GEMM epilogue, for producers whose
    reduction runs in a library collective."""
    T = x.shape[0]
    if x.device.type == "meta":
        return x
    if x.is_cuda:
        _native.call("norm", 0, a, x, None, None, None, ss, None, 1.0, T, x.shape[1], 1, a.stride(0), x.stride(0),
                     0, 0.0)
    else:
        x.copy_((x.float() + a.float()).to(x.dtype))
        ss.view(-1)[:T] = ref.sumsq(x)[:, 0]
    return x


def _hint_next(next_w: Optional[torch.Tensor]) -> None:
    """Tell the next fused decode GEMM launch which weight the GEMM behind it will stream, so that
    its producers warm L2 with that weight's first tiles while their own epilogue runs."""
    if next_w is None or not next_w.is_cuda or next_w.dtype != torch.bfloat16 or not F._flags().decode_l2_prefetch:
        return
    import ctypes
    fn = _native.kernels().gv_gemm_decode_next
    fn(ctypes.c_void_p(next_w.data_ptr()), ctypes.c_longlong(next_w.shape[0]), ctypes.c_longlong(next_w.shape[1]),
       ctypes.c_longlong(next_w.stride(0)))


def _tiles(ss: Optional[torch.Tensor], tiles: Optional[int]):
    """(number of partial sums per token, their pitch) as the kernels take them."""
    if ss is None:
        return 0, 0
    if tiles == 1:
        return 1, 1
    return (ss.shape[1] if tiles is None else tiles), ss.stride(0)


@F._dry
def linear_scaled(x: torch.Tensor, w: torch.Tensor, ss: Optional[torch.Tensor], norm_h: int, eps: float,
                  bias: Optional[torch.Tensor] = None, swiglu: bool = False, tiles: Optional[int] = None,
                  out: Optional[torch.Tensor] = None, splitk: int = 0,
                  next_w: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = s_t * (x @ w^T) (+ bias), s_t from `ss`; with `swiglu`, w holds [64 gate | 64 up] row
    blocks (``F.interleave_gate_up``) and out [T, N / 2] = silu(gate) * up."""
    M, K = x.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty(M, N // 2 if swiglu else N, dtype=x.dtype, device=x.device)
    nt, ld = _tiles(ss, tiles)
    if not x.is_cuda:
        y = x.float() @ w.float().t()
        if ss is not None:
            y = y * token_scale(ss, M, norm_h, eps, tiles)[:, None]
        if bias is not None:
            y = y + bias.float()
        y = y.to(x.dtype)
        if swiglu:
            y = ref.silu_and_mul(F.deinterleave_gate_up_cols(y))
        out.copy_(y)
        return out
    F._check_bf16(x, w, bias)
    assert M <= MAX_TOKENS and x.stride(1) == 1 and w.stride(1) == 1
    _hint_next(next_w)
    _native.call("gemm_decode", x, w, bias, out, M, N, K, x.stride(0), w.stride(0), out.stride(0), ss, nt, ld,
                 norm_h, float(eps), int(swiglu), splitk)
    return out


def linear_residual(a: torch.Tensor, w: torch.Tensor, x: torch.Tensor, ss_out: Optional[torch.Tensor],
                    bias: Optional[torch.Tensor] = None, splitk: int = 0,
                    next_w: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x += a @ w^T (+ bias) in place; ss_out[t, i] = sum of squares of the new x[t, 128 i : 128 i + 128]."""
    M, K = a.shape
    N = w.shape[0]
    if a.device.type == "meta":
        return x
    if not a.is_cuda:
        y = a.float() @ w.float().t()
        if bias is not None:
            y = y + bias.float()
        x.copy_((x.float() + y).to(x.dtype))
        if ss_out is not None:
            ss_out[:M, :N // 128] = x.float().reshape(M, N // 128, 128).pow(2).sum(-1)
        return x
    F._check_bf16(a, w, x, bias)
    assert M <= MAX_TOKENS and a.stride(1) == 1 and x.stride(1) == 1
    _hint_next(next_w)
    _native.call("gemm_decode_residual", a, w, bias, x, x, ss_out, M, N, K, a.stride(0), w.stride(0),
                 x.stride(0), ss_out.stride(0) if ss_out is not None else 0, splitk)
    return x


def rope_fusable(cfg, hd: int, mrope_mode: int) -> bool:
    """The fused QKV epilogue covers 128-wide heads with full NeoX rotation and one position row."""
    return (hd == 128 and cfg.rot_dim == 128 and not cfg.rope_interleaved and mrope_mode == 0
            and not cfg.attn_output_gate and not cfg.qk_norm_full)


@F._dry
def linear_rope(x: torch.Tensor, w: torch.Tensor, meta: "F.AttnMeta", cos_sin: torch.Tensor, k_cache, v_cache,
                nq: int, nkv: int, ss: Optional[torch.Tensor], norm_h: int, eps: float,
                bias: Optional[torch.Tensor] = None, q_norm_w=None, k_norm_w=None, qk_eps: float = 1e-6,
                q_scale: Optional[float] = None, tiles: Optional[int] = None,
                out: Optional[torch.Tensor] = None, splitk: int = 0) -> torch.Tensor:
    """QKV projection + (bias, q/k RMSNorm,) RoPE + q scaling + paged K/V write in one kernel for
    128-wide heads: returns q [T, nq * 128]; K and V of token t land in cache slot
    ``meta.slot_mapping[t]``."""
    hd = 128
    M, K = x.shape
    q_scale = hd ** -0.5 if q_scale is None else q_scale
    if out is None:
        out = torch.empty(M, nq * hd, dtype=x.dtype, device=x.device)
    nt, ld = _tiles(ss, tiles)
    if not x.is_cuda:
        qkv = linear_scaled(x, w, ss, norm_h, eps, tiles=tiles)
        q = ref.rope_kvwrite(qkv, meta.positions[..., :M], meta.slot_mapping[:M], cos_sin, k_cache, v_cache, nq,
                             nkv, hd, hd, q_scale, bias, q_norm_w, k_norm_w, qk_eps, 0, (0, 0, 0), False)
        out.copy_(q)
        return out
    F._check_bf16(x, w, bias, q_norm_w, k_norm_w, k_cache, v_cache)
    assert M <= MAX_TOKENS and w.shape[0] == (nq + 2 * nkv) * hd
    assert cos_sin.dtype == torch.float32 and cos_sin.shape[1] == hd and meta.positions.dim() == 1
    num_slots = k_cache.numel() // (nkv * hd)
    _native.call("gemm_decode_rope", x, w, bias, out, k_cache, v_cache, cos_sin, meta.positions, meta.slot_mapping,
                 q_norm_w, k_norm_w, M, K, x.stride(0), w.stride(0), nq, nkv, float(q_scale), float(qk_eps),
                 cos_sin.shape[0], num_slots, ss, nt, ld, norm_h, float(eps), splitk)
    return out
