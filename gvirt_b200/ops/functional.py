"""Public op layer: each function runs the hand-written sm_100a kernel when its input lives on
a CUDA device and the fp32 PyTorch definition (``ops.reference``) otherwise.

On CUDA there is no fall-back: a missing kernel library or an unsupported shape raises.
Outputs may be passed in (``out=``) so that the model runner can place them in the activation
arena (fixed addresses => CUDA-graph replay); otherwise they come from torch's allocator.

Role of the reference's host op layer ``XliteOp*`` (xlite/csrc/op.h:16-189, op.cpp), minus the
per-dtype dispatch (bf16 storage only on the GPU path) and the dummy-runtime short-circuit
(sizing is done by ``engine.arena`` dry runs instead).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from .. import _native
from ..config import flags as _flags
from . import reference as ref

_KIND = {"rms": 0, "layer": 1, "l2": 2}


def _dry(fn):
    """Dry-run short-circuit: when the first tensor argument is a *meta* tensor (arena sizing
    pass) nothing is computed and the caller-provided ``out`` is returned, as every op of the
    reference returns early under its dummy runtime (e.g. xlite/csrc/op.cpp:208-220)."""
    import functools

    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        first = next((a for a in args if isinstance(a, torch.Tensor)), None)
        if first is not None and first.device.type == "meta":
            out = kwargs.get("out")
            if out is None:
                raise RuntimeError(f"{fn.__name__}: dry run needs an explicit out= tensor")
            return out
        return fn(*args, **kwargs)

    return wrapper


def _is_cuda(t: torch.Tensor) -> bool:
    return t.is_cuda


def _check_bf16(*ts):
    for t in ts:
        if t is not None and t.dtype != torch.bfloat16:
            raise TypeError(f"CUDA path is bf16-only, got {t.dtype}")


# --------------------------------------------------------------------------- GEMM
@_dry
def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out: Optional[torch.Tensor] = None, splitk: int = 0) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T (+ bias). tcgen05 GEMM on CUDA. An int8 weight carrying a
    ``gv_scale`` attribute (per-output-channel scales) runs as W8A8: the activations are quantised
    per token — or with the weight's fixed per-channel factor ``gv_in_scale_recip`` (static mode) —
    and the int8 tensor-core GEMM de-quantises in its epilogue."""
    if w.dtype == torch.int8:
        from . import quant_ops
        x2 = x.reshape(-1, x.shape[-1])
        if out is None:
            out = torch.empty(*x.shape[:-1], w.shape[0], dtype=x.dtype, device=x.device)
        o2 = out.reshape(-1, w.shape[0])
        qb = getattr(w, "gv_bias", None)       # static checkpoints: quant_bias x deq_scale, fp32 [N]
        if qb is not None:
            bias = qb if bias is None else qb + bias.float()
        y = quant_ops.linear_w8a8(x2, w, w.gv_scale, None if bias is None else bias.float(),
                                  input_scale_recip=getattr(w, "gv_in_scale_recip", None),
                                  input_offset=getattr(w, "gv_in_offset", None), out=o2)
        return out if out is not None else y.reshape(*x.shape[:-1], w.shape[0])
    if not _is_cuda(x):
        y = ref.linear(x, w, bias)
        if out is not None:
            out.copy_(y)
            return out
        return y
    _check_bf16(x, w, bias)
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    M, K = x2.shape
    N = w.shape[0]
    assert w.shape[1] == K and w.stride(1) == 1
    if out is None:
        out = torch.empty(*lead, N, dtype=x.dtype, device=x.device)
    o2 = out.reshape(-1, N)
    assert o2.stride(-1) == 1
    if M > 0:
        mode = _flags().prefill_gemm_persistent if M >= 1024 else 0
        if mode == 3:
            # measured at 8192 tokens (Llama-3-8B shapes): the persistent kernel wins on the narrow
            # outputs (qkv 359 vs 429 us, o_proj 230 vs 249, down 727 vs 824) and loses on the wide
            # gate/up (1972 vs 1766), whose many tiles already hide the epilogue
            mode = 2 if N <= 8192 else 0
        if mode == 2 and N % 8 == 0 and o2.stride(0) % 8 == 0 and o2.data_ptr() % 16 == 0:
            # token-major 128 x 256 tiles, one CTA per SM walking the tile list with the accumulator
            # double-buffered in TMEM: a tile's epilogue overlaps the next tile's main loop
            _native.call("gemm_bf16_persistent", x2, w, bias, o2, M, N, K, x2.stride(0), w.stride(0),
                         o2.stride(0))
            return out
        if (mode == 1 and bias is None and x2.stride(0) == K and w.stride(0) == K and o2.stride(0) == N):
            # one segment through the persistent grouped kernel (weight-major 128 x 128 tiles)
            _native.call("grouped_gemm_bf16", x2, w, _one_segment(M, x.device), o2, M, N, K, 1)
            return out
        _native.call("gemm_bf16", x2, w, bias, o2, M, N, K, x2.stride(0), w.stride(0), o2.stride(0),
                     splitk)
    return out


_SEGMENTS: dict = {}


def _one_segment(M: int, device) -> torch.Tensor:
    key = (M, str(device))
    t = _SEGMENTS.get(key)
    if t is None:
        if len(_SEGMENTS) > 64:
            _SEGMENTS.clear()
        t = _SEGMENTS[key] = torch.tensor([0, M], dtype=torch.int32, device=device)
    return t


# --------------------------------------------------------------------------- norms
@_dry
def norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float, kind: str = "rms",
         bias: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
         cnt: int = 1, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Normalise the last dimension (split into `cnt` independent sub-rows). With `residual`,
    first does residual += x in place and normalises the updated residual."""
    if not _is_cuda(x):
        y = ref.norm(x, w, bias, eps, kind, residual, cnt)
        if out is not None:
            out.copy_(y)
            return out
        return y
    _check_bf16(x, w, bias, residual)
    cols_total = x.shape[-1]
    x2 = x.reshape(-1, cols_total)
    rows = x2.shape[0]
    if out is None:
        out = torch.empty_like(x)
    o2 = out.reshape(-1, cols_total)
    r2 = residual.reshape(-1, cols_total) if residual is not None else None
    _native.call("norm", _KIND[kind], x2, r2, w, bias, o2, None, None, 1.0, rows, cols_total // cnt,
                 cnt, x2.stride(0), r2.stride(0) if r2 is not None else 0, o2.stride(0), float(eps))
    return out


def rmsnorm(x, w, eps, out=None):
    return norm(x, w, eps, "rms", out=out)


def add_rmsnorm(x, residual, w, eps, out=None):
    """residual += x (in place); returns rmsnorm(residual) * w."""
    return norm(x, w, eps, "rms", residual=residual, out=out)


def sumsq(x: torch.Tensor, cnt: int = 1) -> torch.Tensor:
    """Per (row, sub-row) sum of squares in fp32 (the variance-only mode of the norm kernel)."""
    if not _is_cuda(x):
        return ref.sumsq(x, cnt)
    _check_bf16(x)
    cols_total = x.shape[-1]
    x2 = x.reshape(-1, cols_total)
    out = torch.empty(x2.shape[0], cnt, dtype=torch.float32, device=x.device)
    _native.call("norm", 0, x2, None, None, None, None, out, None, 1.0, x2.shape[0],
                 cols_total // cnt, cnt, x2.stride(0), 0, 0, 0.0)
    return out.reshape(*x.shape[:-1], cnt)


@_dry
def rmsnorm_extvar(x, w, var_sum, scale, eps, cnt=1, out=None):
    """RMSNorm whose sum of squares comes from outside (already reduced across ranks);
    `scale` = how many times wider the full row is than the local slice."""
    if not _is_cuda(x):
        cols = x.shape[-1] // cnt
        xf = x.float().reshape(*x.shape[:-1], cnt, cols)
        y = xf * torch.rsqrt(var_sum.float().reshape(*x.shape[:-1], cnt, 1) / (scale * cols) + eps)
        y = (y * w.float()).reshape(x.shape).to(x.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    cols_total = x.shape[-1]
    x2 = x.reshape(-1, cols_total)
    if out is None:
        out = torch.empty_like(x)
    o2 = out.reshape(-1, cols_total)
    _native.call("norm", 0, x2, None, w, None, o2, None, var_sum.float().contiguous(), float(scale),
                 x2.shape[0], cols_total // cnt, cnt, x2.stride(0), 0, o2.stride(0), float(eps))
    return out


# --------------------------------------------------------------------------- attention metadata
@dataclass
class AttnMeta:
    """Device-side description of one engine step (see csrc/runtime/attn_meta.h)."""
    query_start_loc: torch.Tensor   # int32 [batch_cap + 1]
    cached_lens: torch.Tensor       # int32 [batch_cap]
    seq_lens: torch.Tensor          # int32 [batch_cap]
    last_token_idx: torch.Tensor    # int32 [batch_cap]
    slot_mapping: torch.Tensor      # int32 [token_cap]
    block_tables: torch.Tensor      # int32 [batch_cap, max_blocks]
    positions: torch.Tensor         # int64 [token_cap] (or [3, token_cap] for M-RoPE)
    batch: int = 0
    num_tokens: int = 0
    max_q_len: int = 0
    max_seq_len: int = 0
    decode_step: bool = False
    block_size: int = 16
    num_splits: int = 1
    split_scratch: Optional[tuple] = None  # (part_o fp32, part_lse fp32) for split-KV decode
    extra: dict = field(default_factory=dict)


# --------------------------------------------------------------------------- RoPE + KV write
@_dry
def rope_kvwrite(qkv, meta: AttnMeta, cos_sin, k_cache, v_cache, nq, nkv, hd, rot_dim=None,
                 q_scale=None, bias=None, q_norm_w=None, k_norm_w=None, eps=1e-6, mrope_mode=0,
                 mrope_sections=(0, 0, 0), interleaved=False, out=None):
    """qkv [T, (nq + 2 nkv) * hd] -> q [T, nq * hd] (rotated, scaled); k/v written to the cache."""
    rot_dim = hd if rot_dim is None else rot_dim
    q_scale = hd ** -0.5 if q_scale is None else q_scale
    T = qkv.shape[0]
    pos = meta.positions[..., :T]
    slots = meta.slot_mapping[:T]
    if not _is_cuda(qkv):
        q = ref.rope_kvwrite(qkv, pos, slots, cos_sin, k_cache, v_cache, nq, nkv, hd, rot_dim,
                             q_scale, bias, q_norm_w, k_norm_w, eps, mrope_mode, mrope_sections,
                             interleaved)
        if out is not None:
            out.copy_(q)
            return out
        return q
    _check_bf16(qkv, bias, q_norm_w, k_norm_w, k_cache, v_cache)
    assert cos_sin.dtype == torch.float32 and cos_sin.shape[1] == rot_dim
    if out is None:
        out = torch.empty(T, nq * hd, dtype=qkv.dtype, device=qkv.device)
    if pos.dim() > 1 and not pos.is_contiguous():
        pos = pos.contiguous()
    num_slots = k_cache.numel() // (nkv * hd) if nkv > 0 else 0
    _native.call("rope_kvwrite", qkv, bias, q_norm_w, k_norm_w, cos_sin, pos, slots, k_cache, v_cache,
                 out, T, nq, nkv, hd, rot_dim, qkv.stride(0), float(q_scale), float(eps),
                 cos_sin.shape[0], num_slots, mrope_mode, int(mrope_sections[0]),
                 int(mrope_sections[1]), int(mrope_sections[2]), int(bool(interleaved)))
    return out


# --------------------------------------------------------------------------- paged attention
_COUNTERS: dict = {}


def _decode_counters(device, n: int) -> torch.Tensor:
    """Zeroed int32 ticket counters for the in-kernel split merge, one array per (device, stream):
    the kernel returns them to zero, so calls ordered on one stream share the array."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    t = _COUNTERS.get(key)
    if t is None or t.numel() < n:
        t = _COUNTERS[key] = torch.zeros(max(n, 4096), dtype=torch.int32, device=device)
    return t


@_dry
def paged_attention(q, k_cache, v_cache, meta: AttnMeta, nq, nkv, hd, scale=1.0, out=None):
    """Causal GQA attention over the paged KV cache. q [T, nq*hd] pre-scaled."""
    T = q.shape[0]
    if not _is_cuda(q):
        y = ref.paged_attention(q, k_cache, v_cache, meta.block_tables, meta.query_start_loc,
                                meta.cached_lens, nq, nkv, hd, meta.block_size, scale,
                                batch=meta.batch)
        if out is not None:
            out.copy_(y)
            return out
        return y
    _check_bf16(q, k_cache, v_cache)
    if out is None:
        out = torch.empty_like(q)
    num_blocks = k_cache.shape[0]
    max_blocks = meta.block_tables.shape[1]
    if meta.decode_step:
        # one token per request; token index == request index (padding requests have seq_len 0)
        ns = meta.num_splits
        po = pl = None
        if ns > 1:
            if meta.split_scratch is None:
                po = torch.empty(T * nq * ns * hd, dtype=torch.float32, device=q.device)
                pl = torch.empty(T * nq * ns, dtype=torch.float32, device=q.device)
            else:
                po, pl = meta.split_scratch
                assert po.numel() >= T * nq * ns * hd and pl.numel() >= T * nq * ns
        # the CTA that finishes a (request, kv head) last merges its splits: one launch
        cnt = _decode_counters(q.device, T * nkv) if ns > 1 else None
        _native.call("paged_attention_decode_merged", q, k_cache, v_cache, meta.block_tables,
                     meta.seq_lens, out, po, pl, cnt, T, nq, nkv, hd, meta.block_size, max_blocks, ns,
                     float(scale), num_blocks)
    elif (hd == 128 and _flags().prefill_attn_tc and meta.block_size >= 8
          and meta.block_size & (meta.block_size - 1) == 0 and q.is_contiguous() and out.is_contiguous()):
        # tcgen05 / TMEM / TMA flash attention (attention_prefill_tc.cu)
        _native.call("paged_attention_prefill_tc", q, k_cache, v_cache, meta.block_tables,
                     meta.query_start_loc, meta.cached_lens, out, T, meta.batch, meta.max_q_len, nq,
                     nkv, hd, meta.block_size, max_blocks, float(scale), num_blocks)
    else:
        _native.call("paged_attention_prefill", q, k_cache, v_cache, meta.block_tables,
                     meta.query_start_loc, meta.cached_lens, out, meta.batch, meta.max_q_len, nq,
                     nkv, hd, meta.block_size, max_blocks, float(scale), num_blocks)
    return out


# --------------------------------------------------------------------------- elementwise
def interleave_gate_up(w: torch.Tensor) -> torch.Tensor:
    """[gate (I rows) ; up (I rows)] -> blocks of 128 rows = [64 gate | 64 up] of the same 64
    features: the row order the SwiGLU-epilogue GEMM wants. I % 64 == 0."""
    inter = w.shape[-2] // 2
    assert inter % 64 == 0
    lead = w.shape[:-2]
    g = w[..., :inter, :].reshape(*lead, inter // 64, 1, 64, w.shape[-1])
    u = w[..., inter:, :].reshape(*lead, inter // 64, 1, 64, w.shape[-1])
    return torch.cat([g, u], dim=-3).reshape(*lead, 2 * inter, w.shape[-1]).contiguous()


def pad_gate_up_down(w_gate_up: torch.Tensor, w_down: torch.Tensor, multiple: int = 64):
    """Zero-pad the intermediate dimension of a SwiGLU FFN to a multiple of `multiple`.

    w_gate_up [2 I, H] = [gate rows ; up rows], w_down [H, I]  ->  ([2 I', H], [H, I'], I' - I).
    A padded feature has gate = up = 0, so silu(0) * 0 = 0 enters the down projection against a
    zero weight column: the FFN output is unchanged bit for bit. Tensor-parallel shards whose
    local I is not a multiple of 64 (29568 / 8 = 3696) get the SwiGLU-epilogue GEMM this way."""
    inter = w_gate_up.shape[-2] // 2
    pad = (-inter) % multiple
    if pad == 0:
        return w_gate_up, w_down, 0
    zr = w_gate_up.new_zeros(*w_gate_up.shape[:-2], pad, w_gate_up.shape[-1])
    gu = torch.cat([w_gate_up[..., :inter, :], zr, w_gate_up[..., inter:, :], zr], dim=-2).contiguous()
    zc = w_down.new_zeros(*w_down.shape[:-1], pad)
    return gu, torch.cat([w_down, zc], dim=-1).contiguous(), pad


def unpad_gate_up_down(w_gate_up: torch.Tensor, w_down: torch.Tensor, pad: int):
    """Inverse of ``pad_gate_up_down`` on [gate ; up]-ordered weights."""
    if pad == 0:
        return w_gate_up, w_down
    ip = w_gate_up.shape[-2] // 2
    gu = torch.cat([w_gate_up[..., :ip - pad, :], w_gate_up[..., ip:2 * ip - pad, :]], dim=-2).contiguous()
    return gu, w_down[..., :ip - pad].contiguous()


def deinterleave_gate_up_rows(w: torch.Tensor) -> torch.Tensor:
    """Inverse of ``interleave_gate_up``: back to [gate rows ; up rows]."""
    return deinterleave_gate_up_cols(w.transpose(-1, -2)).transpose(-1, -2).contiguous()


def deinterleave_gate_up_cols(x: torch.Tensor) -> torch.Tensor:
    """Inverse permutation on the columns of an activation produced with interleaved weights."""
    inter = x.shape[-1] // 2
    b = x.reshape(*x.shape[:-1], inter // 64, 2, 64)
    return torch.cat([b[..., 0, :].reshape(*x.shape[:-1], inter), b[..., 1, :].reshape(*x.shape[:-1], inter)], -1)


@_dry
def linear_swiglu(x, w_il, out=None, splitk: int = 0):
    """out [T, I] = silu(x @ gate^T) * (x @ up^T) with w_il = interleave_gate_up([gate; up]):
    one tcgen05 GEMM whose epilogue applies the activation (CUDA), or the definition (CPU)."""
    inter = w_il.shape[0] // 2
    x2 = x.reshape(-1, x.shape[-1])
    if out is None:
        out = torch.empty(x2.shape[0], inter, dtype=x.dtype, device=x.device)
    if not _is_cuda(x):
        gu = deinterleave_gate_up_cols(ref.linear(x2, w_il, None))
        out.copy_(ref.silu_and_mul(gu))
        return out
    _check_bf16(x, w_il)
    M, K = x2.shape
    _native.call("gemm_bf16_swiglu", x2, w_il, out, M, w_il.shape[0], K, x2.stride(0), w_il.stride(0),
                 out.stride(0), splitk)
    return out


@_dry
def silu_and_mul(x, out=None, num=None, clamp: float = 0.0, interleaved: bool = False):
    if not _is_cuda(x):
        if interleaved:
            x = deinterleave_gate_up_cols(x)
        y = ref.silu_and_mul(x, num, clamp)
        if out is not None:
            out.copy_(y)
            return out
        return y
    _check_bf16(x)
    d = x.shape[-1] // 2
    x2 = x.reshape(-1, 2 * d)
    if out is None:
        out = torch.empty(*x.shape[:-1], d, dtype=x.dtype, device=x.device)
    o2 = out.reshape(-1, d)
    _native.call("silu_and_mul", x2, o2, x2.shape[0], d, x2.stride(0), o2.stride(0), num,
                 float(clamp), int(bool(interleaved)))
    return out


def _binary(mode, a, b, scale=1.0, out=None):
    a2 = a.reshape(-1, a.shape[-1])
    if out is None:
        out = torch.empty_like(a)
    o2 = out.reshape(-1, a.shape[-1])
    b2 = None
    ldb = 0
    if b is not None:
        b2 = b.reshape(-1, b.shape[-1]) if mode != 3 else b
        ldb = b2.stride(0) if mode != 3 else 0
    _native.call("binary", mode, a2, b2, o2, a2.shape[0], a2.shape[1], a2.stride(0), ldb,
                 o2.stride(0), float(scale))
    return out


@_dry
def add(a, b, out=None):
    if not _is_cuda(a):
        y = (a.float() + b.float()).to(a.dtype)
        return y if out is None else out.copy_(y)
    return _binary(0, a, b, out=out)


@_dry
def sigmoid_gate_mul(a, gate, out=None):
    if not _is_cuda(a):
        y = ref.sigmoid_gate_mul(a, gate)
        return y if out is None else out.copy_(y)
    return _binary(1, a, gate, out=out)


def softmax(x, calc_len: int):
    """In-place causal row softmax of x [rows, cols]: row m over its first calc_len + m entries,
    zeros behind them. The reference's stand-alone `softmax(rt, x, calc_len, is_long)`
    (xlite/xlite/_C.pyi:1545); there is one kernel for short and long rows here. On CUDA: bf16,
    cols a multiple of 8."""
    if x.dim() != 2:
        raise ValueError("softmax expects [rows, cols]")
    if x.device.type == "meta":
        return x
    if not _is_cuda(x):
        return x.copy_(ref.causal_softmax(x, int(calc_len)))
    _check_bf16(x)
    if x.stride(1) != 1:
        raise ValueError("softmax needs unit stride along the row")
    _native.call("causal_softmax", x, x.shape[0], x.shape[1], x.stride(0), int(calc_len))
    return x


@_dry
def muls(a, scale, out=None):
    if not _is_cuda(a):
        y = (a.float() * scale).to(a.dtype)
        return y if out is None else out.copy_(y)
    return _binary(2, a, None, scale, out=out)


@_dry
def add_bias(a, bias, out=None):
    if not _is_cuda(a):
        y = (a.float() + bias.float()).to(a.dtype)
        return y if out is None else out.copy_(y)
    return _binary(3, a, bias, out=out)


def cast(x, dtype):
    if not _is_cuda(x) or {x.dtype, dtype} != {torch.bfloat16, torch.float32}:
        return x.to(dtype)
    x = x.contiguous()
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    _native.call("cast", int(dtype == torch.float32), x, out, x.numel())
    return out


def transpose12(x):
    """[B, S, C] -> [B, C, S]"""
    if not _is_cuda(x) or x.element_size() != 2:
        return x.transpose(1, 2).contiguous()
    x = x.contiguous()
    B, S, C = x.shape
    out = torch.empty(B, C, S, dtype=x.dtype, device=x.device)
    _native.call("transpose12", x, out, B, S, C)
    return out


@_dry
def embed(ids, table, vstart=0, vend=None, out=None):
    vend = vstart + table.shape[0] if vend is None else vend
    if not _is_cuda(table):
        y = ref.embed(ids, table, vstart, vend)
        return y if out is None else out.copy_(y)
    _check_bf16(table)
    assert ids.dtype == torch.int32
    T = ids.shape[0]
    if out is None:
        out = torch.empty(T, table.shape[1], dtype=table.dtype, device=table.device)
    _native.call("embed", ids, table, out, T, table.shape[1], vstart, vend)
    return out


@_dry
def gather_rows(src, idx, out=None):
    if not _is_cuda(src):
        y = src[idx.long()]
        return y if out is None else out.copy_(y)
    _check_bf16(src)
    assert idx.dtype == torch.int32
    n = idx.shape[0]
    if out is None:
        out = torch.empty(n, src.shape[1], dtype=src.dtype, device=src.device)
    _native.call("gather_rows", src, idx, out, n, src.shape[1], src.stride(0), src.shape[0])
    return out


# --------------------------------------------------------------------------- sampling
def sample(logits, temperature=None, top_k=None, top_p=None, seed=0, step=0, index_offset=0,
           return_scores=False, step_tensor=None):
    """Greedy (temperature None / <= 0) or Gumbel-max sampling with optional top-k / top-p.
    Returns int32 token ids [batch] (and the winning scores when `return_scores`)."""
    B, V = logits.shape
    if not _is_cuda(logits):
        lf = logits.float()
        if temperature is None:
            idx = lf.argmax(-1)
            val = lf.gather(1, idx[:, None])[:, 0]
        else:
            t = temperature.float().clamp_min(1e-6)[:, None]
            g = torch.Generator(device="cpu").manual_seed(int(seed) * 1000003 + int(step))
            u = torch.rand(lf.shape, generator=g).clamp_min(1e-10)
            z = lf / t
            if top_k is not None or top_p is not None:
                srt, order = z.sort(-1, descending=True)
                keep = torch.ones_like(srt, dtype=torch.bool)
                if top_k is not None:
                    kk = top_k.long().clamp_min(1)[:, None]
                    keep &= torch.arange(V)[None, :] < torch.where(kk > 0, kk, torch.full_like(kk, V))
                if top_p is not None:
                    pr = torch.softmax(srt, -1)
                    keep &= (pr.cumsum(-1) - pr) < top_p.float()[:, None]
                z = torch.full_like(z, float("-inf")).scatter(1, order, srt.masked_fill(~keep, float("-inf")))
            noisy = z - torch.log(-torch.log(u))
            greedy = temperature <= 0
            noisy = torch.where(greedy[:, None], lf, noisy)
            idx = noisy.argmax(-1)
            val = noisy.gather(1, idx[:, None])[:, 0]
        idx = (idx + index_offset).to(torch.int32)
        return (idx, val) if return_scores else idx
    assert logits.stride(1) == 1
    out_idx = torch.empty(B, dtype=torch.int32, device=logits.device)
    out_val = torch.empty(B, dtype=torch.float32, device=logits.device) if return_scores else None
    _native.call("sample", logits, int(logits.dtype == torch.float32), logits.stride(0), B, V,
                 temperature, top_k, top_p, int(seed), int(step), step_tensor, int(index_offset),
                 out_val, out_idx)
    return (out_idx, out_val) if return_scores else out_idx
