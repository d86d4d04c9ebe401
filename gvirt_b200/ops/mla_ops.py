"""MLA ops: ``mla_prepare``, query absorption (+ q_pe RoPE), absorbed attention over the latent
cache, un-absorption. CUDA kernels in csrc/kernels/mla.cu and bmm.cu; fp32 PyTorch otherwise.

Reference kernels: ``mla_prepare_<T>`` (xlite/csrc/kernels/mla_prepare.h:41),
``rope_complex_and_cache_<T>`` (rope_complex_and_cache.h:243), ``einsum_mht_htd_mhd_<T>``
(einsum_mht_htd_mhd.h:40), ``mla_v2`` / ``flash_mla_v2`` (mla_v2.h:762, flash_mla_v2.h:914).
"""
from __future__ import annotations

import torch

from .. import _native
from . import functional as F
from . import reference as ref


def _rope_interleaved(x, cos_sin, pos):
    """x [T, ..., d] with adjacent (re, im) pairs -> rotated, de-interleaved [re.. | im..]."""
    d = x.shape[-1]
    half = d // 2
    cs = cos_sin.float()[pos.long()]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c, s = cs[:, :half].reshape(shape), cs[:, half:].reshape(shape)
    x1, x2 = x[..., 0::2].float(), x[..., 1::2].float()
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)


@F._dry
def mla_prepare(a, q_norm_w, kv_norm_w, cos_sin, meta, kv_cache, ql, dc, dr, eps, out=None):
    """a [T, ql + dc + dr] -> out [T, ql] = RMSNorm(q latent); writes [RMSNorm(kv latent) |
    RoPE(k_pe)] into the paged latent cache at the step's slots."""
    T = a.shape[0]
    pos = meta.positions[:T]
    slots = meta.slot_mapping[:T]
    if not a.is_cuda:
        if ql > 0:
            qn = ref.norm(a[:, :ql], q_norm_w, None, eps)
            out[:, :ql].copy_(qn) if out is not None else None
        kvc = ref.norm(a[:, ql:ql + dc], kv_norm_w, None, eps).float()
        kpe = _rope_interleaved(a[:, ql + dc:ql + dc + dr], cos_sin, pos)
        row = torch.cat([kvc, kpe], -1).to(kv_cache.dtype)
        valid = slots >= 0
        kv_cache.view(-1, dc + dr)[slots[valid].long()] = row[valid]
        return out
    _native.call("mla_prepare", a, q_norm_w, kv_norm_w, cos_sin, pos, slots, kv_cache, out, T, ql, dc, dr,
                 a.stride(0), out.stride(0), float(eps), cos_sin.shape[0],
                 kv_cache.numel() // (dc + dr))
    return out


@F._dry
def absorb_q(q, w_uk_t, cos_sin, meta, hl, dn, dr, dc, out=None):
    """q [T, hl * (dn + dr)] -> out [T, hl, dc + dr] = [q_nope . W_UK | RoPE(q_pe)]."""
    T = q.shape[0]
    pos = meta.positions[:T]
    q3 = q.view(T, hl, dn + dr)
    if not q.is_cuda:
        qa = torch.einsum("thd,hcd->thc", q3[..., :dn].float(), w_uk_t.float())
        qp = _rope_interleaved(q3[..., dn:], cos_sin, pos)
        out.copy_(torch.cat([qa, qp], -1).to(out.dtype))
        return out
    # q_pe: interleaved RoPE written straight into out[..., dc:]
    _native.call("rope_interleaved", q, cos_sin, pos, out, T, hl, dn + dr, dn, dr, dc + dr, dc,
                 cos_sin.shape[0])
    # q_abs: per-head GEMM  out[t, h, :dc] = q3[t, h, :dn] @ w_uk_t[h]^T
    bmm(q3[..., :dn], w_uk_t, out[..., :dc])
    return out


@F._dry
def unabsorb_o(oa, w_uv, out=None):
    """oa [T, hl, dc], w_uv [hl, dv, dc] -> out [T, hl, dv]."""
    if not oa.is_cuda:
        out.copy_(torch.einsum("thc,hvc->thv", oa.float(), w_uv.float()).to(out.dtype))
        return out
    bmm(oa, w_uv, out)
    return out


def bmm(x, w, out):
    """Per-head GEMM: out[t, h, :] = x[t, h, :] @ w[h]^T with x [T, H, K] (any row/head strides,
    unit inner stride), w [H, N, K] contiguous, out [T, H, N] (strided)."""
    T, Hh, K = x.shape
    N = w.shape[1]
    if not x.is_cuda:
        out.copy_(torch.einsum("thk,hnk->thn", x.float(), w.float()).to(out.dtype))
        return out
    assert x.stride(2) == 1 and out.stride(2) == 1 and w.is_contiguous()
    _native.call("bmm_bf16", x, w, out, T, Hh, N, K, x.stride(0), x.stride(1), out.stride(0), out.stride(1))
    return out


@F._dry
def mla_attention(qf, kv_cache, meta, hl, dc, dr, scale, out=None, topk_idx=None):
    """Absorbed attention: qf [T, hl, dc + dr], latent cache [blocks, block, 1, dc + dr] ->
    out [T, hl, dc]. Causal over cached + new tokens of each request. With `topk_idx` (int32
    [T, K], ascending, -1 padded) a query token whose context is longer than K only attends to
    the listed positions (DeepSeek sparse attention)."""
    T = qf.shape[0]
    if not qf.is_cuda:
        qsl = meta.query_start_loc.tolist()
        cl = meta.cached_lens.tolist()
        for b in range(meta.batch):
            s, e = qsl[b], qsl[b + 1]
            n = e - s
            if n <= 0:
                continue
            total = cl[b] + n
            K = ref.gather_paged(kv_cache, meta.block_tables[b], total, meta.block_size)[:, 0].float()
            sc = torch.einsum("qhd,kd->hqk", qf[s:e].float(), K) * scale
            kpos = torch.arange(total)[None, :]
            qpos = (cl[b] + torch.arange(n))[:, None]
            sc = sc.masked_fill((kpos > qpos)[None], float("-inf"))
            if topk_idx is not None:
                Kt = topk_idx.shape[1]
                for i in range(n):
                    if cl[b] + i + 1 > Kt:
                        keep = torch.zeros(total, dtype=torch.bool)
                        sel = topk_idx[s + i]
                        keep[sel[sel >= 0].long()] = True
                        sc[:, i, ~keep] = float("-inf")
            o = torch.einsum("hqk,kc->qhc", sc.softmax(-1), K[:, :dc])
            out[s:e] = o.to(out.dtype)
        return out
    ns = meta.num_splits if meta.decode_step else 1
    po = pl = None
    if ns > 1:
        po = torch.empty(T * hl * ns * dc, dtype=torch.float32, device=qf.device)
        pl = torch.empty(T * hl * ns, dtype=torch.float32, device=qf.device)
    if (meta.decode_step and topk_idx is None and dc == 512 and dr == 64 and hl % 128 == 0
            and meta.block_size % 32 == 0 and F._flags().mla_attn_tc and qf.is_contiguous() and out.is_contiguous()):
        # tcgen05 / TMEM / TMA kernel: the 128 heads of a request on the TMEM lanes (mla_tc.cu)
        _native.call("mla_attention_tc", qf, kv_cache, meta.block_tables, meta.seq_lens, out, po, pl, T, hl, dc, dr,
                     meta.block_size, meta.block_tables.shape[1], ns, float(scale), kv_cache.shape[0])
        return out
    _native.call("mla_attention", qf, kv_cache, meta.block_tables, meta.query_start_loc,
                 meta.cached_lens, out, po, pl, T, meta.batch, hl, dc, dr, meta.block_size,
                 meta.block_tables.shape[1], ns, float(scale), kv_cache.shape[0],
                 topk_idx, 0 if topk_idx is None else topk_idx.shape[1])
    return out


def rope_partial_interleaved(x, cos_sin, pos, dr):
    """x [T, heads, D]: adjacent-pair rotation of the first `dr` dims of every head (written
    de-interleaved), remaining dims copied. Returns a new tensor."""
    T, Hh, D = x.shape
    out = x.clone()
    if not x.is_cuda:
        out[..., :dr] = _rope_interleaved(x[..., :dr], cos_sin, pos).to(x.dtype)
        return out
    _native.call("rope_interleaved", x, cos_sin, pos, out, T, Hh, D, 0, dr, D, 0, cos_sin.shape[0])
    return out


def scatter_rows(src, slots, cache):
    """cache.view(-1, W)[slots[t]] = src[t] for slots[t] >= 0."""
    T, W = src.shape
    if not src.is_cuda:
        ok = slots >= 0
        cache.view(-1, W)[slots[ok].long()] = src[ok].to(cache.dtype)
        return
    _native.call("scatter_rows", src.contiguous(), slots, cache, T, W * src.element_size(),
                 cache.numel() // W)
