"""DeepSeek sparse attention ops: lightning-indexer scores, top-K selection (ascending indices),
gather of selected cache rows (csrc/kernels/dsa.cu); PyTorch definitions for CPU.

Reference goldens: xlite/tests/kernels/indexer_topk.py:25-57 (64 heads x 128, K in {512, 2048},
pass criterion: < 3 % of indices differ), topk.py:13-30, gather_sparse_kv_cache.py:136 (exact)."""
from __future__ import annotations

import torch

from .. import _native
from . import reference as ref


def indexer_scores(q, w, k_cache, meta, relu=True):
    """q [T, Hi, D] bf16, w fp32 [T, Hi], paged k cache [blocks, bs, 1, D] -> fp32 [T, L] with
    L = max context rounded up to 128; positions beyond a token's context are -inf."""
    T, Hi, D = q.shape
    L = (max(meta.max_seq_len, 1) + 127) // 128 * 128
    if not q.is_cuda:
        out = torch.full((T, L), float("-inf"))
        qsl, cl = meta.query_start_loc.tolist(), meta.cached_lens.tolist()
        for b in range(meta.batch):
            for t in range(qsl[b], qsl[b + 1]):
                n = cl[b] + (t - qsl[b]) + 1
                K = ref.gather_paged(k_cache, meta.block_tables[b], n, meta.block_size)[:, 0].float()
                dots = torch.einsum("hd,nd->hn", q[t].float(), K)
                if relu:
                    dots = dots.clamp_min(0)
                out[t, :n] = (w[t].float()[:, None] * dots).sum(0)
        return out
    out = torch.empty(T, L, dtype=torch.float32, device=q.device)
    bs = meta.block_size
    from ..config import flags
    if (D == 128 and Hi % 16 == 0 and 16 <= Hi <= 128 and bs >= 8 and bs & (bs - 1) == 0 and T <= 65535
            and q.dtype == torch.bfloat16 and flags().dsa_indexer_tc):
        # keys on the TMEM lanes, heads on the columns: tcgen05 indexer (dsa_tc.cu)
        _native.call("indexer_scores_tc", q.contiguous(), w.float().contiguous(), k_cache, meta.block_tables,
                     meta.query_start_loc, meta.cached_lens, out, T, meta.batch, Hi, D, bs,
                     meta.block_tables.shape[1], L, int(relu), k_cache.shape[0])
        return out
    _native.call("indexer_scores", q.contiguous(), w.contiguous(), k_cache, meta.block_tables,
                 meta.query_start_loc, meta.cached_lens, out, T, meta.batch, Hi, D, meta.block_size,
                 meta.block_tables.shape[1], L, int(relu), k_cache.shape[0])
    return out


def topk_select(scores, lens, K):
    """Row-wise top-K positions among the first lens[row] scores, ascending, padded with -1."""
    rows = scores.shape[0]
    if not scores.is_cuda:
        out = torch.full((rows, K), -1, dtype=torch.int32)
        for r in range(rows):
            n = int(lens[r])
            if n <= K:
                out[r, :n] = torch.arange(n, dtype=torch.int32)
            else:
                # ties broken towards the lower index: stable sort of the negated scores
                order = torch.sort(-scores[r, :n].float(), stable=True)[1][:K]
                out[r] = torch.sort(order)[0].to(torch.int32)
        return out
    out = torch.empty(rows, K, dtype=torch.int32, device=scores.device)
    _native.call("topk_select", scores, scores.stride(0), lens, rows, K, out)
    return out


def gather_paged_rows(cache, block_tables, idx, block_size):
    """dense[b, i] = cache row of position idx[b, i] of request b (zeros where idx < 0).
    cache [blocks, bs, 1, W]; idx int32 [B, K] -> [B, K, W]."""
    B, K = idx.shape
    W = cache.shape[-1]
    if not cache.is_cuda:
        flat = cache.view(-1, W)
        out = torch.zeros(B, K, W, dtype=cache.dtype)
        for b in range(B):
            sel = idx[b]
            ok = sel >= 0
            p = sel[ok].long()
            slot = block_tables[b].long()[p // block_size] * block_size + p % block_size
            out[b, ok] = flat[slot]
        return out
    out = torch.empty(B, K, W, dtype=cache.dtype, device=cache.device)
    _native.call("gather_paged_rows", cache, block_tables, idx, out, B, K, W * cache.element_size(), block_size,
                 block_tables.shape[1], cache.shape[0])
    return out
