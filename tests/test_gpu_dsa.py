"""Sparse-attention kernels: indexer scores, radix top-K (exact, ascending), paged gather, and
the index-masked absorbed attention; the masked kernel must agree with attention over the
gathered dense cache (the reference's mla_v3 path, xlite/tests/kernels/mla_v3.py:35-53)."""
import pytest
import torch

from gvirt_b200.ops import dsa_ops, mla_ops
from gvirt_b200.ops import functional as F
from tests.gpu_util import close, status_ok
from tests.test_gpu_attention import build

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _to_dev(mc):
    m = F.AttnMeta(*(t.to(DEV) for t in (mc.query_start_loc, mc.cached_lens, mc.seq_lens, mc.last_token_idx,
                                         mc.slot_mapping, mc.block_tables, mc.positions)),
                   batch=mc.batch, num_tokens=mc.num_tokens, max_q_len=mc.max_q_len, max_seq_len=mc.max_seq_len,
                   decode_step=mc.decode_step, block_size=mc.block_size)
    return m


@pytest.mark.parametrize("Hi,D", [(64, 128), (8, 64)])
@pytest.mark.parametrize("relu", [True, False])
def test_indexer_scores(Hi, D, relu):
    lens, cached = [1, 1, 7], [300, 0, 1200]
    _, _, _, mc, _ = build(lens, cached, 1, 1, 64, 64)
    m = _to_dev(mc)
    T = sum(lens)
    g = torch.Generator().manual_seed(0)
    nblk = int(mc.block_tables.max()) + 1
    kc = (torch.randn(nblk, 64, 1, D, generator=g) * 0.3).bfloat16()
    q = (torch.randn(T, Hi, D, generator=g) * 0.3).bfloat16()
    w = torch.randn(T, Hi, generator=g)
    want = dsa_ops.indexer_scores(q, w, kc, mc, relu)
    got = dsa_ops.indexer_scores(q.to(DEV), w.to(DEV), kc.to(DEV), m, relu)
    fin = torch.isfinite(want)
    assert torch.equal(torch.isfinite(got.cpu()), fin)
    close(got.cpu()[fin], want[fin], atol=5e-2, rtol=2e-2, what="indexer scores")
    status_ok()


@pytest.mark.parametrize("n,K", [(13542, 2048), (13542, 512), (100, 512), (131072, 2048), (2049, 2048)])
def test_topk_select_exact(n, K):
    g = torch.Generator().manual_seed(1)
    scores = torch.randn(3, (n + 127) // 128 * 128, generator=g)
    scores[1] = torch.round(scores[1] * 4) / 4          # many ties
    lens = torch.tensor([n, n, max(1, n // 2)], dtype=torch.int32)
    want = dsa_ops.topk_select(scores, lens, K)
    got = dsa_ops.topk_select(scores.to(DEV), lens.to(DEV), K).cpu()
    assert torch.equal(got, want)
    status_ok()


def test_gather_paged_rows_exact():
    lens, cached = [1, 1], [500, 90]
    _, _, _, mc, _ = build(lens, cached, 1, 1, 64, 64)
    nblk = int(mc.block_tables.max()) + 1
    cache = torch.randn(nblk, 64, 1, 576).bfloat16()
    idx = torch.full((2, 128), -1, dtype=torch.int32)
    idx[0, :100] = torch.sort(torch.randperm(501)[:100])[0].to(torch.int32)
    idx[1, :91] = torch.arange(91, dtype=torch.int32)
    want = dsa_ops.gather_paged_rows(cache, mc.block_tables, idx, 64)
    got = dsa_ops.gather_paged_rows(cache.to(DEV), mc.block_tables.to(DEV), idx.to(DEV), 64).cpu()
    assert torch.equal(got, want)
    status_ok()


@pytest.mark.parametrize("mode", ["decode", "prefill"])
def test_masked_attention_matches_reference_and_gathered(mode):
    heads, dc, dr, bs, K = 16, 512, 64, 64, 128
    if mode == "decode":
        lens, cached = [1, 1, 1], [400, 50, 127]
    else:
        lens, cached = [6, 3], [300, 126]
    _, _, _, mc, _ = build(lens, cached, 1, 1, 64, bs)
    mc.decode_step = mode == "decode"
    m = _to_dev(mc)
    T = sum(lens)
    g = torch.Generator().manual_seed(2)
    nblk = int(mc.block_tables.max()) + 1
    cache = (torch.randn(nblk, bs, 1, dc + dr, generator=g) * 0.5).bfloat16()
    qf = (torch.randn(T, heads, dc + dr, generator=g) * 0.3).bfloat16()
    scores = torch.randn(T, (mc.max_seq_len + 127) // 128 * 128, generator=g)
    qsl, cl = mc.query_start_loc.tolist(), mc.cached_lens.tolist()
    tok_len = torch.tensor([cl[b] + (t - qsl[b]) + 1 for b in range(len(lens)) for t in range(qsl[b], qsl[b + 1])],
                           dtype=torch.int32)
    idx = dsa_ops.topk_select(scores, tok_len, K)
    scale = (dc + dr) ** -0.5
    want = torch.zeros(T, heads, dc, dtype=torch.bfloat16)
    mla_ops.mla_attention(qf, cache, mc, heads, dc, dr, scale, out=want, topk_idx=idx)
    got = torch.zeros(T, heads, dc, device=DEV, dtype=torch.bfloat16)
    mla_ops.mla_attention(qf.to(DEV), cache.to(DEV), m, heads, dc, dr, scale, out=got, topk_idx=idx.to(DEV))
    close(got, want, atol=1e-2, rtol=3e-2, what="index-masked attention")
    if mode == "decode":
        # same result through gather + dense attention (one block of K rows per request)
        dense = dsa_ops.gather_paged_rows(cache.to(DEV), m.block_tables, idx.to(DEV), bs)  # [B, K, W]
        B = len(lens)
        z = torch.zeros(1, dtype=torch.int32, device=DEV)
        n_sel = torch.minimum(tok_len, torch.tensor(K)).to(torch.int32).to(DEV)
        md = F.AttnMeta(torch.arange(B + 1, dtype=torch.int32, device=DEV), n_sel - 1, n_sel, z, z,
                        torch.arange(B, dtype=torch.int32, device=DEV).view(B, 1), z.long(), batch=B,
                        num_tokens=B, max_q_len=1, max_seq_len=K, decode_step=True, block_size=K)
        got2 = torch.zeros(T, heads, dc, device=DEV, dtype=torch.bfloat16)
        mla_ops.mla_attention(qf.to(DEV), dense.view(B, K, 1, dc + dr), md, heads, dc, dr, scale, out=got2)
        close(got2, want, atol=1e-2, rtol=3e-2, what="gathered dense attention")
    status_ok()


@pytest.mark.parametrize("Hi,bs", [(64, 64), (32, 128), (128, 16)])
def test_indexer_scores_tensor_core_path_long_context(Hi, bs):
    """tcgen05 indexer (keys on the TMEM lanes) over a long and two short contexts, several key
    tiles per CTA, against the CUDA-core kernel and the fp32 definition."""
    from gvirt_b200 import _native
    D = 128
    lens, cached = [1, 3, 1], [9000, 130, 0]
    _, _, _, mc, _ = build(lens, cached, 1, 1, 64, bs)
    m = _to_dev(mc)
    T = sum(lens)
    g = torch.Generator().manual_seed(Hi)
    nblk = int(mc.block_tables.max()) + 1
    kc = (torch.randn(nblk, bs, 1, D, generator=g) * 0.3).bfloat16()
    q = (torch.randn(T, Hi, D, generator=g) * 0.3).bfloat16()
    w = torch.randn(T, Hi, generator=g)
    want = dsa_ops.indexer_scores(q, w, kc, mc, True)
    got = dsa_ops.indexer_scores(q.to(DEV), w.to(DEV), kc.to(DEV), m, True)
    L = want.shape[1]
    old = torch.empty(T, L, dtype=torch.float32, device=DEV)
    _native.call("indexer_scores", q.to(DEV), w.to(DEV), kc.to(DEV), m.block_tables, m.query_start_loc,
                 m.cached_lens, old, T, m.batch, Hi, D, bs, m.block_tables.shape[1], L, 1, nblk)
    fin = torch.isfinite(want)
    assert torch.equal(torch.isfinite(got.cpu()), fin) and torch.equal(torch.isfinite(old.cpu()), fin)
    close(got.cpu()[fin], want[fin], atol=5e-2, rtol=2e-2, what="tcgen05 indexer vs definition")
    close(got.cpu()[fin], old.cpu()[fin], atol=5e-2, rtol=2e-2, what="tcgen05 indexer vs CUDA-core kernel")
    status_ok()
