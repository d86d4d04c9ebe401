"""MLA kernels vs fp32 definitions. Configurations follow xlite/tests/kernels/mla.py:54-76
((heads, rope, nope, v, kv_rank) such as (16, 64, 128, 128, 512)) and mla_prepare.py:59-142."""
import pytest
import torch

from gvirt_b200.ops import functional as F
from gvirt_b200.ops import mla_ops
from gvirt_b200.ops import reference as ref
from tests.gpu_util import close, status_ok
from tests.test_gpu_attention import build

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _meta_for(lens, cached, bs, dq):
    q, kc, vc, mc, m = build(lens, cached, 1, 1, 64, bs)  # only the metadata is used
    return mc, m


def _cpu(meta):
    return meta


@pytest.mark.parametrize("ql,dc,dr", [(1536, 512, 64), (0, 512, 64), (2048, 128, 64)])
def test_mla_prepare(ql, dc, dr):
    T, bs, nblk = 80, 64, 4
    a = (torch.randn(T, ql + dc + dr, device=DEV)).bfloat16()
    qw = torch.randn(max(ql, 1), device=DEV).bfloat16()
    kw = torch.randn(dc, device=DEV).bfloat16()
    tab = ref.rope_table(512, dr, 10000.0, device=DEV)
    pos = torch.randint(0, 512, (T,), dtype=torch.int64)
    slots = torch.randperm(bs * nblk)[:T].to(torch.int32)
    slots[5] = -1
    z = torch.zeros(1, dtype=torch.int32)
    meta_c = F.AttnMeta(z, z, z, z, slots, z.view(1, 1), pos, batch=1, num_tokens=T)
    meta_g = F.AttnMeta(z.cuda(), z.cuda(), z.cuda(), z.cuda(), slots.cuda(), z.view(1, 1).cuda(), pos.cuda(),
                        batch=1, num_tokens=T)
    cache_g = torch.zeros(nblk, bs, 1, dc + dr, device=DEV, dtype=torch.bfloat16)
    cache_c = torch.zeros(nblk, bs, 1, dc + dr, dtype=torch.bfloat16)
    qn_g = torch.zeros(T, max(ql, 8), device=DEV, dtype=torch.bfloat16)
    qn_c = torch.zeros(T, max(ql, 8), dtype=torch.bfloat16)
    mla_ops.mla_prepare(a, qw if ql else None, kw, tab, meta_g, cache_g, ql, dc, dr, 1e-6, out=qn_g)
    mla_ops.mla_prepare(a.cpu(), qw.cpu() if ql else None, kw.cpu(), tab.cpu(), meta_c, cache_c, ql, dc, dr, 1e-6,
                        out=qn_c)
    if ql:
        close(qn_g, qn_c, what="q latent norm")
    close(cache_g, cache_c, what="latent cache")
    status_ok()


@pytest.mark.parametrize("T,H,N,K", [(3, 4, 512, 128), (3, 8, 128, 512), (963, 4, 256, 192), (130, 16, 512, 128),
                                     (64, 128, 128, 512)])
def test_bmm(T, H, N, K):
    g = torch.Generator(device=DEV).manual_seed(0)
    xfull = (torch.randn(T, H, K + 64, device=DEV, generator=g) * 0.5).bfloat16()
    x = xfull[..., :K]                      # strided rows, like q_nope inside [q_nope | q_pe]
    w = (torch.randn(H, N, K, device=DEV, generator=g) * 0.05).bfloat16()
    outfull = torch.zeros(T, H, N + 64, device=DEV, dtype=torch.bfloat16)
    mla_ops.bmm(x, w, outfull[..., :N])
    want = torch.einsum("thk,hnk->thn", x.float(), w.float())
    close(outfull[..., :N], want, atol=3e-2, rtol=2e-2, what="bmm")
    assert (outfull[..., N:] == 0).all()
    status_ok()


@pytest.mark.parametrize("heads,dc,dr", [(16, 512, 64), (1, 64, 64), (8, 512, 64), (128, 512, 64), (20, 128, 64)])
@pytest.mark.parametrize("mode", ["decode", "decode_split", "prefill"])
def test_mla_attention(heads, dc, dr, mode):
    bs = 64
    if mode == "prefill":
        lens, cached = [5, 70, 1, 33], [0, 130, 64, 7]
    else:
        lens, cached = [1, 1, 1, 1, 1], [0, 63, 64, 1000, 257]
    if heads == 128 and mode == "prefill":
        lens, cached = [3, 9], [10, 100]
    mc, m = _meta_for(lens, cached, bs, dc + dr)
    m.decode_step = mode != "prefill"
    m.num_splits = 3 if mode == "decode_split" else 1
    T = sum(lens)
    g = torch.Generator().manual_seed(1)
    nblk = int(mc.block_tables.max()) + 1
    cache = (torch.randn(nblk, bs, 1, dc + dr, generator=g) * 0.5).bfloat16()
    qf = (torch.randn(T, heads, dc + dr, generator=g) * 0.3).bfloat16()
    scale = (dc + dr) ** -0.5
    want = torch.zeros(T, heads, dc, dtype=torch.bfloat16)
    mla_ops.mla_attention(qf, cache, mc, heads, dc, dr, scale, out=want)
    got = torch.zeros(T, heads, dc, device=DEV, dtype=torch.bfloat16)
    mla_ops.mla_attention(qf.to(DEV), cache.to(DEV), m, heads, dc, dr, scale, out=got)
    close(got, want, atol=1e-2, rtol=3e-2, what=f"mla attention {mode}")
    status_ok()


def test_absorb_and_unabsorb_paths():
    T, hl, dn, dr, dc, dv = 7, 16, 128, 64, 512, 128
    g = torch.Generator().manual_seed(2)
    q = (torch.randn(T, hl * (dn + dr), generator=g) * 0.5).bfloat16()
    w_uk_t = (torch.randn(hl, dc, dn, generator=g) * 0.05).bfloat16()
    w_uv = (torch.randn(hl, dv, dc, generator=g) * 0.05).bfloat16()
    tab = ref.rope_table(256, dr, 10000.0)
    pos = torch.randint(0, 256, (T,), dtype=torch.int64)
    z = torch.zeros(1, dtype=torch.int32)
    mc = F.AttnMeta(z, z, z, z, z, z.view(1, 1), pos, batch=1, num_tokens=T)
    mg = F.AttnMeta(z.cuda(), z.cuda(), z.cuda(), z.cuda(), z.cuda(), z.view(1, 1).cuda(), pos.cuda(), batch=1,
                    num_tokens=T)
    want = torch.zeros(T, hl, dc + dr, dtype=torch.bfloat16)
    mla_ops.absorb_q(q, w_uk_t, tab, mc, hl, dn, dr, dc, out=want)
    got = torch.zeros(T, hl, dc + dr, device=DEV, dtype=torch.bfloat16)
    mla_ops.absorb_q(q.cuda(), w_uk_t.cuda(), tab.cuda(), mg, hl, dn, dr, dc, out=got)
    close(got, want, atol=2e-2, rtol=2e-2, what="absorb_q")
    oa = (torch.randn(T, hl, dc, generator=g) * 0.5).bfloat16()
    want2 = torch.zeros(T, hl, dv, dtype=torch.bfloat16)
    mla_ops.unabsorb_o(oa, w_uv, out=want2)
    got2 = torch.zeros(T, hl, dv, device=DEV, dtype=torch.bfloat16)
    mla_ops.unabsorb_o(oa.cuda(), w_uv.cuda(), out=got2)
    close(got2, want2, atol=3e-2, rtol=2e-2, what="unabsorb_o")
    status_ok()


@pytest.mark.parametrize("ctx", [33000, 131071])
def test_mla_decode_long_caches(ctx):
    """The long end of the reference's sweep (xlite/tests/kernels/mla.py:61-76): 128 heads over one
    long and one short cache, split-KV with the number of splits a serving step would pick."""
    heads, dc, dr, bs = 128, 512, 64, 64
    lens, cached = [1, 1], [ctx - 1, 700]
    mc, m = _meta_for(lens, cached, bs, dc + dr)
    m.decode_step = True
    m.num_splits = 16
    g = torch.Generator().manual_seed(ctx % 89)
    nblk = int(mc.block_tables.max()) + 1
    cache = (torch.randn(nblk, bs, 1, dc + dr, generator=g) * 0.5).bfloat16()
    qf = (torch.randn(2, heads, dc + dr, generator=g) * 0.3).bfloat16()
    scale = (dc + dr) ** -0.5
    want = torch.zeros(2, heads, dc, dtype=torch.bfloat16)
    mla_ops.mla_attention(qf, cache, mc, heads, dc, dr, scale, out=want)
    got = torch.zeros(2, heads, dc, device=DEV, dtype=torch.bfloat16)
    mla_ops.mla_attention(qf.to(DEV), cache.to(DEV), m, heads, dc, dr, scale, out=got)
    close(got, want, atol=1e-2, rtol=3e-2, what=f"mla decode over {ctx} cached tokens")
    status_ok()


def test_mla_tc_rescales_its_output_when_the_maximum_climbs():
    """Scores that grow along the sequence force the lazily moved maximum (and with it the
    accumulated output in tensor memory) to be rescaled many times; padding rows give zeros."""
    heads, dc, dr, bs = 128, 512, 64, 64
    lens, cached = [1, 1, 1], [900, 0, 300]
    mc, m = _meta_for(lens, cached, bs, dc + dr)
    m.decode_step = True
    g = torch.Generator().manual_seed(4)
    nblk = int(mc.block_tables.max()) + 1
    cache = (torch.randn(nblk, bs, 1, dc + dr, generator=g) * 0.5).bfloat16()
    for b in range(3):
        total = cached[b] + 1
        for j in range((total + bs - 1) // bs):
            blk = int(mc.block_tables[b, j])
            pos = torch.arange(j * bs, (j + 1) * bs).float()
            cache[blk] = (cache[blk].float() * (0.3 + pos / 60.0)[:, None, None]).bfloat16()
    qf = (torch.randn(3, heads, dc + dr, generator=g) * 0.6).bfloat16()
    scale = 0.3
    want = torch.zeros(3, heads, dc, dtype=torch.bfloat16)
    mla_ops.mla_attention(qf, cache, mc, heads, dc, dr, scale, out=want)
    for ns in (1, 2):
        m.num_splits = ns
        got = torch.full((3, heads, dc), 7.0, device=DEV, dtype=torch.bfloat16)
        mla_ops.mla_attention(qf.to(DEV), cache.to(DEV), m, heads, dc, dr, scale, out=got)
        close(got, want, atol=2e-2, rtol=3e-2, what=f"mla tc with rescaling, {ns} split(s)")
    m.seq_lens[1] = 0              # a padding row: zeros, nothing read
    m.num_splits = 1
    got = torch.full((3, heads, dc), 7.0, device=DEV, dtype=torch.bfloat16)
    mla_ops.mla_attention(qf.to(DEV), cache.to(DEV), m, heads, dc, dr, scale, out=got)
    assert (got[1] == 0).all()
    close(got[0], want[0], atol=2e-2, rtol=3e-2, what="row beside a padding row")
    status_ok()
