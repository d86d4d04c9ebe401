"""tcgen05 / TMEM / TMA flash attention for prefill (attention_prefill_tc.cu) against the fp32
definition on the same bf16 inputs: block sizes, GQA groups, cached prefixes, ragged batches, a
case that forces the lazy rescaling of O, and the long-context end of the reference's sweep
(a 32 769-token prefill, decode over caches of 33 000 / 60 000 / 131 071 tokens;
xlite/tests/kernels/attention.py:42-60). Long cases use an fp32 PyTorch reference evaluated on the
GPU in query chunks (the CPU definition would take minutes there)."""
import pytest
import torch

from gvirt_b200 import _native
from gvirt_b200.ops import functional as F
from gvirt_b200.ops import reference as ref
from tests.gpu_util import close, status_ok
from tests.test_gpu_attention import build

pytestmark = pytest.mark.gpu
DEV = "cuda"
DEFAULT_WG = 4      # 64-key tiles, two CTAs per SM; 1 / 2 = 128-key tiles with one / two softmax warp groups


def _tc(q, kc, vc, m, nq, nkv, hd, bs, wg=None):
    """`wg`: shape of the kernel (1, 2 or 4, see DEFAULT_WG); None keeps the library default."""
    out = torch.empty_like(q)
    lib = _native.kernels()
    if wg is not None:
        lib.gv_set_prefill_tc_warpgroups(wg)
    try:
        _native.call("paged_attention_prefill_tc", q, kc, vc, m.block_tables, m.query_start_loc, m.cached_lens, out,
                     q.shape[0], m.batch, m.max_q_len, nq, nkv, hd, bs, m.block_tables.shape[1], 1.0, kc.shape[0])
    finally:
        if wg is not None:
            lib.gv_set_prefill_tc_warpgroups(DEFAULT_WG)
    return out


def _ref_gpu(q, kc, vc, mc, nq, nkv, hd, bs, chunk=2048):
    """fp32 causal attention over the paged cache, evaluated on the device."""
    out = torch.zeros(q.shape, dtype=torch.float32, device=DEV)
    G = nq // nkv
    kc, vc = kc.to(DEV), vc.to(DEV)
    for b in range(mc.batch):
        qs, qe = int(mc.query_start_loc[b]), int(mc.query_start_loc[b + 1])
        cached = int(mc.cached_lens[b])
        total = cached + qe - qs
        nblk = (total + bs - 1) // bs
        blocks = mc.block_tables[b, :nblk].long().to(DEV)
        k = kc[blocks].reshape(nblk * bs, nkv, hd)[:total].float()
        v = vc[blocks].reshape(nblk * bs, nkv, hd)[:total].float()
        for h in range(nq):
            kh, vh = k[:, h // G], v[:, h // G]
            for c0 in range(qs, qe, chunk):
                c1 = min(qe, c0 + chunk)
                qq = q[c0:c1, h * hd:(h + 1) * hd].to(DEV).float()
                s = qq @ kh.t()
                lim = cached + torch.arange(c0 - qs, c1 - qs, device=DEV)[:, None]
                s = s.masked_fill(torch.arange(total, device=DEV)[None, :] > lim, float("-inf"))
                out[c0:c1, h * hd:(h + 1) * hd] = torch.softmax(s, -1) @ vh
    return out


@pytest.mark.parametrize("bs", [16, 32, 64, 128, 256])
@pytest.mark.parametrize("nq,nkv", [(8, 2), (4, 4), (5, 1)])
def test_prefill_tc_block_sizes_and_groups(bs, nq, nkv):
    hd = 128
    lens = [1, 127, 128, 129, 300, 7, 513]
    cached = [0, 0, 5, 130, 0, 900, 64]
    q, kc, vc, mc, m = build(lens, cached, nq, nkv, hd, bs, seed=bs + nq)
    want = ref.paged_attention(q, kc, vc, mc.block_tables, mc.query_start_loc, mc.cached_lens, nq, nkv, hd, bs)
    for wg in (1, 2, 4):
        got = _tc(q.to(DEV), kc.to(DEV), vc.to(DEV), m, nq, nkv, hd, bs, wg=wg)
        close(got, want, atol=1e-2, rtol=2e-2, what=f"prefill tc bs={bs} {nq}/{nkv} shape={wg}")
    status_ok()


def test_prefill_tc_forces_lazy_rescale_of_the_output():
    """Keys grow with their position, so the row maximum climbs by far more than 2^8 from tile to
    tile and the accumulated output has to be read back and rescaled several times."""
    nq, nkv, hd, bs = 2, 1, 128, 128
    lens, cached = [700, 300], [0, 260]
    q, kc, vc, mc, m = build(lens, cached, nq, nkv, hd, bs, seed=5)
    # per request, scale key rows by their position: logits spread over hundreds of log2 units
    for b in range(2):
        total = lens[b] + cached[b]
        for j in range((total + bs - 1) // bs):
            blk = int(mc.block_tables[b, j])
            pos = torch.arange(j * bs, (j + 1) * bs).float()
            kc[blk] = (kc[blk].float() * (0.2 + pos / 40.0)[:, None, None]).bfloat16()
    q = (q.float() * 3).bfloat16()
    want = ref.paged_attention(q, kc, vc, mc.block_tables, mc.query_start_loc, mc.cached_lens, nq, nkv, hd, bs)
    for wg in (1, 2, 4):
        got = _tc(q.to(DEV), kc.to(DEV), vc.to(DEV), m, nq, nkv, hd, bs, wg=wg)
        close(got, want, atol=2e-2, rtol=2e-2, what=f"prefill tc with rescaling, warp groups={wg}")
    status_ok()


def test_prefill_tc_is_the_default_path_and_matches_the_mma_sync_kernel():
    nq, nkv, hd, bs = 32, 8, 128, 128
    lens, cached = [1024, 300, 77], [0, 128, 1000]
    q, kc, vc, mc, m = build(lens, cached, nq, nkv, hd, bs, seed=11)
    qd, kd, vd = q.to(DEV), kc.to(DEV), vc.to(DEV)
    before = _native.LAUNCHES
    a = F.paged_attention(qd, kd, vd, m, nq, nkv, hd)
    assert _native.LAUNCHES == before + 1
    old = torch.empty_like(qd)
    _native.call("paged_attention_prefill", qd, kd, vd, m.block_tables, m.query_start_loc, m.cached_lens, old,
                 m.batch, m.max_q_len, nq, nkv, hd, bs, m.block_tables.shape[1], 1.0, kd.shape[0])
    assert torch.equal(a, _tc(qd, kd, vd, m, nq, nkv, hd, bs))
    close(a, old, atol=1e-2, rtol=2e-2, what="tc vs mma.sync")
    status_ok()


def test_prefill_tc_32769_tokens():
    nq, nkv, hd, bs = 2, 1, 128, 128
    q, kc, vc, mc, m = build([32769], [0], nq, nkv, hd, bs, seed=2)
    want = _ref_gpu(q, kc, vc, mc, nq, nkv, hd, bs)
    for wg in (1, 2, 4):
        got = _tc(q.to(DEV), kc.to(DEV), vc.to(DEV), m, nq, nkv, hd, bs, wg=wg)
        close(got, want, atol=1e-2, rtol=2e-2, what=f"32769-token prefill, warp groups={wg}")
    status_ok()


@pytest.mark.parametrize("ctx", [33000, 60000, 131071])
def test_decode_long_caches(ctx):
    """Split-KV decode with the in-kernel merge over long caches, splits chosen by the tuner."""
    nq, nkv, hd, bs = 8, 1, 128, 128
    rt = _native.runtime()
    ns = rt.pick_decode_splits(2, nkv, ctx, 148, 1, 32).splits
    assert ns > 1
    q, kc, vc, mc, m = build([1, 1], [ctx - 1, ctx // 3], nq, nkv, hd, bs, seed=ctx % 97, decode=True, splits=ns)
    want = _ref_gpu(q, kc, vc, mc, nq, nkv, hd, bs)
    got = F.paged_attention(q.to(DEV), kc.to(DEV), vc.to(DEV), m, nq, nkv, hd)
    close(got, want, atol=1e-2, rtol=2e-2, what=f"decode over {ctx} cached tokens ({ns} splits)")
    status_ok()
