"""Memory-bound kernels vs their fp32 PyTorch definitions (shapes from the reference's
per-op tests: rmsnorm.py, add_and_rmsnorm.py, rope_and_cache.py, silu_and_mul.py)."""
import pytest
import torch

from gvirt_b200.ops import functional as F
from gvirt_b200.ops import reference as ref
from tests.gpu_util import close, status_ok

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rnd(*shape, scale=1.0, seed=0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(*shape, device=DEV, generator=g) * scale).bfloat16()


@pytest.mark.parametrize("kind", ["rms", "layer", "l2"])
@pytest.mark.parametrize("rows,cols", [(64, 8192), (5, 256), (3, 6144), (2, 32768)])
def test_norm(kind, rows, cols):
    x, w, b = rnd(rows, cols), rnd(cols, seed=1), rnd(cols, seed=2)
    y = F.norm(x, w, 1e-6, kind, bias=b)
    close(y, ref.norm(x.cpu(), w.cpu(), b.cpu(), 1e-6, kind), what=f"norm {kind}")


def test_add_rmsnorm_updates_residual_in_place():
    x, res, w = rnd(64, 6144), rnd(64, 6144, seed=3), rnd(6144, seed=1)
    res_ref = res.cpu().clone()
    want = ref.norm(x.cpu(), w.cpu(), None, 1e-5, "rms", residual=res_ref)
    y = F.add_rmsnorm(x, res, w, 1e-5)
    close(res, res_ref, atol=1e-2, what="residual")
    close(y, want, what="add_rmsnorm")


def test_per_head_norm_strided():
    # [64, 128 * (8 + 2)] with 8 sub-norms of width 128 on the first 1024 columns
    x = rnd(64, 1280)
    w = rnd(128, seed=1)
    y = F.norm(x[:, :1024], w, 1e-6, "rms", cnt=8)
    close(y, ref.norm(x[:, :1024].cpu(), w.cpu(), None, 1e-6, "rms", cnt=8), what="per-head norm")


def test_sumsq_and_extvar():
    x, w = rnd(16, 1024), rnd(1024, seed=1)
    ss = F.sumsq(x)
    close(ss, ref.sumsq(x.cpu()), atol=1e-1, rtol=1e-2, what="sumsq")
    y = F.rmsnorm_extvar(x, w, ss * 2, 2.0, 1e-6)
    want = ref.norm(x.cpu(), w.cpu(), None, 1e-6, "rms")
    close(y, want, what="extvar")


def _meta(T, slots, pos, device=DEV):
    z = torch.zeros(1, dtype=torch.int32, device=device)
    return F.AttnMeta(z, z, z, z, slots.to(device), z.view(1, 1), pos.to(device), batch=1, num_tokens=T)


@pytest.mark.parametrize("hd,rot,bias,qkn,inter", [(128, 128, False, False, False), (128, 64, True, False, False),
                                                   (64, 64, False, True, False), (128, 128, True, True, False),
                                                   (64, 64, False, False, True)])
def test_rope_kvwrite(hd, rot, bias, qkn, inter):
    T, nq, nkv, bs, nblk = 80, 32, 8, 128, 4
    qkv = rnd(T, (nq + 2 * nkv) * hd)
    b = rnd((nq + 2 * nkv) * hd, seed=5, scale=0.1) if bias else None
    qn = rnd(hd, seed=6) if qkn else None
    kn = rnd(hd, seed=7) if qkn else None
    tab = ref.rope_table(512, rot, 10000.0, device=DEV)
    pos = torch.randint(0, 512, (T,), dtype=torch.int64)
    slots = torch.randperm(bs * nblk)[:T].to(torch.int32)
    slots[3] = -1
    kc = torch.zeros(nblk, bs, nkv, hd, device=DEV, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    meta = _meta(T, slots, pos)
    q = F.rope_kvwrite(qkv, meta, tab, kc, vc, nq, nkv, hd, rot, hd ** -0.5, b, qn, kn, 1e-6, interleaved=inter)
    kc_r, vc_r = torch.zeros_like(kc).cpu(), torch.zeros_like(vc).cpu()
    q_r = ref.rope_kvwrite(qkv.cpu(), pos, slots, tab.cpu(), kc_r, vc_r, nq, nkv, hd, rot, hd ** -0.5,
                           b.cpu() if bias else None, qn.cpu() if qkn else None, kn.cpu() if qkn else None,
                           1e-6, interleaved=inter)
    close(q, q_r, what="rope q")
    close(kc, kc_r, what="k cache")
    close(vc, vc_r, atol=1e-2, what="v cache")
    status_ok()


def test_mrope_sections():
    T, nq, nkv, hd = 16, 4, 2, 128
    qkv = rnd(T, (nq + 2 * nkv) * hd)
    tab = ref.rope_table(256, hd, 10000.0, device=DEV)
    pos = torch.randint(0, 256, (3, T), dtype=torch.int64)
    slots = torch.arange(T, dtype=torch.int32)
    for mode in (1, 2):
        kc = torch.zeros(1, 128, nkv, hd, device=DEV, dtype=torch.bfloat16)
        vc = torch.zeros_like(kc)
        meta = _meta(T, slots, pos)
        q = F.rope_kvwrite(qkv, meta, tab, kc, vc, nq, nkv, hd, mrope_mode=mode, mrope_sections=(24, 20, 20))
        kr, vr = torch.zeros_like(kc).cpu(), torch.zeros_like(kc).cpu()
        qr = ref.rope_kvwrite(qkv.cpu(), pos, slots, tab.cpu(), kr, vr, nq, nkv, hd, hd, hd ** -0.5,
                              mrope_mode=mode, mrope_sections=(24, 20, 20))
        close(q, qr, what=f"mrope mode {mode}")
        close(kc, kr, what=f"mrope k mode {mode}")


@pytest.mark.parametrize("rows,d", [(41, 2304), (41, 6400), (1, 8)])
def test_silu_and_mul(rows, d):
    x = rnd(rows, 2 * d)
    close(F.silu_and_mul(x), ref.silu_and_mul(x.cpu()), atol=2e-2, rtol=2e-2, what="swiglu")
    num = torch.tensor([rows // 2], dtype=torch.int32, device=DEV)
    out = torch.zeros(rows, d, device=DEV, dtype=torch.bfloat16)
    F.silu_and_mul(x, out=out, num=num)
    assert (out[rows // 2:] == 0).all()
    close(F.silu_and_mul(x, clamp=1.0), ref.silu_and_mul(x.cpu(), clamp=1.0), what="clamped swiglu")


def test_elementwise_set():
    a, b = rnd(33, 1024), rnd(33, 1024, seed=1)
    close(F.add(a, b), a.float() + b.float(), what="add")
    close(F.sigmoid_gate_mul(a, b), a.float() * torch.sigmoid(b.float()), what="gate")
    close(F.muls(a, 0.37), a.float() * 0.37, what="muls")
    bias = rnd(1024, seed=2)
    close(F.add_bias(a, bias), a.float() + bias.float(), what="add_bias")
    assert torch.equal(F.cast(F.cast(a, torch.float32), torch.bfloat16), a)
    t = rnd(3, 70, 45)
    assert torch.equal(F.transpose12(t), t.transpose(1, 2).contiguous())


def test_embed_and_gather():
    table = rnd(1000, 512)
    ids = torch.randint(0, 2000, (77,), dtype=torch.int32, device=DEV)
    out = F.embed(ids, table, 500, 1500)
    assert torch.equal(out.cpu(), ref.embed(ids.cpu(), table.cpu(), 500, 1500))
    idx = torch.randint(0, 1000, (9,), dtype=torch.int32, device=DEV)
    assert torch.equal(F.gather_rows(table, idx), table[idx.long()])
    status_ok()


def test_sampling():
    logits = rnd(7, 50000, scale=3.0)
    lf = logits.float()
    mx = lf.max(-1)[0]

    def is_argmax(tok):
        return torch.equal(lf.gather(1, tok.long()[:, None])[:, 0], mx)

    assert is_argmax(F.sample(logits))
    assert is_argmax(F.sample(lf))
    temp = torch.full((7,), 0.8, device=DEV)
    topk = torch.full((7,), 5, dtype=torch.int32, device=DEV)
    topp = torch.full((7,), 1.0, device=DEV)
    a = F.sample(logits, temp, topk, topp, seed=1, step=3)
    b = F.sample(logits, temp, topk, topp, seed=1, step=3)
    assert torch.equal(a, b)
    fifth = lf.topk(5, -1)[0][:, -1]
    seen = set()
    for step in range(20):
        s = F.sample(logits, temp, topk, topp, seed=1, step=step).long()
        assert (lf.gather(1, s[:, None])[:, 0] >= fifth).all(), "sample outside the top-k set"
        seen.add(tuple(s.tolist()))
    assert len(seen) > 1
    # top-p = tiny -> always the arg-max
    topp0 = torch.full((7,), 1e-4, device=DEV)
    assert is_argmax(F.sample(logits, temp, None, topp0, seed=2, step=1))
    # greedy rows mixed with sampled rows
    temp2 = temp.clone()
    temp2[::2] = 0
    s = F.sample(logits, temp2, topk, topp, seed=3, step=0)
    assert torch.equal(lf.gather(1, s.long()[:, None])[:, 0][::2], mx[::2])


@pytest.mark.parametrize("bias,qkn,mode", [(False, False, 0), (True, True, 0), (False, False, 1), (False, True, 2)])
def test_rope_kvwrite_row_tiled(bias, qkn, mode):
    """One warp per token (chunks of 256 tokens or more): same results as the per-head kernels,
    including tokens without a cache slot, the folded bias / qk-norm and M-RoPE position rows."""
    T, nq, nkv, hd, bs = 300, 8, 2, 128, 128
    nblk = 4
    qkv = rnd(T, (nq + 2 * nkv) * hd)
    b = rnd((nq + 2 * nkv) * hd, seed=5, scale=0.1) if bias else None
    qn = rnd(hd, seed=6) if qkn else None
    kn = rnd(hd, seed=7) if qkn else None
    tab = ref.rope_table(512, hd, 10000.0, device=DEV)
    pos = torch.randint(0, 512, (T,) if mode == 0 else (3, T), dtype=torch.int64)
    slots = torch.randperm(bs * nblk)[:T].to(torch.int32)
    slots[3] = -1
    slots[257] = -1
    kc = torch.zeros(nblk, bs, nkv, hd, device=DEV, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    meta = _meta(T, slots, pos)
    kw = dict(mrope_mode=mode, mrope_sections=(24, 20, 20)) if mode else {}
    q = F.rope_kvwrite(qkv, meta, tab, kc, vc, nq, nkv, hd, hd, hd ** -0.5, b, qn, kn, 1e-6, **kw)
    kc_r, vc_r = torch.zeros_like(kc).cpu(), torch.zeros_like(vc).cpu()
    q_r = ref.rope_kvwrite(qkv.cpu(), pos, slots, tab.cpu(), kc_r, vc_r, nq, nkv, hd, hd, hd ** -0.5,
                           b.cpu() if bias else None, qn.cpu() if qkn else None, kn.cpu() if qkn else None,
                           1e-6, **kw)
    close(q, q_r, what="rope q (rows)")
    close(kc, kc_r, what="k cache (rows)")
    close(vc, vc_r, atol=1e-2, what="v cache (rows)")
    status_ok()
