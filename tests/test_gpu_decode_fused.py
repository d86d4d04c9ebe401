"""Fused decode-step kernels (gemm_decode.cu, the in-kernel split merge of attention_decode.cu)
against the fp32 definitions evaluated on the same bf16 inputs, and the fused layer loop of the
model against the generic loop on the same weights."""
import os

import pytest
import torch

from gvirt_b200 import _native
from gvirt_b200.ops import decode_ops as D
from gvirt_b200.ops import functional as F
from gvirt_b200.ops import reference as ref
from tests.gpu_util import close, status_ok

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).bfloat16().to(DEV)


def _ss_tiles(x):
    """Per-128-feature sums of squares in the producer layout [128 tokens, H / 128]."""
    T, H = x.shape
    ss = D.new_sumsq(H, x.device)
    ss[:T] = x.float().reshape(T, H // 128, 128).pow(2).sum(-1)
    return ss


@pytest.mark.parametrize("M", [1, 7, 16, 33, 64, 100, 128])
@pytest.mark.parametrize("splitk", [0, 1, 3])
def test_scaled_gemm_plain_bias_swiglu(M, splitk):
    H, N, eps = 1024, 768, 1e-5
    x, w, b = rnd(M, H, seed=1), rnd(N, H, seed=2, scale=0.05), rnd(N, seed=3)
    ss = _ss_tiles(x)
    s = D.token_scale(ss, M, H, eps)[:, None]
    want = (x.float() @ w.float().t()) * s
    close(D.linear_scaled(x, w, ss, H, eps, splitk=splitk), want, atol=3e-2, rtol=2e-2, what="scaled gemm")
    close(D.linear_scaled(x, w, ss, H, eps, bias=b, splitk=splitk), want + b.float(), atol=3e-2, rtol=2e-2,
          what="scaled gemm + bias")
    close(D.linear_scaled(x, w, None, H, eps, splitk=splitk), x.float() @ w.float().t(), atol=3e-2, rtol=2e-2,
          what="unscaled")
    # whole-row form of the sums of squares (one tile), as written by the stand-alone producer
    ss1 = torch.full_like(ss, 123.0)
    D.row_sumsq(x, ss1)
    close(D.linear_scaled(x, w, ss1, H, eps, tiles=1, splitk=splitk), want, atol=3e-2, rtol=2e-2, what="one tile")
    wil = F.interleave_gate_up(w)
    gu = (want).bfloat16().float()
    close(D.linear_scaled(x, wil, ss, H, eps, swiglu=True, splitk=splitk),
          torch.nn.functional.silu(gu[:, :N // 2]) * gu[:, N // 2:], atol=3e-2, rtol=3e-2, what="swiglu")
    status_ok()


@pytest.mark.parametrize("M,N,K", [(1, 512, 256), (64, 4096, 1024), (100, 1024, 3584), (128, 256, 64)])
@pytest.mark.parametrize("splitk", [0, 1, 4])
def test_residual_gemm_updates_in_place_and_emits_sumsq(M, N, K, splitk):
    a, w, b = rnd(M, K, seed=4, scale=0.5), rnd(N, K, seed=5, scale=0.05), rnd(N, seed=6)
    x0 = rnd(M, N, seed=7)
    for bias in (None, b):
        x = x0.clone()
        ss = torch.full((128, N // 128), -1.0, device=DEV)
        D.linear_residual(a, w, x, ss, bias=bias, splitk=splitk)
        want = x0.float() + a.float() @ w.float().t() + (bias.float() if bias is not None else 0)
        close(x, want, atol=3e-2, rtol=2e-2, what="residual gemm")
        want_ss = x.float().reshape(M, N // 128, 128).pow(2).sum(-1)          # of the rows as stored
        close(ss[:M], want_ss, atol=1e-3, rtol=1e-4, what="tile sums of squares")
        assert (ss[M:] == -1).all()
    status_ok()


@pytest.mark.parametrize("M", [1, 5, 64, 128])
@pytest.mark.parametrize("bias,qkn", [(False, False), (True, False), (False, True)])
def test_qkv_gemm_with_rope_and_cache_write(M, bias, qkn):
    H, nq, nkv, hd, bs, nblk, eps = 512, 4, 2, 128, 128, 3, 1e-5
    x = rnd(M, H, seed=8)
    w = rnd((nq + 2 * nkv) * hd, H, seed=9, scale=0.05)
    b = rnd((nq + 2 * nkv) * hd, seed=10, scale=0.1) if bias else None
    qn = (1 + 0.2 * rnd(hd, seed=11).float()).bfloat16() if qkn else None
    kn = (1 + 0.2 * rnd(hd, seed=12).float()).bfloat16() if qkn else None
    tab = ref.rope_table(512, hd, 10000.0, device=DEV)
    g = torch.Generator().manual_seed(M)
    pos = torch.randint(0, 512, (M,), generator=g, dtype=torch.int64).to(DEV)
    slots = torch.randperm(bs * nblk, generator=g)[:M].to(torch.int32)
    if M > 3:
        slots[3] = -1
    slots = slots.to(DEV)
    z = torch.zeros(1, dtype=torch.int32, device=DEV)
    meta = F.AttnMeta(z, z, z, z, slots, z.view(1, 1), pos, batch=1, num_tokens=M)
    ss = _ss_tiles(x)
    kc = torch.zeros(nblk, bs, nkv, hd, device=DEV, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    q = D.linear_rope(x, w, meta, tab, kc, vc, nq, nkv, ss, H, eps, bias=b, q_norm_w=qn, k_norm_w=kn, qk_eps=1e-6)
    # the same arithmetic in two launches: scaled GEMM (rounded to bf16), then the RoPE kernel's definition
    qkv = D.linear_scaled(x, w, ss, H, eps)
    kc_r, vc_r = torch.zeros_like(kc).cpu(), torch.zeros_like(vc).cpu()
    q_r = ref.rope_kvwrite(qkv.cpu(), pos.cpu(), slots.cpu(), tab.cpu(), kc_r, vc_r, nq, nkv, hd, hd, hd ** -0.5,
                           b.cpu() if bias else None, qn.cpu() if qkn else None, kn.cpu() if qkn else None, 1e-6)
    close(q, q_r, atol=2e-2, rtol=2e-2, what="q")
    close(kc, kc_r, atol=3e-2, rtol=2e-2, what="k cache")
    close(vc, vc_r, atol=3e-2, rtol=2e-2, what="v cache")
    status_ok()


def test_in_kernel_split_merge_matches_the_two_launch_form():
    from tests.test_gpu_attention import build
    nq, nkv, hd, bs = 32, 8, 128, 128
    lens = [1, 130, 1060, 517, 2048, 77, 900, 4000]
    q, kc, vc, _, m = build([1] * len(lens), [n - 1 for n in lens], nq, nkv, hd, bs, seed=3, decode=True)
    q, kc, vc, bt, sl = q.to(DEV), kc.to(DEV), vc.to(DEV), m.block_tables, m.seq_lens
    B = len(lens)
    for ns in (2, 3, 7):
        po = torch.empty(B * nq * ns * hd, dtype=torch.float32, device=DEV)
        pl = torch.empty(B * nq * ns, dtype=torch.float32, device=DEV)
        two = torch.empty_like(q)
        _native.call("paged_attention_decode", q, kc, vc, bt, sl, two, po, pl, B, nq, nkv, hd, bs, bt.shape[1], ns,
                     1.0, kc.shape[0])
        cnt = torch.zeros(B * nkv, dtype=torch.int32, device=DEV)
        for _ in range(2):          # the second call finds the counters back at zero
            one = torch.empty_like(q)
            _native.call("paged_attention_decode_merged", q, kc, vc, bt, sl, one, po, pl, cnt, B, nq, nkv, hd, bs,
                         bt.shape[1], ns, 1.0, kc.shape[0])
            assert torch.equal(one, two)
        assert int(cnt.abs().sum()) == 0
    status_ok()


def _tiny_llama(**kw):
    from gvirt_b200.models import presets
    over = dict(num_layers=3, hidden_size=512, intermediate_size=1408, num_heads=4, num_kv_heads=2, head_dim=128,
                vocab_size=4096, max_seq_len=512, max_batch_size=8, max_num_batched_tokens=256, block_size=128,
                max_position_embeddings=1024)
    over.update(kw)
    return presets.get("llama-3-8b", **over)


@pytest.mark.parametrize("kw", [dict(), dict(qkv_bias=True), dict(qk_norm=True), dict(head_dim=64, num_heads=8,
                                                                                     num_kv_heads=4)])
def test_fused_layer_loop_matches_generic_loop(kw):
    """Same weights, same prompts: the engine with the fused decode loop against the engine with
    GVIRT_FUSED_DECODE=0, both judged by the fp32 oracle on the same (bf16-rounded) weights: the
    first-step logits of the fused loop must be as close to the oracle as those of the generic
    loop (both are bf16 pipelines that round at different points, so they are not compared
    element by element with each other). Greedy tokens of the first steps agree, and the CUDA
    graph replay of the fused loop reproduces its eager tokens exactly."""
    import copy

    from gvirt_b200 import config
    from gvirt_b200.engine.llm import LLM
    from gvirt_b200.engine.scheduler import SamplingParams
    from gvirt_b200.models import weights as W
    from gvirt_b200.models.transformer import Transformer
    from gvirt_b200.parallel.state import ParallelContext
    from gvirt_b200.reference_cpu.oracle import NaiveDecoder
    cfg = _tiny_llama(**kw)
    ctx = ParallelContext(device=torch.device(DEV))
    w0 = W.init_random(cfg, ctx, seed=2, device=DEV, std=0.05)
    g = torch.Generator().manual_seed(1)
    for lw in w0.layers:
        lw.attn_norm = (1 + 0.3 * torch.randn(cfg.hidden_size, generator=g)).bfloat16().to(DEV)
        lw.mlp_norm = (1 + 0.3 * torch.randn(cfg.hidden_size, generator=g)).bfloat16().to(DEV)
    prompts = [torch.randint(1, cfg.vocab_size, (n,), generator=g).tolist() for n in (40, 7, 60, 3)]
    sp = SamplingParams(max_tokens=8, ignore_eos=True)
    # oracle: fp32 arithmetic on the CPU over the same weights
    ccfg = copy.copy(cfg)
    ccfg.dtype = "float32"
    wc = copy.deepcopy(w0)
    for obj in [wc] + list(wc.layers):
        for k2, v in list(vars(obj).items()):
            if isinstance(v, torch.Tensor):
                setattr(obj, k2, v.float().cpu())
    oracle = NaiveDecoder(ccfg, wc)
    want = torch.stack([oracle.logits(torch.tensor([p]))[0, -1] for p in prompts])
    res = {}
    for mode in ("0", "1"):
        os.environ["GVIRT_FUSED_DECODE"] = mode
        config.reload_flags()
        try:
            m = Transformer(cfg, copy.deepcopy(w0), ctx)
            assert m.fused_decode == (mode == "1")
            seen = []
            orig = m.compute_logits
            m.compute_logits = lambda hidden, meta, ws=None, batch=None, _o=orig, _s=seen: (
                lambda lg: (_s.append(lg.detach().float().cpu()) if lg.device.type != "meta" else None, lg)[1])(
                    _o(hidden, meta, ws, batch))
            llm = LLM(m, num_blocks=32, use_graphs=False)
            res[mode] = ([o.output for o in llm.generate(prompts, sp)], seen[0])
            if mode == "1":
                llm2 = LLM(Transformer(cfg, copy.deepcopy(w0), ctx), num_blocks=32, use_graphs=True)
                res["graph"] = [o.output for o in llm2.generate(prompts, sp)]
        finally:
            os.environ.pop("GVIRT_FUSED_DECODE", None)
            config.reload_flags()
    top = want.abs().max().item()
    err = {k: (res[k][1] - want).abs().max().item() / top for k in ("0", "1")}
    assert res["1"][1].shape == want.shape and torch.isfinite(res["1"][1]).all()
    assert err["1"] <= 1.5 * err["0"] + 0.01, err          # the fused loop is no further from the oracle
    assert err["1"] <= 0.06, err
    # greedy tokens: the first one follows from the compared logits; later ones may flip on bf16
    # near-ties between the two loops, so most of the first four have to agree, not all
    assert [o[0] for o in res["0"][0]] == [o[0] for o in res["1"][0]]
    same = sum(int(a == b) for p, q in zip(res["0"][0], res["1"][0]) for a, b in zip(p[:4], q[:4]))
    assert same >= 13, (same, res["0"][0], res["1"][0])
    assert res["graph"] == res["1"][0]          # graph replay of the fused loop == eager fused loop
    status_ok()
