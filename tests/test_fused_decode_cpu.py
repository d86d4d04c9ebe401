"""The fused decode path on the CPU: RMSNorm folded into the consumer GEMMs (norm weight in the
weight columns, per-token factor from partial sums of squares), residual add in the producer, RoPE
and cache write behind the QKV projection. The fp32 definitions of the fused ops must agree with
the unfused composition, the folded model with the plain one, and a checkpoint written from a
folded model must hold the original weights."""
import copy

import pytest
import torch

from gvirt_b200.engine.llm import LLM
from gvirt_b200.engine.scheduler import SamplingParams
from gvirt_b200.models import loader
from gvirt_b200.models import weights as W
from gvirt_b200.models.transformer import Transformer
from gvirt_b200.ops import decode_ops as D
from gvirt_b200.ops import functional as F
from gvirt_b200.ops import reference as ref
from gvirt_b200.parallel.state import ParallelContext
from tests.test_engine_cpu import tiny_cfg


def _meta(T, slots, pos):
    z = torch.zeros(1, dtype=torch.int32)
    return F.AttnMeta(z, z, z, z, slots, z.view(1, 1), pos, batch=1, num_tokens=T)


def test_fused_op_definitions_match_the_unfused_composition():
    g = torch.Generator().manual_seed(3)
    T, H, N = 7, 256, 384
    x = torch.randn(T, H, generator=g)
    gw = 1 + 0.3 * torch.randn(H, generator=g)
    w = torch.randn(N, H, generator=g) * 0.05
    eps = 1e-6
    h = ref.norm(x, gw, None, eps)
    wf = D.fold_norm_weight(w, gw)
    # sums of squares as a fused producer leaves them (per 128-feature tile) and as the stand-alone form
    ss = D.new_sumsq(H, "cpu")
    ss[:T] = x.reshape(T, H // 128, 128).pow(2).sum(-1)
    assert torch.allclose(D.linear_scaled(x, wf, ss, H, eps), h @ w.t(), atol=1e-5, rtol=1e-5)
    ss1 = torch.full((128, H // 128), 7.0)
    D.row_sumsq(x, ss1)
    assert torch.allclose(D.linear_scaled(x, wf, ss1, H, eps, tiles=1), h @ w.t(), atol=1e-5, rtol=1e-5)
    b = torch.randn(N, generator=g)
    assert torch.allclose(D.linear_scaled(x, wf, ss, H, eps, bias=b), h @ w.t() + b, atol=1e-5, rtol=1e-5)
    # SwiGLU epilogue over the block-interleaved layout
    wgu = torch.randn(2 * 128, H, generator=g) * 0.05
    want = ref.silu_and_mul(h @ wgu.t())
    got = D.linear_scaled(x, F.interleave_gate_up(D.fold_norm_weight(wgu, gw)), ss, H, eps, swiglu=True)
    assert torch.allclose(got, want, atol=1e-5, rtol=1e-5)
    # producer: residual add in place + per-tile sums of squares
    a = torch.randn(T, 96, generator=g)
    wo = torch.randn(H, 96, generator=g) * 0.1
    x2 = x.clone()
    ss2 = torch.zeros_like(ss)
    D.linear_residual(a, wo, x2, ss2)
    assert torch.allclose(x2, x + a @ wo.t(), atol=1e-5)
    assert torch.allclose(ss2[:T].sum(1), x2.pow(2).sum(-1), rtol=1e-5)
    x3, ss3 = x.clone(), torch.zeros_like(ss)
    D.add_residual_sumsq(a @ wo.t(), x3, ss3)
    assert torch.allclose(x3, x2, atol=1e-5) and torch.allclose(ss3.view(-1)[:T], ss2[:T].sum(1), rtol=1e-5)
    assert torch.allclose(D.unfold_norm_weight(wf, gw), w, atol=1e-6)


@pytest.mark.parametrize("bias,qkn", [(False, False), (True, True)])
def test_fused_qkv_rope_definition(bias, qkn):
    """QKV GEMM + RoPE + cache write in one op == scaled GEMM followed by the RoPE op."""
    g = torch.Generator().manual_seed(5)
    T, H, nq, nkv, hd, bs, nblk = 9, 256, 4, 2, 128, 16, 3
    x = torch.randn(T, H, generator=g)
    w = torch.randn((nq + 2 * nkv) * hd, H, generator=g) * 0.05
    b = torch.randn((nq + 2 * nkv) * hd, generator=g) * 0.1 if bias else None
    qn = 1 + 0.2 * torch.randn(hd, generator=g) if qkn else None
    kn = 1 + 0.2 * torch.randn(hd, generator=g) if qkn else None
    tab = ref.rope_table(64, hd, 10000.0)
    pos = torch.randint(0, 64, (T,), generator=g, dtype=torch.int64)
    slots = torch.randperm(bs * nblk, generator=g)[:T].to(torch.int32)
    slots[2] = -1
    ss = D.new_sumsq(H, "cpu")
    D.row_sumsq(x, ss)
    kc, vc = torch.zeros(nblk, bs, nkv, hd), torch.zeros(nblk, bs, nkv, hd)
    q = D.linear_rope(x, w, _meta(T, slots, pos), tab, kc, vc, nq, nkv, ss, H, 1e-6, bias=b, q_norm_w=qn,
                      k_norm_w=kn, tiles=1)
    kc2, vc2 = torch.zeros_like(kc), torch.zeros_like(vc)
    qkv = ref.norm(x, None, None, 1e-6) @ w.t()
    q2 = ref.rope_kvwrite(qkv, pos, slots, tab, kc2, vc2, nq, nkv, hd, hd, hd ** -0.5, b, qn, kn, 1e-6)
    assert torch.allclose(q, q2, atol=1e-5) and torch.allclose(kc, kc2, atol=1e-5) and torch.allclose(vc, vc2, atol=1e-5)


def _random_norms(w, seed):
    g = torch.Generator().manual_seed(seed)
    for lw in w.layers:
        lw.attn_norm = (1 + 0.3 * torch.randn(lw.attn_norm.shape, generator=g)).to(lw.attn_norm.dtype)
        lw.mlp_norm = (1 + 0.3 * torch.randn(lw.mlp_norm.shape, generator=g)).to(lw.mlp_norm.dtype)


@pytest.mark.parametrize("kw", [dict(), dict(head_dim=128, num_heads=2, num_kv_heads=1, qkv_bias=False, qk_norm=True)])
def test_folded_model_matches_plain_model_and_saves_original_weights(tmp_path, kw):
    """Hidden states of the fused loop (prefill chunk of 19 tokens, then decode steps through the
    engine) agree with the generic loop; heads of 128 also take the fused QKV + RoPE op."""
    cfg = tiny_cfg(**kw)
    ctx = ParallelContext()
    w_plain = W.init_random(cfg, ctx, seed=4, device="cpu")
    _random_norms(w_plain, 1)
    w_fold = copy.deepcopy(w_plain)
    m_plain, m_fold = Transformer(cfg, w_plain, ctx), Transformer(cfg, w_fold, ctx)
    m_fold._prepare_device_layouts(force=True)
    assert m_fold.fused_decode and not m_plain.fused_decode
    assert m_fold.rope_fused == (cfg.head_dim == 128)
    assert all(torch.equal(lw.attn_norm, torch.ones_like(lw.attn_norm)) for lw in w_fold.layers)
    g = torch.Generator().manual_seed(9)
    prompts = [torch.randint(1, cfg.vocab_size, (n,), generator=g).tolist() for n in (13, 6)]
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    seen = {}
    for name, m in (("plain", m_plain), ("fold", m_fold)):
        llm = LLM(m)
        hs = []
        orig = m.compute_logits
        m.compute_logits = lambda hidden, meta, ws=None, batch=None, _o=orig, _h=hs: (
            _h.append(hidden.detach().clone()), _o(hidden, meta, ws, batch))[1]
        outs = [o.output for o in llm.generate(prompts, sp)]
        seen[name] = (outs, hs)
    assert seen["plain"][0] == seen["fold"][0]
    for a, b in zip(seen["plain"][1], seen["fold"][1]):
        assert a.shape == b.shape and torch.allclose(a, b, atol=2e-4, rtol=2e-4)
    loader.save_hf_checkpoint(cfg, w_fold, str(tmp_path))
    _, w_back, _, _ = loader.load_pretrained(str(tmp_path), ctx, device="cpu", dtype="float32")
    for a, b in zip(w_back.layers, w_plain.layers):
        assert torch.allclose(a.w_qkv, b.w_qkv, atol=1e-6) and torch.allclose(a.w_gate_up, b.w_gate_up, atol=1e-6)
        assert torch.equal(a.attn_norm, b.attn_norm) and torch.equal(a.mlp_norm, b.mlp_norm)


def test_interleave16_round_trip_and_cpu_definition():
    """Expert gate / up rows in blocks of [16 gate | 16 up]: the permutation inverts exactly and the
    CPU definition of the fused grouped GEMM equals GEMM -> SwiGLU on the original order."""
    import torch
    from gvirt_b200.ops import moe_ops
    from gvirt_b200.ops import reference as ref
    g = torch.Generator().manual_seed(0)
    E, I, K = 3, 48, 32
    w13 = torch.randn(E, 2 * I, K, generator=g)
    il = moe_ops.interleave16(w13)
    assert torch.equal(moe_ops.deinterleave16(il), w13)
    # block b of 32 rows = gate rows 16 b .. 16 b + 15, then up rows 16 b .. 16 b + 15
    assert torch.equal(il[:, 32:48], w13[:, 16:32]) and torch.equal(il[:, 48:64], w13[:, I + 16:I + 32])
    xs = torch.randn(10, K, generator=g)
    off = torch.tensor([0, 4, 4, 10], dtype=torch.int32)
    act = torch.zeros(10, I)
    moe_ops.grouped_gemm_swiglu(xs, il, off, act, clamp=0.7)
    gu = torch.zeros(10, 2 * I)
    moe_ops.grouped_gemm(xs, w13, off, gu)
    assert torch.allclose(act, ref.silu_and_mul(gu, None, 0.7))
    T = 6
    wts = torch.rand(T, 2, generator=g)
    ids = torch.tensor([[0, 1], [2, 0], [1, 2], [0, 2], [1, 0], [2, 1]], dtype=torch.int32)
    x = torch.randn(T, K, generator=g)
    w2 = torch.randn(E, K, I, generator=g)
    a = moe_ops.experts_forward(x, wts, ids, il, w2, 0, 0.0, il16=True)
    b = moe_ops.experts_forward(x, wts, ids, w13, w2, 0, 0.0)
    assert torch.allclose(a, b)


def test_moe_model_with_interleaved_expert_rows_matches_and_saves_original_weights(tmp_path):
    """A tiny MoE model whose expert gate / up rows were re-ordered for the fused grouped GEMM samples
    the same tokens as the plain one, and a checkpoint written from it holds the original rows."""
    kw = dict(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, swiglu_clamp=2.0)
    cfg = tiny_cfg(**kw)
    ctx = ParallelContext()
    w_plain = W.init_random(cfg, ctx, seed=8, device="cpu")
    w_il = copy.deepcopy(w_plain)
    m_plain, m_il = Transformer(cfg, w_plain, ctx), Transformer(cfg, w_il, ctx)
    m_il._prepare_device_layouts(force=True)
    moe_layers = [lw for lw in w_il.layers if getattr(lw, "w13", None) is not None]
    assert moe_layers and all(getattr(lw, "w13_il16", False) for lw in moe_layers)
    assert not torch.equal(moe_layers[0].w13, [lw for lw in w_plain.layers if getattr(lw, "w13", None) is not None][0].w13)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(1, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 4)]
    sp = SamplingParams(max_tokens=5, ignore_eos=True)
    a = [o.output for o in LLM(m_plain).generate(prompts, sp)]
    b = [o.output for o in LLM(m_il).generate(prompts, sp)]
    assert a == b
    loader.save_hf_checkpoint(cfg, w_il, str(tmp_path))
    _, w_back, _, _ = loader.load_pretrained(str(tmp_path), ctx, device="cpu", dtype="float32")
    for l0, l1 in zip(w_plain.layers, w_back.layers):
        if getattr(l0, "w13", None) is not None:
            assert torch.equal(l0.w13, l1.w13)
