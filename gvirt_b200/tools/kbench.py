"""Single-GPU kernel micro-benchmarks with roofline fractions.

    python -m gvirt_b200.tools.kbench gemm --m 64 --n 6144 --k 4096
    python -m gvirt_b200.tools.kbench swiglu --m 64 --n 28672 --k 4096
    python -m gvirt_b200.tools.kbench attn --batch 64 --ctx 1060 --nq 32 --nkv 8
    python -m gvirt_b200.tools.kbench mla --batch 32 --ctx 2048 --heads 128
    python -m gvirt_b200.tools.kbench layer --tp 1            # one Llama-3-8B decode layer, by parts
    python -m gvirt_b200.tools.kbench prefill_gemm --m 8192   # token-major / persistent kernels / cuBLAS
    python -m gvirt_b200.tools.kbench rope --tokens 8192      # RoPE + cache write on a prefill chunk
    python -m gvirt_b200.tools.kbench prefill_attn --batch 8 --tokens 1024   # tcgen05 vs mma.sync prefill attention

Each case runs `--chain` calls with rotating operands (so that nothing is served from L2) inside
one CUDA graph, times `--reps` replays with CUDA events after warm-up and prints one JSON line
with microseconds per call, achieved GB/s and the fraction of the HBM peak given by ``--hbm-gbs``
(default: ``hbm_gbs`` of MEASURED_PEAKS.json in the working directory when present, else 6650).
``--eager`` launches without a graph (what a profiler capture wants: ``--chain 1 --reps 1``).
The reference's counterpart is its ``matmul_bench`` binding (xlite/xlite/_C.cpp:1001-1029).
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from .. import _native
from ..ops import functional as F
from ..ops import mla_ops


def _peak(args) -> float:
    if args.hbm_gbs:
        return args.hbm_gbs
    try:
        with open("MEASURED_PEAKS.json") as f:
            return float(json.load(f)["hbm_gbs"])
    except Exception:  # noqa: BLE001 - optional file
        return 6650.0


def _time_us(fn, args) -> float:
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    if args.eager:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.reps):
            for i in range(args.chain):
                fn(i)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / (args.chain * args.reps)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(args.chain):
            fn(i)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (args.chain * args.reps)


def _report(name, us, nbytes, args, **extra):
    gbs = nbytes / us / 1e3
    print(json.dumps({"case": name, "us": round(us, 2), "GB_s": round(gbs, 1),
                      "hbm_fraction_of_measured": round(gbs / _peak(args), 3), **extra}), flush=True)


def _meta(batch, ctx, block, dev):
    """Decode-step metadata: one new token per request, ctx - 1 cached, shuffled block ids."""
    nblk = (ctx + block - 1) // block
    perm = torch.randperm(batch * nblk + 1)[: batch * nblk].view(batch, nblk).int()
    qsl = torch.arange(batch + 1, dtype=torch.int32)
    cached = torch.full((batch,), ctx - 1, dtype=torch.int32)
    seq = torch.full((batch,), ctx, dtype=torch.int32)
    slots = (perm[:, (ctx - 1) // block].long() * block + (ctx - 1) % block).int()
    pos = torch.full((batch,), ctx - 1, dtype=torch.int64)
    m = F.AttnMeta(qsl.to(dev), cached.to(dev), seq.to(dev), (qsl[1:] - 1).to(dev), slots.to(dev),
                   perm.to(dev), pos.to(dev), batch=batch, num_tokens=batch, max_q_len=1, max_seq_len=ctx,
                   decode_step=True, block_size=block, num_splits=1)
    return m, batch * nblk + 1


def case_gemm(args, swiglu=False):
    dev = "cuda"
    M, N, K = args.m, args.n, args.k
    copies = max(2, int(400e6 / (N * K * 2)) + 1)
    ws = [(torch.randn(N, K, device=dev) * 0.02).bfloat16() for _ in range(copies)]
    x = torch.randn(M, K, device=dev).bfloat16()
    if swiglu:
        out = torch.empty(M, N // 2, device=dev, dtype=torch.bfloat16)
        us = _time_us(lambda i: F.linear_swiglu(x, ws[i % copies], out=out, splitk=args.splitk), args)
    else:
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        us = _time_us(lambda i: F.linear(x, ws[i % copies], out=out, splitk=args.splitk), args)
    _report("swiglu" if swiglu else "gemm", us, N * K * 2, args, M=M, N=N, K=K, splitk=args.splitk,
            tflops=round(2.0 * M * N * K / us / 1e6, 1))


def case_attn(args):
    dev = "cuda"
    B, ctx, nq, nkv, hd = args.batch, args.ctx, args.nq, args.nkv, 128
    m, nblk = _meta(B, ctx, 128, dev)
    m.num_splits = args.splits
    copies = 4
    kcs = [(torch.randn(nblk, 128, nkv, hd, device=dev) * 0.5).bfloat16() for _ in range(copies)]
    vcs = [(torch.randn(nblk, 128, nkv, hd, device=dev) * 0.5).bfloat16() for _ in range(copies)]
    q = (torch.randn(B, nq * hd, device=dev) * 0.3).bfloat16()
    o = torch.empty_like(q)
    m.split_scratch = (torch.empty(B * nq * 32 * hd, device=dev), torch.empty(B * nq * 32, device=dev))
    if args.variant >= 0:
        # tile shape of the decode kernel: 1 / 2 / 3 = 16 tokens x 2 / 3 / 4 stages, 4 = 32 x 3, 0 = 32 x 2
        _native.kernels().gv_set_decode_variant(args.variant)
    us = _time_us(lambda i: F.paged_attention(q, kcs[i % copies], vcs[i % copies], m, nq, nkv, hd, out=o), args)
    _report("attn_decode", us, B * ctx * nkv * hd * 2 * 2, args, batch=B, ctx=ctx, nq=nq, nkv=nkv,
            splits=args.splits, variant=args.variant)


def case_mla(args):
    dev = "cuda"
    B, ctx, H, dc, dr = args.batch, args.ctx, args.heads, 512, 64
    m, nblk = _meta(B, ctx, 64, dev)
    m.num_splits = args.splits
    copies = 4
    caches = [(torch.randn(nblk, 64, 1, dc + dr, device=dev) * 0.3).bfloat16() for _ in range(copies)]
    qf = (torch.randn(B, H, dc + dr, device=dev) * 0.1).bfloat16()
    out = torch.empty(B, H, dc, device=dev, dtype=torch.bfloat16)
    us = _time_us(lambda i: mla_ops.mla_attention(qf, caches[i % copies], m, H, dc, dr, 0.07, out=out), args)
    flops = 2.0 * B * H * ctx * (2 * dc + dr)
    _report("mla_decode", us, B * ctx * (dc + dr) * 2, args, batch=B, ctx=ctx, heads=H, splits=args.splits,
            tflops=round(flops / us / 1e6, 1))


def case_layer(args):
    """One Llama-3-8B decode layer (64 requests, context 1060) split into its parts: g = the four
    GEMMs, a = attention, s = the small kernels; with and without programmatic dependent launch."""
    dev = "cuda"
    TP = args.tp
    B, ctx, H = args.batch, args.ctx, 4096
    nq, nkv, inter, L = 32 // TP, max(1, 8 // TP), 14336 // TP, 8
    m, nblk = _meta(B, ctx, 128, dev)
    kcs = [(torch.randn(nblk, 128, nkv, 128, device=dev) * 0.5).bfloat16() for _ in range(L)]
    vcs = [(torch.randn(nblk, 128, nkv, 128, device=dev) * 0.5).bfloat16() for _ in range(L)]

    def mk(n, k):
        return (torch.randn(n, k, device=dev) * 0.02).bfloat16()

    wqkv = [mk((nq + 2 * nkv) * 128, H) for _ in range(L)]
    wo = [mk(H, nq * 128) for _ in range(L)]
    wgu = [F.interleave_gate_up(mk(2 * inter, H)) for _ in range(L)]
    wd = [mk(H, inter) for _ in range(L)]
    nw = torch.ones(H, device=dev, dtype=torch.bfloat16)
    x = torch.randn(B, H, device=dev).bfloat16()
    res, h, x0 = x.clone(), torch.empty_like(x), x.clone()
    qkv = torch.empty(B, (nq + 2 * nkv) * 128, device=dev, dtype=torch.bfloat16)
    qd = torch.empty(B, nq * 128, device=dev, dtype=torch.bfloat16)
    ao = torch.empty_like(qd)
    gu = torch.empty(B, 2 * inter, device=dev, dtype=torch.bfloat16)
    act = torch.empty(B, inter, device=dev, dtype=torch.bfloat16)
    cos_sin = torch.randn(8192, 128, device=dev)

    def layer(li, parts, fused):
        if "s" in parts:
            F.add_rmsnorm(x, res, nw, 1e-5, out=h)
        if "g" in parts:
            F.linear(h, wqkv[li], out=qkv)
        if "s" in parts:
            F.rope_kvwrite(qkv, m, cos_sin, kcs[li], vcs[li], nq, nkv, 128, out=qd)
        if "a" in parts:
            F.paged_attention(qd, kcs[li], vcs[li], m, nq, nkv, 128, out=ao)
        if "g" in parts:
            F.linear(ao, wo[li], out=x)
        if "s" in parts:
            F.add_rmsnorm(x, res, nw, 1e-5, out=h)
        if fused and "g" in parts:
            F.linear_swiglu(h, wgu[li], out=act)
        else:
            if "g" in parts:
                F.linear(h, wgu[li], out=gu)
            if "s" in parts:
                F.silu_and_mul(gu, out=act, interleaved=True)
        if "g" in parts:
            F.linear(act, wd[li], out=x)

    from ..ops import decode_ops as D
    m.num_splits = args.splits
    if args.splits > 1:
        m.split_scratch = (torch.empty(B * nq * args.splits * 128, device=dev),
                           torch.empty(B * nq * args.splits, device=dev))
    ss = D.new_sumsq(H, dev)
    D.linear_residual(ao, wo[0], res, ss)

    def layer5(li):
        """The fused loop: QKV GEMM with RoPE + cache write, attention, o_proj with the residual add,
        gate/up GEMM with SwiGLU, down_proj with the residual add; RMSNorm inside the epilogues."""
        D.linear_rope(res, wqkv[li], m, cos_sin, kcs[li], vcs[li], nq, nkv, ss, H, 1e-5, out=qd)
        F.paged_attention(qd, kcs[li], vcs[li], m, nq, nkv, 128, out=ao)
        D.linear_residual(ao, wo[li], res, ss, next_w=wgu[li])
        D.linear_scaled(res, wgu[li], ss, H, 1e-5, swiglu=True, out=act, next_w=wd[li])
        D.linear_residual(act, wd[li], res, ss, next_w=wqkv[(li + 1) % L])

    wbytes = (wqkv[0].numel() + wo[0].numel() + wgu[0].numel() + wd[0].numel()) * 2
    kvbytes = B * ctx * nkv * 128 * 2 * 2
    peak = _peak(args)
    res_out = {"case": "layer", "tp": TP, "ideal_us": {"gemm": round(wbytes / peak / 1e3, 1),
                                                        "attn": round(kvbytes / peak / 1e3, 1)}}
    for pdl in (1, 0):
        _native.kernels().gv_set_pdl(pdl)
        row = {}
        for parts, fused in (("gsa", True), ("gsa", False), ("g", False), ("a", False), ("s", False)):
            def run(_i, parts=parts, fused=fused):
                for li in range(L):
                    layer(li, parts, fused)
            saved = args.chain
            args.chain = 1
            row[parts + ("+fused_swiglu" if fused else "")] = round(_time_us(run, args) / L, 1)
            args.chain = saved

        def run5(_i):
            for li in range(L):
                layer5(li)
            res.copy_(x0)           # the residual stream grows layer by layer: start every replay alike
        saved, args.chain = args.chain, 1
        row["fused_5_launches"] = round(_time_us(run5, args) / L, 1)
        args.chain = saved
        res_out["pdl_on" if pdl else "pdl_off"] = row
    _native.kernels().gv_set_pdl(1)
    print(json.dumps(res_out), flush=True)


def _plain_us(fn, n=10, warm=3) -> float:
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / n * 1e3


def case_prefill_gemm(args):
    """The four projection shapes of a Llama-3-8B layer at M tokens: the default token-major kernel,
    the persistent grouped kernel with one segment, the persistent token-major kernel
    (`--with-persistent`, gemm_persist.cu) and cuBLAS through torch.matmul; operands of one shape
    (60 - 400 MB) exceed what the previous launch left in L2."""
    dev = "cuda"
    M = args.m
    out = {"case": "prefill_gemm", "M": M}
    for name, N, K in (("qkv", 6144, 4096), ("o_proj", 4096, 4096), ("gate_up", 28672, 4096), ("down", 4096, 14336)):
        x = (torch.randn(M, K, device=dev) * 0.1).bfloat16()
        w = (torch.randn(N, K, device=dev) * 0.02).bfloat16()
        y0 = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        y1, y2 = torch.empty_like(y0), torch.empty_like(y0)
        off = torch.tensor([0, M], dtype=torch.int32, device=dev)
        fl = 2.0 * M * N * K
        row = {}
        t = _plain_us(lambda: _native.call("gemm_bf16", x, w, None, y0, M, N, K, K, K, N, 0))
        row["token_major"] = {"us": round(t, 1), "tflops": round(fl / t / 1e6, 1)}
        t = _plain_us(lambda: _native.call("grouped_gemm_bf16", x, w.view(1, N, K), off, y1, M, N, K, 1))
        row["grouped_one_segment"] = {"us": round(t, 1), "tflops": round(fl / t / 1e6, 1),
                                      "maxdiff": (y0.float() - y1.float()).abs().max().item()}
        if args.with_persistent:
            t = _plain_us(lambda: _native.call("gemm_bf16_persistent", x, w, None, y2, M, N, K, K, K, N))
            row["persistent_token_major"] = {"us": round(t, 1), "tflops": round(fl / t / 1e6, 1),
                                             "maxdiff": (y0.float() - y2.float()).abs().max().item()}
        t = _plain_us(lambda: torch.matmul(x, w.t()))
        row["cublas"] = {"us": round(t, 1), "tflops": round(fl / t / 1e6, 1)}
        out[name] = row
    print(json.dumps(out), flush=True)


def case_rope(args):
    """RoPE + query scaling + paged cache write over `--tokens` tokens of 32 q / 8 k / 8 v heads of
    128. Run once as is and once with GVIRT_DISABLE_ROPE_FAST=1 to compare the two kernels."""
    from ..ops import reference as ref
    dev = "cuda"
    T, nq, nkv, hd = args.tokens, args.nq, args.nkv, 128
    qkv = torch.randn(T, (nq + 2 * nkv) * hd, device=dev).bfloat16()
    tab = ref.rope_table(8192, hd, 10000.0, device=dev)
    pos = torch.arange(T, dtype=torch.int64, device=dev) % 1024
    slots = torch.arange(T, dtype=torch.int32, device=dev)
    nblk = (T + 127) // 128
    kc = torch.zeros(nblk, 128, nkv, hd, device=dev, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    z = torch.zeros(1, dtype=torch.int32, device=dev)
    meta = F.AttnMeta(z, z, z, z, slots, z.view(1, 1), pos, batch=1, num_tokens=T)
    us = _plain_us(lambda: F.rope_kvwrite(qkv, meta, tab, kc, vc, nq, nkv, hd))
    nbytes = 2 * qkv.numel() * 2
    _report("rope", us, nbytes, args, tokens=T, generic_kernel=bool(os.environ.get("GVIRT_DISABLE_ROPE_FAST")))


def case_decode_gemm(args):
    """The fused decode GEMMs of one Llama-3-8B layer at `--tp` shapes, each timed on its own over
    rotating weights: QKV + RoPE + cache write, o_proj + residual, gate/up + SwiGLU, down + residual."""
    from ..ops import decode_ops as D
    dev = "cuda"
    TP, B, H = args.tp, args.batch, 4096
    nq, nkv, inter = 32 // TP, max(1, 8 // TP), 14336 // TP
    m, nblk = _meta(B, args.ctx, 128, dev)
    copies = 2 if args.eager else 6          # a profiler capture wants a small footprint
    kc = (torch.randn(nblk, 128, nkv, 128, device=dev) * 0.5).bfloat16()
    vc = torch.zeros_like(kc)

    def mk(n, k):
        return [(torch.randn(n, k, device=dev) * 0.02).bfloat16() for _ in range(copies)]

    wqkv, wo, wgu, wd = mk((nq + 2 * nkv) * 128, H), mk(H, nq * 128), mk(2 * inter, H), mk(H, inter)
    x = torch.randn(B, H, device=dev).bfloat16()
    ss = D.new_sumsq(H, dev)
    qd = torch.empty(B, nq * 128, device=dev, dtype=torch.bfloat16)
    ao = torch.randn(B, nq * 128, device=dev).bfloat16()
    act = torch.randn(B, inter, device=dev).bfloat16()
    act_o = torch.empty_like(act)
    cos_sin = torch.randn(8192, 128, device=dev)
    D.linear_residual(ao, wo[0], x, ss)
    out = {"case": "decode_gemm", "tp": TP, "batch": B}
    peak = _peak(args)
    for name, fn, nbytes in (
            ("qkv_rope", lambda i: D.linear_rope(x, wqkv[i % copies], m, cos_sin, kc, vc, nq, nkv, ss, H, 1e-5, out=qd),
             wqkv[0].numel() * 2),
            ("o_proj_residual", lambda i: D.linear_residual(ao, wo[i % copies], x, ss), wo[0].numel() * 2),
            ("gate_up_swiglu", lambda i: D.linear_scaled(x, wgu[i % copies], ss, H, 1e-5, swiglu=True, out=act_o),
             wgu[0].numel() * 2),
            ("down_residual", lambda i: D.linear_residual(act, wd[i % copies], x, ss), wd[0].numel() * 2)):
        us = _time_us(fn, args)
        out[name] = {"us": round(us, 2), "GB_s": round(nbytes / us / 1e3, 1),
                     "hbm_fraction_of_measured": round(nbytes / us / 1e3 / peak, 3)}
    print(json.dumps(out), flush=True)


def case_prefill_attn(args):
    """Causal prefill attention over `--batch` requests of `--tokens` new tokens each (no cached
    prefix), 128-wide heads: the tcgen05 kernel against the mma.sync kernel, TFLOP/s counted as
    4 * tokens^2 / 2 * head_dim per (request, head) (the causal half)."""
    dev = "cuda"
    B, S, nq, nkv, hd, bs = args.batch, args.tokens, args.nq, args.nkv, 128, 128
    nblk = (S + bs - 1) // bs
    bt = torch.randperm(B * nblk, device=dev).view(B, nblk).int()
    qsl = (torch.arange(B + 1, device=dev) * S).int()
    cached = torch.zeros(B, dtype=torch.int32, device=dev)
    kc = (torch.randn(B * nblk, bs, nkv, hd, device=dev) * 0.5).bfloat16()
    vc = (torch.randn(B * nblk, bs, nkv, hd, device=dev) * 0.5).bfloat16()
    q = (torch.randn(B * S, nq * hd, device=dev) * 0.3).bfloat16()
    o1, o2 = torch.empty_like(q), torch.empty_like(q)
    flops = 4.0 * B * nq * hd * S * (S + 1) / 2
    res = {}
    # kernel shapes: 1 / 2 = 128-key tiles with one / two softmax warp groups, 4 = 64-key tiles, two
    # CTAs per SM (the default); the last one timed leaves its output in o1 for the comparison
    for wg in (1, 2, 4):
        _native.kernels().gv_set_prefill_tc_warpgroups(wg)
        t = _plain_us(lambda: _native.call("paged_attention_prefill_tc", q, kc, vc, bt, qsl, cached, o1, B * S, B, S,
                                           nq, nkv, hd, bs, nblk, 1.0, B * nblk))
        res[wg] = t
    t_tc = res[4]
    t_old = _plain_us(lambda: _native.call("paged_attention_prefill", q, kc, vc, bt, qsl, cached, o2, B, S, nq, nkv,
                                           hd, bs, nblk, 1.0, B * nblk))
    print(json.dumps({"case": "prefill_attn", "batch": B, "tokens": S, "nq": nq, "nkv": nkv,
                      "tcgen05": {"us": round(t_tc, 1), "tflops": round(flops / t_tc / 1e6, 1)},
                      "tcgen05_128_key_tiles_two_softmax_warpgroups": {"us": round(res[2], 1), "tflops": round(flops / res[2] / 1e6, 1)},
                      "tcgen05_128_key_tiles_one_softmax_warpgroup": {"us": round(res[1], 1), "tflops": round(flops / res[1] / 1e6, 1)},
                      "mma_sync": {"us": round(t_old, 1), "tflops": round(flops / t_old / 1e6, 1)},
                      "maxdiff": (o1.float() - o2.float()).abs().max().item()}), flush=True)


def case_fused1(args):
    """The kernels that fuse a GEMM with its collective, on a one-rank symmetric heap (the rank is
    its own peer: staging, flags, generation counters and the reduce phase all run; nothing crosses
    NVLink). Meant for single-GPU profiler captures of these kernels' compute side
    (``--eager --chain 1 --reps 1``); multi-rank timings come from ``tools.comm_bench``."""
    from types import SimpleNamespace
    from ..config import ModelConfig
    from ..ops import decode_ops as D
    from ..ops import moe_ops
    from ..parallel.moe_a2a import MoEA2A
    from ..parallel.symm import SymmetricHeap
    dev = torch.device("cuda", torch.cuda.current_device())
    heap = SymmetricHeap(None, 0, 1, dev, nbytes=1 << 30)
    out = {"case": "fused1"}
    B, H, P = args.batch, 4096, args.tokens
    x = (torch.randn(B, H, device=dev) * 0.1).bfloat16()
    w = (torch.randn(H, H, device=dev) * 0.02).bfloat16()
    res = torch.randn(B, H, device=dev).bfloat16()
    ss = D.new_sumsq(H, dev)
    out["gemm_allreduce_residual_sumsq_us"] = round(_time_us(
        lambda i: heap.gemm_allreduce(x, w, out=res, residual=res, ss_out=ss), args), 2)
    xp = (torch.randn(P, H, device=dev) * 0.1).bfloat16()
    o1 = torch.empty(P, H, device=dev, dtype=torch.bfloat16)
    out["gemm_rs_us"] = round(_time_us(lambda i: heap.gemm_reduce_scatter(xp, w, out=o1), args), 2)
    out["ag_gemm_us"] = round(_time_us(lambda i: heap.allgather_gemm(xp, w, out=o1), args), 2)
    E, K, inter, T = 32, 8, 768, 128
    cfg = ModelConfig(hidden_size=2048, num_experts=E, num_experts_per_tok=K, moe_intermediate_size=inter)
    a2a = MoEA2A(heap, cfg, SimpleNamespace(), tokens_cap=T, fp8=False)
    L = SimpleNamespace(w13=moe_ops.interleave16((torch.randn(E, 2 * inter, 2048, device=dev) * 0.05).bfloat16()),
                        w2=(torch.randn(E, 2048, inter, device=dev) * 0.05).bfloat16(), w13_il16=True)
    xt = (torch.randn(T, 2048, device=dev) * 0.5).bfloat16()
    wts, ids = moe_ops.softmax_topk(torch.randn(T, E, device=dev), K, True)
    ot = torch.empty_like(xt)
    out["moe_exchange_and_experts_us"] = round(_time_us(lambda i: a2a.forward(xt, wts, ids, L, ot), args), 2)
    print(json.dumps(out), flush=True)


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("case", choices=["gemm", "swiglu", "attn", "mla", "layer", "prefill_gemm", "rope", "prefill_attn", "decode_gemm", "fused1"])
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--with-persistent", action="store_true",
                    help="prefill_gemm: also time gemm_persist.cu (GVIRT_PREFILL_GEMM_PERSISTENT=2)")
    ap.add_argument("--m", type=int, default=64)
    ap.add_argument("--n", type=int, default=6144)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--splitk", type=int, default=0)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=1060)
    ap.add_argument("--nq", type=int, default=32)
    ap.add_argument("--nkv", type=int, default=8)
    ap.add_argument("--heads", type=int, default=128)
    ap.add_argument("--splits", type=int, default=1)
    ap.add_argument("--variant", type=int, default=-1, help="attn: decode kernel tile shape (-1 = library default)")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--chain", type=int, default=16)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--eager", action="store_true")
    ap.add_argument("--hbm-gbs", type=float, default=0.0)
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("kbench needs a CUDA device")
    torch.manual_seed(0)
    {"gemm": case_gemm, "swiglu": lambda a: case_gemm(a, True), "attn": case_attn, "mla": case_mla,
     "layer": case_layer, "prefill_gemm": case_prefill_gemm, "rope": case_rope,
     "prefill_attn": case_prefill_attn, "decode_gemm": case_decode_gemm, "fused1": case_fused1}[args.case](args)
    st = _native.read_status()
    if st:
        print(json.dumps({"status_word": st, "meaning": _native.describe_status(st)}))
        return 1
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
