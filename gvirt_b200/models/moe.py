"""Mixture-of-experts FFN: routing, expert-parallel dispatch, grouped expert GEMMs, combine.

Reference dataflow (xlite/csrc/model.cpp:1209-1332): gate GEMM -> ``softmax_topk`` /
``sigmoid_topk`` -> dispatch (default: all-gather of packed [hidden | weights | routing] over
the DP group then ``permutation`` of the local experts' rows; or the all-to-all mode with a
host-side count exchange) -> grouped GEMM up/gate -> SwiGLU -> grouped GEMM down ->
``unpermutation`` (+ reduce-scatter / all-to-all back) -> shared expert -> TP all-reduce.

Here routing produces compact ``[T, K]`` ids + weights instead of dense ``[T, E]`` weights and
a bitmap; the expert-parallel exchange has two implementations:

* *replicate-then-filter* (library collectives; any backend, used by the CPU / gloo tests and
  as the baseline): tokens are made visible to every EP rank (already true when attention is
  tensor-parallel; all-gather over DP otherwise), each rank runs its local experts on the
  rows routed to them, partial outputs are summed by all-reduce / reduce-scatter;
* *fused dispatch / combine* (``parallel.moe_a2a``; CUDA + symmetric heap): the routing
  kernel writes each (token, expert) row straight into the destination rank's receive region
  over NVLink, the grouped GEMM consumes expert-major segments, and the combine kernel pulls
  the weighted rows back — no host synchronisation, no count-exchange collective. With
  data-parallel attention every rank dispatches its own tokens; with tensor-parallel attention
  (tokens replicated) rank r dispatches the r-th 1/tp slice of the tokens and the finished
  slices are all-gathered, which replaces the all-reduce of ``[T, H]`` partial sums (each row
  crosses the links once, already summed) and runs every routed row on one rank only.
"""
from __future__ import annotations

import torch

from ..config import ScoringFunc, flags
from ..ops import functional as F
from ..ops import moe_ops
from ..parallel import collectives as coll


def route(model, lw, h):
    """-> (weights fp32 [T, K], ids int32 [T, K])"""
    cfg = model.cfg
    logits = moe_ops.router_logits(h, lw.w_router)
    lb = getattr(lw, "router_logit_bias", None)
    if lb is not None:
        logits = logits + lb      # benchmark knob: skewed expert popularity (see weights.zipf_router_bias)
    if cfg.scoring_func == ScoringFunc.SOFTMAX:
        return moe_ops.softmax_topk(logits, cfg.num_experts_per_tok, cfg.norm_topk_prob)
    return moe_ops.sigmoid_topk(logits, lw.router_bias, cfg.num_experts_per_tok, cfg.n_group,
                                cfg.topk_group, cfg.norm_topk_prob, cfg.routed_scaling_factor)


def forward(model, li, lw, h, ws, out):
    cfg, ctx = model.cfg, model.ctx
    if h.device.type == "meta":
        return _dry(model, lw, h, ws, out)
    T = h.shape[0]
    e_local = cfg.num_experts // ctx.ep
    e_start = ctx.ep_rank * e_local

    a2a = getattr(ctx, "moe_a2a", None)
    a2a_ok = a2a is not None and flags().moe_alltoall and (h.is_cuda or getattr(a2a, "any_device", False))
    if a2a_ok and ctx.dp == 1 and ctx.tp > 1 and ctx.ep == ctx.tp and a2a.supports(-(-T // ctx.tp)):
        # tensor-parallel attention: the tokens are the same on every rank; this rank routes and
        # dispatches its 1/tp slice, the slices of finished rows are gathered
        tl = -(-T // ctx.tp)
        lo = min(T, ctx.tp_rank * tl)
        n = min(T, lo + tl) - lo
        hs = h[lo:lo + n]
        weights, ids = route(model, lw, hs)
        mine = ws.get((tl, cfg.hidden_size), model.dtype)
        a2a.forward(hs, weights, ids, lw, out=mine[:n], clamp=cfg.swiglu_clamp)
        if tl * ctx.tp == T:
            coll.all_gather(mine, ctx.tp_group, ctx, out=out)
        else:
            full = ws.get((tl * ctx.tp, cfg.hidden_size), model.dtype)
            coll.all_gather(mine, ctx.tp_group, ctx, out=full)
            out.copy_(full[:T])
            ws.put(full)
        ws.put(mine)
        summed_over_ep = True
        return _add_shared(model, lw, h, ws, out, summed_over_ep)
    weights, ids = route(model, lw, h)
    if a2a_ok and ctx.dp > 1 and a2a.supports(T):
        a2a.forward(h, weights, ids, lw, out=out, clamp=cfg.swiglu_clamp)
        summed_over_ep = True
    elif ctx.dp > 1 and ctx.ep > 1:
        # attention is data parallel: gather every DP rank's tokens, run local experts, scatter back
        tmax = _max_tokens_dp(T, ctx)
        hp = _pad_rows(h, tmax)
        wp = _pad_rows(weights, tmax)
        ip = _pad_rows(ids, tmax, fill=-1)
        hg = coll.all_gather(hp, ctx.dp_group)
        wg = coll.all_gather(wp, ctx.dp_group)
        ig = coll.all_gather(ip, ctx.dp_group)
        yg = moe_ops.experts_forward(hg, wg, ig, lw.w13, lw.w2, e_start, cfg.swiglu_clamp,
                                     w13_scale=getattr(lw, "w13_scale", None),
                                     w2_scale=getattr(lw, "w2_scale", None), il16=getattr(lw, "w13_il16", False))
        y = coll.reduce_scatter(yg, ctx.dp_group)
        out.copy_(y[:T])
        summed_over_ep = True
    else:
        moe_ops.experts_forward(h, weights, ids, lw.w13, lw.w2, e_start, cfg.swiglu_clamp, out=out,
                                w13_scale=getattr(lw, "w13_scale", None),
                                w2_scale=getattr(lw, "w2_scale", None), il16=getattr(lw, "w13_il16", False))
        summed_over_ep = ctx.ep == 1
    return _add_shared(model, lw, h, ws, out, summed_over_ep)


def _add_shared(model, lw, h, ws, out, summed_over_ep):
    """Shared expert and the reduction that is still owed over the EP / TP group."""
    cfg, ctx = model.cfg, model.ctx
    T = h.shape[0]
    # shared expert: partial sum on every TP rank (weights TP-sharded), joins the final reduce
    if getattr(lw, "ws_gate_up", None) is not None:
        sh = ws.get((T, cfg.hidden_size), model.dtype)
        shared = type("S", (), {"w_gate_up": lw.ws_gate_up, "w_down": lw.ws_down})
        model._mlp(shared, h, ws, sh, reduce=False)
        if getattr(lw, "ws_gate", None) is not None:
            # sigmoid(h . w) per token; the same on every rank, so it may scale the partial sums.
            # One output column is below the GEMM kernels' granularity: a fused multiply-reduce.
            gate = torch.sigmoid((h.float() * lw.ws_gate.float()).sum(-1, keepdim=True))
            sh.mul_(gate.to(sh.dtype))
        if summed_over_ep and ctx.tp > 1:
            # routed part is already complete on every rank: reduce the shared part alone
            coll.all_reduce(sh, ctx.tp_group, ctx)
        F.add(out, sh, out=out)
        ws.put(sh)
    if not summed_over_ep:
        # tokens replicated over the EP group (TP attention): sum the local-expert partials
        coll.all_reduce(out, ctx.ep_group if ctx.ep_group is not None else ctx.tp_group, ctx)
    return out


def _dry(model, lw, h, ws, out):
    """Arena sizing pass: account for the big temporaries of the expert path."""
    cfg = model.cfg
    T = h.shape[0]
    rows = T * cfg.num_experts_per_tok
    inter = lw.w13.shape[1] // 2
    a = ws.get((rows, cfg.hidden_size), model.dtype)
    b = ws.get((rows, 2 * inter), model.dtype)
    c = ws.get((rows, inter), model.dtype)
    d = ws.get((rows, cfg.hidden_size), model.dtype)
    for t in (a, b, c, d):
        ws.put(t)
    return out


def _max_tokens_dp(T, ctx):
    t = torch.tensor([T], dtype=torch.int64, device="cpu" if ctx.device.type == "cpu" else ctx.device)
    import torch.distributed as dist
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=ctx.dp_group)
    return int(t.item())


def _pad_rows(x, n, fill=0):
    if x.shape[0] == n:
        return x.contiguous()
    pad = torch.full((n - x.shape[0],) + tuple(x.shape[1:]), fill, dtype=x.dtype, device=x.device)
    return torch.cat([x, pad], 0)
