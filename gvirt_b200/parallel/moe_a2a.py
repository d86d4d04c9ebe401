"""Expert-parallel MoE exchange on the symmetric heap: fused dispatch -> grouped expert GEMMs ->
fused combine (kernels in csrc/kernels/moe_a2a.cu, grouped_gemm.cu, gemm_fp8.cu).

One instance serves every MoE layer of a model: all layers share the receive regions, because a
rank only starts the next layer's dispatch after the current layer's combine has come back from
every expert rank (see the header of moe_a2a.cu). With fp8 expert weights the token rows travel as
e4m3 + per-128-column scales (half the NVLink bytes) and feed the block-scaled grouped GEMM
directly; with bf16 weights they travel as bf16.
"""
from __future__ import annotations

import ctypes

import torch

from .. import _native
from ..config import flags as env_flags
from ..ops import functional as F
from ..ops import moe_ops


def a2a_capacity(cfg, R: int, tokens_cap: int) -> int:
    """Slots per local expert in the receive region. The worst case is every token of every rank
    (R * tokens_cap); GVIRT_ACTIVE_TOKENS_RATIO_PER_EP scales it down, never below four times the
    expected load. Because the buffers between the two expert GEMMs are addressed by slot, their
    size follows this capacity too: it is cut further when they would exceed
    GVIRT_A2A_SCRATCH_GB. With the default ratio of 1 nothing is ever dropped: where memory cuts
    the capacity, `attach_device_comm` lowers the step size (`max_num_batched_tokens`) to
    `a2a_exact_tokens`, so that even the worst routing fits. A ratio below 1 is the reference's
    approximate mode (its ACTIVE_TOKENS_RATIO knob): rows beyond the capacity are dropped and
    counted in the status word."""
    E = max(cfg.num_experts, 1)
    worst = R * tokens_cap
    expect = R * tokens_cap * cfg.num_experts_per_tok / E
    floor = max(16, int(4 * expect))
    ratio = env_flags().active_tokens_ratio_per_ep
    cap = worst if ratio >= 1.0 else max(floor, int(worst * ratio))
    inter = cfg.moe_intermediate_size // max(getattr(cfg, "moe_tp_size", 1) or 1, 1)
    per_row = 2 * inter * 2 + inter * 2 + 2 * cfg.hidden_size * 2     # gate/up, act, down out, received row
    e_local = max(E // R, 1)
    fit = int(env_flags().a2a_scratch_gb * (1 << 30)) // (per_row * e_local)
    if cap > fit:
        cap = max(floor, fit)
    return int(min(worst, cap))


def a2a_exact_tokens(cfg, R: int, tokens_cap: int) -> int:
    """Most tokens one rank may dispatch per step such that no routing whatsoever can overflow an
    expert's receive region (every token of every rank to the same expert: R * tokens slots)."""
    return min(int(tokens_cap), a2a_capacity(cfg, R, tokens_cap) // max(R, 1))


class MoEA2A:
    def __init__(self, heap, cfg, ctx, tokens_cap: int, fp8: bool):
        """heap: SymmetricHeap of the EP group; tokens_cap: most tokens one rank dispatches per
        step (larger steps use the library-collective path)."""
        self.heap, self.cfg, self.ctx = heap, cfg, ctx
        self.R, self.rank = heap.world, heap.rank
        self.H, self.K = cfg.hidden_size, cfg.num_experts_per_tok
        self.e_local = cfg.num_experts // self.R
        self.fp8 = bool(fp8)
        self.tokens_cap = int(tokens_cap)
        expect = self.R * self.tokens_cap * self.K / cfg.num_experts
        self.cap = a2a_capacity(cfg, self.R, self.tokens_cap)
        rows = self.e_local * self.cap
        rb = self.H if self.fp8 else 2 * self.H
        take = heap._take
        self.x_off = take(rows * rb)
        self.scale_off = take((self.H // 128) * rows * 4) if self.fp8 else 0
        self.meta_off = take(rows * 4)
        self.cnt_off = take(self.e_local * 4)
        self.ret_off = take(self.tokens_cap * self.K * self.H * 2)
        self.flag_off = take(2 * 16 * 4)
        dev = heap.device
        self.state = torch.zeros(2, dtype=torch.int32, device=dev)
        self.offs = (ctypes.c_longlong * 6)(self.x_off, self.scale_off, self.meta_off, self.cnt_off,
                                            self.ret_off, self.flag_off)
        self.dims = (ctypes.c_longlong * 6)(self.rank, self.R, self.cap, self.H, self.e_local, int(self.fp8))
        self.seg_start = torch.zeros(self.e_local, dtype=torch.int32, device=dev)
        self.seg_end = torch.zeros(self.e_local, dtype=torch.int32, device=dev)
        slab = heap.slab
        if self.fp8:
            self.xs = slab[self.x_off: self.x_off + rows * rb].view(torch.float8_e4m3fn).view(rows, self.H)
            self.xscale = slab[self.scale_off: self.scale_off + (self.H // 128) * rows * 4].view(torch.float32).view(self.H // 128, rows)
        else:
            self.xs = slab[self.x_off: self.x_off + rows * rb].view(torch.bfloat16).view(rows, self.H)
            self.xscale = None
        self.ret = slab[self.ret_off: self.ret_off + self.tokens_cap * self.K * self.H * 2].view(torch.bfloat16).view(self.tokens_cap * self.K, self.H)
        self.rows = rows
        self.row_of = torch.empty(self.tokens_cap, self.K, dtype=torch.int32, device=dev)
        self.avg_rows = max(1, int(expect + 0.5))
        self._scratch: dict = {}       # buffers between the two expert GEMMs, shared by all layers

    def _buf(self, name: str, shape, dtype) -> torch.Tensor:
        """Slot-addressed intermediate of fixed worst-case size: allocated once (all layers run one
        after the other on one stream), so a step allocates nothing."""
        key = (name, tuple(shape), dtype)
        t = self._scratch.get(key)
        if t is None:
            t = self._scratch[key] = torch.empty(tuple(shape), dtype=dtype, device=self.heap.device)
        return t

    def supports(self, T: int) -> bool:
        return T <= self.tokens_cap

    def forward(self, h: torch.Tensor, weights: torch.Tensor, ids: torch.Tensor, lw, out: torch.Tensor,
                clamp: float = 0.0) -> torch.Tensor:
        """out[t] = sum_k weights[t, k] * Expert_{ids[t, k]}(h[t]) with experts spread over the EP group."""
        T = h.shape[0]
        dev = h.device
        peers = self.heap.peers
        row_of = self.row_of[:max(T, 1)]
        _native.call("moe_a2a_dispatch", h, ids, row_of, T, self.K, peers, self.offs, self.state, self.dims)
        _native.call("moe_a2a_recv_prepare", self.seg_start, self.seg_end, peers, self.offs, self.state, self.dims)
        inter = lw.w13.shape[1] // 2
        rows, E = self.rows, self.e_local
        # token-tile width of the grouped GEMMs from this step's expected rows per expert (assuming
        # the other ranks run a similar step): decode steps get narrow tiles, so the padding rows of
        # the activation tile do not double the bytes streamed next to the weights
        avg_rows = max(1, int(self.R * max(T, 1) * self.K / max(self.cfg.num_experts, 1) + 0.5))
        w13s, w2s = getattr(lw, "w13_scale", None), getattr(lw, "w2_scale", None)
        if getattr(lw, "w13_il16", False) and not self.fp8:
            # gate / up rows interleaved: SwiGLU runs in the grouped GEMM's epilogue
            act = self._buf("act", (rows, inter), torch.bfloat16)
            ys = self._buf("ys", (rows, self.H), torch.bfloat16)
            _native.call("grouped_gemm_bf16_swiglu_seg", self.xs, lw.w13, self.seg_start, self.seg_end, act, rows,
                         2 * inter, self.H, E, E, avg_rows, float(clamp))
            _native.call("grouped_gemm_bf16_seg", act, lw.w2, self.seg_start, self.seg_end, ys, rows, self.H,
                         inter, E, E, avg_rows)
            return self._combine(ys, peers, weights, row_of, out, T)
        gu = self._buf("gu", (rows, 2 * inter), torch.bfloat16)
        if self.fp8:
            _native.call("grouped_gemm_fp8_seg", self.xs, self.xscale, lw.w13, w13s, self.seg_start, self.seg_end,
                         gu, rows, 2 * inter, self.H, E, E, rows, avg_rows)
        else:
            _native.call("grouped_gemm_bf16_seg", self.xs, lw.w13, self.seg_start, self.seg_end, gu, rows,
                         2 * inter, self.H, E, E, avg_rows)
        ys = self._buf("ys", (rows, self.H), torch.bfloat16)
        # SwiGLU (and, for fp8 experts, the activation quantisation) over the live rows only
        seg_ok = inter % 128 == 0 and E <= 512
        if self.fp8:
            if seg_ok:
                aq = self._buf("aq", (rows, inter), torch.float8_e4m3fn)
                asc = self._buf("asc", (inter // 128, rows), torch.float32)
                _native.call("moe_act_seg", gu, None, aq, asc, self.seg_start, self.seg_end, E, inter,
                             gu.stride(0), rows, float(clamp), 1)
            else:
                act = self._buf("act", (rows, inter), torch.bfloat16)
                F.silu_and_mul(gu, out=act, clamp=clamp)
                aq, asc = moe_ops.quant_fp8(act)
            _native.call("grouped_gemm_fp8_seg", aq, asc, lw.w2, w2s, self.seg_start, self.seg_end, ys, rows,
                         self.H, inter, E, E, asc.shape[1], avg_rows)
        else:
            act = self._buf("act", (rows, inter), torch.bfloat16)
            if seg_ok:
                _native.call("moe_act_seg", gu, act, None, None, self.seg_start, self.seg_end, E, inter,
                             gu.stride(0), rows, float(clamp), 0)
            else:
                F.silu_and_mul(gu, out=act, clamp=clamp)
            _native.call("grouped_gemm_bf16_seg", act, lw.w2, self.seg_start, self.seg_end, ys, rows, self.H,
                         inter, E, E, avg_rows)
        return self._combine(ys, peers, weights, row_of, out, T)

    def _combine(self, ys, peers, weights, row_of, out, T):
        _native.call("moe_a2a_combine_push", ys, self.seg_end, peers, self.offs, self.state, self.dims)
        _native.call("moe_a2a_combine_wait", peers, self.offs, self.state, self.dims)
        if T > 0:
            _native.call("moe_unpermute", self.ret, weights, row_of, out, T, self.H, self.K)
        return out


def attach_moe_a2a(ctx, cfg, tokens_cap: int) -> None:
    """Enable the fused dispatch / combine path on `ctx` (needs the EP-group symmetric heap)."""
    heap = ctx.symm_ep
    if heap is None or not cfg.is_moe:
        return
    ctx.moe_a2a = MoEA2A(heap, cfg, ctx, tokens_cap, fp8=(cfg.quant == "fp8_block"))
