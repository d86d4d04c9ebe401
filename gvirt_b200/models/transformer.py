"""The decoder forward graph: one class configured by ``ModelConfig`` runs every supported
family (Llama / Qwen2 / Qwen3 dense, Qwen3-MoE, GLM-4-MoE / MiniMax-M2, DeepSeek-V3 MLA+MoE,
Qwen3.5 hybrid linear attention), as the reference's single ``XModel`` does
(xlite/csrc/model.h:119-201, forward in xlite/csrc/model.cpp:1408-1533).

Layer loop (xlite/csrc/model.cpp:1413-1433): ``h = norm0(x)``; per layer ``h = attn(h)``;
``x += h; h = norm_mlp(x)`` (fused add+RMSNorm, residual updated in place); ``h = ffn(h)``;
``x += h; h = norm_next(x)``. Temporaries come from a ``Workspace`` (arena) so addresses repeat
step to step. Tensor parallelism: column-parallel fused QKV / gate-up, row-parallel o_proj /
down_proj followed by an all-reduce (or reduce-scatter + all-gather in the sequence-parallel
path for long prefills), vocab-parallel embedding and lm_head.
"""
from __future__ import annotations

from types import SimpleNamespace
from typing import List, Optional, Tuple

import torch

from ..config import AttnType, ModelConfig, flags
from ..engine.arena import TorchWorkspace, Workspace
from ..ops import decode_ops as D
from ..ops import functional as F
from ..ops import moe_ops
from ..ops import reference as ref
from ..parallel import collectives as coll
from ..parallel import fused
from ..parallel.state import ParallelContext, context
from . import linear_attn, mla, moe


def _dtype(cfg: ModelConfig) -> torch.dtype:
    return {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}[cfg.dtype]


class Transformer:
    def __init__(self, cfg: ModelConfig, weights: SimpleNamespace, ctx: Optional[ParallelContext] = None):
        cfg.validate()
        self.cfg = cfg
        self.ctx = ctx or context()
        self.w = weights
        self.dtype = _dtype(cfg)
        self.device = weights.embed.device
        self.nq, self.nkv = cfg.local_heads()
        self.hd = cfg.head_dim
        self.vocab_local = weights.embed.shape[0]
        self.vocab_start = self.ctx.tp_rank * self.vocab_local
        if cfg.attn_type == AttnType.MHA or cfg.attn_type == AttnType.HYBRID:
            self.cos_sin = ref.rope_table(cfg.max_position_embeddings, cfg.rot_dim, cfg.rope_theta,
                                          device=self.device, scaling=cfg.rope_scaling)
        else:
            self.cos_sin = ref.rope_table(cfg.max_position_embeddings, cfg.qk_rope_head_dim,
                                          cfg.rope_theta, device=self.device, scaling=cfg.rope_scaling)
        self.mrope_mode = 0
        if cfg.mrope_sections is not None:
            self.mrope_mode = 2 if cfg.mrope_interleaved else 1
        self.debug_hook = None  # callable(tag, layer, tensor) for layer-level A/B diffing
        self.fused_decode = False   # set by _fold_norms: steps of <= 128 tokens take _forward_decode_fused
        self.rope_fused = False
        self._prepare_device_layouts()

    def _prepare_device_layouts(self, force: bool = False) -> None:
        """On CUDA the dense gate/up weights are re-ordered once into blocks of [64 gate | 64 up]
        rows so that the gate/up GEMM can apply SwiGLU in its epilogue (``F.linear_swiglu``); the
        layer is marked ``gu_il``. A local intermediate size that is not a multiple of 64 is first
        zero-padded to one (``F.pad_gate_up_down``, the layer records ``gu_pad``; the FFN output
        does not change). Skipped for clamped SwiGLU, quantised weights and off the GPU
        (``force`` runs it anywhere: the CPU definition of the fused op takes the same layout)."""
        cfg = self.cfg
        if not force and (self.device.type != "cuda" or self.dtype != torch.bfloat16):
            return
        if not flags().fuse_swiglu:
            return
        # routed experts (bf16): gate / up rows in blocks of [16 gate | 16 up], the layout whose
        # grouped GEMM applies SwiGLU (clamped or not) in its epilogue; marked ``w13_il16``
        for lw in self.w.layers:
            w13 = getattr(lw, "w13", None)
            if (w13 is None or getattr(lw, "w13_il16", False) or w13.dtype != self.dtype
                    or getattr(lw, "w13_scale", None) is not None or (w13.shape[1] // 2) % 16):
                continue
            lw.w13 = moe_ops.interleave16(w13)
            lw.w13_il16 = True
        if cfg.swiglu_clamp > 0:
            return
        for lw in self.w.layers:
            w = getattr(lw, "w_gate_up", None)
            if w is None or getattr(lw, "gu_il", False) or w.dtype != self.dtype:
                continue
            if (w.shape[0] // 2) % 64 != 0:
                wd = getattr(lw, "w_down", None)
                if not flags().pad_swiglu or wd is None or wd.dtype != w.dtype:
                    continue
                w, lw.w_down, lw.gu_pad = F.pad_gate_up_down(w, wd, 64)
            lw.w_gate_up = F.interleave_gate_up(w)
            lw.gu_il = True
        self._fold_norms()

    def _fold_norms(self) -> None:
        """Dense RMSNorm + MHA models: fold each layer's norm weights into w_qkv / w_gate_up so that
        steps of up to 128 tokens can run without norm launches (``_forward_decode_fused``). Every
        other path keeps working on the folded weights because the norm weights become ones."""
        cfg = self.cfg
        self.fused_decode = False
        if not flags().fused_decode or cfg.attn_type != AttnType.MHA or cfg.is_moe or cfg.qk_norm_full:
            return
        if cfg.attn_output_gate or any(cfg.layer_is_linear_attn(i) for i in range(cfg.num_layers)):
            return
        if cfg.hidden_size % 128 or any(getattr(lw, "norm_folded", False) for lw in self.w.layers):
            return
        for lw in self.w.layers:
            if (not getattr(lw, "gu_il", False) or lw.w_qkv.dtype != self.dtype or lw.w_o.dtype != self.dtype
                    or lw.w_down.dtype != self.dtype or lw.w_o.shape[0] % 128):
                return
        for lw in self.w.layers:
            D.fold_layer_norms(lw)
        self.fused_decode = True
        self.rope_fused = D.rope_fusable(cfg, self.hd, self.mrope_mode)

    # ------------------------------------------------------------------ KV cache
    def kv_cache_shapes(self, num_blocks: int) -> List[Tuple[Tuple[int, ...], ...]]:
        """Per layer, the shapes of the cache tensors the caller must allocate (the caller owns
        KV memory, xlite/csrc/model.cpp:1583-1637)."""
        cfg = self.cfg
        shapes = []
        for i in range(cfg.num_layers):
            if cfg.layer_is_linear_attn(i):
                shapes.append(linear_attn.state_shapes(cfg, self.ctx))
            elif cfg.attn_type in (AttnType.MLA, AttnType.DSA):
                shapes.append(mla.cache_shapes(cfg, num_blocks))
            else:
                s = (num_blocks, cfg.block_size, self.nkv, self.hd)
                shapes.append((s, s))
        return shapes

    def alloc_kv_cache(self, num_blocks: int):
        caches = []
        for i, shapes in enumerate(self.kv_cache_shapes(num_blocks)):
            dt = torch.float32 if self.cfg.layer_is_linear_attn(i) else self.dtype  # recurrent state stays fp32
            caches.append(tuple(torch.zeros(s, dtype=dt, device=self.device) for s in shapes))
        return caches

    # ------------------------------------------------------------------ pieces
    def _dbg(self, tag, layer, t):
        if self.debug_hook is not None and t.device.type != "meta":
            self.debug_hook(tag, layer, t)

    def _embed(self, tokens, ws: Workspace):
        cfg, ctx = self.cfg, self.ctx
        T = tokens.shape[0]
        x = ws.get((T, cfg.hidden_size), self.dtype)
        F.embed(tokens, self.w.embed, self.vocab_start, self.vocab_start + self.vocab_local, out=x)
        if ctx.tp > 1:
            coll.all_reduce(x, ctx.tp_group, ctx)
        return x

    def _attn_mha(self, li, lw, h, meta, cache, ws: Workspace, out):
        cfg = self.cfg
        T = h.shape[0]
        nq, nkv, hd = self.nq, self.nkv, self.hd
        gate_w = nq * hd if cfg.attn_output_gate else 0
        qkv = ws.get((T, (nq + 2 * nkv) * hd + gate_w), self.dtype)
        F.linear(h, lw.w_qkv, None, out=qkv)
        q = ws.get((T, nq * hd), self.dtype)
        qk_nw = (lw.q_norm, lw.k_norm) if (cfg.qk_norm and not cfg.qk_norm_full) else (None, None)
        if cfg.qk_norm_full:
            self._full_width_qk_norm(lw, qkv, ws)
        F.rope_kvwrite(qkv, meta, self.cos_sin, cache[0], cache[1], nq, nkv, hd, cfg.rot_dim,
                       hd ** -0.5, lw.b_qkv, qk_nw[0], qk_nw[1], cfg.rms_norm_eps, self.mrope_mode,
                       cfg.mrope_sections or (0, 0, 0), cfg.rope_interleaved, out=q)
        o = ws.get((T, nq * hd), self.dtype)
        F.paged_attention(q, cache[0], cache[1], meta, nq, nkv, hd, 1.0, out=o)
        ws.put(q)
        if cfg.attn_output_gate:
            gate = qkv[:, (nq + 2 * nkv) * hd:]
            F.sigmoid_gate_mul(o, gate, out=o)
        ws.put(qkv)
        fused.row_parallel_linear(o, lw.w_o, self.ctx, out=out, ws=ws)
        ws.put(o)
        return out

    def _full_width_qk_norm(self, lw, qkv, ws):
        """RMSNorm over the *whole* q (and k) width, which is split across TP ranks: each rank
        computes its sum of squares, one packed [2T] fp32 all-reduce combines them, the norm
        then uses the external variance (xlite/csrc/model.cpp:521-543)."""
        cfg, ctx = self.cfg, self.ctx
        nq, nkv, hd = self.nq, self.nkv, self.hd
        if qkv.device.type == "meta":
            return
        qv = qkv[:, : nq * hd]
        kv = qkv[:, nq * hd: (nq + nkv) * hd]
        ss = torch.cat([F.sumsq(qv), F.sumsq(kv)], dim=0).contiguous()
        if ctx.tp > 1:
            coll.all_reduce(ss, ctx.tp_group, None)
        T = qkv.shape[0]
        kv_rep = max(ctx.tp // cfg.num_kv_heads, 1)  # replicated kv heads were counted kv_rep times
        F.rmsnorm_extvar(qv, lw.q_norm, ss[:T], float(ctx.tp), cfg.rms_norm_eps, out=qv)
        F.rmsnorm_extvar(kv, lw.k_norm, ss[T:] / kv_rep, float(ctx.tp) / kv_rep, cfg.rms_norm_eps, out=kv)

    def _mlp(self, lw, h, ws: Workspace, out, reduce=True):
        T = h.shape[0]
        inter = lw.w_gate_up.shape[0] // 2
        a = ws.get((T, inter), self.dtype)
        if getattr(lw, "gu_il", False):
            F.linear_swiglu(h, lw.w_gate_up, out=a)     # SwiGLU in the GEMM epilogue
        else:
            gu = ws.get((T, 2 * inter), self.dtype)
            F.linear(h, lw.w_gate_up, None, out=gu)
            F.silu_and_mul(gu, out=a, clamp=self.cfg.swiglu_clamp)
            ws.put(gu)
        if reduce:
            fused.row_parallel_linear(a, lw.w_down, self.ctx, out=out, ws=ws)
        else:
            F.linear(a, lw.w_down, None, out=out)
        ws.put(a)
        return out

    # ------------------------------------------------------------------ fused decode forward
    def _residual_linear(self, a, w, x, ss, ws, next_w=None) -> int:
        """x += all_reduce_tp(a @ w^T) in place with the sums of squares of the new rows in `ss`.
        Returns how many tiles of `ss` are valid (all of them from a fused producer, one from the
        stand-alone add)."""
        ctx = self.ctx
        tiles = w.shape[0] // 128
        if ctx.tp == 1:
            D.linear_residual(a, w, x, ss, next_w=next_w)
            return tiles
        if a.device.type == "meta":
            tmp = ws.get(tuple(x.shape), self.dtype)       # the unfused fall-back sizes the arena
            ws.put(tmp)
            return tiles
        heap = ctx.symm
        fusable = heap is not None and a.is_cuda and heap.can_fuse_gemm_ar(a, w)
        if fusable and flags().fused_ar_residual:
            heap.gemm_allreduce(a, w, out=x, residual=x, ss_out=ss, next_w=next_w)
            return tiles
        tmp = ws.get(tuple(x.shape), self.dtype)
        if fusable:
            heap.gemm_allreduce(a, w, out=tmp)          # GEMM + all-reduce in one kernel, add behind it
        else:
            F.linear(a, w, None, out=tmp)
            coll.all_reduce(tmp, ctx.tp_group, ctx)
        D.add_residual_sumsq(tmp, x, ss)
        ws.put(tmp)
        return 1

    def _forward_decode_fused(self, tokens, meta, kv_caches, ws):
        """Layer loop for steps of up to 128 tokens of a dense model with folded norm weights: five
        launches per layer (QKV GEMM with RoPE + cache write, attention, o_proj, gate/up GEMM with
        SwiGLU, down_proj) against the nine of the generic loop. The residual stream `x` is updated
        in place by the o_proj / down_proj epilogues (under tensor parallelism: by the reduce phase
        of the fused GEMM + all-reduce), which also leave the sums of squares that the next GEMM
        turns into the RMSNorm factor."""
        cfg = self.cfg
        T = tokens.shape[0]
        H, eps = cfg.hidden_size, cfg.rms_norm_eps
        nq, nkv, hd = self.nq, self.nkv, self.hd
        x = self._embed(tokens, ws)
        ss = ws.get((D.MAX_TOKENS, H // 128), torch.float32)
        D.row_sumsq(x, ss)
        nt = 1
        for li, lw in enumerate(self.w.layers):
            cache = kv_caches[li]
            q = ws.get((T, nq * hd), self.dtype)
            qk_nw = (lw.q_norm, lw.k_norm) if cfg.qk_norm else (None, None)
            if self.rope_fused:
                D.linear_rope(x, lw.w_qkv, meta, self.cos_sin, cache[0], cache[1], nq, nkv, ss, H, eps,
                              bias=lw.b_qkv, q_norm_w=qk_nw[0], k_norm_w=qk_nw[1], qk_eps=eps, tiles=nt, out=q)
            else:
                qkv = ws.get((T, (nq + 2 * nkv) * hd), self.dtype)
                D.linear_scaled(x, lw.w_qkv, ss, H, eps, tiles=nt, out=qkv)
                F.rope_kvwrite(qkv, meta, self.cos_sin, cache[0], cache[1], nq, nkv, hd, cfg.rot_dim, hd ** -0.5,
                               lw.b_qkv, qk_nw[0], qk_nw[1], eps, self.mrope_mode, cfg.mrope_sections or (0, 0, 0),
                               cfg.rope_interleaved, out=q)
                ws.put(qkv)
            o = ws.get((T, nq * hd), self.dtype)
            F.paged_attention(q, cache[0], cache[1], meta, nq, nkv, hd, 1.0, out=o)
            ws.put(q)
            nt = self._residual_linear(o, lw.w_o, x, ss, ws, next_w=lw.w_gate_up)
            ws.put(o)
            a = ws.get((T, lw.w_gate_up.shape[0] // 2), self.dtype)
            D.linear_scaled(x, lw.w_gate_up, ss, H, eps, swiglu=True, tiles=nt, out=a, next_w=lw.w_down)
            nxt = self.w.layers[li + 1].w_qkv if li + 1 < len(self.w.layers) else None
            nt = self._residual_linear(a, lw.w_down, x, ss, ws, next_w=nxt)
            ws.put(a)
        ws.put(ss)
        h = ws.get((T, H), self.dtype)
        F.rmsnorm(x, self.w.final_norm, eps, out=h)
        ws.put(x)
        return h

    # ------------------------------------------------------------------ sequence-parallel forward
    def _use_sp(self, T: int) -> bool:
        cfg, ctx = self.cfg, self.ctx
        return (1 < ctx.tp <= flags().sp_max_ranks and T >= flags().comm_optimize_len
                and cfg.attn_type == AttnType.MHA and not cfg.is_moe and not cfg.qk_norm_full)

    def _forward_sp(self, tokens, meta, kv_caches, ws):
        """Layer loop with the residual stream and the norms sharded over tokens (Megatron-style
        sequence parallelism, the reference's "comm optimize" loop, xlite/csrc/model.cpp:1343-1406):
        row-parallel GEMMs end in a reduce-scatter, column-parallel GEMMs start with an all-gather,
        add+RMSNorm runs on T / tp rows. Tokens are padded to a multiple of 128 * tp."""
        cfg, ctx = self.cfg, self.ctx
        R = ctx.tp
        T = tokens.shape[0]
        unit = 128 * R
        Tp = (T + unit - 1) // unit * unit
        Tl = Tp // R
        H = cfg.hidden_size
        dt = self.dtype
        meta_dev = tokens.device.type == "meta"
        # embedding: vocab-parallel rows, reduce-scatter instead of all-reduce
        xfull = ws.get((Tp, H), dt)
        F.embed(tokens, self.w.embed, self.vocab_start, self.vocab_start + self.vocab_local, out=xfull[:T])
        if not meta_dev and Tp > T:
            xfull[T:].zero_()
        x = ws.get((Tl, H), dt)
        coll.reduce_scatter(xfull, ctx.tp_group, ctx, out=x)
        ws.put(xfull)
        h = ws.get((Tl, H), dt)
        F.rmsnorm(x, self.w.layers[0].attn_norm, cfg.rms_norm_eps, out=h)
        nq, nkv, hd = self.nq, self.nkv, self.hd
        for li, lw in enumerate(self.w.layers):
            qkv = ws.get((Tp, (nq + 2 * nkv) * hd), dt)
            fused.allgather_linear(h, lw.w_qkv, ctx, out=qkv, ws=ws)
            q = ws.get((T, nq * hd), dt)
            qk_nw = (lw.q_norm, lw.k_norm) if cfg.qk_norm else (None, None)
            F.rope_kvwrite(qkv[:T], meta, self.cos_sin, kv_caches[li][0], kv_caches[li][1], nq, nkv, hd,
                           cfg.rot_dim, hd ** -0.5, lw.b_qkv, qk_nw[0], qk_nw[1], cfg.rms_norm_eps,
                           self.mrope_mode, cfg.mrope_sections or (0, 0, 0), cfg.rope_interleaved, out=q)
            ws.put(qkv)
            o = ws.get((Tp, nq * hd), dt)
            F.paged_attention(q, kv_caches[li][0], kv_caches[li][1], meta, nq, nkv, hd, 1.0, out=o[:T])
            if not meta_dev and Tp > T:
                o[T:].zero_()
            ws.put(q)
            a = ws.get((Tl, H), dt)
            fused.row_parallel_linear_rs(o, lw.w_o, ctx, out=a, ws=ws)
            ws.put(o)
            F.add_rmsnorm(a, x, lw.mlp_norm, cfg.rms_norm_eps, out=h)
            inter = lw.w_gate_up.shape[0] // 2
            gu = ws.get((Tp, 2 * inter), dt)
            fused.allgather_linear(h, lw.w_gate_up, ctx, out=gu, ws=ws)
            act = ws.get((Tp, inter), dt)
            F.silu_and_mul(gu, out=act, clamp=cfg.swiglu_clamp, interleaved=getattr(lw, "gu_il", False))
            ws.put(gu)
            fused.row_parallel_linear_rs(act, lw.w_down, ctx, out=a, ws=ws)
            ws.put(act)
            nxt = self.w.layers[li + 1].attn_norm if li + 1 < len(self.w.layers) else self.w.final_norm
            F.add_rmsnorm(a, x, nxt, cfg.rms_norm_eps, out=h)
            ws.put(a)
        ws.put(x)
        hfull = ws.get((Tp, H), dt)
        coll.all_gather(h, ctx.tp_group, ctx, out=hfull)
        ws.put(h)
        return hfull

    # ------------------------------------------------------------------ forward
    def forward(self, tokens: torch.Tensor, meta: F.AttnMeta, kv_caches, ws: Optional[Workspace] = None,
                inputs_embeds: Optional[torch.Tensor] = None, deepstack: Optional[list] = None,
                mm_override=None) -> torch.Tensor:
        """tokens int32 [T] -> final-normed hidden states [T, H].

        Multimodal inputs (xlite/xlite/_C.cpp:1988-2001): `inputs_embeds` replaces the embedding
        lookup for the whole step and `deepstack[i]` ([T, H]) is added after layer i; or, for steps
        that mix text and image tokens, `mm_override = (rows, embeds, [deepstack...])` replaces the
        embedding of the listed rows only and adds the DeepStack features to those rows."""
        g = self.forward_phases(tokens, meta, kv_caches, ws, inputs_embeds, deepstack, mm_override)
        while True:
            try:
                next(g)
            except StopIteration as done:
                return done.value

    def forward_phases(self, tokens: torch.Tensor, meta: F.AttnMeta, kv_caches, ws: Optional[Workspace] = None,
                       inputs_embeds: Optional[torch.Tensor] = None, deepstack: Optional[list] = None,
                       mm_override=None, allow_sp: bool = True):
        """`forward` as a generator that pauses after the attention half and after the FFN half of
        every layer and returns the hidden states at the end. A driver that alternates two such
        generators on two streams overlaps one micro-batch's collectives with the other's GEMMs
        (the reference's dual-runtime "multi task parallel" prefill, xlite/tests/models/llama.py:368-416):
        a later micro-batch's attention at layer L only needs the earlier one's cache rows of
        layer L, which are written before the earlier one's pause after that attention."""
        cfg = self.cfg
        ws = ws or TorchWorkspace(self.device)
        T = tokens.shape[0] if inputs_embeds is None else inputs_embeds.shape[0]
        plain = inputs_embeds is None and deepstack is None and mm_override is None
        if (plain and self.fused_decode and 0 < T <= D.MAX_TOKENS
                and self.debug_hook is None):
            return self._forward_decode_fused(tokens, meta, kv_caches, ws)
        if allow_sp and plain and self._use_sp(T):
            return self._forward_sp(tokens, meta, kv_caches, ws)
        if inputs_embeds is not None:
            x = ws.get((T, cfg.hidden_size), self.dtype)
            if x.device.type != "meta":
                x.copy_(inputs_embeds)
        else:
            x = self._embed(tokens, ws)
            if mm_override is not None and x.device.type != "meta":
                x.index_copy_(0, mm_override[0], mm_override[1].to(x.dtype))
        h = ws.get((T, cfg.hidden_size), self.dtype)
        F.rmsnorm(x, self.w.layers[0].attn_norm, cfg.rms_norm_eps, out=h)
        for li, lw in enumerate(self.w.layers):
            self._dbg("in", li, x)
            a = ws.get((T, cfg.hidden_size), self.dtype)
            if cfg.layer_is_linear_attn(li):
                linear_attn.forward(self, li, lw, h, meta, kv_caches[li], ws, a)
            elif cfg.attn_type in (AttnType.MLA, AttnType.DSA):
                mla.forward(self, li, lw, h, meta, kv_caches[li], ws, a)
            else:
                self._attn_mha(li, lw, h, meta, kv_caches[li], ws, a)
            self._dbg("after_attn", li, a)
            yield ("attn", li)
            F.add_rmsnorm(a, x, lw.mlp_norm, cfg.rms_norm_eps, out=h)
            if cfg.layer_is_moe(li):
                moe.forward(self, li, lw, h, ws, a)
            else:
                self._mlp(lw, h, ws, a)
            self._dbg("after_ffn", li, a)
            if deepstack is not None and li < len(deepstack) and a.device.type != "meta":
                F.add(a, deepstack[li], out=a)
            if mm_override is not None and li < len(mm_override[2]) and a.device.type != "meta":
                a.index_add_(0, mm_override[0], mm_override[2][li].to(a.dtype))
            nxt = self.w.layers[li + 1].attn_norm if li + 1 < len(self.w.layers) else self.w.final_norm
            F.add_rmsnorm(a, x, nxt, cfg.rms_norm_eps, out=h)
            ws.put(a)
            yield ("ffn", li)
        ws.put(x)
        return h

    def compute_logits(self, hidden: torch.Tensor, meta: F.AttnMeta, ws: Optional[Workspace] = None,
                       batch: Optional[int] = None, gather: bool = True) -> torch.Tensor:
        """Logits of each request's last new token: gather rows -> vocab-parallel lm_head ->
        all-gather over TP (xlite/csrc/model.cpp:1458-1475). Returns [B, V]; with `gather=False`
        this rank's vocabulary shard [B, V / tp] (token ids offset by `vocab_start`)."""
        cfg, ctx = self.cfg, self.ctx
        ws = ws or TorchWorkspace(self.device)
        B = batch if batch is not None else meta.batch
        rows = ws.get((B, cfg.hidden_size), self.dtype)
        F.gather_rows(hidden, meta.last_token_idx[:B], out=rows)
        lm = self.w.lm_head if self.w.lm_head is not None else self.w.embed
        logits = ws.get((B, self.vocab_local), self.dtype)
        F.linear(rows, lm, None, out=logits)
        ws.put(rows)
        if ctx.tp > 1 and gather:
            full = ws.get((ctx.tp, B, self.vocab_local), self.dtype)
            coll.all_gather(logits, ctx.tp_group, ctx, out=full.view(ctx.tp * B, self.vocab_local))
            ws.put(logits)
            merged = ws.get((B, ctx.tp * self.vocab_local), self.dtype)
            if full.device.type != "meta":
                merged.view(B, ctx.tp, self.vocab_local).copy_(full.permute(1, 0, 2))
            ws.put(full)
            return merged
        return logits

    def greedy_tokens(self, hidden: torch.Tensor, meta: F.AttnMeta, ws: Optional[Workspace] = None,
                      batch: Optional[int] = None) -> torch.Tensor:
        """argmax of the logits without assembling them: every rank takes the best token of its
        vocabulary shard, the (score, id) pairs (8 bytes per request and rank) are all-gathered and
        the best pair wins, the lowest rank on a tie, which is what argmax over the concatenated
        vocabulary returns. Replaces the all-gather of [B, V] logits, their re-ordering and a
        full-vocabulary pass of the sampler. Returns int32 [B]."""
        ctx = self.ctx
        logits = self.compute_logits(hidden, meta, ws, batch, gather=False)
        if ctx.tp == 1:
            out = F.sample(logits)
        else:
            idx, val = F.sample(logits, index_offset=self.vocab_start, return_scores=True)
            # rows of 16 bytes (score, id, 0, 0): the push collective moves whole 16-byte lines
            zero = torch.zeros_like(val, dtype=torch.float32)
            pair = torch.stack([val.float(), idx.view(torch.float32), zero, zero], 1).contiguous()
            allp = coll.all_gather(pair, ctx.tp_group, ctx).view(ctx.tp, -1, 4)
            best = allp[:, :, 0].argmax(0, keepdim=True)                                     # first max = lowest rank
            out = allp[:, :, 1].contiguous().view(torch.int32).gather(0, best)[0]
        if getattr(logits, "_gv_off", None) is not None and ws is not None:
            ws.put(logits)
        return out
