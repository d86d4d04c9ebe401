"""Same-box floor: the identical decoder graph written with stock PyTorch ops — cuBLAS GEMMs
(``torch.matmul``), ``scaled_dot_product_attention`` over a dense preallocated KV cache,
``torch.distributed`` (NCCL) all-reduce for tensor parallelism — with random-init weights and
synthetic token ids. None of this repository's kernels, engine or scheduler is on this path.
The decode step has static shapes (the cache up to the next multiple of 64 positions under a
length mask, the position a device scalar), so the library attention keeps a cached plan instead
of building one per context length, and the step is replayed from a CUDA graph per 64-position
bucket (``GVIRT_FLOOR_GRAPH=0`` runs it eagerly).
Used by ``bench.py --impl torch``; reports the same JSON fields as the main arm.
"""
from __future__ import annotations

import time

import torch
import torch.distributed as dist
import torch.nn.functional as TF


def _rope(x, cos, sin):
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1)


class TorchLlama:
    def __init__(self, cfg, ctx, batch, max_len, seed=0):
        self.cfg, self.ctx = cfg, ctx
        dev, dt = ctx.device, torch.bfloat16
        tp = ctx.tp
        g = torch.Generator(device=dev).manual_seed(seed + ctx.rank)
        H, hd = cfg.hidden_size, cfg.head_dim
        self.nq, self.nkv = cfg.num_heads // tp, max(cfg.num_kv_heads // tp, 1)

        def w(*s):
            t = torch.empty(*s, dtype=dt, device=dev)
            t.normal_(0, 0.02, generator=g)
            return t

        self.embed = w(cfg.vocab_size, H)
        self.lm_head = w(cfg.vocab_size // tp, H)
        self.layers = []
        for _ in range(cfg.num_layers):
            self.layers.append(dict(
                n1=torch.ones(H, dtype=dt, device=dev), n2=torch.ones(H, dtype=dt, device=dev),
                qkv=w((self.nq + 2 * self.nkv) * hd, H), o=w(H, self.nq * hd),
                b_qkv=w((self.nq + 2 * self.nkv) * hd) if getattr(cfg, "qkv_bias", False) else None,
                gu=w(2 * cfg.intermediate_size // tp, H), down=w(H, cfg.intermediate_size // tp)))
        self.norm = torch.ones(H, dtype=dt, device=dev)
        self.k = [torch.zeros(batch, self.nkv, max_len, hd, dtype=dt, device=dev) for _ in range(cfg.num_layers)]
        self.v = [torch.zeros(batch, self.nkv, max_len, hd, dtype=dt, device=dev) for _ in range(cfg.num_layers)]
        half = hd // 2
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, half, device=dev).float() * 2 / hd))
        ang = torch.outer(torch.arange(max_len, device=dev).float(), inv)
        self.cos, self.sin = ang.cos().to(dt), ang.sin().to(dt)
        # static decode step: inputs and outputs live at fixed addresses
        self.max_len = max_len
        self.tok = torch.zeros(batch, 1, dtype=torch.int64, device=dev)
        self.pos_t = torch.zeros(1, dtype=torch.int64, device=dev)
        self.out = torch.zeros(batch, dtype=torch.int64, device=dev)
        self.arange = torch.arange(max_len, device=dev)
        self.graphs = {}                      # cache length bucket -> captured step
        self.pos_host = 0

    def _rms(self, x, w):
        return TF.rms_norm(x, (x.shape[-1],), w, self.cfg.rms_norm_eps)

    @torch.no_grad()
    def decode_static(self, Lb):
        """One decode step of static shape over the first `Lb` cache positions: token ids in
        ``self.tok``, position in ``self.pos_t`` (advanced by one here), next ids into ``self.out``."""
        cfg, ctx = self.cfg, self.ctx
        B, hd = self.tok.shape[0], cfg.head_dim
        pos = self.pos_t
        x = self.embed[self.tok]
        cos, sin = self.cos.index_select(0, pos)[None, :, None, :], self.sin.index_select(0, pos)[None, :, None, :]
        mask = (self.arange[:Lb] <= pos).view(1, 1, 1, Lb)
        G = self.nq // self.nkv
        for i, L in enumerate(self.layers):
            h = self._rms(x, L["n1"])
            qkv = h @ L["qkv"].t()
            if L["b_qkv"] is not None:
                qkv = qkv + L["b_qkv"]
            q, k, v = qkv.split([self.nq * hd, self.nkv * hd, self.nkv * hd], -1)
            q = _rope(q.view(B, 1, self.nq, hd), cos, sin).transpose(1, 2)
            k = _rope(k.view(B, 1, self.nkv, hd), cos, sin).transpose(1, 2)
            v = v.view(B, 1, self.nkv, hd).transpose(1, 2)
            self.k[i].index_copy_(2, pos, k)
            self.v[i].index_copy_(2, pos, v)
            o = TF.scaled_dot_product_attention(q.reshape(B, self.nkv, G, hd), self.k[i][:, :, :Lb], self.v[i][:, :, :Lb],
                                                    attn_mask=mask)
            o = o.reshape(B, 1, self.nq * hd) @ L["o"].t()
            if ctx.tp > 1:
                dist.all_reduce(o, group=ctx.tp_group)
            x = x + o
            h = self._rms(x, L["n2"])
            gu = h @ L["gu"].t()
            d = gu.shape[-1] // 2
            m = (TF.silu(gu[..., :d]) * gu[..., d:]) @ L["down"].t()
            if ctx.tp > 1:
                dist.all_reduce(m, group=ctx.tp_group)
            x = x + m
        h = self._rms(x[:, -1], self.norm)
        logits = h @ self.lm_head.t()
        if ctx.tp > 1:
            full = torch.empty(ctx.tp, *logits.shape, dtype=logits.dtype, device=logits.device)
            dist.all_gather_into_tensor(full, logits, group=ctx.tp_group)
            logits = full.permute(1, 0, 2).reshape(B, -1)
        self.out.copy_(logits.argmax(-1))
        self.pos_t.add_(1)

    def bucket(self, pos):
        return min(self.max_len, (pos + 64) // 64 * 64)

    def capture(self, first_pos, last_pos):
        """Record the static decode step into one CUDA graph per cache-length bucket that the
        positions first_pos..last_pos need (a side stream warms each up first)."""
        keep = self.pos_t.clone()
        for Lb in sorted({self.bucket(p) for p in range(first_pos, last_pos + 1)}):
            if Lb in self.graphs:
                continue
            self.pos_t.fill_(Lb - 1)
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self.decode_static(Lb)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            self.pos_t.fill_(Lb - 1)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self.decode_static(Lb)
            self.graphs[Lb] = g
        self.pos_t.copy_(keep)

    def seek(self, pos):
        self.pos_host = pos
        self.pos_t.fill_(pos)

    def step(self, tokens):
        """tokens [B] (device) -> next ids [B] at the current position, which moves on by one."""
        self.tok.copy_(tokens.view(-1, 1))
        Lb = self.bucket(self.pos_host)
        g = self.graphs.get(Lb)
        if g is not None:
            g.replay()
        else:
            self.decode_static(Lb)
        self.pos_host += 1
        return self.out

    @torch.no_grad()
    def forward(self, tokens, start):
        """tokens [B, S] at positions start..start+S-1 -> next token ids [B]."""
        cfg, ctx = self.cfg, self.ctx
        B, S = tokens.shape
        hd = cfg.head_dim
        x = self.embed[tokens]
        cos, sin = self.cos[start:start + S][None, :, None, :], self.sin[start:start + S][None, :, None, :]
        for i, L in enumerate(self.layers):
            h = self._rms(x, L["n1"])
            qkv = h @ L["qkv"].t()
            if L["b_qkv"] is not None:
                qkv = qkv + L["b_qkv"]
            q, k, v = qkv.split([self.nq * hd, self.nkv * hd, self.nkv * hd], -1)
            q = _rope(q.view(B, S, self.nq, hd), cos, sin).transpose(1, 2)
            k = _rope(k.view(B, S, self.nkv, hd), cos, sin).transpose(1, 2)
            v = v.view(B, S, self.nkv, hd).transpose(1, 2)
            self.k[i][:, :, start:start + S] = k
            self.v[i][:, :, start:start + S] = v
            kk, vv = self.k[i][:, :, :start + S], self.v[i][:, :, :start + S]
            if S == 1:
                # decode: the query heads that share a kv head become the rows of one attention
                # problem per kv head ([B, nkv, G, hd] against [B, nkv, L, hd]); this shape takes a
                # fused SDPA kernel, whereas enable_gqa on a one-token query falls back to the
                # unfused math path
                G = self.nq // self.nkv
                o = TF.scaled_dot_product_attention(q.reshape(B, self.nkv, G, hd), kk, vv, is_causal=False)
                o = o.reshape(B, 1, self.nq * hd) @ L["o"].t()
            else:
                o = TF.scaled_dot_product_attention(q, kk, vv, is_causal=True, enable_gqa=True)
                o = o.transpose(1, 2).reshape(B, S, self.nq * hd) @ L["o"].t()
            if ctx.tp > 1:
                dist.all_reduce(o, group=ctx.tp_group)
            x = x + o
            h = self._rms(x, L["n2"])
            gu = h @ L["gu"].t()
            d = gu.shape[-1] // 2
            m = (TF.silu(gu[..., :d]) * gu[..., d:]) @ L["down"].t()
            if ctx.tp > 1:
                dist.all_reduce(m, group=ctx.tp_group)
            x = x + m
        h = self._rms(x[:, -1], self.norm)
        logits = h @ self.lm_head.t()
        if ctx.tp > 1:
            full = torch.empty(ctx.tp, *logits.shape, dtype=logits.dtype, device=logits.device)
            dist.all_gather_into_tensor(full, logits, group=ctx.tp_group)
            logits = full.permute(1, 0, 2).reshape(B, -1)
        return logits.argmax(-1)


def run_floor(cfg, ctx, B, P, K, W, advance=0):
    """`advance`: decode positions skipped after the warm-up so that the timed steps sit at the
    same context as the main arm's (the skipped cache rows stay zero: same bytes, same work)."""
    if cfg.is_moe or cfg.attn_type.name != "MHA":
        raise SystemExit("--impl torch covers the dense MHA decoders (Llama, Qwen2, Qwen2.5)")
    dev = ctx.device
    max_len = (P + W + advance + K + 2 + 64) // 64 * 64
    model = TorchLlama(cfg, ctx, B, max_len)
    g = torch.Generator().manual_seed(1234)
    prompts = torch.randint(0, cfg.vocab_size, (B, P), generator=g)
    host_tok = torch.empty(B, dtype=torch.int64, pin_memory=True)
    t0 = time.perf_counter()
    chunk = 8
    nxt = torch.empty(B, dtype=torch.int64, device=dev)
    # prefill in request chunks of 8 x P tokens (same token budget as the main arm)
    ks, vs = model.k, model.v
    for s in range(0, B, chunk):
        model.k = [t[s:s + chunk] for t in ks]
        model.v = [t[s:s + chunk] for t in vs]
        nxt[s:s + chunk] = model.forward(prompts[s:s + chunk].to(dev), 0)
    model.k, model.v = ks, vs
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0
    pos = P

    def barrier():
        if ctx.world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    import os
    graphed = os.environ.get("GVIRT_FLOOR_GRAPH", "1") != "0"
    if graphed:
        model.capture(pos, pos + W)
        model.capture(pos + W + advance, pos + W + advance + K + 2)
    model.seek(pos)
    for _ in range(W):
        nxt = model.step(nxt)
        pos += 1
    pos += advance
    model.seek(pos)
    barrier()
    pos0 = pos
    # end to end: token ids come from pinned host memory each step, result is read back
    host_tok.copy_(nxt)
    t0 = time.perf_counter()
    for _ in range(K):
        d = host_tok.to(dev, non_blocking=True)
        out = model.step(d)
        host_tok.copy_(out, non_blocking=True)
        torch.cuda.synchronize()
        pos += 1
    barrier()
    e2e_s = time.perf_counter() - t0
    nxt = host_tok.to(dev)
    pos = pos0                                # the device-timed loop covers the same positions again
    model.seek(pos)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(K):
        nxt = model.step(nxt)
        pos += 1
    ev1.record()
    barrier()
    dev_ms = ev0.elapsed_time(ev1)
    t = torch.tensor([dev_ms, e2e_s * 1e3], dtype=torch.float64, device=dev)
    if ctx.world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = t.tolist()
    return {"metric": "decode_output_tok_s", "value": round(B * K / (dev_ms / 1e3), 1), "unit": "tok/s",
            "n_gpus": ctx.world, "steps": K, "warmup": W, "ms_per_step": round(dev_ms / K, 4),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "impl": "torch",
            "config": {"model": cfg.name, "global_batch": B, "seq_len": P, "parallelism": f"tp{ctx.world}",
                       "layers": cfg.num_layers, "decode_context": pos,
                       "note": "PyTorch ops: cuBLAS + SDPA + NCCL, dense KV cache, static-shape decode step"
                               + (" replayed from a CUDA graph" if graphed else " run eagerly")},
            "e2e": {"value": round(B * K / (e2e_ms / 1e3), 1), "unit": "tok/s", "ms_per_step": round(e2e_ms / K, 4),
                    "h2d_bytes_per_step": B * 8, "d2h_bytes_per_step": B * 8},
            "gpu_launches": 0, "prefill_tok_s": round(B * P / prefill_s, 1)}
