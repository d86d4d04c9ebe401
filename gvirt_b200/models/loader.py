"""Hugging Face checkpoint loading: ``config.json`` -> ``ModelConfig``, ``*.safetensors``
(single file or sharded with ``model.safetensors.index.json``) -> the engine's weight namespace,
sliced for this rank while reading (lazy ``get_slice`` — a rank never materialises tensors it
does not own).

Follows the reference loaders: lazy safetensors iteration with TP shard loading
(xlite/tests/models/weight_utils.py:169-309), q/k/v -> fused ``qkv_proj`` and gate/up -> fused
``gate_up_proj`` (xlite/tests/models/llama.py:446-509), expert slicing per EP rank
(xlite/tests/models/qwen3_moe.py:720-803), DeepSeek ``kv_b_proj`` split into ``W_UK^T`` / ``W_UV``
(xlite/tests/models/deepseek_v3.py:1501-1515) and fp8 checkpoints with ``weight_scale_inv``
128x128 block scales (xlite/xlite/tools/fp8_cast_bf16.py:21-61), which are either kept as fp8 +
scales (``quant == "fp8_block"``) or dequantised to bf16 on the fly.
"""
from __future__ import annotations

import json
import os
from pathlib import Path
from types import SimpleNamespace
from typing import Dict, Optional

import torch

from ..config import AttnType, ModelConfig
from ..ops import reference as ref
from ..parallel.state import ParallelContext, context
from . import weights as W


class CheckpointReader:
    """name -> tensor (or row / column slice) across all safetensors shards of a directory."""

    def __init__(self, path: str):
        from safetensors import safe_open
        self.path = Path(path)
        self._open = safe_open
        idx = self.path / "model.safetensors.index.json"
        self.where: Dict[str, str] = {}
        if idx.exists():
            with open(idx) as f:
                self.where = dict(json.load(f)["weight_map"])
        else:
            for fn in sorted(self.path.glob("*.safetensors")):
                with safe_open(str(fn), framework="pt") as f:
                    for k in f.keys():
                        self.where[k] = fn.name
        # torch-pickle checkpoints (`pytorch_model*.bin`, `*.pt`) as a fall-back, held in memory
        # (the reference's iterator has the same fall-backs, xlite/tests/models/weight_utils.py:169-241)
        self._mem: Dict[str, torch.Tensor] = {}
        if not self.where:
            for fn in sorted(self.path.glob("*.bin")) + sorted(self.path.glob("*.pt")):
                sd = torch.load(str(fn), map_location="cpu", weights_only=True)
                if isinstance(sd, dict):
                    for k, v in sd.items():
                        if isinstance(v, torch.Tensor):
                            self._mem[k] = v
                            self.where[k] = ":memory:"
        if not self.where:
            raise FileNotFoundError(f"no safetensors / .bin / .pt weights under {path}")
        # multimodal checkpoints nest the decoder under `model.language_model.`
        self.alias: Dict[str, str] = {}
        for k in self.where:
            if k.startswith("model.language_model."):
                self.alias["model." + k[len("model.language_model."):]] = k
        self._handles = {}

    def _h(self, fn):
        if fn not in self._handles:
            self._handles[fn] = self._open(str(self.path / fn), framework="pt")
        return self._handles[fn]

    def _n(self, name: str) -> str:
        return name if name in self.where else self.alias.get(name, name)

    def has(self, name: str) -> bool:
        return self._n(name) in self.where

    def get(self, name: str) -> torch.Tensor:
        name = self._n(name)
        if name in self._mem:
            return self._mem[name]
        return self._h(self.where[name]).get_tensor(name)

    def rows(self, name: str, a: int, b: int) -> torch.Tensor:
        name = self._n(name)
        if name in self._mem:
            return self._mem[name][a:b]
        return self._h(self.where[name]).get_slice(name)[a:b]

    def cols(self, name: str, a: int, b: int) -> torch.Tensor:
        name = self._n(name)
        if name in self._mem:
            return self._mem[name][:, a:b]
        return self._h(self.where[name]).get_slice(name)[:, a:b]

    def shape(self, name: str):
        name = self._n(name)
        if name in self._mem:
            return tuple(self._mem[name].shape)
        return tuple(self._h(self.where[name]).get_slice(name).get_shape())

    def dequant(self, name: str) -> torch.Tensor:
        """Full tensor; fp8 weights with a `<name>_scale_inv` companion are block-dequantised,
        int8 weights with a `<name>_scale` (or `deq_scale` / `input_scale`) companion are
        de-quantised per output channel."""
        w = self.get(name)
        s = name + "_scale_inv"
        if w.dtype == torch.float8_e4m3fn and self.has(s):
            return ref.dequant_fp8_block(w, self.get(s).float())
        if w.dtype == torch.int8:
            q = self.int8_params(name[: -len("weight")] if name.endswith("weight") else name + ".")
            wf = w.float() * q["scale"][:, None]
            if q["in_scale"] is not None:          # static: deq_scale = weight scale x input scale
                wf = wf / q["in_scale"].reshape(1, -1)
            return wf.to(torch.bfloat16)
        return w

    def int8_params(self, prefix: str) -> dict:
        """Quantisation tensors stored beside `<prefix>weight` (names of the reference's int8
        checkpoints, xlite/tests/models/deepseek_v3.py:1226-1238): dynamic layers carry
        `weight_scale` [N]; static layers carry `input_scale`, `input_offset`, `quant_bias` [N]
        (int32) and `deq_scale` [N]. Returns fp32 tensors (None where absent)."""
        def opt(n):
            return self.get(prefix + n) if self.has(prefix + n) else None
        scale = opt("deq_scale")
        static = scale is not None
        if scale is None:
            scale = opt("weight_scale")
        if scale is None:
            raise KeyError(f"int8 tensor {prefix}weight has neither weight_scale nor deq_scale")
        if scale.dtype == torch.int64:              # fp32 bits kept in the low half of an int64
            scale = (scale & 0xFFFFFFFF).to(torch.int32).view(torch.float32)
        ins, off, qb = opt("input_scale"), opt("input_offset"), opt("quant_bias")
        return {"scale": scale.float().reshape(-1), "static": static,
                "in_scale": None if ins is None else ins.float().reshape(-1),
                "in_offset": None if off is None else off.float().reshape(-1),
                "quant_bias": None if qb is None else qb.float().reshape(-1)}


def load_pretrained(path: str, ctx: Optional[ParallelContext] = None, device=None, **overrides):
    """-> (ModelConfig, weights namespace, tokenizer or None, eos token id or None)"""
    ctx = ctx or context()
    device = torch.device(device) if device is not None else ctx.device
    overrides.setdefault("tp_size", ctx.tp)
    overrides.setdefault("dp_size", ctx.dp)
    overrides.setdefault("ep_size", ctx.ep)
    overrides.setdefault("moe_tp_size", ctx.moe_tp)
    cfg = ModelConfig.from_pretrained(path, **overrides)
    if cfg.quant == "fp8_block" and not overrides.get("keep_fp8", True):
        cfg.quant = "none"
    rd = CheckpointReader(path)
    weights = _load(cfg, rd, ctx, device)
    if cfg.quant == "w8a8_int8":
        for L in weights.layers:          # projections the checkpoint holds in floating point
            W.quantize_dense_layer_w8a8(L)
    tok, eos = None, None
    try:
        from transformers import AutoTokenizer
        tok = AutoTokenizer.from_pretrained(path)
        eos = tok.eos_token_id
    except Exception:  # noqa: BLE001 - a checkpoint without tokenizer files is fine
        with open(Path(path) / "config.json") as f:
            e = json.load(f).get("eos_token_id")
        eos = e[0] if isinstance(e, list) else e
    return cfg, weights, tok, eos


def _load(cfg: ModelConfig, rd: CheckpointReader, ctx: ParallelContext, device) -> SimpleNamespace:
    dt = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}[cfg.dtype]
    tp, r = cfg.tp_size, ctx.tp_rank
    hd, H = cfg.head_dim, cfg.hidden_size
    nq_l, nkv_l = cfg.local_heads()
    k0, k1 = W.kv_head_range(cfg, r)

    def put(t):
        if t.dtype == torch.int8:
            return t.to(device).contiguous()
        return t.to(dt).to(device).contiguous()

    def fused(pieces, cols=None, keep_bias=True):
        """A projection assembled from checkpoint tensors. `pieces`: [(name prefix, row lo, row
        hi)] concatenated along the output dimension; `cols` = (lo, hi) slices the input dimension
        (row-parallel layers). bf16 / fp8 checkpoints give a tensor of the model dtype. int8
        checkpoints keep their int8 values when the engine runs W8A8 (`quant == "w8a8_int8"`) and
        every piece agrees on its activation quantisation; the per-channel scales, the static
        activation factors and the folded `quant_bias` travel as attributes of the tensor
        (`gv_scale`, `gv_in_scale_recip`, `gv_in_offset`, `gv_bias`). Otherwise they are
        de-quantised."""
        raw = [rd.rows(p + "weight", lo, hi) for p, lo, hi in pieces]
        if cols is not None:
            raw = [t[:, cols[0]:cols[1]] for t in raw]
        if raw[0].dtype != torch.int8:
            if raw[0].dtype == torch.float8_e4m3fn:
                raw = [rd.dequant(p + "weight")[lo:hi] for p, lo, hi in pieces]
                if cols is not None:
                    raw = [t[:, cols[0]:cols[1]] for t in raw]
            return put(torch.cat(raw, 0))
        qs = [rd.int8_params(p) for p, _, _ in pieces]
        K = raw[0].shape[1]

        def kvec(v):      # per-tensor or per-channel value as a [K] vector of this rank's columns
            v = v.expand(rd.shape(pieces[0][0] + "weight")[1]) if v.numel() == 1 else v
            return v[cols[0]:cols[1]] if cols is not None else v

        same = all(q["static"] == qs[0]["static"] for q in qs)
        if same and qs[0]["static"]:
            same = all(torch.equal(q["in_scale"], qs[0]["in_scale"]) and
                       (q["in_offset"] is None) == (qs[0]["in_offset"] is None) and
                       (q["in_offset"] is None or torch.equal(q["in_offset"], qs[0]["in_offset"])) for q in qs)
        if cfg.quant != "w8a8_int8" or not same or K % 16:
            deq = [rd.dequant(p + "weight")[lo:hi] for p, lo, hi in pieces]
            if cols is not None:
                deq = [t[:, cols[0]:cols[1]] for t in deq]
            return put(torch.cat(deq, 0))
        w = put(torch.cat(raw, 0))
        w.gv_scale = torch.cat([q["scale"][lo:hi] for q, (_, lo, hi) in zip(qs, pieces)]).to(device).contiguous()
        if qs[0]["static"]:
            w.gv_in_scale_recip = (1.0 / kvec(qs[0]["in_scale"])).to(device).contiguous()
            if qs[0]["in_offset"] is not None:
                w.gv_in_offset = kvec(qs[0]["in_offset"]).to(device).contiguous()
            if keep_bias and all(q["quant_bias"] is not None for q in qs):
                qb = torch.cat([q["quant_bias"][lo:hi] for q, (_, lo, hi) in zip(qs, pieces)])
                w.gv_bias = (qb.to(device) * w.gv_scale).contiguous()
        return w

    def pre(i):
        return f"model.layers.{i}."

    def norm(name):
        """RMSNorm weight; checkpoints of the (1 + w) convention are folded to plain weights
        (xlite/tests/models/qwen3_5.py:56-59)."""
        w = rd.get(name)
        return put(w.float() + 1.0) if cfg.norm_plus_one else put(w)

    out = SimpleNamespace()
    V = cfg.vocab_size
    vl = V // tp
    out.embed = put(rd.rows("model.embed_tokens.weight", r * vl, (r + 1) * vl))
    if cfg.tie_word_embeddings or not rd.has("lm_head.weight"):
        out.lm_head = None
    else:
        out.lm_head = put(rd.rows("lm_head.weight", r * vl, (r + 1) * vl))
    out.final_norm = norm("model.norm.weight")
    def load_layer(i, moe):
        p = pre(i)
        L = SimpleNamespace()
        L.attn_norm = norm(p + "input_layernorm.weight")
        L.mlp_norm = norm(p + "post_attention_layernorm.weight")
        a = p + "self_attn."
        if cfg.layer_is_linear_attn(i):
            _load_linear_attn(cfg, rd, L, p + "linear_attn.", r, put)
        elif cfg.attn_type in (AttnType.MLA, AttnType.DSA):
            _load_mla(cfg, rd, L, a, r, put)
        else:
            k = v = None
            if not cfg.attn_output_gate:
                L.w_qkv = fused([(a + "q_proj.", r * nq_l * hd, (r + 1) * nq_l * hd),
                                 (a + "k_proj.", k0 * hd, k1 * hd), (a + "v_proj.", k0 * hd, k1 * hd)])
            else:
                k = rd.rows(a + "k_proj.weight", k0 * hd, k1 * hd)
                v = rd.rows(a + "v_proj.weight", k0 * hd, k1 * hd)
            if cfg.attn_output_gate:
                # q_proj holds [q | gate] per head (xlite/tests/models/qwen3_5.py:39-53); the
                # engine's fused row is [q heads | k | v | gate heads]
                qg = rd.rows(a + "q_proj.weight", r * nq_l * 2 * hd, (r + 1) * nq_l * 2 * hd).view(nq_l, 2, hd, H)
                L.w_qkv = put(torch.cat([qg[:, 0].reshape(nq_l * hd, H), k, v, qg[:, 1].reshape(nq_l * hd, H)], 0))
            if rd.has(a + "q_proj.bias") and not cfg.attn_output_gate:
                L.b_qkv = put(torch.cat([rd.rows(a + "q_proj.bias", r * nq_l * hd, (r + 1) * nq_l * hd),
                                         rd.rows(a + "k_proj.bias", k0 * hd, k1 * hd),
                                         rd.rows(a + "v_proj.bias", k0 * hd, k1 * hd)], 0))
            else:
                L.b_qkv = None
            if rd.has(a + "q_norm.weight"):
                qn, kn = rd.get(a + "q_norm.weight"), rd.get(a + "k_norm.weight")
                if cfg.qk_norm_full:
                    qn, kn = qn[r * nq_l * hd:(r + 1) * nq_l * hd], kn[k0 * hd:k1 * hd]
                if cfg.norm_plus_one:
                    qn, kn = qn.float() + 1.0, kn.float() + 1.0
                L.q_norm, L.k_norm = put(qn), put(kn)
            else:
                L.q_norm = L.k_norm = None
            L.w_o = fused([(a + "o_proj.", 0, H)], cols=(r * nq_l * hd, (r + 1) * nq_l * hd), keep_bias=(r == 0))
        m = p + "mlp."
        if moe:
            _load_moe(cfg, rd, ctx, L, m, put, device)
        else:
            I = cfg.intermediate_size
            il = I // tp
            L.w_gate_up = fused([(m + "gate_proj.", r * il, (r + 1) * il), (m + "up_proj.", r * il, (r + 1) * il)])
            L.w_down = fused([(m + "down_proj.", 0, H)], cols=(r * il, (r + 1) * il), keep_bias=(r == 0))
        return L

    out.layers = [load_layer(i, cfg.layer_is_moe(i)) for i in range(cfg.num_layers)]
    # multi-token-prediction module stored as one more "layer" (DeepSeek-V3: index num_hidden_layers)
    mp = pre(cfg.num_layers)
    if rd.has(mp + "eh_proj.weight") and not cfg.layer_is_linear_attn(cfg.num_layers):
        out.mtp = SimpleNamespace(layer=load_layer(cfg.num_layers, cfg.is_moe), enorm=norm(mp + "enorm.weight"),
                                  hnorm=norm(mp + "hnorm.weight"), eh_proj=put(rd.dequant(mp + "eh_proj.weight")),
                                  shared_norm=norm(mp + "shared_head.norm.weight"))
    else:
        out.mtp = None
    return out


def _load_linear_attn(cfg, rd, L, a, r, put):
    """Gated DeltaNet layer (names of xlite/tests/models/qwen3_5.py:341-356): in_proj_qkv
    [q | k | v], in_proj_z, in_proj_b, in_proj_a, depthwise conv1d [C, 1, K], A_log, dt_bias, the
    gated norm and out_proj. Every part is sharded by heads and packed as the engine's fused
    input projection [q | k | v | z | b | a]."""
    tp = cfg.tp_size
    Hk, Hv = cfg.linear_num_key_heads, cfg.linear_num_value_heads
    dk, dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
    kd, vd = Hk * dk, Hv * dv
    kl, vl, hl = kd // tp, vd // tp, Hv // tp
    qkv = a + "in_proj_qkv.weight"
    parts = [rd.rows(qkv, r * kl, (r + 1) * kl), rd.rows(qkv, kd + r * kl, kd + (r + 1) * kl),
             rd.rows(qkv, 2 * kd + r * vl, 2 * kd + (r + 1) * vl),
             rd.rows(a + "in_proj_z.weight", r * vl, (r + 1) * vl),
             rd.rows(a + "in_proj_b.weight", r * hl, (r + 1) * hl),
             rd.rows(a + "in_proj_a.weight", r * hl, (r + 1) * hl)]
    L.w_in = put(torch.cat(parts, 0))
    conv = rd.get(a + "conv1d.weight")
    conv = conv.reshape(conv.shape[0], conv.shape[-1])
    L.conv_w = put(torch.cat([conv[r * kl:(r + 1) * kl], conv[kd + r * kl:kd + (r + 1) * kl],
                              conv[2 * kd + r * vl:2 * kd + (r + 1) * vl]], 0))
    L.conv_b = None
    dev = L.conv_w.device
    L.A_log = rd.get(a + "A_log")[r * hl:(r + 1) * hl].float().to(dev).contiguous()
    L.dt_bias = rd.get(a + "dt_bias")[r * hl:(r + 1) * hl].float().to(dev).contiguous()
    L.gdn_norm = put(rd.get(a + "norm.weight"))
    L.w_o = put(rd.cols(a + "out_proj.weight", r * vl, (r + 1) * vl))


def _load_mla(cfg, rd, L, a, r, put):
    hl = cfg.num_heads // cfg.tp_size
    dn, dr, dv, dc = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim, cfg.kv_lora_rank
    kv_a = rd.dequant(a + "kv_a_proj_with_mqa.weight")
    if cfg.q_lora_rank > 0:
        L.w_qkv_a = put(torch.cat([rd.dequant(a + "q_a_proj.weight"), kv_a], 0))
        L.q_a_norm = put(rd.get(a + "q_a_layernorm.weight"))
        qb = rd.dequant(a + "q_b_proj.weight")
    else:
        L.w_qkv_a = put(kv_a)
        L.q_a_norm = None
        qb = rd.dequant(a + "q_proj.weight")
    L.w_q_b = put(qb[r * hl * (dn + dr):(r + 1) * hl * (dn + dr)])
    L.kv_a_norm = put(rd.get(a + "kv_a_layernorm.weight"))
    kvb = rd.dequant(a + "kv_b_proj.weight").view(cfg.num_heads, dn + dv, dc)[r * hl:(r + 1) * hl]
    L.w_uk_t = put(kvb[:, :dn, :].transpose(1, 2))
    L.w_uv = put(kvb[:, dn:, :])
    ow = rd.dequant(a + "o_proj.weight")
    L.w_o = put(ow[:, r * hl * dv:(r + 1) * hl * dv])


def _load_moe(cfg, rd, ctx, L, m, put, device):
    E, I = cfg.num_experts, cfg.moe_intermediate_size
    e_local = E // ctx.ep
    e0 = ctx.ep_rank * e_local
    mtp, mr = ctx.moe_tp, ctx.moe_tp_rank
    il = I // mtp
    L.w_router = put(rd.get(m + "gate.weight"))
    bias_name = m + "gate.e_score_correction_bias"
    L.router_bias = rd.get(bias_name).float().to(device) if rd.has(bias_name) else None
    keep_fp8 = cfg.quant == "fp8_block"
    w13, w2, s13, s2 = [], [], [], []
    for e in range(e0, e0 + e_local):
        ep = f"{m}experts.{e}."
        if keep_fp8 and rd.get(ep + "gate_proj.weight").dtype == torch.float8_e4m3fn and mtp == 1:
            g, u, d = (rd.get(ep + n + ".weight") for n in ("gate_proj", "up_proj", "down_proj"))
            sg, su, sd = (rd.get(ep + n + ".weight_scale_inv").float() for n in ("gate_proj", "up_proj", "down_proj"))
            w13.append(torch.cat([g, u], 0))
            s13.append(torch.cat([sg, su], 0))
            w2.append(d)
            s2.append(sd)
        else:
            g = rd.dequant(ep + "gate_proj.weight")[mr * il:(mr + 1) * il]
            u = rd.dequant(ep + "up_proj.weight")[mr * il:(mr + 1) * il]
            d = rd.dequant(ep + "down_proj.weight")[:, mr * il:(mr + 1) * il]
            w13.append(torch.cat([g, u], 0))
            w2.append(d)
    if s13:
        L.w13, L.w2 = torch.stack(w13).to(device), torch.stack(w2).to(device)
        L.w13_scale, L.w2_scale = torch.stack(s13).to(device), torch.stack(s2).to(device)
    else:
        L.w13, L.w2 = put(torch.stack(w13)), put(torch.stack(w2))
        if keep_fp8:
            W.quantize_moe_layer_fp8(L)
    sp = m + "shared_experts."
    if not rd.has(sp + "gate_proj.weight") and rd.has(m + "shared_expert.gate_proj.weight"):
        sp = m + "shared_expert."          # Qwen-MoE naming, with a per-token gate beside it
    L.ws_gate = put(rd.dequant(m + "shared_expert_gate.weight")) if rd.has(m + "shared_expert_gate.weight") else None
    if rd.has(sp + "gate_proj.weight"):
        Is = rd.shape(sp + "gate_proj.weight")[0]
        stp, sr = (cfg.tp_size, ctx.tp_rank) if ctx.dp == 1 else (1, 0)
        sl = Is // stp
        g = rd.dequant(sp + "gate_proj.weight")[sr * sl:(sr + 1) * sl]
        u = rd.dequant(sp + "up_proj.weight")[sr * sl:(sr + 1) * sl]
        L.ws_gate_up = put(torch.cat([g, u], 0))
        L.ws_down = put(rd.dequant(sp + "down_proj.weight")[:, sr * sl:(sr + 1) * sl])
    else:
        L.ws_gate_up = L.ws_down = None


def save_hf_checkpoint(cfg: ModelConfig, weights: SimpleNamespace, path: str, shards: int = 2,
                       mtp: Optional[SimpleNamespace] = None) -> None:
    """Write a TP=1 / EP=1 weight namespace as a Hugging Face style directory (config.json +
    sharded safetensors + index). Used by tests and for exporting random-init models. `mtp`: a
    multi-token-prediction module (``engine.mtp``) stored as layer ``num_hidden_layers``."""
    from safetensors.torch import save_file
    assert cfg.tp_size == 1 and cfg.ep_size == 1
    os.makedirs(path, exist_ok=True)
    hd, nq, nkv = cfg.head_dim, cfg.num_heads, cfg.num_kv_heads
    def nrm(w):
        return (w.float() - 1.0).to(w.dtype) if cfg.norm_plus_one else w

    t: Dict[str, torch.Tensor] = {"model.embed_tokens.weight": weights.embed, "model.norm.weight": nrm(weights.final_norm)}
    if weights.lm_head is not None:
        t["lm_head.weight"] = weights.lm_head
    def emit(prefix, w, lo, hi):
        """Rows [lo, hi) of a (possibly fused) projection as `<prefix>weight`; an int8 projection
        also writes its scales in the int8 checkpoint layout `CheckpointReader.int8_params` reads."""
        t[prefix + "weight"] = w[lo:hi]
        if w.dtype != torch.int8:
            return
        scale = w.gv_scale[lo:hi]
        recip = getattr(w, "gv_in_scale_recip", None)
        if recip is None:
            t[prefix + "weight_scale"] = scale
            return
        t[prefix + "deq_scale"] = scale
        t[prefix + "input_scale"] = 1.0 / recip
        if getattr(w, "gv_in_offset", None) is not None:
            t[prefix + "input_offset"] = w.gv_in_offset
        if getattr(w, "gv_bias", None) is not None:
            t[prefix + "quant_bias"] = torch.round(w.gv_bias[lo:hi] / scale).to(torch.int32)

    def save_layer(i, L, moe):
        p = f"model.layers.{i}."
        if getattr(L, "norm_folded", False):    # norm weights folded into w_qkv / w_gate_up: undo
            from ..ops.decode_ops import unfolded_layer
            L = unfolded_layer(L)
        t[p + "input_layernorm.weight"] = nrm(L.attn_norm)
        t[p + "post_attention_layernorm.weight"] = nrm(L.mlp_norm)
        a = p + "self_attn."
        if cfg.layer_is_linear_attn(i):
            la = p + "linear_attn."
            kd = cfg.linear_num_key_heads * cfg.linear_key_head_dim
            vd = cfg.linear_num_value_heads * cfg.linear_value_head_dim
            Hv = cfg.linear_num_value_heads
            t[la + "in_proj_qkv.weight"] = L.w_in[: 2 * kd + vd]
            t[la + "in_proj_z.weight"] = L.w_in[2 * kd + vd: 2 * kd + 2 * vd]
            t[la + "in_proj_b.weight"] = L.w_in[2 * kd + 2 * vd: 2 * kd + 2 * vd + Hv]
            t[la + "in_proj_a.weight"] = L.w_in[2 * kd + 2 * vd + Hv:]
            t[la + "conv1d.weight"] = L.conv_w.unsqueeze(1)
            t[la + "A_log"], t[la + "dt_bias"] = L.A_log, L.dt_bias
            t[la + "norm.weight"] = L.gdn_norm
            t[la + "out_proj.weight"] = L.w_o
        elif cfg.attn_type in (AttnType.MLA, AttnType.DSA):
            dn, dr, dv, dc, ql = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim, cfg.kv_lora_rank, cfg.q_lora_rank
            if ql > 0:
                t[a + "q_a_proj.weight"] = L.w_qkv_a[:ql]
                t[a + "q_a_layernorm.weight"] = L.q_a_norm
                t[a + "q_b_proj.weight"] = L.w_q_b
            else:
                t[a + "q_proj.weight"] = L.w_q_b
            t[a + "kv_a_proj_with_mqa.weight"] = L.w_qkv_a[ql:]
            t[a + "kv_a_layernorm.weight"] = L.kv_a_norm
            t[a + "kv_b_proj.weight"] = torch.cat([L.w_uk_t.transpose(1, 2), L.w_uv], 1).reshape(nq * (dn + dv), dc)
            t[a + "o_proj.weight"] = L.w_o
        else:
            if cfg.attn_output_gate:
                qw, gw = L.w_qkv[: nq * hd], L.w_qkv[(nq + 2 * nkv) * hd:]
                t[a + "q_proj.weight"] = torch.stack([qw.view(nq, hd, -1), gw.view(nq, hd, -1)], 1).reshape(2 * nq * hd, -1)
                emit(a + "k_proj.", L.w_qkv, nq * hd, (nq + nkv) * hd)
                emit(a + "v_proj.", L.w_qkv, (nq + nkv) * hd, (nq + 2 * nkv) * hd)
            else:
                emit(a + "q_proj.", L.w_qkv, 0, nq * hd)
                emit(a + "k_proj.", L.w_qkv, nq * hd, (nq + nkv) * hd)
                emit(a + "v_proj.", L.w_qkv, (nq + nkv) * hd, (nq + 2 * nkv) * hd)
            if L.b_qkv is not None:
                t[a + "q_proj.bias"] = L.b_qkv[: nq * hd]
                t[a + "k_proj.bias"] = L.b_qkv[nq * hd:(nq + nkv) * hd]
                t[a + "v_proj.bias"] = L.b_qkv[(nq + nkv) * hd:]
            if L.q_norm is not None:
                t[a + "q_norm.weight"], t[a + "k_norm.weight"] = nrm(L.q_norm), nrm(L.k_norm)
            emit(a + "o_proj.", L.w_o, 0, L.w_o.shape[0])
        m = p + "mlp."
        if moe:
            t[m + "gate.weight"] = L.w_router
            if L.router_bias is not None:
                t[m + "gate.e_score_correction_bias"] = L.router_bias
            w13 = L.w13
            if getattr(L, "w13_il16", False):   # device layout [16 gate | 16 up] blocks -> HF order
                from ..ops.moe_ops import deinterleave16
                w13 = deinterleave16(w13)
            I = w13.shape[1] // 2
            for e in range(w13.shape[0]):
                t[f"{m}experts.{e}.gate_proj.weight"] = w13[e, :I]
                t[f"{m}experts.{e}.up_proj.weight"] = w13[e, I:]
                t[f"{m}experts.{e}.down_proj.weight"] = L.w2[e]
            if getattr(L, "ws_gate_up", None) is not None:
                Is = L.ws_gate_up.shape[0] // 2
                sp = m + ("shared_expert." if cfg.shared_expert_gate else "shared_experts.")
                t[sp + "gate_proj.weight"] = L.ws_gate_up[:Is]
                t[sp + "up_proj.weight"] = L.ws_gate_up[Is:]
                t[sp + "down_proj.weight"] = L.ws_down
                if getattr(L, "ws_gate", None) is not None:
                    t[m + "shared_expert_gate.weight"] = L.ws_gate
        else:
            gu = L.w_gate_up
            if getattr(L, "gu_il", False):      # device layout [64 gate | 64 up] blocks -> HF order
                from ..ops.functional import deinterleave_gate_up_rows
                gu = deinterleave_gate_up_rows(gu)
            wd = L.w_down
            if getattr(L, "gu_pad", 0):         # zero rows / columns added for the fused SwiGLU GEMM
                from ..ops.functional import unpad_gate_up_down
                gu, wd = unpad_gate_up_down(gu, wd, L.gu_pad)
            I = gu.shape[0] // 2
            emit(m + "gate_proj.", gu, 0, I)
            emit(m + "up_proj.", gu, I, 2 * I)
            emit(m + "down_proj.", wd, 0, wd.shape[0])

    for i, L in enumerate(weights.layers):
        save_layer(i, L, cfg.layer_is_moe(i))
    if mtp is not None:
        mp = f"model.layers.{cfg.num_layers}."
        save_layer(cfg.num_layers, mtp.layer, cfg.is_moe)
        t[mp + "enorm.weight"], t[mp + "hnorm.weight"] = nrm(mtp.enorm), nrm(mtp.hnorm)
        t[mp + "eh_proj.weight"] = mtp.eh_proj
        t[mp + "shared_head.norm.weight"] = nrm(mtp.shared_norm)
    names = sorted(t)
    index = {"metadata": {}, "weight_map": {}}
    for s in range(shards):
        part = {n: t[n].detach().cpu().contiguous() for n in names[s::shards]}
        fn = f"model-{s + 1:05d}-of-{shards:05d}.safetensors"
        save_file(part, os.path.join(path, fn))
        for n in part:
            index["weight_map"][n] = fn
    with open(os.path.join(path, "model.safetensors.index.json"), "w") as f:
        json.dump(index, f)
    hf = _hf_config(cfg)
    if any(v.dtype == torch.int8 for v in t.values()):
        hf["quantization_config"] = {"quant_method": "w8a8_int8"}
    if mtp is not None:
        hf["num_nextn_predict_layers"] = 1
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(hf, f)


def _hf_config(cfg: ModelConfig) -> dict:
    mt = "llama"
    if cfg.attn_type in (AttnType.MLA, AttnType.DSA):
        mt = "deepseek_v3"
    elif cfg.is_moe:
        mt = "qwen3_moe" if cfg.qk_norm else "qwen2_moe"
    elif cfg.qk_norm:
        mt = "qwen3"
    elif cfg.qkv_bias:
        mt = "qwen2"
    if cfg.full_attention_interval > 0:
        mt = "qwen3_5_moe" if cfg.is_moe else "qwen3_5"
    d = {"model_type": mt, "architectures": [mt], "vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
         "intermediate_size": cfg.intermediate_size, "num_hidden_layers": cfg.num_layers,
         "num_attention_heads": cfg.num_heads, "num_key_value_heads": cfg.num_kv_heads, "head_dim": cfg.head_dim,
         "rms_norm_eps": cfg.rms_norm_eps, "tie_word_embeddings": cfg.tie_word_embeddings,
         "rope_theta": cfg.rope_theta, "max_position_embeddings": cfg.max_position_embeddings,
         "rope_scaling": cfg.rope_scaling, "torch_dtype": cfg.dtype, "eos_token_id": 0}
    if cfg.is_moe:
        d.update({"num_experts" if mt != "deepseek_v3" else "n_routed_experts": cfg.num_experts,
                  "num_experts_per_tok": cfg.num_experts_per_tok, "moe_intermediate_size": cfg.moe_intermediate_size,
                  "n_shared_experts": cfg.num_shared_experts, "first_k_dense_replace": cfg.first_k_dense,
                  "norm_topk_prob": cfg.norm_topk_prob, "routed_scaling_factor": cfg.routed_scaling_factor,
                  "n_group": cfg.n_group, "topk_group": cfg.topk_group,
                  "scoring_func": "sigmoid" if int(cfg.scoring_func) == 1 else "softmax"})
    if cfg.shared_expert_gate:
        d["shared_expert_intermediate_size"] = cfg.num_shared_experts * cfg.moe_intermediate_size
    if cfg.rotary_dim and cfg.rotary_dim < cfg.head_dim:
        d["partial_rotary_factor"] = cfg.rotary_dim / cfg.head_dim
    if cfg.full_attention_interval > 0:
        d.update({"full_attention_interval": cfg.full_attention_interval,
                  "linear_num_key_heads": cfg.linear_num_key_heads, "linear_num_value_heads": cfg.linear_num_value_heads,
                  "linear_key_head_dim": cfg.linear_key_head_dim, "linear_value_head_dim": cfg.linear_value_head_dim,
                  "linear_conv_kernel_dim": cfg.linear_conv_kernel, "attn_output_gate": cfg.attn_output_gate})
    if mt == "deepseek_v3":
        d.update({"q_lora_rank": cfg.q_lora_rank or None, "kv_lora_rank": cfg.kv_lora_rank,
                  "qk_nope_head_dim": cfg.qk_nope_head_dim, "qk_rope_head_dim": cfg.qk_rope_head_dim,
                  "v_head_dim": cfg.v_head_dim})
    return d
