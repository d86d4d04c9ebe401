"""Model / engine configuration and the environment-flag registry.

``ModelConfig`` is the flat description of a decoder the engine can run — the counterpart of
the reference's ``XModelConfig`` (xlite/csrc/model.h:22-96, mirrored 1:1 as the Python
``ModelConfig`` in xlite/csrc/_C.cpp:1924-1986): sizes, attention flavour (MHA / MLA / DSA /
hybrid linear attention), RoPE flavour, q/k-norm flavours, MoE routing, parallel sizes and
the serving limits fixed at init (max_seq_len, max_batch_size, max_num_batched_tokens,
block_size). ``from_hf`` fills it from a Hugging Face ``config.json``.

Environment flags follow the reference's grammar (xlite/doc/ENVIRONMENT_VARIABLES.md:7-16,
bool parsing xlite/csrc/base.h:181-207: true/1/yes/on) with the prefix ``GVIRT_``.
"""
from __future__ import annotations

import enum
import json
import os
from dataclasses import dataclass, field, asdict
from pathlib import Path
from typing import Any, Dict, List, Optional, Tuple


class AttnType(enum.IntEnum):
    MHA = 0      # multi-head / grouped-query attention
    MLA = 1      # multi-head latent attention (DeepSeek-V2/V3)
    DSA = 2      # MLA + lightning-indexer sparse attention (DeepSeek-V3.2 / GLM-5)
    HYBRID = 3   # interleaved full attention and gated-delta-net linear attention (Qwen3.5)


class ScoringFunc(enum.IntEnum):
    SOFTMAX = 0
    SIGMOID = 1


@dataclass
class ModelConfig:
    # ---- sizes
    name: str = "model"
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 32
    head_dim: int = 128
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = False
    dtype: str = "bfloat16"
    # ---- attention
    attn_type: AttnType = AttnType.MHA
    qkv_bias: bool = False
    qk_norm: bool = False             # per-head RMSNorm on q and k (Qwen3)
    qk_norm_full: bool = False        # RMSNorm over the full q / k width across TP (MiniMax-M2)
    attn_output_gate: bool = False    # out = attn * sigmoid(gate) (Qwen3.5 full-attention layers)
    # ---- RoPE
    rope_theta: float = 10000.0
    rotary_dim: Optional[int] = None  # partial rotary; None = head_dim
    rope_interleaved: bool = False    # adjacent-pair ("complex") rotation instead of NeoX halves
    rope_scaling: Optional[Dict[str, Any]] = None
    mrope_sections: Optional[Tuple[int, int, int]] = None
    mrope_interleaved: bool = False
    max_position_embeddings: int = 8192
    # ---- MLA
    q_lora_rank: int = 0
    kv_lora_rank: int = 0
    qk_nope_head_dim: int = 0
    qk_rope_head_dim: int = 0
    v_head_dim: int = 0
    # ---- DSA indexer
    index_n_heads: int = 0
    index_head_dim: int = 0
    index_topk: int = 0
    # ---- linear attention (gated delta net)
    full_attention_interval: int = 0  # every n-th layer is full attention; others linear
    linear_num_key_heads: int = 0
    linear_num_value_heads: int = 0
    linear_key_head_dim: int = 0
    linear_value_head_dim: int = 0
    linear_conv_kernel: int = 4
    # ---- MoE
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    num_shared_experts: int = 0
    norm_plus_one: bool = False       # checkpoint stores RMSNorm weights as w - 1 (Qwen3.5 / Qwen3-Next); folded at load
    shared_expert_gate: bool = False  # shared expert output scaled by sigmoid(h . w_gate) per token (Qwen3.5-MoE)
    first_k_dense: int = 0            # leading layers with a dense FFN
    scoring_func: ScoringFunc = ScoringFunc.SOFTMAX
    norm_topk_prob: bool = True
    routed_scaling_factor: float = 1.0
    n_group: int = 1
    topk_group: int = 1
    router_bias: bool = False         # e_score_correction_bias
    swiglu_clamp: float = 0.0
    # ---- quantisation
    quant: str = "none"               # none | fp8_block (e4m3, 128x128 weight blocks) | w8a8_int8
    # ---- parallel sizes
    tp_size: int = 1
    dp_size: int = 1
    ep_size: int = 1
    moe_tp_size: int = 1
    # ---- serving limits
    max_seq_len: int = 4096
    max_batch_size: int = 64
    max_num_batched_tokens: int = 8192
    block_size: int = 128

    # -- derived
    @property
    def rot_dim(self) -> int:
        if self.attn_type in (AttnType.MLA, AttnType.DSA):
            return self.qk_rope_head_dim
        return self.rotary_dim or self.head_dim

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    def layer_is_moe(self, i: int) -> bool:
        return self.is_moe and i >= self.first_k_dense

    def layer_is_linear_attn(self, i: int) -> bool:
        if self.attn_type != AttnType.HYBRID or self.full_attention_interval <= 0:
            return False
        return (i + 1) % self.full_attention_interval != 0

    @property
    def max_blocks_per_seq(self) -> int:
        return (self.max_seq_len + self.block_size - 1) // self.block_size

    def local_heads(self) -> Tuple[int, int]:
        """(q heads, kv heads) on one TP rank; kv heads are replicated when tp > num_kv_heads
        (xlite/csrc/model.cpp:490-499: max(n_kv / tp, 1))."""
        assert self.num_heads % self.tp_size == 0
        return self.num_heads // self.tp_size, max(self.num_kv_heads // self.tp_size, 1)

    def validate(self) -> None:
        if self.num_heads % self.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if self.num_heads % self.tp_size:
            raise ValueError("num_heads must be divisible by tp_size")
        if self.tp_size > self.num_kv_heads and self.tp_size % self.num_kv_heads:
            raise ValueError("tp_size must be a multiple of num_kv_heads when larger")
        if self.is_moe:
            if self.num_experts % self.ep_size:
                raise ValueError("num_experts must be divisible by ep_size")
            if self.num_experts_per_tok <= 0:
                raise ValueError("MoE needs num_experts_per_tok > 0")
            if self.n_group > 1 and self.num_experts % self.n_group:
                raise ValueError("num_experts must be divisible by n_group")
        if self.max_num_batched_tokens < self.max_batch_size:
            raise ValueError("max_num_batched_tokens must be >= max_batch_size")

    def to_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        d["attn_type"] = int(self.attn_type)
        d["scoring_func"] = int(self.scoring_func)
        return d

    # -- Hugging Face config.json
    @classmethod
    def from_hf(cls, hf: Dict[str, Any], **overrides) -> "ModelConfig":
        arch = (hf.get("architectures") or [hf.get("model_type", "")])[0].lower()
        mt = hf.get("model_type", "").lower()
        text = hf.get("text_config", hf)
        g = text.get
        heads = g("num_attention_heads", 32)
        hidden = g("hidden_size", 4096)
        c = cls(
            name=mt or arch,
            vocab_size=g("vocab_size", 32000),
            hidden_size=hidden,
            intermediate_size=g("intermediate_size", 4 * hidden),
            num_layers=g("num_hidden_layers", 32),
            num_heads=heads,
            num_kv_heads=g("num_key_value_heads", heads) or heads,
            head_dim=g("head_dim") or hidden // heads,
            rms_norm_eps=g("rms_norm_eps", 1e-6),
            tie_word_embeddings=bool(g("tie_word_embeddings", False)),
            rope_theta=float(g("rope_theta", 10000.0)),
            max_position_embeddings=g("max_position_embeddings", 8192),
            rope_scaling=g("rope_scaling"),
        )
        prf = g("partial_rotary_factor")
        if prf and prf < 1.0:
            c.rotary_dim = int(c.head_dim * prf)
        if "qwen2" in mt and "moe" not in mt:
            c.qkv_bias = True
        if mt in ("qwen3", "qwen3_moe") or mt.startswith(("qwen3_next", "qwen3_5")):
            c.qk_norm = True
        if mt.startswith(("qwen3_next", "qwen3_5")):
            c.norm_plus_one = True
        if g("attention_bias") and "qwen" not in mt:
            c.qkv_bias = True
        if g("use_qk_norm"):
            c.qk_norm = True
        # MoE
        ne = g("num_experts") or g("n_routed_experts") or g("num_local_experts") or 0
        if ne:
            c.num_experts = ne
            c.num_experts_per_tok = g("num_experts_per_tok", 8)
            c.moe_intermediate_size = g("moe_intermediate_size", c.intermediate_size)
            c.num_shared_experts = g("n_shared_experts", 0) or 0
            if g("shared_expert_intermediate_size"):
                # Qwen-MoE naming: one gated shared expert of its own width
                c.num_shared_experts = max(1, int(g("shared_expert_intermediate_size")) // max(c.moe_intermediate_size, 1))
                c.shared_expert_gate = True
            c.first_k_dense = g("first_k_dense_replace", 0) or 0
            c.norm_topk_prob = bool(g("norm_topk_prob", True))
            c.routed_scaling_factor = float(g("routed_scaling_factor", 1.0) or 1.0)
            c.n_group = g("n_group", 1) or 1
            c.topk_group = g("topk_group", 1) or 1
            if g("scoring_func", "softmax") == "sigmoid" or mt in ("deepseek_v3", "glm4_moe", "minimax_m2"):
                c.scoring_func = ScoringFunc.SIGMOID
                c.router_bias = True
        # MLA
        if g("kv_lora_rank"):
            c.attn_type = AttnType.MLA
            c.q_lora_rank = g("q_lora_rank", 0) or 0
            c.kv_lora_rank = g("kv_lora_rank")
            c.qk_nope_head_dim = g("qk_nope_head_dim", 128)
            c.qk_rope_head_dim = g("qk_rope_head_dim", 64)
            c.v_head_dim = g("v_head_dim", 128)
            c.head_dim = c.qk_nope_head_dim + c.qk_rope_head_dim
            c.rope_interleaved = True
            if g("index_topk"):
                c.attn_type = AttnType.DSA
                c.index_topk = g("index_topk")
                c.index_n_heads = g("index_n_heads", 64)
                c.index_head_dim = g("index_head_dim", 128)
        if mt == "minimax_m2":
            c.qk_norm_full = True
        qc = g("quantization_config") or {}
        if qc.get("quant_method") == "fp8" and qc.get("weight_block_size"):
            c.quant = "fp8_block"
        if qc.get("quant_method") in ("w8a8_int8", "w8a8", "int8"):
            c.quant = "w8a8_int8"
        # hybrid linear attention
        if g("full_attention_interval"):
            c.attn_type = AttnType.HYBRID
            c.full_attention_interval = g("full_attention_interval")
            c.linear_num_key_heads = g("linear_num_key_heads", 16)
            c.linear_num_value_heads = g("linear_num_value_heads", 32)
            c.linear_key_head_dim = g("linear_key_head_dim", 128)
            c.linear_value_head_dim = g("linear_value_head_dim", 128)
            c.linear_conv_kernel = g("linear_conv_kernel_dim", 4)
            c.attn_output_gate = bool(g("attn_output_gate", True))
        rs = g("rope_scaling") or {}
        if rs.get("mrope_section"):
            sec = list(rs["mrope_section"]) + [0, 0, 0]
            c.mrope_sections = (sec[0], sec[1], sec[2])
            c.mrope_interleaved = bool(rs.get("mrope_interleaved", False))
        for k, v in overrides.items():
            setattr(c, k, v)
        return c

    @classmethod
    def from_pretrained(cls, path: str, **overrides) -> "ModelConfig":
        with open(Path(path) / "config.json") as f:
            return cls.from_hf(json.load(f), **overrides)


# --------------------------------------------------------------------------- env flags
def parse_bool(s: Optional[str], default: bool = False) -> bool:
    if s is None:
        return default
    v = s.strip().lower()
    if v in ("true", "1", "yes", "on"):
        return True
    if v in ("false", "0", "no", "off"):
        return False
    return default


@dataclass
class EnvFlags:
    """Run-time knobs read once from the environment (all optional)."""
    devs_per_node: int = 8               # GVIRT_DEVS_PER_NODE
    node_ips: List[str] = field(default_factory=list)  # GVIRT_NODE_IPS (comma separated)
    port: int = 10266                    # GVIRT_PORT (base port of the TCP bootstrap)
    comm_optimize_len: int = 6144        # GVIRT_COMM_OPTIMIZE_LEN: tokens from which the
    #                                      sequence-parallel RS/AG residual path replaces AR
    disable_symm: bool = False           # GVIRT_DISABLE_SYMM: use NCCL instead of own collectives
    enable_graph: bool = True            # GVIRT_ENABLE_GRAPH: CUDA-graph decode buckets
    moe_alltoall: bool = True            # GVIRT_MOE_ALLTOALL: fused dispatch/combine vs AG/RS
    moe_a2a_tp_slices: bool = False      # GVIRT_MOE_A2A_TP_SLICES: with tensor-parallel attention, run the
                                         # dispatch/combine exchange on 1/tp token slices instead of
                                         # local experts + all-reduce (measured slower at EP2: the
                                         # replicated tokens need no dispatch, and K rows travel per token)
    active_tokens_ratio_per_ep: float = 1.0  # GVIRT_ACTIVE_TOKENS_RATIO_PER_EP: receive-region
    #                                      size as a fraction of the worst case tokens * top_k
    deterministic: bool = True           # GVIRT_DETERMINISTIC: fixed-order reductions
    debug_on: str = ""                   # GVIRT_DEBUG_ON: forward,tuner,gettensor,misc,base,comm,all
    paranoid: bool = False               # GVIRT_PARANOID: census every op output for NaN/Inf
    paranoid_ops: bool = False           # GVIRT_PARANOID_OPS: every op call is compared with its CPU definition
    fuse_swiglu: bool = True             # GVIRT_FUSE_SWIGLU: SwiGLU in the gate/up GEMM epilogue
    decode_l2_prefetch: bool = False     # GVIRT_DECODE_L2_PREFETCH: a decode GEMM warms L2 with the next GEMM's first
                                         # tiles (measured: +3.6 us per Llama-3-8B layer at TP1, so off)
    vocab_parallel_greedy: bool = True   # GVIRT_VOCAB_PARALLEL_GREEDY: all-greedy steps under TP pick the best
                                         # token per vocabulary shard and all-gather (score, id) pairs
                                         # instead of the logits
    tp_pdl: bool = False                 # GVIRT_TP_PDL: keep programmatic dependent launch on for dense models
                                         # under tensor parallelism (measured slower across GPUs: Llama-3-8B
                                         # TP4 16.5 k tok/s with it, 21.5 k without; MoE models keep it on:
                                         # Qwen3-30B-A3B on 4 GPUs 14.9 k with, 14.4 k without)
    fused_ar_residual: bool = True       # GVIRT_FUSED_AR_RESIDUAL: under TP the fused GEMM + all-reduce also adds the
                                         # residual and emits the RMSNorm sums of squares (false: a small kernel behind it)
    prefill_attn_tc: bool = True         # GVIRT_PREFILL_ATTN_TC: tcgen05 flash attention for 128-wide heads
    dsa_indexer_tc: bool = True          # GVIRT_DSA_INDEXER_TC: tcgen05 lightning-indexer scores (head_dim 128)
    mla_attn_tc: bool = True             # GVIRT_MLA_ATTN_TC: tcgen05 absorbed MLA decode (128 local heads)
    fused_decode: bool = True            # GVIRT_FUSED_DECODE: dense layers at <= 128 tokens run norm, RoPE + cache
                                         # write and residual add inside the GEMM epilogues (norm weights folded)
    pad_swiglu: bool = True              # GVIRT_PAD_SWIGLU: zero-pad a local intermediate size to a multiple of 64 for it
    a2a_scratch_gb: float = 16.0         # GVIRT_A2A_SCRATCH_GB: cap on the slot-addressed MoE exchange buffers
    async_scheduling: bool = True        # GVIRT_ASYNC_SCHEDULING: prepare step k + 1 on the host during step k
    symm_max_bytes: int = 8 << 20        # GVIRT_SYMM_MAX_BYTES: largest payload of the own collectives
    sp_max_ranks: int = 8                # GVIRT_SP_MAX_RANKS: sequence-parallel layer loop up to this TP size
    prefill_gemm_persistent: int = 3     # GVIRT_PREFILL_GEMM_PERSISTENT: GEMMs with >= 1024 rows through a persistent
                                         # kernel with a double-buffered accumulator: 0 = never, 1 = the grouped kernel
                                         # with one segment (128 x 128 tiles, bias-free only), 2 = token-major 128 x 256
                                         # tiles always, 3 = token-major 128 x 256 tiles for outputs up to 8192 wide
    nvtx: bool = False                   # GVIRT_NVTX: an NVTX range around every kernel launcher call and engine step
    cpu_binding: bool = False            # GVIRT_CPU_BINDING: pin each rank to the host cores next to its GPU
    mixed_batches: bool = False          # GVIRT_MIXED_BATCHES: decoding requests ride along with prefill chunks
    dual_stream_prefill: bool = False    # GVIRT_DUAL_STREAM_PREFILL: two micro-batches on two streams (TP > 1)
    dual_stream_min_tokens: int = 2048   # GVIRT_DUAL_STREAM_MIN_TOKENS: smallest prefill step that is split

    @classmethod
    def from_env(cls, env=None) -> "EnvFlags":
        e = os.environ if env is None else env
        f = cls()
        f.devs_per_node = int(e.get("GVIRT_DEVS_PER_NODE", f.devs_per_node))
        ips = e.get("GVIRT_NODE_IPS", "")
        f.node_ips = [x.strip() for x in ips.split(",") if x.strip()]
        f.port = int(e.get("GVIRT_PORT", f.port))
        f.comm_optimize_len = int(e.get("GVIRT_COMM_OPTIMIZE_LEN", f.comm_optimize_len))
        f.disable_symm = parse_bool(e.get("GVIRT_DISABLE_SYMM"), f.disable_symm)
        f.enable_graph = parse_bool(e.get("GVIRT_ENABLE_GRAPH"), f.enable_graph)
        f.moe_alltoall = parse_bool(e.get("GVIRT_MOE_ALLTOALL"), f.moe_alltoall)
        f.moe_a2a_tp_slices = parse_bool(e.get("GVIRT_MOE_A2A_TP_SLICES"), f.moe_a2a_tp_slices)
        f.active_tokens_ratio_per_ep = float(e.get("GVIRT_ACTIVE_TOKENS_RATIO_PER_EP",
                                                   f.active_tokens_ratio_per_ep))
        f.deterministic = parse_bool(e.get("GVIRT_DETERMINISTIC"), f.deterministic)
        f.debug_on = e.get("GVIRT_DEBUG_ON", "")
        f.paranoid = parse_bool(e.get("GVIRT_PARANOID"), f.paranoid)
        f.paranoid_ops = parse_bool(e.get("GVIRT_PARANOID_OPS"), f.paranoid_ops)
        f.fuse_swiglu = parse_bool(e.get("GVIRT_FUSE_SWIGLU"), f.fuse_swiglu)
        f.fused_decode = parse_bool(e.get("GVIRT_FUSED_DECODE"), f.fused_decode)
        f.prefill_attn_tc = parse_bool(e.get("GVIRT_PREFILL_ATTN_TC"), f.prefill_attn_tc)
        f.fused_ar_residual = parse_bool(e.get("GVIRT_FUSED_AR_RESIDUAL"), f.fused_ar_residual)
        f.tp_pdl = parse_bool(e.get("GVIRT_TP_PDL"), f.tp_pdl)
        f.vocab_parallel_greedy = parse_bool(e.get("GVIRT_VOCAB_PARALLEL_GREEDY"), f.vocab_parallel_greedy)
        f.decode_l2_prefetch = parse_bool(e.get("GVIRT_DECODE_L2_PREFETCH"), f.decode_l2_prefetch)
        f.mla_attn_tc = parse_bool(e.get("GVIRT_MLA_ATTN_TC"), f.mla_attn_tc)
        f.dsa_indexer_tc = parse_bool(e.get("GVIRT_DSA_INDEXER_TC"), f.dsa_indexer_tc)
        f.pad_swiglu = parse_bool(e.get("GVIRT_PAD_SWIGLU"), f.pad_swiglu)
        f.a2a_scratch_gb = float(e.get("GVIRT_A2A_SCRATCH_GB", f.a2a_scratch_gb))
        f.async_scheduling = parse_bool(e.get("GVIRT_ASYNC_SCHEDULING"), f.async_scheduling)
        f.symm_max_bytes = int(e.get("GVIRT_SYMM_MAX_BYTES", f.symm_max_bytes))
        f.sp_max_ranks = int(e.get("GVIRT_SP_MAX_RANKS", f.sp_max_ranks))
        v = (e.get("GVIRT_PREFILL_GEMM_PERSISTENT") or "").strip().lower()
        if v:
            f.prefill_gemm_persistent = int(v) if v.isdigit() else int(parse_bool(v, False))
        f.nvtx = parse_bool(e.get("GVIRT_NVTX"), f.nvtx)
        f.cpu_binding = parse_bool(e.get("GVIRT_CPU_BINDING"), f.cpu_binding)
        f.mixed_batches = parse_bool(e.get("GVIRT_MIXED_BATCHES"), f.mixed_batches)
        f.dual_stream_prefill = parse_bool(e.get("GVIRT_DUAL_STREAM_PREFILL"), f.dual_stream_prefill)
        f.dual_stream_min_tokens = int(e.get("GVIRT_DUAL_STREAM_MIN_TOKENS", f.dual_stream_min_tokens))
        return f


_FLAGS: Optional[EnvFlags] = None


def flags() -> EnvFlags:
    global _FLAGS
    if _FLAGS is None:
        _FLAGS = EnvFlags.from_env()
    return _FLAGS


def reload_flags(env=None) -> EnvFlags:
    global _FLAGS
    _FLAGS = EnvFlags.from_env(env)
    return _FLAGS
