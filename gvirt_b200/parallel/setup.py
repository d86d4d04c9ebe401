"""One call that gives a CUDA process group its device-side communication: the symmetric heaps
(tensor-parallel and expert-parallel) and, for data-parallel attention + expert-parallel MoE, the
fused dispatch / combine exchange. The reference does the equivalent inside ``XRuntime::Init``
(IPC export of the tensor pool and flag pages, xlite/csrc/runtime.cpp:228-278, ccl.cpp:44-80).
"""
from __future__ import annotations

from ..config import ModelConfig, flags
from .moe_a2a import attach_moe_a2a
from .symm import attach_symmetric_heap


def heap_bytes(cfg: ModelConfig, world: int) -> int:
    """Tensor-parallel heap: fused GEMM + all-reduce receive regions (2 parities x R sources x 128
    tokens x hidden x 4 bytes, one per distinct row-parallel projection), the push collectives'
    regions (<= 1 MiB payloads) and, when sequence parallelism is on, its staging."""
    H = cfg.hidden_size
    gemm_ar = 4 * (2 * (world + 1) * 128 * H * 4)
    push = 6 * (2 * 16 * world * (1 << 17))
    sp = 0
    if cfg.max_num_batched_tokens >= flags().comm_optimize_len and world <= flags().sp_max_ranks:
        # GEMM -> reduce-scatter receive region and all-gather -> GEMM staging, each 2 parities x R
        # sources x rows-per-rank x H bf16 (the two projections of a kind share a region); the
        # widest activation that is gathered or scattered has H columns
        cap = sp_rows_per_rank(cfg, world)
        sp = 2 * (2 * world * cap * H * 2) + (8 << 20)
    return max(1 << 30, gemm_ar + push + sp + (64 << 20))


def sp_rows_per_rank(cfg: ModelConfig, world: int) -> int:
    """Token rows per rank that the sequence-parallel regions hold: one full step, padded to the
    128 * world rows the fused kernels work in."""
    return max(128, -(-cfg.max_num_batched_tokens // (128 * world)) * 128)


def a2a_bytes(cfg: ModelConfig, world: int, tokens_cap: int) -> int:
    """Expert-parallel heap for the fused MoE exchange (receive rows + return rows)."""
    from .moe_a2a import a2a_capacity
    H, K, E = cfg.hidden_size, cfg.num_experts_per_tok, max(cfg.num_experts, 1)
    e_local = max(E // world, 1)
    cap = a2a_capacity(cfg, world, tokens_cap)
    rows = e_local * cap
    return rows * (2 * H + 8 + (H // 128) * 4) + tokens_cap * K * H * 2 + (64 << 20)


def fit_step_to_exchange(cfg: ModelConfig, world: int, slices: int = 1) -> int:
    """Keep the fused MoE exchange exact: when the slot-addressed buffers behind the receive regions
    cannot hold the worst case of a full step (every token of every rank routed to one expert),
    shrink the step (`cfg.max_num_batched_tokens`: prefill chunks get smaller) until they can.
    `slices`: ranks that share one step's tokens (tensor-parallel attention: each dispatches
    1/slices of them; 1 with data-parallel attention). With
    GVIRT_ACTIVE_TOKENS_RATIO_PER_EP < 1 the caller has asked for the approximate mode and nothing
    is changed. Returns the step size in force."""
    from .moe_a2a import a2a_exact_tokens
    if flags().active_tokens_ratio_per_ep < 1.0:
        return cfg.max_num_batched_tokens
    per_rank = -(-cfg.max_num_batched_tokens // slices)
    exact = a2a_exact_tokens(cfg, world, per_rank)
    if exact < per_rank:
        step = exact * slices
        if step < cfg.max_batch_size:
            raise ValueError(f"the fused MoE exchange cannot hold a decode step of {cfg.max_batch_size} requests "
                             f"exactly ({step} tokens fit): raise GVIRT_A2A_SCRATCH_GB or lower max_batch_size")
        cfg.max_num_batched_tokens = max(step // 128 * 128, cfg.max_batch_size) if step >= 128 else step
    return cfg.max_num_batched_tokens


def attach_device_comm(ctx, cfg: ModelConfig) -> None:
    """No-op on CPU or a single process."""
    if ctx.device.type != "cuda" or ctx.world == 1:
        return
    ep_bytes = 0
    # the fused exchange serves data-parallel attention (every rank dispatches its own tokens) and,
    # on request (GVIRT_MOE_A2A_TP_SLICES), tensor-parallel attention over the same ranks as the
    # experts (every rank dispatches a 1/tp slice of the replicated tokens)
    sliced = ctx.dp == 1 and ctx.tp > 1 and ctx.ep == ctx.tp and flags().moe_a2a_tp_slices
    use_a2a = cfg.is_moe and ctx.ep > 1 and flags().moe_alltoall and (ctx.dp > 1 or sliced)
    tokens_cap = cfg.max_num_batched_tokens
    if use_a2a:
        fit_step_to_exchange(cfg, ctx.ep, ctx.tp if sliced else 1)
        tokens_cap = -(-cfg.max_num_batched_tokens // ctx.tp) if sliced else cfg.max_num_batched_tokens
        ep_bytes = a2a_bytes(cfg, ctx.ep, tokens_cap)
    attach_symmetric_heap(ctx, nbytes=heap_bytes(cfg, ctx.tp) if ctx.tp > 1 else 0, ep_nbytes=ep_bytes)
    if getattr(ctx, "symm", None) is not None:
        ctx.symm.sp_rows_cap = sp_rows_per_rank(cfg, ctx.tp)
    if ctx.tp > 1 and not flags().tp_pdl and not cfg.is_moe:
        # Across GPUs a kernel that starts before the one in front has drained shares SMs and HBM
        # with the fused GEMM + all-reduce, whose push phase every peer waits for: in the dense
        # decode loop (two such kernels among five per layer) the early starts cost more than they
        # hide. They still pay on one GPU and in MoE layers, whose many short kernels gain more.
        from .. import _native
        _native.kernels().gv_set_pdl(0)
    if use_a2a:
        attach_moe_a2a(ctx, cfg, tokens_cap=tokens_cap)
