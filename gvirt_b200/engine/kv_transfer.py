"""KV connector: move a request together with its KV cache from one engine to another —
disaggregated prefill (one engine prefills, another decodes) and request migration.

The reference's serving integration lists "disaggregated prefill (non-layerwise KV connector)" and
"KV cache pool" among its features (xlite/doc/feature_matrix.md:12-35); the engine there only sees
block tables, the connector lives in the serving framework. Here the engine owns the blocks, so it
offers the two halves itself:

    payload = export_request(llm_a, req_id)           # after prefill: blocks -> contiguous tensors
    send_payload(payload, dst=1, group=g)              # optional: ship over torch.distributed
    rid = import_request(llm_b, payload)               # allocate blocks, scatter, join the decode batch

The transfer is non-layerwise: all layers of the request are gathered after the step that
produced its first token. Linear-attention layers carry their recurrent state instead of blocks.
Both engines must hold the same model with the same parallel layout (the payload holds this
rank's shard of every layer).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import torch

from .scheduler import Request, SamplingParams


@dataclass
class KVPayload:
    prompt: List[int]
    output: List[int]
    params: SamplingParams
    num_computed: int                          # tokens whose KV is in `layers`
    block_size: int
    layers: List[Tuple[torch.Tensor, ...]] = field(default_factory=list)
    # per layer: paged layers -> tensors [n_blocks, block, ...]; linear-attention layers -> state rows


def export_request(llm, req_id: int, release: bool = True) -> KVPayload:
    """Take a running request (between steps) out of `llm` with its KV. With release=True the
    request leaves the engine and its blocks are freed."""
    sch, runner, cfg = llm.scheduler, llm.runner, llm.cfg
    req = next((r for r in sch.running if r.req_id == req_id), None)
    if req is None:
        raise KeyError(f"request {req_id} is not running")
    if req.num_computed != req.total_len - 1 and req.num_computed != len(req.prompt):
        raise RuntimeError("export needs a request whose prefill is complete")
    blocks = list(sch.bm.block_table(req_id))
    need = (req.num_computed + cfg.block_size - 1) // cfg.block_size
    idx = torch.tensor(blocks[:need], dtype=torch.long, device=runner.device)
    layers = []
    for li, caches in enumerate(runner.kv_caches):
        if cfg.layer_is_linear_attn(li):
            layers.append(tuple(c[req.state_slot].clone() for c in caches))
        else:
            layers.append(tuple(c.index_select(0, idx) for c in caches))
    payload = KVPayload(list(req.prompt), list(req.output), req.params, req.num_computed, cfg.block_size, layers)
    if release:
        sch.abort(req)
        req.finished = False      # it lives on elsewhere
    return payload


def _check_payload(llm, payload: KVPayload, need: int) -> None:
    """Everything that can be wrong with a payload is found here, before a block is taken."""
    sch, runner, cfg = llm.scheduler, llm.runner, llm.cfg
    from .scheduler import validate_request
    total = len(payload.prompt) + len(payload.output)
    validate_request(list(payload.prompt), payload.params, cfg.max_seq_len, cfg.vocab_size)
    for t in payload.output:
        if not isinstance(t, int) or not 0 <= t < cfg.vocab_size:
            raise ValueError(f"output token id {t!r} is outside [0, {cfg.vocab_size})")
    if total > cfg.max_seq_len:
        raise ValueError(f"request of {total} tokens exceeds max_seq_len {cfg.max_seq_len}")
    if payload.num_computed != total - 1 and payload.num_computed != len(payload.prompt):
        raise ValueError(f"num_computed {payload.num_computed} does not match a request of {total} tokens")
    if len(payload.layers) != len(runner.kv_caches):
        raise ValueError(f"payload has {len(payload.layers)} layers, the engine {len(runner.kv_caches)}")
    for li, (caches, src) in enumerate(zip(runner.kv_caches, payload.layers)):
        if len(src) != len(caches):
            raise ValueError(f"layer {li}: payload has {len(src)} tensors, the engine {len(caches)}")
        linear = cfg.layer_is_linear_attn(li)
        for c, t in zip(caches, src):
            if not isinstance(t, torch.Tensor):
                raise ValueError(f"layer {li}: not a tensor")
            want = tuple(c.shape[1:]) if linear else (need,) + tuple(c.shape[1:])
            if tuple(t.shape) != want:
                raise ValueError(f"layer {li}: payload tensor {tuple(t.shape)}, expected {want}")
            if t.dtype != c.dtype:
                raise ValueError(f"layer {li}: payload dtype {t.dtype}, engine {c.dtype}")


def import_request(llm, payload: KVPayload) -> int:
    """Admit a request whose KV was computed elsewhere; it joins the next decode step. The payload
    is validated against this engine (lengths, layer count, tensor shapes and dtypes) before any
    block is allocated, and a failure after the allocation returns the blocks and the state slot."""
    sch, runner, cfg = llm.scheduler, llm.runner, llm.cfg
    if payload.block_size != cfg.block_size:
        raise ValueError(f"block size mismatch: payload {payload.block_size}, engine {cfg.block_size}")
    need = (payload.num_computed + cfg.block_size - 1) // cfg.block_size
    _check_payload(llm, payload, need)
    if len(sch.running) >= cfg.max_batch_size:
        raise RuntimeError("decode batch is full")
    if sch.uses_state_slots and not sch.free_state_slots:
        raise RuntimeError("no free recurrent-state slot for the imported request")
    rid = llm._next_id
    llm._next_id += 1
    req = Request(rid, list(payload.prompt), payload.params, output=list(payload.output))
    tokens = req.all_tokens
    if sch.bm.allocate(rid, tokens) < 0:
        raise RuntimeError("not enough free KV blocks for the imported request")
    try:
        blocks = list(sch.bm.block_table(rid))[:need]
        idx = torch.tensor(blocks, dtype=torch.long, device=runner.device)
        if sch.uses_state_slots:
            req.state_slot = sch.free_state_slots.pop()
        for li, (caches, src) in enumerate(zip(runner.kv_caches, payload.layers)):
            if cfg.layer_is_linear_attn(li):
                for c, t in zip(caches, src):
                    c[req.state_slot].copy_(t.to(c.device))
            else:
                for c, t in zip(caches, src):
                    c.index_copy_(0, idx, t.to(c.device, c.dtype))
    except BaseException:
        sch.bm.release(rid)
        sch._free_slot(req)
        raise
    req.num_computed = payload.num_computed
    import time
    req.arrival = time.perf_counter()
    if req.output:
        req.first_token_time = req.arrival
        req.token_times = [req.arrival] * len(req.output)
    sch.running.append(req)
    sch.epoch += 1
    return rid


# ---------------------------------------------------------------------------- transport
def send_payload(payload: KVPayload, dst: int, group=None) -> None:
    """Ship a payload to rank `dst`: metadata as an object, tensors with point-to-point sends."""
    import torch.distributed as dist
    meta = dict(prompt=payload.prompt, output=payload.output, params=payload.params,
                num_computed=payload.num_computed, block_size=payload.block_size,
                shapes=[[(tuple(t.shape), str(t.dtype).replace("torch.", "")) for t in ts] for ts in payload.layers])
    dist.send_object_list([meta], dst=dst, group=group)
    for ts in payload.layers:
        for t in ts:
            dist.send(t.contiguous(), dst=dst, group=group)


def recv_payload(src: int, device, group=None) -> KVPayload:
    import torch.distributed as dist
    box: List[Optional[dict]] = [None]
    dist.recv_object_list(box, src=src, group=group)
    meta = box[0]
    layers = []
    for ts in meta["shapes"]:
        got = []
        for shape, dt in ts:
            t = torch.empty(shape, dtype=getattr(torch, dt), device=device)
            dist.recv(t, src=src, group=group)
            got.append(t)
        layers.append(tuple(got))
    return KVPayload(meta["prompt"], meta["output"], meta["params"], meta["num_computed"], meta["block_size"],
                     layers)
