"""Model runner: owns the weights' forward graph, the paged KV cache, the activation arena, the
per-step metadata staging buffers and the CUDA graphs of the decode buckets.

One ``execute`` call is one engine step, the unit the reference exposes as
``Model.forward`` + ``Model.forward_get_logits`` (xlite/csrc/_C.cpp:604-664,
xlite/tests/models/llama.py:359-365) — plus sampling, which the reference leaves to Python.
Per step the host does: build the attention metadata into one pinned blob (C++), copy token
ids + blob to the device (2 async H2D copies), launch (eager for prefill; a graph replay for
decode), and read back the sampled token ids (1 D2H copy). There is no other host<->device
synchronisation inside a step.

Decode steps are captured once per batch bucket (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, ...):
all tensors a captured step touches live at fixed addresses (arena, staging blob, token
buffers), padding requests have seq_len 0 / slot -1.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from .. import _native
from ..config import AttnType, ModelConfig, flags
from ..models.transformer import Transformer
from ..ops import functional as F
from .arena import Arena, TorchWorkspace

DEFAULT_BUCKETS = (1, 2, 4, 8, 12, 16, 24, 32, 48, 64, 96, 128, 192, 256, 384, 512)


@dataclass
class StepInput:
    tokens: List[int]                 # flat new token ids of all requests
    lens: List[int]                   # new tokens per request
    cached_lens: List[int]            # tokens already in the KV cache per request
    block_tables: List[List[int]]     # physical block ids per request
    temperature: Optional[List[float]] = None
    top_k: Optional[List[int]] = None
    top_p: Optional[List[float]] = None
    sample: bool = True               # False: run the step for its KV side effect only (chunk)
    all_logits: bool = False          # sample at every input row, not only each request's last one
                                      # (verification step of speculative decoding; greedy only)
    logprobs: int = 0                 # N > 0: also return log-probabilities (chosen token + N most likely)
    penalties: Optional[dict] = None  # presence / frequency / repetition adjustments (Scheduler._penalties)
    state_slots: Optional[List[int]] = None  # per request: recurrent-state slot (linear attention)
    step_id: int = 0
    # multimodal (see scheduler.MultiModalInputs); all optional
    mm_rows: Optional[List[int]] = None       # rows of the flat token dimension whose embedding is given
    mm_embeds: Optional[torch.Tensor] = None  # [len(mm_rows), hidden]
    mm_deepstack: Optional[List[torch.Tensor]] = None   # per early layer: [len(mm_rows), hidden]
    positions3: Optional[torch.Tensor] = None  # int64 [3, tokens]: explicit M-RoPE positions (prefill)
    pos_delta: Optional[List[int]] = None      # decode: per request offset added to the position


class ModelRunner:
    def __init__(self, model: Transformer, num_blocks: int, seed: int = 0,
                 use_graphs: Optional[bool] = None, use_arena: bool = True,
                 buckets: Sequence[int] = DEFAULT_BUCKETS, logit_rows: int = 0,
                 dual_stream: Optional[bool] = None):
        """`logit_rows`: the largest number of rows a step may ask logits for (0 = one per
        request); verification steps of speculative decoding sample at every input row.
        `dual_stream`: run large prefill steps as two micro-batches on two streams (default:
        GVIRT_DUAL_STREAM_PREFILL; collective over the world when it creates communicators)."""
        self.model = model
        self.cfg: ModelConfig = model.cfg
        self.ctx = model.ctx
        self.device = model.device
        self.cuda = self.device.type == "cuda"
        self.num_blocks = num_blocks
        self.seed = seed
        self.rt = _native.runtime()
        self.kv_caches = model.alloc_kv_cache(num_blocks)
        cfg = self.cfg
        self.use_graphs = (flags().enable_graph if use_graphs is None else use_graphs) and self.cuda
        self.buckets = tuple(b for b in buckets if b <= cfg.max_batch_size)
        if not self.buckets or self.buckets[-1] < cfg.max_batch_size:
            self.buckets = self.buckets + (cfg.max_batch_size,)
        # ---- staging: one layout sized for the largest step
        self.layout = self.rt.attn_meta_layout(cfg.max_batch_size, cfg.max_num_batched_tokens,
                                               cfg.max_blocks_per_seq)
        nbytes = self.layout.total_bytes
        # two pinned copies: the next step's metadata can be built while the previous step's copy
        # may still be in flight (see `stage`)
        self.host_blobs = [torch.empty(nbytes, dtype=torch.uint8, pin_memory=self.cuda) for _ in range(2)]
        self._blob_idx = 0
        self.host_blob = self.host_blobs[0]
        self.dev_blob = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.host_tokens = torch.empty(cfg.max_num_batched_tokens, dtype=torch.int32, pin_memory=self.cuda)
        self.dev_tokens = torch.zeros(cfg.max_num_batched_tokens, dtype=torch.int32, device=self.device)
        self.host_samp = torch.zeros(3, cfg.max_batch_size, dtype=torch.float32, pin_memory=self.cuda)
        self.dev_samp = torch.zeros(3, cfg.max_batch_size, dtype=torch.float32, device=self.device)
        self.dev_topk = torch.zeros(cfg.max_batch_size, dtype=torch.int32, device=self.device)
        self.logit_rows = min(max(logit_rows, cfg.max_batch_size), max(cfg.max_num_batched_tokens, cfg.max_batch_size))
        self.dev_out = torch.zeros(self.logit_rows, dtype=torch.int32, device=self.device)
        self.dev_all_rows = torch.arange(self.logit_rows, dtype=torch.int32, device=self.device)
        self.dev_step = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.dev_state_slots = torch.full((cfg.max_batch_size,), cfg.max_batch_size, dtype=torch.int32,
                                          device=self.device)  # padding requests use the spare slot
        self.host_out = torch.zeros(self.logit_rows, dtype=torch.int32, pin_memory=self.cuda)
        self._views = self._make_views(self.dev_blob)
        # ---- arena sized by dry runs of the largest prefill and the largest decode
        self.arena = None
        if use_arena:
            need = max(self.dry_run_bytes(cfg.max_num_batched_tokens, cfg.max_batch_size),
                       self.dry_run_bytes(cfg.max_batch_size, cfg.max_batch_size))
            if self.logit_rows > cfg.max_batch_size:
                need = max(need, self.dry_run_bytes(self.logit_rows, cfg.max_batch_size, self.logit_rows))
            self.arena_bytes = need
            self.arena = Arena(need, device=self.device)
        self.ws = self.arena if self.arena is not None else TorchWorkspace(self.device)
        # split-KV scratch for decode (sized for the worst bucket)
        self.max_splits = 32
        nq = model.nq
        if cfg.attn_type in (AttnType.MHA, AttnType.HYBRID) and self.cuda:
            self.split_o = torch.empty(cfg.max_batch_size * nq * self.max_splits * cfg.head_dim,
                                       dtype=torch.float32, device=self.device)
            self.split_lse = torch.empty(cfg.max_batch_size * nq * self.max_splits, dtype=torch.float32,
                                         device=self.device)
        else:
            self.split_o = self.split_lse = None
        self.graphs: Dict[tuple, torch.cuda.CUDAGraph] = {}
        self.graph_launches: Dict[tuple, int] = {}
        self._graph_addrs: Dict[tuple, tuple] = {}
        self.last_graph_key = None
        self.launch_count = 0
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.num_sms = torch.cuda.get_device_properties(self.device).multi_processor_count if self.cuda else 148
        # ---- dual-stream prefill: second metadata blob, second arena (made on first use), side stream
        self.dual_stream = flags().dual_stream_prefill if dual_stream is None else dual_stream
        self.dual_stream = bool(self.dual_stream) and self.ctx.dp == 1 and cfg.full_attention_interval == 0
        self.dual_min_tokens = flags().dual_stream_min_tokens
        self.dual_steps = 0
        self._side = None
        from ..utils import debug as _dbg
        self._dbg_tuner = _dbg.enabled("tuner")
        self.hold_hidden = False      # set by a draft head (engine/mtp.py)
        self._held = None
        self._lp_dev = None           # device tensors of the last step's log-probabilities
        self.last_logprobs = None     # ... as host lists, after `collect`
        if self.dual_stream:
            self.ctx.make_side_groups()
            self.dev_blob_b = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
            self._views_b = self._make_views(self.dev_blob_b)
            self.ws_b = None

    # ------------------------------------------------------------------ sizing
    def dry_run_bytes(self, tokens: int, batch: int, logit_rows: int = 0) -> int:
        """Arena bytes needed by a step of `tokens` new tokens over `batch` requests that asks
        for logits at `logit_rows` rows (default: one per request)."""
        arena = Arena(dry_run=True)
        cfg = self.cfg
        meta = F.AttnMeta(*(torch.empty(0, device="meta") for _ in range(7)), batch=batch,
                          num_tokens=tokens, max_q_len=tokens, max_seq_len=cfg.max_seq_len,
                          decode_step=(tokens == batch and not logit_rows), block_size=cfg.block_size)
        meta.last_token_idx = torch.empty(max(batch, logit_rows), dtype=torch.int32, device="meta")
        meta.extra["state_slots"] = torch.empty(batch, dtype=torch.int32, device="meta")
        toks = torch.empty(tokens, dtype=torch.int32, device="meta")
        kv = [tuple(torch.empty(0, device="meta") for _ in c) for c in self.kv_caches]
        h = self.model.forward(toks, meta, kv, arena)
        logits = self.model.compute_logits(h, meta, arena, batch=logit_rows or batch)
        return arena.high_water + (1 << 20)

    # ------------------------------------------------------------------ metadata
    def _make_views(self, blob: torch.Tensor):
        L = self.layout

        def v(off, n, dtype):
            sz = torch.tensor([], dtype=dtype).element_size()
            return blob[off: off + n * sz].view(dtype)

        return dict(
            query_start_loc=v(L.query_start_loc, L.batch_cap + 1, torch.int32),
            cached_lens=v(L.cached_lens, L.batch_cap, torch.int32),
            seq_lens=v(L.seq_lens, L.batch_cap, torch.int32),
            last_token_idx=v(L.last_token_idx, L.batch_cap, torch.int32),
            slot_mapping=v(L.slot_mapping, L.token_cap, torch.int32),
            block_tables=v(L.block_tables, L.batch_cap * L.max_blocks, torch.int32).view(L.batch_cap, L.max_blocks),
            positions=v(L.positions, L.token_cap, torch.int64),
        )

    def _meta(self, info, batch_rows: int, num_splits: int = 1, views=None) -> F.AttnMeta:
        vw = views or self._views
        m = F.AttnMeta(vw["query_start_loc"], vw["cached_lens"][:batch_rows], vw["seq_lens"][:batch_rows],
                       vw["last_token_idx"], vw["slot_mapping"], vw["block_tables"][:batch_rows],
                       vw["positions"], batch=info.batch if not isinstance(info, dict) else info["batch"],
                       num_tokens=info.num_tokens if not isinstance(info, dict) else info["num_tokens"],
                       max_q_len=info.max_q_len if not isinstance(info, dict) else info["max_q_len"],
                       max_seq_len=info.max_seq_len if not isinstance(info, dict) else info["max_seq_len"],
                       decode_step=info.decode_step if not isinstance(info, dict) else info["decode_step"],
                       block_size=self.cfg.block_size, num_splits=num_splits)
        if num_splits > 1:
            m.split_scratch = (self.split_o, self.split_lse)
        m.extra["state_slots"] = self.dev_state_slots
        return m

    def _bucket(self, batch: int) -> int:
        for b in self.buckets:
            if b >= batch:
                return b
        return self.cfg.max_batch_size

    def _pick_splits(self, batch: int, max_len: int) -> int:
        ns = self._pick_splits_quiet(batch, max_len)
        if self._dbg_tuner:
            from ..utils import debug as dbg
            dbg.log("tuner", f"decode batch {batch} max_len {max_len} sms {self.num_sms}: {ns} KV split(s)")
        return ns

    def _pick_splits_quiet(self, batch: int, max_len: int) -> int:
        if not self.cuda:
            return 1
        if self.cfg.attn_type in (AttnType.MLA, AttnType.DSA):
            hl = self.cfg.num_heads // self.cfg.tp_size
            if (self.cfg.attn_type == AttnType.MLA and hl % 128 == 0 and self.cfg.kv_lora_rank == 512
                    and self.cfg.qk_rope_head_dim == 64 and self.cfg.block_size % 32 == 0
                    and flags().mla_attn_tc):
                # tcgen05 kernel: one CTA per (request, 128 heads, output half, split), one CTA per
                # SM: as many splits as fill one wave, each at least 512 keys long
                tasks = max(1, batch * 2 * (hl // 128))
                return max(1, min(8, self.num_sms // tasks, max(max_len, 1) // 512))
            # the mma.sync kernel runs one CTA per (token, group of 32 heads, split)
            groups = max(1, (hl + 31) // 32)
            c = self.rt.pick_decode_splits(batch, groups, max(max_len, 1), self.num_sms, 1, 8)
            return max(1, c.splits)
        c = self.rt.pick_decode_splits(batch, self.model.nkv, max(max_len, 1), self.num_sms, 1,
                                       self.max_splits)
        return max(1, c.splits)

    # ------------------------------------------------------------------ the step
    def _forward_and_sample(self, ntok: int, meta: F.AttnMeta, rows: int, want_sample: bool,
                            stochastic: bool, step_id: int, mm=None, logprobs: int = 0, penalties=None):
        toks = self.dev_tokens[:ntok]
        h = self.model.forward(toks, meta, self.kv_caches, self.ws, mm_override=mm)
        if (want_sample and not stochastic and penalties is None and logprobs == 0 and self.model.ctx.tp > 1
                and flags().vocab_parallel_greedy and hasattr(self.model, "greedy_tokens")):
            # all-greedy step under tensor parallelism: pick the token per vocabulary shard
            self.dev_out[:rows].copy_(self.model.greedy_tokens(h, meta, self.ws, batch=rows))
        elif want_sample:
            logits = self.model.compute_logits(h, meta, self.ws, batch=rows)
            if penalties is not None:
                self._apply_penalties(logits, penalties)
            if stochastic:
                F_out = F.sample(logits, self.dev_samp[0, :rows], self.dev_topk[:rows],
                                 self.dev_samp[2, :rows], seed=self.seed, step=step_id,
                                 step_tensor=self.dev_step if self.cuda else None)
            else:
                F_out = F.sample(logits)
            self.dev_out[:rows].copy_(F_out)
            if logprobs > 0:
                # eager steps only (never captured): a handful of library element-wise ops
                lp = torch.log_softmax(logits.float(), dim=-1)
                chosen = lp.gather(1, self.dev_out[:rows].long().unsqueeze(1)).squeeze(1)
                topv, topi = lp.topk(min(logprobs, lp.shape[-1]), dim=-1)
                self._lp_dev = (chosen, topv, topi)
            if getattr(logits, "_gv_off", None) is not None:
                self.ws.put(logits)
        if self.hold_hidden:
            # a draft head reads this step's hidden states after sampling; returned to the arena
            # at the start of the next launch
            self._held = (h, meta, ntok)
        else:
            self.ws.put(h)

    def _apply_penalties(self, logits: torch.Tensor, pen: dict) -> None:
        """Adjust the step's logits in place (eager steps only): repetition penalty on tokens seen
        in prompt or output, then `frequency * count + presence` off the generated tokens."""
        dev = logits.device
        n = len(pen["presence"])

        def col(x, dt):
            return torch.tensor(x, dtype=dt, device=dev)

        if pen["rep_rows"]:
            r, t = col(pen["rep_rows"], torch.long), col(pen["rep_toks"], torch.long)
            rep = col(pen["repetition"], torch.float32)[r]
            v = logits[r, t].float()
            logits[r, t] = torch.where(v > 0, v / rep, v * rep).to(logits.dtype)
        if pen["rows"]:
            r, t = col(pen["rows"], torch.long), col(pen["toks"], torch.long)
            off = col(pen["frequency"], torch.float32)[r] * col(pen["counts"], torch.float32) \
                + col(pen["presence"], torch.float32)[r]
            logits[r, t] = (logits[r, t].float() - off).to(logits.dtype)
        assert n <= logits.shape[0]

    def release_held(self) -> None:
        if self._held is not None:
            self.ws.put(self._held[0])
            self._held = None

    def stage(self, inp: StepInput) -> None:
        """Build the step's metadata blob ahead of time (into the pinned copy the step in flight
        is not using). `launch` picks it up; the token ids may be filled in later."""
        self._blob_idx ^= 1
        blob = self.host_blobs[self._blob_idx]
        info = self.rt.build_attn_meta(self.layout, blob.data_ptr(), inp.lens, inp.cached_lens,
                                       inp.block_tables, self.cfg.block_size, self.num_blocks)
        inp._staged = (self._blob_idx, info)

    def execute(self, inp: StepInput) -> Optional[List[int]]:
        """Run one step; returns the sampled token id per request (or None when sample=False)."""
        return self.collect(self.launch(inp))

    def launch(self, inp: StepInput):
        """Enqueue one step (copies, forward, sampling, read-back) without waiting for it.
        Returns a handle for `collect`."""
        cfg = self.cfg
        batch = len(inp.lens)
        ntok = len(inp.tokens)
        self.release_held()
        self._lp_dev = None
        self.last_logprobs = None
        staged = getattr(inp, "_staged", None)
        if staged is None:
            self.stage(inp)
            staged = inp._staged
        self.host_blob = self.host_blobs[staged[0]]
        info = staged[1]
        assert info.num_tokens == ntok
        if inp.pos_delta is not None and ntok == batch and not getattr(inp, "_delta_applied", False):
            # decode of requests with an M-RoPE delta: shift this step's positions in the host blob
            L = self.layout
            pos = self.host_blob[L.positions: L.positions + 8 * ntok].view(torch.int64)
            pos += torch.tensor(inp.pos_delta, dtype=torch.int64)
            inp._delta_applied = True
        stochastic = inp.temperature is not None and any(t > 0 for t in inp.temperature)
        self.host_tokens[:ntok] = torch.tensor(inp.tokens, dtype=torch.int32)
        # an empty step (a data-parallel rank with nothing to run) is a fully padded decode step:
        # it joins the step's collectives and touches no KV slot
        decode = info.decode_step or batch == 0
        rows = self._bucket(max(batch, 1)) if decode else batch
        if decode and rows > ntok:
            self.host_tokens[ntok:rows] = 0
        n_copy = rows if decode else ntok
        self.dev_tokens[:n_copy].copy_(self.host_tokens[:n_copy], non_blocking=True)
        self.dev_blob.copy_(self.host_blob, non_blocking=True)
        self.h2d_bytes += n_copy * 4 + self.host_blob.numel()
        if inp.state_slots is not None:
            fresh = [s for s, c in zip(inp.state_slots, inp.cached_lens) if c == 0]
            if fresh:  # a request starting from scratch: its recurrent state starts at zero
                idx = torch.tensor(fresh, dtype=torch.long, device=self.device)
                for li in range(cfg.num_layers):
                    if cfg.layer_is_linear_attn(li):
                        for t in self.kv_caches[li]:
                            t.index_fill_(0, idx, 0)
            sl = list(inp.state_slots) + [cfg.max_batch_size] * (cfg.max_batch_size - batch)
            self.dev_state_slots.copy_(torch.tensor(sl, dtype=torch.int32), non_blocking=True)
            self.h2d_bytes += 4 * cfg.max_batch_size
        if stochastic:
            self.host_samp.zero_()
            self.host_samp[0, :batch] = torch.tensor(inp.temperature, dtype=torch.float32)
            self.host_samp[2, :batch] = torch.tensor(inp.top_p or [1.0] * batch, dtype=torch.float32)
            self.dev_samp.copy_(self.host_samp, non_blocking=True)
            self.dev_topk[:batch].copy_(torch.tensor(inp.top_k or [0] * batch, dtype=torch.int32))
            self.dev_step.fill_(int(inp.step_id) & 0x7fffffff)
            self.h2d_bytes += self.host_samp.numel() * 4 + batch * 4
        if decode:
            ns = self._pick_splits(batch, info.max_seq_len)
            meta = self._meta(dict(batch=rows, num_tokens=rows, max_q_len=1, max_seq_len=info.max_seq_len,
                                   decode_step=True), rows, ns)
            key = (rows, ns, stochastic)
            if self.use_graphs and not inp.logprobs and inp.penalties is None:
                g = self.graphs.get(key)
                if g is None:
                    g = self._capture(key, rows, meta, stochastic, inp.step_id)
                elif self._graph_addrs.get(key) != self._fixed_addresses():
                    # a captured graph replays raw pointers: refuse to run on moved buffers
                    # (the reference's replay guard, xlite/csrc/runtime.cpp:653-662)
                    raise RuntimeError(f"fixed-address violation: buffers of graph {key} moved since capture")
                g.replay()
                self.last_graph_key = key
                self.launch_count += self.graph_launches[key]
            else:
                self._forward_and_sample(rows, meta, rows, True, stochastic, inp.step_id, logprobs=inp.logprobs,
                                         penalties=inp.penalties)
        elif self._dual_eligible(inp, ntok, stochastic):
            return self._launch_dual(inp, stochastic)
        else:
            meta = self._meta(info, batch, 1)
            mm = None
            if inp.positions3 is not None:
                meta.positions = inp.positions3.to(self.device, non_blocking=True).contiguous()
                self.h2d_bytes += inp.positions3.numel() * 8
            if inp.mm_rows:
                rows_dev = torch.tensor(inp.mm_rows, dtype=torch.long, device=self.device)
                emb = inp.mm_embeds.to(self.device, self.model.dtype)
                deep = [d.to(self.device, self.model.dtype) for d in (inp.mm_deepstack or [])]
                mm = (rows_dev, emb, deep)
                self.h2d_bytes += emb.numel() * emb.element_size() * (1 + len(deep))
            n_out = batch
            if inp.all_logits:
                if stochastic:
                    raise ValueError("all_logits steps sample greedily")
                if ntok > self.logit_rows:
                    raise ValueError(f"step asks for logits at {ntok} rows; the runner was built for {self.logit_rows}")
                meta.last_token_idx = self.dev_all_rows
                n_out = ntok
            self._forward_and_sample(ntok, meta, n_out, inp.sample, stochastic, inp.step_id, mm=mm,
                                     logprobs=0 if inp.all_logits else inp.logprobs,
                                     penalties=None if inp.all_logits else inp.penalties)
            batch = n_out
        if not inp.sample or batch == 0:
            return None
        self.host_out[:batch].copy_(self.dev_out[:batch], non_blocking=True)
        self.d2h_bytes += batch * 4
        return batch

    # ------------------------------------------------------------------ dual-stream prefill
    def _dual_eligible(self, inp: StepInput, ntok: int, stochastic: bool) -> bool:
        return (self.dual_stream and not self.hold_hidden and ntok >= self.dual_min_tokens and not inp.all_logits
                and not inp.logprobs and inp.penalties is None
                and inp.mm_rows is None and inp.positions3 is None and inp.state_slots is None
                and max(inp.lens) >= 2)

    @staticmethod
    def split_step(inp: StepInput):
        """Cut a prefill step along the sequence: micro-batch A holds the first half of every
        request's new tokens, B the rest on top of A's rows in the cache. Requests with a single
        new token go to B whole. Returns (A, B, rows of `inp`'s requests that A contains)."""
        la = [n // 2 for n in inp.lens]
        in_a = [i for i, n in enumerate(la) if n > 0]
        tok_a: List[int] = []
        tok_b: List[int] = []
        base = 0
        for n, a in zip(inp.lens, la):
            tok_a.extend(inp.tokens[base: base + a])
            tok_b.extend(inp.tokens[base + a: base + n])
            base += n
        A = StepInput(tokens=tok_a, lens=[la[i] for i in in_a], cached_lens=[inp.cached_lens[i] for i in in_a],
                      block_tables=[inp.block_tables[i] for i in in_a], sample=False, step_id=inp.step_id)
        B = StepInput(tokens=tok_b, lens=[n - a for n, a in zip(inp.lens, la)],
                      cached_lens=[c + a for c, a in zip(inp.cached_lens, la)], block_tables=inp.block_tables,
                      temperature=inp.temperature, top_k=inp.top_k, top_p=inp.top_p, sample=inp.sample,
                      step_id=inp.step_id)
        return A, B, in_a

    def _launch_dual(self, inp: StepInput, stochastic: bool):
        """One prefill step as two micro-batches that leapfrog through the layers: A on the
        current stream, B on a side stream, B's phase i ordered after A's phase i (which wrote the
        cache rows B's attention reads). A's tensor-parallel collectives overlap B's GEMMs and
        vice versa. The reference runs the two halves of a prompt on two runtimes / threads with
        cross notifies (xlite/tests/models/llama.py:368-416, xlite/csrc/_C.cpp:637-657)."""
        cfg = self.cfg
        A, B, _ = self.split_step(inp)
        na, nb = len(A.tokens), len(B.tokens)
        batch = len(B.lens)
        info_a = self.rt.build_attn_meta(self.layout, self.host_blobs[0].data_ptr(), A.lens, A.cached_lens,
                                         A.block_tables, cfg.block_size, self.num_blocks)
        info_b = self.rt.build_attn_meta(self.layout, self.host_blobs[1].data_ptr(), B.lens, B.cached_lens,
                                         B.block_tables, cfg.block_size, self.num_blocks)
        # tokens were copied in request order by `launch`; lay them out as [A | B]
        self.host_tokens[:na] = torch.tensor(A.tokens, dtype=torch.int32)
        self.host_tokens[na:na + nb] = torch.tensor(B.tokens, dtype=torch.int32)
        self.dev_tokens[:na + nb].copy_(self.host_tokens[:na + nb], non_blocking=True)
        self.dev_blob.copy_(self.host_blobs[0], non_blocking=True)
        self.dev_blob_b.copy_(self.host_blobs[1], non_blocking=True)
        self.h2d_bytes += (na + nb) * 4 + 2 * self.host_blobs[0].numel()
        meta_a = self._meta(info_a, len(A.lens), 1)
        meta_b = self._meta(info_b, batch, 1, views=self._views_b)
        if self.ws_b is None:
            self.ws_b = (Arena(self.arena_bytes, device=self.device) if self.arena is not None
                         else TorchWorkspace(self.device))
        model, ctx = self.model, self.ctx
        ga = model.forward_phases(self.dev_tokens[:na], meta_a, self.kv_caches, self.ws, allow_sp=False)
        gb = model.forward_phases(self.dev_tokens[na:na + nb], meta_b, self.kv_caches, self.ws_b, allow_sp=False)

        def advance(g):
            try:
                next(g)
                return None
            except StopIteration as done:
                return done.value

        main = torch.cuda.current_stream() if self.cuda else None
        if self.cuda and self._side is None:
            self._side = torch.cuda.Stream(device=self.device)
        side = self._side
        h_a = advance(ga)
        h_b = None
        while h_b is None:
            if self.cuda:
                side.wait_stream(main)          # B's phase i after A's phase i (and after the copies)
                with ctx.side_lane(), torch.cuda.stream(side):
                    h_b = advance(gb)
            else:
                with ctx.side_lane():
                    h_b = advance(gb)
            if h_a is None:
                h_a = advance(ga)
        if h_a is None:
            raise RuntimeError("micro-batches fell out of step")
        if self.cuda:
            main.wait_stream(side)
        self.ws.put(h_a)
        self.dual_steps += 1
        if inp.sample:
            logits = model.compute_logits(h_b, meta_b, self.ws_b, batch=batch)
            if stochastic:
                out = F.sample(logits, self.dev_samp[0, :batch], self.dev_topk[:batch], self.dev_samp[2, :batch],
                               seed=self.seed, step=inp.step_id, step_tensor=self.dev_step if self.cuda else None)
            else:
                out = F.sample(logits)
            self.dev_out[:batch].copy_(out)
            if getattr(logits, "_gv_off", None) is not None:
                self.ws_b.put(logits)
        self.ws_b.put(h_b)
        if not inp.sample:
            return None
        self.host_out[:batch].copy_(self.dev_out[:batch], non_blocking=True)
        self.d2h_bytes += batch * 4
        return batch

    def collect(self, handle) -> Optional[List[int]]:
        """Wait for the step enqueued by `launch` and return its sampled tokens."""
        if handle is None:
            if self.cuda:
                torch.cuda.current_stream().synchronize()
            return None
        if self.cuda:
            torch.cuda.current_stream().synchronize()
        if self._lp_dev is not None:
            c, v, i = self._lp_dev
            self.last_logprobs = (c[:handle].tolist(), v[:handle].tolist(), i[:handle].tolist())
            self._lp_dev = None
        return self.host_out[:handle].tolist()

    def idle_step(self) -> None:
        """Take part in one engine step without any request (data-parallel lockstep)."""
        self.execute(StepInput(tokens=[], lens=[], cached_lens=[], block_tables=[], sample=False))

    def warmup_graphs(self, batches: Optional[Sequence[int]] = None, seq_lens: Sequence[int] = (1024,)) -> int:
        """Capture decode graphs ahead of traffic, so that the first request of a batch size does
        not pay for the capture (serving stacks capture a list of sizes at start-up; the
        reference's deployment uses [1, 4, 8, 12, 16, 24, 32, 48, 64, 96],
        xlite/tests/e2e/online_api_server.sh:101). Each capture runs a fully padded step (no
        request, no KV slot written), so it is safe while requests are in flight between steps.
        `seq_lens` are the context lengths whose split-KV choice should be covered. Returns the
        number of graphs captured."""
        if not self.use_graphs:
            return 0
        cfg = self.cfg
        done = 0
        for b in (batches or self.buckets):
            b = min(int(b), cfg.max_batch_size)
            rows = self._bucket(b)
            for L in seq_lens:
                ns = self._pick_splits(b, min(int(L), cfg.max_seq_len))
                key = (rows, ns, False)
                if key in self.graphs:
                    continue
                blob = self.host_blobs[self._blob_idx]
                self.rt.build_attn_meta(self.layout, blob.data_ptr(), [], [], [], cfg.block_size, self.num_blocks)
                self.dev_blob.copy_(blob, non_blocking=True)
                self.dev_tokens[:rows].zero_()
                meta = self._meta(dict(batch=rows, num_tokens=rows, max_q_len=1, max_seq_len=int(L),
                                       decode_step=True), rows, ns)
                self._capture(key, rows, meta, False, 0)
                done += 1
        return done

    def _capture(self, key, rows, meta, stochastic, step_id):
        # warm-up run outside capture (lazy initialisation: smem attributes, tensor maps, status word)
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self._forward_and_sample(rows, meta, rows, True, stochastic, step_id)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        before = _native.LAUNCHES
        with torch.cuda.graph(g):
            self._forward_and_sample(rows, meta, rows, True, stochastic, step_id)
        self.graph_launches[key] = _native.LAUNCHES - before
        self.graphs[key] = g
        self._graph_addrs[key] = self._fixed_addresses()
        return g

    def _fixed_addresses(self) -> tuple:
        """Addresses every captured graph depends on: step inputs, metadata, outputs, the arena
        slab and the KV cache set (a handful of pointer reads: this runs before every replay)."""
        slab = getattr(self.arena, "slab", None)
        kv0 = self.kv_caches[0][0] if self.kv_caches else None
        return (self.dev_tokens.data_ptr(), self.dev_blob.data_ptr(), self.dev_out.data_ptr(),
                0 if slab is None else slab.data_ptr(), id(self.kv_caches),
                0 if kv0 is None else kv0.data_ptr())

    def update_sm_fraction(self, fraction: float) -> int:
        """Plan the following steps of the calling thread for a share of the device: persistent
        kernels size their grids and the split-KV tuner counts CTAs slots by it (the reference's
        ``Runtime.update_core_num``, xlite/csrc/runtime.cpp:749-755). Captured graphs keep the
        shape they were captured with, so callers that change shares run eagerly. Returns the SM
        count now planned with."""
        total = torch.cuda.get_device_properties(self.device).multi_processor_count if self.cuda else 148
        sms = total if fraction >= 1.0 else max(1, int(round(total * max(fraction, 0.0))))
        self.num_sms = sms
        if self.cuda:
            _native.set_sm_budget(0 if sms >= total else sms)
        return sms

    def check_status(self) -> int:
        """Device status word (bounded waits that ran out, bad indices). 0 = healthy."""
        return _native.read_status() if self.cuda else 0

    def memory_report(self) -> str:
        from ..models.weights import weight_bytes
        kv = sum(t.numel() * t.element_size() for c in self.kv_caches for t in c)
        ar = self.arena_bytes if self.arena is not None else 0
        return (f"model {weight_bytes(self.model.w) / 2**20:.1f} MiB, kv cache {kv / 2**20:.1f} MiB, "
                f"activation arena {ar / 2**20:.1f} MiB")
