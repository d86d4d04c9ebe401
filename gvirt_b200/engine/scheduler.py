"""Continuous-batching scheduler.

The reference has no scheduler — vLLM drives it with (lens, cached_lens, block_tables) per
step (xlite/doc/feature_matrix.md:10-35; the in-repo harness is a static-batch loop,
xlite/tests/generate.py:51-103). This one provides what a stand-alone runtime needs:

* a waiting queue and a running set; new requests are admitted while KV blocks and the
  ``max_num_batched_tokens`` / ``max_batch_size`` budgets allow;
* prefill-priority iteration-level scheduling: a step is either a prefill step (new prompts,
  optionally *chunked* so a long prompt is fed ``max_num_batched_tokens`` at a time while its
  earlier chunks sit in the cache) or a decode step over every running request;
* automatic prefix caching through the block manager (cached leading blocks shorten the
  prefill) and preemption by recomputation when the cache runs out of blocks.
"""
from __future__ import annotations

import collections
import time
from dataclasses import dataclass, field

import torch  # noqa: F401 - tensors appear in the multimodal input types
from typing import Deque, List, Optional

from .. import _native
from ..config import ModelConfig
from .runner import StepInput


@dataclass
class SamplingParams:
    max_tokens: int = 16
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    stop_token_ids: tuple = ()
    ignore_eos: bool = False
    logprobs: int = 0            # N > 0: record the chosen token's log-probability and the N most likely tokens
    presence_penalty: float = 0.0    # subtracted from the logit of every token generated so far
    frequency_penalty: float = 0.0   # subtracted once per occurrence in the generated text
    repetition_penalty: float = 1.0  # logits of tokens seen in prompt or output: divided (if > 0) or multiplied

    @property
    def has_penalties(self) -> bool:
        return self.presence_penalty != 0.0 or self.frequency_penalty != 0.0 or self.repetition_penalty != 1.0


def validate_request(prompt, params: "SamplingParams", max_seq_len: int, vocab_size: int) -> None:
    """Raise ``ValueError`` for a request that no engine step could run. Called on the client side
    of the serving engine (the HTTP layer answers 400) so that a malformed request never reaches
    the engine thread: token ids outside the vocabulary would index logits and embedding rows out
    of range on the device, and a request longer than ``max_seq_len`` has no block-table row."""
    import math
    n = len(prompt)
    if n == 0:
        raise ValueError("empty prompt")
    if not isinstance(params.max_tokens, int) or params.max_tokens < 1:
        raise ValueError(f"max_tokens must be a positive integer, got {params.max_tokens!r}")
    if n + params.max_tokens > max_seq_len:
        raise ValueError(f"prompt of {n} tokens + max_tokens {params.max_tokens} exceeds max_seq_len {max_seq_len}")
    for name, ids in (("prompt", prompt), ("stop_token_ids", params.stop_token_ids)):
        for t in ids:
            if not isinstance(t, int) or isinstance(t, bool) or not 0 <= t < vocab_size:
                raise ValueError(f"{name}: token id {t!r} is outside [0, {vocab_size})")
    for name in ("temperature", "top_p", "presence_penalty", "frequency_penalty", "repetition_penalty"):
        v = getattr(params, name)
        if not isinstance(v, (int, float)) or not math.isfinite(v):
            raise ValueError(f"{name} must be a finite number, got {v!r}")
    if params.temperature < 0:
        raise ValueError(f"temperature must be >= 0, got {params.temperature}")
    if not 0 < params.top_p <= 1:
        raise ValueError(f"top_p must be in (0, 1], got {params.top_p}")
    if not isinstance(params.top_k, int) or params.top_k < 0:
        raise ValueError(f"top_k must be a non-negative integer, got {params.top_k!r}")
    if params.repetition_penalty <= 0:
        raise ValueError(f"repetition_penalty must be > 0, got {params.repetition_penalty}")
    if not -2.0 <= params.presence_penalty <= 2.0 or not -2.0 <= params.frequency_penalty <= 2.0:
        raise ValueError("presence_penalty and frequency_penalty must be in [-2, 2]")
    if not isinstance(params.logprobs, int) or not 0 <= params.logprobs <= 20:
        raise ValueError(f"logprobs must be in [0, 20], got {params.logprobs!r}")


@dataclass
class MultiModalInputs:
    """Pre-computed embeddings for some prompt positions (image / video patches from a vision
    tower) and, for M-RoPE models, explicit 3-row positions. The reference's full-graph mode
    takes the same inputs: `inputs_embeds`, a 3-row `positions` tensor and DeepStack features
    added to the hidden states after the first layers (xlite/xlite/_C.cpp:1988-2001).

    embed_index    prompt positions whose embedding is replaced (sorted, unique)
    embeds         [len(embed_index), hidden]
    positions      optional int64 [3, len(prompt)] (temporal / height / width); text positions
                   hold the same value in the three rows
    position_delta added to the running position of every token after the prompt (the M-RoPE
                   "rope delta": image grids advance the position by less than their length)
    deepstack      optional list of [len(embed_index), hidden]: entry i is added to the hidden
                   state of the embed_index rows after layer i"""
    embed_index: List[int]
    embeds: "torch.Tensor"
    positions: Optional["torch.Tensor"] = None
    position_delta: int = 0
    deepstack: Optional[List["torch.Tensor"]] = None


@dataclass(eq=False)  # identity semantics: membership tests must not compare token lists
class Request:
    req_id: int
    prompt: List[int]
    params: SamplingParams
    output: List[int] = field(default_factory=list)
    num_computed: int = 0          # tokens whose KV is in the cache
    arrival: float = 0.0
    first_token_time: Optional[float] = None
    finish_time: Optional[float] = None
    token_times: List[float] = field(default_factory=list)
    finished: bool = False
    preemptions: int = 0
    state_slot: int = -1           # recurrent-state slot (models with linear-attention layers)
    mm: Optional[MultiModalInputs] = None
    logprobs: List[tuple] = field(default_factory=list)   # per output token: (logprob, [(token, logprob), ...])

    @property
    def all_tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def hash_tokens(self) -> List[int]:
        """Token ids as the prefix cache sees them: positions whose embedding comes from
        multimodal inputs get a per-request id, so that equal placeholder tokens with different
        images never share cached blocks."""
        if self.mm is None or not self.mm.embed_index:
            return self.all_tokens
        toks = self.all_tokens
        salt = -(self.req_id + 1)
        for i in self.mm.embed_index:
            toks[i] = salt
        return toks

    @property
    def total_len(self) -> int:
        return len(self.prompt) + len(self.output)


@dataclass
class ScheduledStep:
    requests: List[Request]
    inp: StepInput
    is_prefill: bool
    sample_mask: List[bool]  # per request: does this step produce a token for it
    drafts: Optional[List[List[int]]] = None  # verification step: per request the draft tokens after its last token
    emitted: int = 0         # tokens appended to requests by this step (set by `update`)


class Scheduler:
    def __init__(self, cfg: ModelConfig, num_blocks: int, enable_prefix_cache: bool = False,
                 enable_chunked_prefill: bool = True, eos_token_id: Optional[int] = None,
                 proposer=None, spec_tokens: int = 0, kv_pool=None, mixed_batches: bool = False):
        self.cfg = cfg
        # mixed batches: requests in their decode phase ride along with prefill chunks (one token
        # each) instead of waiting for the prompts in front of them; see `_schedule`
        self.mixed = mixed_batches
        self.mixed_steps = 0
        self.bm = _native.runtime().BlockManager(num_blocks, cfg.block_size, enable_prefix_cache)
        # second tier behind the prefix cache (engine/kv_pool.py): evicted blocks are saved to host
        # memory and restored when a later prefix asks for them
        self.kv_pool = kv_pool if (enable_prefix_cache and cfg.full_attention_interval == 0) else None
        if self.kv_pool is not None:
            self.bm.set_eviction_log(True)
        self.waiting: Deque[Request] = collections.deque()
        self.running: List[Request] = []
        self.chunked = enable_chunked_prefill
        self.eos = eos_token_id
        self.step_id = 0
        self.epoch = 0             # bumped whenever the set of requests changes outside a step's update
        self.num_preemptions = 0
        self.free_state_slots = list(range(cfg.max_batch_size - 1, -1, -1))
        self.uses_state_slots = cfg.full_attention_interval > 0
        # speculative decoding (engine/spec_decode.py); a recurrent state cannot be rolled back past
        # rejected drafts, so models with linear-attention layers decode one token at a time
        self.proposer = None if self.uses_state_slots else proposer
        self.spec_tokens = spec_tokens if self.proposer is not None else 0
        self.spec_steps = 0
        self.spec_drafted = 0
        self.spec_accepted = 0

    # -------------------------------------------------------------- admission
    def add(self, req: Request) -> None:
        if len(req.prompt) + req.params.max_tokens > self.cfg.max_seq_len:
            raise ValueError(f"request {req.req_id}: prompt + max_tokens exceeds max_seq_len "
                             f"{self.cfg.max_seq_len}")
        if not req.prompt:
            raise ValueError("empty prompt")
        req.arrival = req.arrival or time.perf_counter()
        self.waiting.append(req)
        self.epoch += 1

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def abort(self, req: Request) -> bool:
        """Drop a request between steps (client went away): frees its blocks and state slot.
        Returns False when the request was not queued or running."""
        now = time.perf_counter()
        if req in self.running:
            self.bm.release(req.req_id)
            self.running.remove(req)
            self._free_slot(req)
        elif req in self.waiting:
            self.waiting.remove(req)
        else:
            return False
        req.finished = True
        req.finish_time = now
        if self.proposer is not None:
            self.proposer.forget(req)
        self.epoch += 1
        return True

    # -------------------------------------------------------------- one step
    def schedule(self) -> Optional[ScheduledStep]:
        step = self._schedule()
        self._sync_pool()      # blocks taken over by appends of this pass
        return step

    def _schedule(self) -> Optional[ScheduledStep]:
        cfg = self.cfg
        self.step_id += 1
        # 0) with mixed batches, requests that are decoding keep their place in every step
        riders: List[Request] = []
        if self.mixed and (self.waiting or any(r.num_computed < self._target_len(r) for r in self.running)):
            cand = [r for r in self.running if r.num_computed >= self._target_len(r)]
            if len(cand) < cfg.max_num_batched_tokens and all(self.bm.append(r.req_id, r.total_len) for r in cand):
                riders = cand      # (no preemption on behalf of riders: otherwise decode alone below)
        # 1) requests still prefilling (admitted earlier, chunked) and new admissions
        budget = cfg.max_num_batched_tokens - len(riders)
        pre: List[Request] = []
        lens: List[int] = []
        for r in self.running:
            if r.num_computed < self._target_len(r):
                if len(pre) + len(riders) >= cfg.max_batch_size or budget <= 0:
                    break
                n = min(self._target_len(r) - r.num_computed, budget)
                if not self.chunked and n < self._target_len(r) - r.num_computed:
                    continue
                pre.append(r)
                lens.append(n)
                budget -= n
        while (self.waiting and budget > 0 and len(self.running) < cfg.max_batch_size
               and len(pre) + len(riders) < cfg.max_batch_size):
            r = self.waiting[0]
            toks = r.all_tokens  # a preempted request recomputes prompt + generated tokens
            cached = self._allocate(r)
            if cached < 0:
                break  # no blocks: wait for running requests to finish
            remaining = len(toks) - cached
            n = min(remaining, budget)
            if not self.chunked and n < remaining:
                self.bm.release(r.req_id)
                break
            self.waiting.popleft()
            r.num_computed = cached
            if self.uses_state_slots:
                r.state_slot = self.free_state_slots.pop()
                r.num_computed = 0  # recurrent state cannot be restored from cached KV blocks
            if r.output:
                # recompute path: treat everything so far as the prompt of this pass
                r._recompute_len = len(toks)
            self.running.append(r)
            pre.append(r)
            lens.append(n)
            budget -= n
        if pre:
            if riders:
                self.mixed_steps += 1
                return self._make_prefill(riders + pre, [1] * len(riders) + lens)
            return self._make_prefill(pre, lens)
        # 2) decode step over all running requests
        if not self.running:
            return None
        dec: List[Request] = []
        for r in list(self.running):
            if r not in self.running:
                continue  # preempted a moment ago to make room for an earlier request
            while not self.bm.append(r.req_id, r.total_len):
                victim = self._preempt_one(exclude=r)
                if victim is None:
                    raise RuntimeError("KV cache too small for a single request")
            dec.append(r)
        dec = [r for r in dec if r in self.running]
        if not dec:
            return None
        if self.spec_tokens > 0:
            ver = self._make_verify(dec)
            if ver is not None:
                return ver
        tokens = [(r.output[-1] if r.output else r.prompt[-1]) for r in dec]
        inp = StepInput(tokens=tokens, lens=[1] * len(dec), cached_lens=[r.total_len - 1 for r in dec],
                        block_tables=[self.bm.block_table(r.req_id) for r in dec], step_id=self.step_id,
                        state_slots=[r.state_slot for r in dec] if self.uses_state_slots else None)
        self._fill_mm_decode(inp, dec)
        self._fill_sampling(inp, dec)
        return ScheduledStep(dec, inp, False, [True] * len(dec))

    def _make_verify(self, dec: List[Request]) -> Optional[ScheduledStep]:
        """Turn the decode step over `dec` into a verification step when the proposer has drafts
        for at least one request. Every request contributes its last token plus its drafts as one
        chunk over its cached context; the step asks for the model's choice at every row.
        Speculation never preempts: a request whose drafts do not fit into its blocks or into the
        step's token budget goes without. Returns None for "decode normally"."""
        cfg = self.cfg
        if any(r.params.temperature > 0 or r.params.logprobs or r.params.has_penalties for r in dec):
            return None   # the acceptance rule below is the greedy one; log-probabilities come from plain steps
        budget = cfg.max_num_batched_tokens - len(dec)
        ks = [max(0, min(self.spec_tokens, r.params.max_tokens - len(r.output) - 1,
                         cfg.max_seq_len - r.total_len - 1)) for r in dec]
        proposals = self.proposer.propose_batch(dec, ks)
        drafts: List[List[int]] = []
        for r, k, d in zip(dec, ks, proposals):
            d = list(d[:max(min(k, budget), 0)])
            if d and not self.bm.append(r.req_id, r.total_len + len(d)):
                d = []
            budget -= len(d)
            drafts.append(d)
        if not any(drafts):
            return None
        tokens: List[int] = []
        for r, d in zip(dec, drafts):
            tokens.append(r.output[-1] if r.output else r.prompt[-1])
            tokens.extend(d)
        lens = [1 + len(d) for d in drafts]
        inp = StepInput(tokens=tokens, lens=lens, cached_lens=[r.total_len - 1 for r in dec],
                        block_tables=[self.bm.block_table(r.req_id) for r in dec], step_id=self.step_id,
                        all_logits=True)
        self._fill_mm_prefill(inp, dec, lens)
        self.spec_steps += 1
        return ScheduledStep(dec, inp, False, [True] * len(dec), drafts=drafts)

    def peek_next_decode(self, cur: ScheduledStep) -> Optional[ScheduledStep]:
        """Prepare the decode step that follows `cur` while `cur` is still running on the device,
        assuming every request of `cur` gets exactly one more token and none of them stops. Returns
        None when that cannot be assumed (admissions waiting, a request about to reach max_tokens,
        no free block without preempting, batch not in steady state); the caller then schedules
        normally. The returned step has no token ids yet (`inp.tokens` is filled in by the caller
        from the sampled tokens of `cur`) and must be dropped if any request of `cur` finished."""
        if cur.is_prefill or self.waiting or len(cur.requests) != len(self.running):
            return None
        if self.spec_tokens > 0:
            return None   # the next step's drafts depend on the tokens this step produces
        if any(r.params.has_penalties for r in cur.requests):
            return None   # ... and so do logit penalties
        reqs = cur.requests
        for r, q in zip(reqs, self.running):
            if r is not q or len(r.output) + 2 > r.params.max_tokens or getattr(r, "_recompute_len", None):
                return None
            if r.num_computed != r.total_len - 1:
                return None
        tables = []
        for r in reqs:
            # after `cur` the request holds total_len + 1 tokens, the new one being the next input
            if not self.bm.append(r.req_id, r.total_len + 1):
                return None   # needs a preemption: leave that to the regular path
            tables.append(self.bm.block_table(r.req_id))
        inp = StepInput(tokens=[0] * len(reqs), lens=[1] * len(reqs), cached_lens=[r.total_len for r in reqs],
                        block_tables=tables, step_id=self.step_id + 1,
                        state_slots=[r.state_slot for r in reqs] if self.uses_state_slots else None)
        self._fill_mm_decode(inp, reqs)
        self._fill_sampling(inp, reqs)
        self._sync_pool()
        return ScheduledStep(list(reqs), inp, False, [True] * len(reqs))

    def adopt(self, step: ScheduledStep) -> None:
        """The caller runs a step prepared by `peek_next_decode` instead of calling `schedule`."""
        self.step_id += 1

    def _allocate(self, r: Request) -> int:
        if self.kv_pool is None:
            return self.bm.allocate(r.req_id, r.hash_tokens)
        toks = r.hash_tokens
        ext = self.kv_pool.present(self.bm.prefix_hashes(toks))
        cached = self.bm.allocate_ext(r.req_id, toks, ext)
        self._sync_pool()
        return cached

    def _sync_pool(self) -> None:
        """Hand the block manager's second-tier events to the pool, evictions first: a block
        may be evicted and promised to a restore within one call."""
        if self.kv_pool is not None:
            self.kv_pool.sync(self.bm.drain_evictions(), self.bm.drain_restores())

    def _free_slot(self, r: Request) -> None:
        if r.state_slot >= 0:
            self.free_state_slots.append(r.state_slot)
            r.state_slot = -1

    def _target_len(self, r: Request) -> int:
        return getattr(r, "_recompute_len", None) or len(r.prompt)

    def _make_prefill(self, reqs: List[Request], lens: List[int]) -> ScheduledStep:
        tokens: List[int] = []
        cached, tables, mask = [], [], []
        for r, n in zip(reqs, lens):
            allt = r.all_tokens
            tokens.extend(allt[r.num_computed:r.num_computed + n])
            cached.append(r.num_computed)
            tables.append(self.bm.block_table(r.req_id))
            mask.append(r.num_computed + n >= self._target_len(r))
        inp = StepInput(tokens=tokens, lens=list(lens), cached_lens=cached, block_tables=tables,
                        sample=any(mask), step_id=self.step_id,
                        state_slots=[r.state_slot for r in reqs] if self.uses_state_slots else None)
        self._fill_mm_prefill(inp, reqs, lens)
        self._fill_sampling(inp, reqs)
        return ScheduledStep(reqs, inp, True, mask)

    # -------------------------------------------------------------- multimodal inputs
    @staticmethod
    def _fill_mm_decode(inp: StepInput, reqs: List[Request]) -> None:
        if any(r.mm is not None and r.mm.position_delta for r in reqs):
            inp.pos_delta = [(r.mm.position_delta if r.mm is not None else 0) for r in reqs]

    @staticmethod
    def _fill_mm_prefill(inp: StepInput, reqs: List[Request], lens: List[int]) -> None:
        """Gather what this chunk needs of every request's multimodal inputs: embedding rows that
        fall into the chunk (as row numbers of the step's flat token dimension) and per-token
        3-row positions."""
        if not any(r.mm is not None for r in reqs):
            return
        import bisect
        import torch
        rows: List[int] = []
        emb, deep = [], []
        pos3 = []
        need_pos = any(r.mm is not None and (r.mm.positions is not None or r.mm.position_delta) for r in reqs)
        base = 0
        for r, n in zip(reqs, lens):
            c0 = r.num_computed
            if r.mm is not None:
                idx = r.mm.embed_index
                lo, hi = bisect.bisect_left(idx, c0), bisect.bisect_left(idx, c0 + n)
                if hi > lo:
                    rows.extend(base + (i - c0) for i in idx[lo:hi])
                    emb.append(r.mm.embeds[lo:hi])
                    if r.mm.deepstack:
                        deep.append([d[lo:hi] for d in r.mm.deepstack])
            if need_pos:
                p = torch.arange(c0, c0 + n, dtype=torch.int64)
                p3 = p.unsqueeze(0).repeat(3, 1)
                if r.mm is not None:
                    plen = len(r.prompt)
                    if r.mm.positions is not None:
                        k = max(0, min(n, plen - c0))          # part of the chunk inside the prompt
                        if k > 0:
                            p3[:, :k] = r.mm.positions[:, c0:c0 + k].to(torch.int64)
                        if k < n:
                            p3[:, k:] += r.mm.position_delta
                    elif r.mm.position_delta:
                        k = max(0, min(n, plen - c0))
                        p3[:, k:] += r.mm.position_delta
                pos3.append(p3)
            base += n
        if rows:
            inp.mm_rows = rows
            inp.mm_embeds = torch.cat(emb, 0)
            if deep:
                if len(deep) != len(emb):
                    raise ValueError("either every request with embeddings in a step carries DeepStack features or none")
                depth = min(len(d) for d in deep)
                inp.mm_deepstack = [torch.cat([d[i] for d in deep], 0) for i in range(depth)]
        if need_pos:
            inp.positions3 = torch.cat(pos3, 1)

    def _fill_sampling(self, inp: StepInput, reqs: List[Request]) -> None:
        inp.logprobs = max((r.params.logprobs for r in reqs), default=0)
        if any(r.params.has_penalties for r in reqs):
            inp.penalties = self._penalties(reqs)
        if any(r.params.temperature > 0 for r in reqs):
            inp.temperature = [r.params.temperature for r in reqs]
            inp.top_k = [r.params.top_k for r in reqs]
            inp.top_p = [r.params.top_p for r in reqs]

    @staticmethod
    def _penalties(reqs: List[Request]) -> dict:
        """Sparse description of the logit adjustments of a step: (row, token, count) triples of
        the generated tokens for the presence / frequency terms, (row, token) pairs of everything
        seen for the repetition term, and the per-row coefficients."""
        rows, toks, cnts, rrows, rtoks = [], [], [], [], []
        for b, r in enumerate(reqs):
            p = r.params
            if p.presence_penalty != 0.0 or p.frequency_penalty != 0.0:
                for t, c in collections.Counter(r.output).items():
                    rows.append(b)
                    toks.append(t)
                    cnts.append(c)
            if p.repetition_penalty != 1.0:
                for t in set(r.prompt) | set(r.output):
                    rrows.append(b)
                    rtoks.append(t)
        return {"rows": rows, "toks": toks, "counts": cnts, "rep_rows": rrows, "rep_toks": rtoks,
                "presence": [r.params.presence_penalty for r in reqs],
                "frequency": [r.params.frequency_penalty for r in reqs],
                "repetition": [r.params.repetition_penalty for r in reqs]}

    def _preempt_one(self, exclude: Request) -> Optional[Request]:
        for r in reversed(self.running):
            if r is not exclude:
                self.bm.release(r.req_id)
                self.running.remove(r)
                self._free_slot(r)
                r.num_computed = 0
                r.preemptions += 1
                self.epoch += 1
                self.num_preemptions += 1
                self.waiting.appendleft(r)
                return r
        return None

    # -------------------------------------------------------------- results
    def update(self, step: ScheduledStep, sampled: Optional[List[int]], logprobs=None) -> List[Request]:
        """Apply the step's results; returns requests that finished in this step. `sampled` holds
        one token per request, or one per input row for a verification step; `logprobs` (when the
        step asked for them) = (chosen [B], top values [B, N], top ids [B, N]) as lists."""
        now = time.perf_counter()
        done: List[Request] = []
        row = 0
        step.emitted = 0
        for i, r in enumerate(step.requests):
            n_in = step.inp.lens[i]
            if step.drafts is not None:
                from .spec_decode import accept
                new = accept(step.drafts[i], sampled[row:row + n_in])
                row += n_in
                self.spec_drafted += len(step.drafts[i])
                self.spec_accepted += len(new) - 1
                r.num_computed += len(new)   # the last token and the accepted drafts hold valid KV
            else:
                r.num_computed += n_in
                if not step.sample_mask[i]:
                    continue
                new = [int(sampled[i])]
                if logprobs is not None and r.params.logprobs:
                    n = r.params.logprobs
                    r.logprobs.append((logprobs[0][i], list(zip(logprobs[2][i][:n], logprobs[1][i][:n]))))
            if getattr(r, "_recompute_len", None):
                r._recompute_len = None
            stop = False
            for tok in new:
                r.output.append(tok)
                r.token_times.append(now)
                step.emitted += 1
                if r.first_token_time is None:
                    r.first_token_time = now
                stop = (not r.params.ignore_eos and self.eos is not None and tok == self.eos) or \
                    tok in r.params.stop_token_ids or len(r.output) >= r.params.max_tokens
                if stop:
                    break
            if stop:
                # tokens accepted after a stop are dropped; the newest token's KV is not in the
                # cache, so only the blocks below it may be shared
                r.num_computed = min(r.num_computed, r.total_len - 1)
                r.finished = True
                r.finish_time = now
                self.bm.commit(r.req_id, r.hash_tokens[:r.num_computed])
                self.bm.release(r.req_id)
                self.running.remove(r)
                self._free_slot(r)
                if self.proposer is not None:
                    self.proposer.forget(r)
                done.append(r)
            elif step.is_prefill:
                self.bm.commit(r.req_id, r.hash_tokens[:r.num_computed])
        return done
