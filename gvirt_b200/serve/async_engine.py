"""Background engine loop: requests arrive from any thread, one thread steps the engine.

The reference is driven by an external serving framework whose scheduler hands the engine
``lens / cached_lens / block_tables`` every step (xlite/xlite/_C.cpp:1988-2001) and whose feature
matrix lists asynchronous scheduling, prefix caching and chunked prefill
(xlite/doc/feature_matrix.md:12-35). This module is the in-tree equivalent: the ``LLM`` engine
already owns scheduling and KV blocks; ``AsyncEngine`` adds the thread that keeps stepping while
requests come and go, per-request completion futures, token streaming callbacks, cancellation and
the serving metrics the reference's benchmark scripts report (QPS, TTFT / TPOT mean and p99,
output tok/s; xlite/tests/e2e/process_data.py:7-46).

Several processes (tensor / expert parallel replicas of one model): every rank holds the same
engine and must see the same requests in the same order, because scheduling is deterministic and
every step is a collective. Rank 0 runs ``AsyncEngine`` and, before every iteration, broadcasts
that iteration's events — new requests, aborts, whether a step follows — over a gloo control
group; the other ranks run ``follower_loop`` and mirror them. Stop strings and client
cancellations are decided on rank 0 and reach the followers as aborts before the next step.
With data-parallel attention (dp > 1) every request belongs to one data-parallel rank (the least
loaded one, chosen by rank 0): only that rank's tensor-parallel group adds it, all ranks still
step together (a rank without work takes the engine's idle step), and after every step the
owners report their new tokens to rank 0 through a gather on the control group.
"""
from __future__ import annotations

import dataclasses
import threading
import time
from concurrent.futures import Future
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

from ..engine.llm import LLM
from ..engine.scheduler import Request, SamplingParams, validate_request


@dataclass
class GenerationResult:
    request_id: int
    prompt_ids: List[int]
    output_ids: List[int]
    finish_reason: str
    ttft_s: Optional[float]
    tpot_s: Optional[float]
    latency_s: float
    text: Optional[str] = None     # decoded output, cut before a matched stop string (tokenizer needed)
    logprobs: Optional[List[tuple]] = None   # per output token: (logprob, [(token, logprob), ...]) when asked for


@dataclass
class _Pending:
    prompt: List[int]
    params: SamplingParams
    future: Future
    on_token: Optional[Callable[[int, int], None]]
    submitted: float = field(default_factory=time.perf_counter)
    stop: tuple = ()               # stop strings; generation ends when the decoded output contains one
    deadline: Optional[float] = None   # perf_counter value after which the request is ended with reason "timeout"
    export: bool = False           # disaggregated prefill: resolve with the request's KV payload after its first token
    payload: object = None         # disaggregated decode: a ``kv_transfer.KVPayload`` to continue from


class ServingMetrics:
    """Counters and latency samples; ``snapshot()`` gives the numbers, ``prometheus()`` the text
    exposition format."""

    def __init__(self, keep: int = 4096):
        self.lock = threading.Lock()
        self.started = time.time()
        self.requests = self.finished = self.cancelled = self.prompt_tokens = self.output_tokens = 0
        self.ttft: List[float] = []
        self.tpot: List[float] = []
        self.latency: List[float] = []
        self.keep = keep

    def _push(self, arr: List[float], v: Optional[float]):
        if v is not None:
            arr.append(v)
            if len(arr) > self.keep:
                del arr[: len(arr) - self.keep]

    def record(self, res: GenerationResult):
        with self.lock:
            self.finished += 1
            self.prompt_tokens += len(res.prompt_ids)
            self.output_tokens += len(res.output_ids)
            self._push(self.ttft, res.ttft_s)
            self._push(self.tpot, res.tpot_s)
            self._push(self.latency, res.latency_s)

    @staticmethod
    def _stat(arr: List[float]) -> Dict[str, Optional[float]]:
        if not arr:
            return {"mean": None, "p50": None, "p99": None}
        s = sorted(arr)
        return {"mean": sum(s) / len(s), "p50": s[len(s) // 2], "p99": s[min(len(s) - 1, int(0.99 * len(s)))]}

    def snapshot(self) -> dict:
        with self.lock:
            up = max(time.time() - self.started, 1e-9)
            return {"uptime_s": up, "requests": self.requests, "finished": self.finished,
                    "cancelled": self.cancelled, "prompt_tokens": self.prompt_tokens,
                    "output_tokens": self.output_tokens, "qps": self.finished / up,
                    "output_tok_s": self.output_tokens / up, "ttft_s": self._stat(self.ttft),
                    "tpot_s": self._stat(self.tpot), "latency_s": self._stat(self.latency)}

    def prometheus(self) -> str:
        s = self.snapshot()
        lines = []
        for k in ("requests", "finished", "cancelled", "prompt_tokens", "output_tokens"):
            lines += [f"# TYPE gvirt_{k}_total counter", f"gvirt_{k}_total {s[k]}"]
        for k in ("qps", "output_tok_s"):
            lines += [f"# TYPE gvirt_{k} gauge", f"gvirt_{k} {s[k]}"]
        for k in ("ttft_s", "tpot_s", "latency_s"):
            for q, v in s[k].items():
                if v is not None:
                    lines.append(f'gvirt_{k}{{stat="{q}"}} {v}')
        return "\n".join(lines) + "\n"


def make_control_group(llm: LLM):
    """gloo group over the whole world for the serving control plane (pickled events). Collective:
    every rank calls it once, after building its engine. None for a single process."""
    import torch.distributed as dist
    if llm.ctx.world <= 1:
        return None
    return dist.new_group(ranks=list(range(llm.ctx.world)), backend="gloo")


def _find_request(llm: LLM, rid: int) -> Optional[Request]:
    for r in llm.scheduler.running:
        if r.req_id == rid:
            return r
    for r in llm.scheduler.waiting:
        if r.req_id == rid:
            return r
    return None


@dataclass
class _Remote:
    """Rank 0's view of a request that another data-parallel rank runs."""
    req_id: int
    prompt: List[int]
    params: SamplingParams
    output: List[int] = field(default_factory=list)
    finished: bool = False
    arrival: float = field(default_factory=time.perf_counter)
    first_token_time: Optional[float] = None
    token_times: List[float] = field(default_factory=list)


class _Owned:
    """Requests this rank runs, by global id, and how much of each has been reported."""

    def __init__(self, llm: LLM):
        self.llm = llm
        self.reqs: Dict[int, list] = {}      # gid -> [Request, tokens reported]

    def add(self, gid: int, prompt, params: SamplingParams) -> Request:
        rid = self.llm.add_request(prompt, params)
        req = next(r for r in reversed(self.llm.scheduler.waiting) if r.req_id == rid)
        self.reqs[gid] = [req, 0]
        return req

    def abort(self, gid: int) -> None:
        ent = self.reqs.pop(gid, None)
        if ent is not None and not ent[0].finished:
            self.llm.scheduler.abort(ent[0])

    def delta(self) -> dict:
        """{gid: (new tokens, finished)} since the last call; finished requests are dropped."""
        out = {}
        for gid in list(self.reqs):
            req, seen = self.reqs[gid]
            if len(req.output) > seen or req.finished:
                out[gid] = (req.output[seen:], req.finished)
                self.reqs[gid][1] = len(req.output)
            if req.finished:
                del self.reqs[gid]
        return out


def follower_loop(llm: LLM, control_group=None) -> int:
    """Ranks other than 0 of a multi-process replica: mirror rank 0's events and steps until it
    shuts down. Returns the number of steps taken."""
    import torch.distributed as dist
    group = control_group if control_group is not None else make_control_group(llm)
    ctx = llm.ctx
    owned = _Owned(llm)
    steps = 0
    while True:
        box = [None]
        dist.broadcast_object_list(box, src=0, group=group)
        ev = box[0]
        if ev.get("exit"):
            return steps
        for gid, dp_rank, prompt, params in ev["new"]:
            if dp_rank == ctx.dp_rank:
                try:
                    owned.add(gid, prompt, SamplingParams(**params))
                except (ValueError, RuntimeError):
                    pass        # rank 0 validated the same request with the same limits and dropped it
        for gid in ev["abort"]:
            owned.abort(gid)
        if ev["step"]:
            llm.step()
            steps += 1
            if ctx.dp > 1:
                # owners' tensor-parallel leaders report; everyone takes part in the gather
                report = owned.delta()
                dist.gather_object(report if ctx.tp_rank == 0 else {}, None, dst=0, group=group)


class QueueFull(RuntimeError):
    """More requests are waiting than the engine was told to accept (`max_pending`)."""


class AsyncEngine:
    def __init__(self, llm: LLM, idle_sleep_s: float = 0.001, health=None, control_group=None,
                 max_pending: int = 0):
        """With more than one process, construct on rank 0 only (the other ranks call
        ``follower_loop``); `control_group` defaults to a fresh gloo group (collective).
        `max_pending` > 0 bounds the requests that are queued or running; `submit` raises
        ``QueueFull`` beyond it (the HTTP layer answers 429)."""
        self.llm = llm
        self.max_pending = int(max_pending)
        self._pending = 0
        self._ctl = control_group if control_group is not None else make_control_group(llm)
        self._aborts: List[int] = []            # aborts decided on this rank that followers must mirror
        self._exit_sent = False
        self._owned = _Owned(llm)               # requests this rank's engine runs, by global id
        self._next_gid = 0
        self._load = [0] * max(llm.ctx.dp, 1)   # live requests per data-parallel rank
        self._dp_of: Dict[int, int] = {}
        self.metrics = ServingMetrics()
        self.health = health                    # optional parallel.health.Heartbeat
        self._inbox: List[_Pending] = []
        self._cancel: List[int] = []
        self._lock = threading.Lock()
        self._wake = threading.Event()
        self._stop = threading.Event()
        self._live: Dict[int, tuple] = {}       # req_id -> (Request, _Pending, tokens already streamed)
        self._idle_sleep = idle_sleep_s
        self.error: Optional[BaseException] = None
        self._thread = threading.Thread(target=self._loop, name="gvirt-engine", daemon=True)
        self._thread.start()

    # ------------------------------------------------------------------ client side (any thread)
    def submit(self, prompt: Sequence[int], params: Optional[SamplingParams] = None,
               on_token: Optional[Callable[[int, int], None]] = None,
               stop: Sequence[str] = (), export_after_prefill: bool = False,
               timeout_s: Optional[float] = None) -> Future:
        """Queue a request. The future resolves to a ``GenerationResult``; ``on_token(req_id,
        token)`` is called from the engine thread for every new token. ``future.request_id`` is
        set once the engine thread has admitted the request. With `export_after_prefill` the
        request leaves the engine right after its first token and the future resolves to its
        ``kv_transfer.KVPayload`` (prompt, first token, KV of every layer): the prefill half of
        disaggregated serving; `submit_payload` is the other half. `timeout_s` ends the request
        with finish reason "timeout" (and what it produced so far) that long after submission."""
        if export_after_prefill and self._ctl is not None:
            raise NotImplementedError("KV export over HTTP is for single-process replicas")
        if self.error is not None:
            raise RuntimeError("engine loop has stopped") from self.error
        params = params or SamplingParams()
        prompt = list(prompt)
        validate_request(prompt, params, self.llm.cfg.max_seq_len, self.llm.cfg.vocab_size)
        fut: Future = Future()
        with self._lock:
            if self.max_pending and self._pending >= self.max_pending:
                raise QueueFull(f"{self._pending} requests pending (limit {self.max_pending})")
            self._pending += 1
            p = _Pending(prompt, params, fut, on_token,
                         stop=tuple(x for x in stop if x), export=export_after_prefill)
            if timeout_s is not None:
                p.deadline = p.submitted + float(timeout_s)
            self._inbox.append(p)
            self.metrics.requests += 1
        fut.add_done_callback(self._one_less)
        self._wake.set()
        return fut

    def submit_payload(self, payload, on_token: Optional[Callable[[int, int], None]] = None,
                       stop: Sequence[str] = ()) -> Future:
        """Continue a request whose prefill ran elsewhere (``kv_transfer.KVPayload``): its KV is
        copied into this engine's cache between steps and it joins the next decode step. The
        result's output includes the token(s) the payload already carried."""
        if self.error is not None:
            raise RuntimeError("engine loop has stopped") from self.error
        if self._ctl is not None:
            raise NotImplementedError("KV import over HTTP is for single-process replicas")
        fut: Future = Future()
        with self._lock:
            if self.max_pending and self._pending >= self.max_pending:
                raise QueueFull(f"{self._pending} requests pending (limit {self.max_pending})")
            self._pending += 1
            self._inbox.append(_Pending(list(payload.prompt), payload.params, fut, on_token,
                                        stop=tuple(x for x in stop if x), payload=payload))
            self.metrics.requests += 1
        fut.add_done_callback(self._one_less)
        self._wake.set()
        return fut

    def _one_less(self, _fut) -> None:
        with self._lock:
            self._pending -= 1

    def cancel(self, request_id: int) -> None:
        with self._lock:
            self._cancel.append(request_id)
        self._wake.set()

    def generate(self, prompt: Sequence[int], params: Optional[SamplingParams] = None,
                 timeout: Optional[float] = None) -> GenerationResult:
        return self.submit(prompt, params).result(timeout)

    def shutdown(self) -> None:
        self._stop.set()
        self._wake.set()
        self._thread.join(timeout=30)
        if self._ctl is not None and not self._exit_sent:
            import torch.distributed as dist
            self._exit_sent = True
            dist.broadcast_object_list([{"exit": True}], src=0, group=self._ctl)

    # ------------------------------------------------------------------ engine thread
    def _admit(self):
        with self._lock:
            inbox, self._inbox = self._inbox, []
            cancels, self._cancel = self._cancel, []
        new = []
        my_dp = self.llm.ctx.dp_rank
        for p in inbox:
            gid = self._next_gid
            self._next_gid += 1
            dp_rank = min(range(len(self._load)), key=lambda d: (self._load[d], d))
            self._load[dp_rank] += 1
            if p.payload is not None:
                from ..engine.kv_transfer import import_request
                try:
                    rid = import_request(self.llm, p.payload)
                except (RuntimeError, ValueError) as e:      # no room / mismatching engine: the client's error
                    self._load[dp_rank] -= 1
                    p.future.set_exception(e)
                    continue
                req = next(r for r in self.llm.scheduler.running if r.req_id == rid)
                self._owned.reqs[gid] = [req, 0]
                p.payload = None
            elif dp_rank == my_dp:
                try:
                    req = self._owned.add(gid, p.prompt, p.params)
                except (ValueError, RuntimeError) as e:     # a bad request fails alone, the engine goes on
                    self._load[dp_rank] -= 1
                    p.future.set_exception(e)
                    continue
            else:
                req = _Remote(gid, p.prompt, p.params)
            p.future.request_id = gid
            self._live[gid] = (req, p, 0)
            self._dp_of[gid] = dp_rank
            new.append((gid, dp_rank, p.prompt, dataclasses.asdict(p.params)))
        aborts, self._aborts = self._aborts, []
        for gid in cancels:
            ent = self._live.pop(gid, None)
            if ent is None:
                continue
            req, p, _ = ent
            self._drop(gid)
            aborts.append(gid)
            self.metrics.cancelled += 1
            self._resolve(req, p, "cancelled")
        if self._ctl is not None:
            import torch.distributed as dist
            dist.broadcast_object_list([{"new": new, "abort": aborts, "step": bool(self._live)}], src=0,
                                       group=self._ctl)

    def _drop(self, gid: int) -> None:
        """Forget a request that ends before its engine finished it (cancel, stop string)."""
        self._owned.abort(gid)
        d = self._dp_of.pop(gid, None)
        if d is not None:
            self._load[d] -= 1

    def _collect_remote(self) -> None:
        """After a step with data-parallel ranks: take in the owners' new tokens."""
        import torch.distributed as dist
        self._owned.delta()          # keeps this rank's own bookkeeping current (nothing to send)
        reports = [None] * self.llm.ctx.world
        dist.gather_object({}, reports, dst=0, group=self._ctl)
        now = time.perf_counter()
        for rep in reports:
            for gid, (toks, finished) in (rep or {}).items():
                ent = self._live.get(gid)
                if ent is None:
                    continue          # ended here already (cancelled / stopped): the abort is on its way
                req = ent[0]
                if toks:
                    if req.first_token_time is None:
                        req.first_token_time = now
                    req.output.extend(toks)
                    req.token_times.extend([now] * len(toks))
                req.finished = req.finished or finished

    def _resolve(self, req: Request, p: _Pending, reason: str, text: Optional[str] = None):
        now = time.perf_counter()
        ttft = (req.first_token_time - req.arrival) if req.first_token_time else None
        tpot = None
        if len(req.token_times) > 1:
            tpot = (req.token_times[-1] - req.token_times[0]) / (len(req.token_times) - 1)
        if text is None and self.llm.tokenizer is not None:
            text = self.llm.tokenizer.decode(req.output)
        res = GenerationResult(req.req_id, p.prompt, list(req.output), reason, ttft, tpot, now - p.submitted, text,
                               list(getattr(req, "logprobs", None) or []) or None)
        if reason != "cancelled":
            self.metrics.record(res)
        if not p.future.done():
            p.future.set_result(res)

    def _stream_and_finish(self):
        done = []
        stopped = []
        exported = []
        timed_out = []
        for rid, (req, p, seen) in self._live.items():
            if p.on_token is not None:
                for tok in req.output[seen:]:
                    try:
                        p.on_token(rid, tok)
                    except Exception:  # noqa: BLE001 - a broken client callback must not stop the engine
                        pass
            grew = len(req.output) > seen
            self._live[rid] = (req, p, len(req.output))
            if p.export and req.output and not req.finished:
                exported.append(rid)
                continue
            if p.deadline is not None and not req.finished and time.perf_counter() > p.deadline:
                timed_out.append(rid)
                continue
            if p.stop and grew and self.llm.tokenizer is not None:
                text = self.llm.tokenizer.decode(req.output)
                cut = min((i for i in (text.find(x) for x in p.stop) if i >= 0), default=-1)
                if cut >= 0:
                    stopped.append((rid, text[:cut]))
                    continue
            if req.finished:
                done.append(rid)
        for rid in exported:
            from ..engine.kv_transfer import export_request
            req, p, _ = self._live.pop(rid)
            payload = export_request(self.llm, req.req_id, release=True)
            self._owned.reqs.pop(rid, None)
            d = self._dp_of.pop(rid, None)
            if d is not None:
                self._load[d] -= 1
            if not p.future.done():
                p.future.set_result(payload)
        for rid in timed_out:
            req, p, _ = self._live.pop(rid)
            self._aborts.append(rid)
            self._drop(rid)
            self._resolve(req, p, "timeout")
        for rid, text in stopped:
            req, p, _ = self._live.pop(rid)
            if not req.finished:
                self._aborts.append(rid)           # its owner (or every mirror) aborts before the next step
            self._drop(rid)                        # frees its blocks here; nothing of it is in flight between steps
            self._resolve(req, p, "stop", text)
        for rid in done:
            req, p, _ = self._live.pop(rid)
            self._drop(rid)
            n = len(req.output)
            reason = "length" if n >= req.params.max_tokens else "stop"
            self._resolve(req, p, reason)

    def _loop(self):
        try:
            while not self._stop.is_set():
                self._admit()
                if not self._live:
                    self._wake.wait(0.05)
                    self._wake.clear()
                    continue
                if self.health is not None:
                    self.health.check()          # a lost peer is reported before the next launch
                self.llm.step()
                if self._ctl is not None and self.llm.ctx.dp > 1:
                    self._collect_remote()
                self._stream_and_finish()
        except BaseException as e:  # noqa: BLE001 - surfaced to every waiting client
            self.error = e
            for rid, (req, p, _) in list(self._live.items()):
                if not p.future.done():
                    p.future.set_exception(e)
            self._live.clear()
            with self._lock:
                for p in self._inbox:
                    p.future.set_exception(e)
                self._inbox = []
            if self._ctl is not None and not self._exit_sent:
                # Best effort, from a thread of its own: followers that are between iterations get
                # the exit; one that already entered the failed step's collectives is released by
                # the process-group time-out or by this process going away, not by this message.
                self._exit_sent = True

                def tell():
                    try:
                        import torch.distributed as dist
                        dist.broadcast_object_list([{"exit": True}], src=0, group=self._ctl)
                    except Exception:  # noqa: BLE001 - the process group itself may be what failed
                        pass
                threading.Thread(target=tell, daemon=True).start()
