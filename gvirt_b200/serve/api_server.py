"""OpenAI-style HTTP front end.

    python -m gvirt_b200.serve.api_server --model /path/to/hf_dir --port 8000
    python -m gvirt_b200.serve.api_server --preset qwen3-0.6b --port 8000        # random weights

Endpoints
  POST /v1/completions        {"prompt": "text" | [ids] | [[ids], ...], "max_tokens", "temperature",
                               "top_p", "top_k", "stop_token_ids", "stop", "n", "echo", "logprobs", "presence_penalty",
                               "frequency_penalty", "repetition_penalty", "ignore_eos", "stream"}
  POST /v1/chat/completions   {"messages": [...]} (needs a tokenizer with a chat template)
  POST /v1/prefill, /v1/decode         the two halves of disaggregated serving (serve/disagg.py)
  GET  /v1/models, /health, /metrics (Prometheus text), /stats (JSON)
  POST /start_profile, /stop_profile   torch.profiler trace of the engine thread's work, the
                                       hooks the reference's benchmark scripts drive
                                       (xlite/tests/e2e/online_server_test.sh:69-98)

The reference has no server of its own: it plugs into an external serving framework
(xlite/tests/e2e/online_api_server.sh:44-105). This is the stand-alone equivalent on top of
``AsyncEngine`` (continuous batching, chunked prefill, prefix cache). A tensor- / expert-parallel
replica is launched with ``torch.distributed.run`` (one process per GPU): rank 0 serves HTTP and
broadcasts every iteration's requests and aborts, the other ranks mirror them
(``async_engine.follower_loop``):

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m gvirt_b200.serve.api_server --preset qwen2.5-72b --port 8000
    ... -m gvirt_b200.serve.api_server --preset deepseek-v3 --dp 8 --port 8000   # DP attention + EP experts

With ``--dp`` every request runs on one data-parallel rank (the least loaded) and its tokens
travel back to rank 0 after every step.
"""
from __future__ import annotations

import argparse
import asyncio
import json
import os
import time
import uuid
from typing import List, Optional

import torch

from ..engine.scheduler import SamplingParams
from .async_engine import AsyncEngine, GenerationResult, QueueFull

try:        # annotations of route handlers are resolved against the module's globals
    from fastapi import Request as HTTPRequest
except ImportError:     # the server needs FastAPI; importing this module does not
    HTTPRequest = None


def build_app(engine: AsyncEngine, model_name: str = "gvirt"):
    from fastapi import FastAPI, HTTPException
    from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

    app = FastAPI(title="gvirt_b200")
    llm = engine.llm
    prof = {"p": None}

    def _n_logprobs(body: dict) -> int:
        lp = body.get("logprobs")
        if lp is True:                       # chat style: logprobs + top_logprobs
            lp = int(body.get("top_logprobs", 1) or 1)
        n = int(lp or 0)
        if n < 0 or n > 20:
            raise HTTPException(400, "logprobs must be between 0 and 20")
        return n

    def _logprobs(r: GenerationResult):
        if not r.logprobs:
            return None
        name = (lambda t: llm.tokenizer.decode([t])) if llm.tokenizer is not None else str
        return {"tokens": [name(t) for t in r.output_ids[:len(r.logprobs)]],
                "token_logprobs": [lp for lp, _ in r.logprobs],
                "top_logprobs": [{name(t): v for t, v in top} for _, top in r.logprobs]}

    def _params(body: dict) -> SamplingParams:
        try:
            return _params_unchecked(body)
        except (TypeError, ValueError) as e:        # "max_tokens": "many", "stop_token_ids": 5, ...
            raise HTTPException(400, f"bad sampling parameter: {e}")

    def _params_unchecked(body: dict) -> SamplingParams:
        return SamplingParams(max_tokens=int(body.get("max_tokens", 16)),
                              temperature=float(body.get("temperature", 0.0)),
                              top_k=int(body.get("top_k", 0)), top_p=float(body.get("top_p", 1.0)),
                              stop_token_ids=tuple(body.get("stop_token_ids", ())),
                              ignore_eos=bool(body.get("ignore_eos", False)),
                              logprobs=_n_logprobs(body),
                              presence_penalty=float(body.get("presence_penalty", 0.0) or 0.0),
                              frequency_penalty=float(body.get("frequency_penalty", 0.0) or 0.0),
                              repetition_penalty=float(body.get("repetition_penalty", 1.0) or 1.0))

    def _prompts(p) -> List[List[int]]:
        if isinstance(p, str):
            p = [p]
        if isinstance(p, list) and p and all(isinstance(t, int) for t in p):
            p = [p]
        out = []
        for item in p or []:
            if isinstance(item, str):
                if llm.tokenizer is None:
                    raise HTTPException(400, "text prompts need a tokenizer; send token ids")
                out.append(llm.tokenizer.encode(item))
            elif isinstance(item, list) and all(isinstance(t, int) for t in item):
                out.append(item)
            else:
                raise HTTPException(400, "prompt must be a string, a list of ids, or a list of those")
        if not out:
            raise HTTPException(400, "empty prompt")
        return out

    def _text(ids: List[int]) -> Optional[str]:
        return llm.tokenizer.decode(ids) if llm.tokenizer is not None else None

    def _choice(i: int, r: GenerationResult, echo: str = "") -> dict:
        text = r.text if r.text is not None else _text(r.output_ids)
        return {"index": i, "text": (echo + text) if (echo and text is not None) else text,
                "token_ids": r.output_ids, "finish_reason": r.finish_reason, "logprobs": _logprobs(r)}

    def _stops(body: dict) -> tuple:
        st = body.get("stop") or ()
        if isinstance(st, str):
            st = (st,)
        if st and llm.tokenizer is None:
            raise HTTPException(400, "stop strings need a tokenizer; use stop_token_ids")
        return tuple(st)

    async def _run(prompts: List[List[int]], sp: SamplingParams, stop: tuple = (),
                   timeout_s: Optional[float] = None) -> List[GenerationResult]:
        try:
            futs = [asyncio.wrap_future(engine.submit(p, sp, stop=stop, timeout_s=timeout_s)) for p in prompts]
        except ValueError as e:
            raise HTTPException(400, str(e))
        except QueueFull as e:
            raise HTTPException(429, str(e))
        return list(await asyncio.gather(*futs))

    @app.get("/health")
    async def health():
        if engine.error is not None:
            return JSONResponse({"status": "error", "error": repr(engine.error)}, status_code=503)
        return {"status": "ok"}

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": model_name, "object": "model", "owned_by": "gvirt_b200",
                                             "max_model_len": llm.cfg.max_seq_len}]}

    @app.get("/metrics")
    async def metrics():
        text = engine.metrics.prometheus()
        for k in ("spec_steps", "spec_drafted", "spec_accepted", "prepared_steps"):
            text += f"# TYPE gvirt_{k}_total counter\ngvirt_{k}_total {llm.stats.get(k, 0)}\n"
        sch = llm.scheduler
        gauges = {"requests_running": len(sch.running), "requests_waiting": len(sch.waiting),
                  "kv_blocks_free": sch.bm.num_free_blocks, "kv_blocks_total": llm.num_blocks,
                  "preemptions_total": sch.num_preemptions, "prefix_cache_hits_total": sch.bm.prefix_hits,
                  "prefix_cache_queries_total": sch.bm.prefix_queries}
        if llm.kv_pool is not None:
            ps = llm.kv_pool.stats()
            gauges.update(kv_pool_resident_blocks=ps["resident_blocks"], kv_pool_saves_total=ps["saves"],
                          kv_pool_loads_total=ps["loads"])
        for k, v in gauges.items():
            kind = "counter" if k.endswith("_total") else "gauge"
            text += f"# TYPE gvirt_{k} {kind}\ngvirt_{k} {v}\n"
        return PlainTextResponse(text)

    @app.get("/stats")
    async def stats():
        s = engine.metrics.snapshot()
        s["engine"] = dict(llm.stats)
        s["kv_blocks_free"] = llm.scheduler.bm.num_free_blocks
        s["kv_blocks_total"] = llm.num_blocks
        s["prefix_cache_hits"] = llm.scheduler.bm.prefix_hits
        s["preemptions"] = llm.scheduler.num_preemptions
        if llm.kv_pool is not None:
            s["kv_pool"] = llm.kv_pool.stats()
        return s

    @app.post("/v1/completions")
    async def completions(body: dict):
        prompts = _prompts(body.get("prompt"))
        sp = _params(body)
        stop = _stops(body)
        n = int(body.get("n", 1))
        if n < 1 or n > 16:
            raise HTTPException(400, "n must be between 1 and 16")
        if n > 1:
            prompts = [p for p in prompts for _ in range(n)]      # choices are grouped by prompt
        rid = "cmpl-" + uuid.uuid4().hex[:24]
        if body.get("stream"):
            if len(prompts) != 1:
                raise HTTPException(400, "streaming takes a single prompt")
            loop = asyncio.get_running_loop()
            q: asyncio.Queue = asyncio.Queue()
            try:
                fut = engine.submit(prompts[0], sp, stop=stop,
                                    on_token=lambda _r, tok: loop.call_soon_threadsafe(q.put_nowait, tok))
            except ValueError as e:
                raise HTTPException(400, str(e))
            except QueueFull as e:
                raise HTTPException(429, str(e))
            fut.add_done_callback(lambda f: loop.call_soon_threadsafe(q.put_nowait, None))

            async def gen():
                try:
                    while True:
                        tok = await q.get()
                        if tok is None:
                            break
                        chunk = {"id": rid, "object": "text_completion", "model": model_name,
                                 "choices": [{"index": 0, "text": _text([tok]), "token_ids": [tok],
                                              "finish_reason": None}]}
                        yield f"data: {json.dumps(chunk)}\n\n"
                    res = fut.result()
                    tail = {"id": rid, "object": "text_completion", "model": model_name,
                            "choices": [{"index": 0, "text": "", "token_ids": [],
                                         "finish_reason": res.finish_reason}]}
                    yield f"data: {json.dumps(tail)}\n\ndata: [DONE]\n\n"
                finally:
                    if not fut.done() and getattr(fut, "request_id", None) is not None:
                        engine.cancel(fut.request_id)       # client went away mid-stream
            return StreamingResponse(gen(), media_type="text/event-stream")
        results = await _run(prompts, sp, stop, body.get("timeout"))
        echo = bool(body.get("echo")) and llm.tokenizer is not None
        return {"id": rid, "object": "text_completion", "created": int(time.time()), "model": model_name,
                "choices": [_choice(i, r, _text(r.prompt_ids) if echo else "") for i, r in enumerate(results)],
                "usage": {"prompt_tokens": sum(len(r.prompt_ids) for r in results),
                          "completion_tokens": sum(len(r.output_ids) for r in results),
                          "total_tokens": sum(len(r.prompt_ids) + len(r.output_ids) for r in results)}}

    # ---- disaggregated prefill (serve/disagg.py): this instance as the prefill or the decode half
    @app.post("/v1/prefill")
    async def prefill(body: dict):
        from fastapi import Response
        from .disagg import payload_to_bytes
        prompts = _prompts(body.get("prompt"))
        if len(prompts) != 1:
            raise HTTPException(400, "one prompt per prefill call")
        try:
            fut = engine.submit(prompts[0], _params(body), export_after_prefill=True)
        except (ValueError, NotImplementedError) as e:
            raise HTTPException(400, str(e))
        res = await asyncio.wrap_future(fut)
        if isinstance(res, GenerationResult):       # finished on its first token: nothing left to decode
            raise HTTPException(409, "the request finished during prefill")
        return Response(content=payload_to_bytes(res), media_type="application/octet-stream")

    @app.post("/v1/decode")
    async def decode(request: HTTPRequest):
        from .disagg import payload_from_bytes
        blob = await request.body()
        try:
            payload = payload_from_bytes(blob)
        except Exception as e:  # noqa: BLE001 - anything unreadable is the client's error
            raise HTTPException(400, f"unreadable KV payload: {e!r}")
        stop = tuple(request.query_params.getlist("stop"))
        if stop and llm.tokenizer is None:
            raise HTTPException(400, "stop strings need a tokenizer; use stop_token_ids")
        try:
            res = await asyncio.wrap_future(engine.submit_payload(payload, stop=stop))
        except (RuntimeError, ValueError, NotImplementedError) as e:
            raise HTTPException(503 if isinstance(e, RuntimeError) else 400, str(e))
        return {"id": "cmpl-" + uuid.uuid4().hex[:24], "object": "text_completion", "created": int(time.time()),
                "model": model_name, "choices": [_choice(0, res)],
                "usage": {"prompt_tokens": len(res.prompt_ids), "completion_tokens": len(res.output_ids),
                          "total_tokens": len(res.prompt_ids) + len(res.output_ids)}}

    @app.post("/v1/chat/completions")
    async def chat(body: dict):
        tok = llm.tokenizer
        if tok is None or not hasattr(tok, "apply_chat_template"):
            raise HTTPException(400, "chat completions need a tokenizer with a chat template")
        ids = list(tok.apply_chat_template(body.get("messages", []), add_generation_prompt=True, tokenize=True))
        sp, stop = _params(body), _stops(body)
        cid = "chatcmpl-" + uuid.uuid4().hex[:24]
        if body.get("stream"):
            loop = asyncio.get_running_loop()
            q: asyncio.Queue = asyncio.Queue()
            try:
                fut = engine.submit(ids, sp, stop=stop,
                                    on_token=lambda _r, t: loop.call_soon_threadsafe(q.put_nowait, t))
            except ValueError as e:
                raise HTTPException(400, str(e))
            except QueueFull as e:
                raise HTTPException(429, str(e))
            fut.add_done_callback(lambda f: loop.call_soon_threadsafe(q.put_nowait, None))

            async def gen():
                try:
                    first = {"id": cid, "object": "chat.completion.chunk", "model": model_name,
                             "choices": [{"index": 0, "delta": {"role": "assistant"}, "finish_reason": None}]}
                    yield f"data: {json.dumps(first)}\n\n"
                    while True:
                        t = await q.get()
                        if t is None:
                            break
                        chunk = {"id": cid, "object": "chat.completion.chunk", "model": model_name,
                                 "choices": [{"index": 0, "delta": {"content": _text([t])}, "finish_reason": None}]}
                        yield f"data: {json.dumps(chunk)}\n\n"
                    res = fut.result()
                    tail = {"id": cid, "object": "chat.completion.chunk", "model": model_name,
                            "choices": [{"index": 0, "delta": {}, "finish_reason": res.finish_reason}]}
                    yield f"data: {json.dumps(tail)}\n\ndata: [DONE]\n\n"
                finally:
                    if not fut.done() and getattr(fut, "request_id", None) is not None:
                        engine.cancel(fut.request_id)
            return StreamingResponse(gen(), media_type="text/event-stream")
        res = (await _run([ids], sp, stop))[0]
        content = res.text if res.text is not None else _text(res.output_ids)
        return {"id": cid, "object": "chat.completion",
                "created": int(time.time()), "model": model_name,
                "choices": [{"index": 0, "message": {"role": "assistant", "content": content},
                             "finish_reason": res.finish_reason}],
                "usage": {"prompt_tokens": len(res.prompt_ids), "completion_tokens": len(res.output_ids),
                          "total_tokens": len(res.prompt_ids) + len(res.output_ids)}}

    @app.post("/start_profile")
    async def start_profile():
        if prof["p"] is not None:
            raise HTTPException(409, "a profile is already running")
        from torch.profiler import ProfilerActivity, profile
        acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
        prof["p"] = profile(activities=acts)
        prof["p"].__enter__()
        return {"status": "started"}

    @app.post("/stop_profile")
    async def stop_profile(body: Optional[dict] = None):
        p = prof["p"]
        if p is None:
            raise HTTPException(409, "no profile is running")
        p.__exit__(None, None, None)
        prof["p"] = None
        path = (body or {}).get("path") or os.path.join(os.getcwd(), f"gvirt_trace_{int(time.time())}.json")
        p.export_chrome_trace(path)
        return {"status": "stopped", "trace": path}

    return app


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    src = ap.add_mutually_exclusive_group(required=True)
    src.add_argument("--model")
    src.add_argument("--preset")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--device", default=None)
    ap.add_argument("--max-batch-size", type=int, default=0)
    ap.add_argument("--max-seq-len", type=int, default=0)
    ap.add_argument("--max-num-batched-tokens", type=int, default=0)
    ap.add_argument("--prefix-cache", action="store_true")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.9)
    ap.add_argument("--spec-tokens", type=int, default=0,
                    help="speculative decoding: prompt-lookup drafts per request and step (0 = off)")
    ap.add_argument("--spec-ngram-max", type=int, default=4)
    ap.add_argument("--spec-method", default="ngram", choices=["ngram", "mtp"],
                    help="draft source: prompt lookup, or the checkpoint's multi-token-prediction module")
    ap.add_argument("--dp", type=int, default=1,
                    help="data-parallel attention ranks of a multi-process replica (MoE models: experts stay "
                         "spread over all ranks); tensor-parallel size = processes / dp")
    ap.add_argument("--mixed-batches", action="store_true",
                    help="decoding requests ride along with prefill chunks instead of waiting for them")
    ap.add_argument("--no-warmup", action="store_true", help="do not capture the decode graphs at start-up")
    ap.add_argument("--max-pending", type=int, default=0,
                    help="answer 429 when this many requests are queued or running (0 = no limit)")
    ap.add_argument("--kv-pool-gb", type=float, default=0.0,
                    help="host-memory KV pool behind the prefix cache, in GiB (needs --prefix-cache)")
    a = ap.parse_args()
    import uvicorn
    from ..engine.llm import LLM
    from ..models import presets
    over = {}
    if a.max_batch_size:
        over["max_batch_size"] = a.max_batch_size
    if a.max_seq_len:
        over["max_seq_len"] = a.max_seq_len
    if a.max_num_batched_tokens:
        over["max_num_batched_tokens"] = a.max_num_batched_tokens
    kw = dict(enable_prefix_cache=a.prefix_cache, use_graphs=not a.no_graph,
              gpu_memory_utilization=a.gpu_memory_utilization)
    if a.kv_pool_gb > 0:
        kw["kv_pool_gb"] = a.kv_pool_gb
    if a.mixed_batches:
        kw["mixed_batches"] = True
    if a.spec_method == "mtp":
        kw["speculative"] = dict(method="mtp", num_tokens=max(a.spec_tokens, 1))
    elif a.spec_tokens > 0:
        kw["speculative"] = dict(method="ngram", num_tokens=a.spec_tokens, ngram_max=a.spec_ngram_max)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    ctx = None
    if world > 1:
        from ..parallel import state as pstate
        from ..parallel.setup import attach_device_comm
        probe = presets.get(a.preset) if a.preset else None
        if probe is None:
            from ..config import ModelConfig
            probe = ModelConfig.from_pretrained(a.model)
        ep = world if probe.is_moe else 1
        if world % max(a.dp, 1):
            raise SystemExit(f"--dp {a.dp} does not divide the {world} processes")
        tp = world // max(a.dp, 1)
        ctx = pstate.init_parallel(tp=tp, dp=a.dp, ep=ep, moe_tp=world // ep, device=a.device)
        over.update(tp_size=tp, dp_size=a.dp, ep_size=ep)
    if a.preset:
        cfg = presets.get(a.preset, **over)
        if ctx is not None:
            attach_device_comm(ctx, cfg)
        llm = LLM.from_config(cfg, ctx, device=a.device, shard_from_full=False, **kw)
        name = a.preset
    else:
        llm = LLM.from_pretrained(a.model, ctx, device=a.device, config_overrides=over, **kw)
        if ctx is not None:
            attach_device_comm(ctx, llm.cfg)
        name = os.path.basename(os.path.normpath(a.model))
    if not a.no_warmup:
        llm.warmup(seq_lens=(min(1024, llm.cfg.max_seq_len), llm.cfg.max_seq_len))
    if ctx is not None and ctx.rank != 0:
        from .async_engine import follower_loop
        follower_loop(llm)
        return 0
    engine = AsyncEngine(llm, max_pending=a.max_pending)
    try:
        uvicorn.run(build_app(engine, name), host=a.host, port=a.port, log_level="info")
    finally:
        engine.shutdown()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
