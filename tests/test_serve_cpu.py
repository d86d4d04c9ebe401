"""Serving layer on CPU with the tiny fp32 model: the async engine loop (concurrent submissions,
streaming callbacks, cancellation, metrics) and the HTTP front end through an in-process client.
Greedy outputs must equal what the synchronous engine produces for the same prompts."""
import json
import threading

import pytest

from gvirt_b200.engine.llm import LLM
from gvirt_b200.engine.scheduler import SamplingParams
from gvirt_b200.models import presets
from gvirt_b200.serve import AsyncEngine
from gvirt_b200.serve.api_server import build_app


def _llm(**kw):
    cfg = presets.get("tiny-qwen2", max_batch_size=4, max_seq_len=128, max_num_batched_tokens=64)
    return LLM.from_config(cfg, seed=0, device="cpu", **kw)


PROMPTS = [[1, 2, 3, 4], [9, 8, 7], list(range(20, 60)), [5]]


@pytest.fixture(scope="module")
def golden():
    llm = _llm()
    return [o.output for o in llm.generate(PROMPTS, SamplingParams(max_tokens=12, ignore_eos=True))]


def test_async_engine_concurrent_submit_stream_and_metrics(golden):
    eng = AsyncEngine(_llm())
    try:
        streamed = {i: [] for i in range(len(PROMPTS))}
        futs = [None] * len(PROMPTS)

        def client(i):
            futs[i] = eng.submit(PROMPTS[i], SamplingParams(max_tokens=12, ignore_eos=True),
                                 on_token=lambda rid, tok, i=i: streamed[i].append(tok))

        ths = [threading.Thread(target=client, args=(i,)) for i in range(len(PROMPTS))]
        [t.start() for t in ths]
        [t.join() for t in ths]
        res = [f.result(timeout=120) for f in futs]
        assert [r.output_ids for r in res] == golden
        assert [streamed[i] for i in range(len(PROMPTS))] == golden
        assert all(r.finish_reason == "length" and r.ttft_s is not None for r in res)
        snap = eng.metrics.snapshot()
        assert snap["finished"] == len(PROMPTS) and snap["output_tokens"] == 12 * len(PROMPTS)
        assert "gvirt_finished_total 4" in eng.metrics.prometheus()
        with pytest.raises(ValueError):
            eng.submit([])
    finally:
        eng.shutdown()


def test_async_engine_cancel_frees_blocks():
    llm = _llm()
    eng = AsyncEngine(llm)
    try:
        seen = threading.Event()
        fut = eng.submit([1, 2, 3], SamplingParams(max_tokens=100, ignore_eos=True),
                         on_token=lambda rid, tok: seen.set())
        assert seen.wait(60)
        eng.cancel(fut.request_id)
        res = fut.result(timeout=60)
        assert res.finish_reason == "cancelled" and 0 < len(res.output_ids) < 100
        # the engine keeps serving and the cancelled request's blocks are back
        out = eng.generate([4, 5, 6], SamplingParams(max_tokens=4, ignore_eos=True), timeout=60)
        assert len(out.output_ids) == 4
        assert llm.scheduler.bm.num_free_blocks == llm.num_blocks
    finally:
        eng.shutdown()


def test_http_completions_stream_and_errors(golden):
    from starlette.testclient import TestClient
    eng = AsyncEngine(_llm())
    try:
        with TestClient(build_app(eng, "tiny")) as c:
            assert c.get("/health").json() == {"status": "ok"}
            assert c.get("/v1/models").json()["data"][0]["id"] == "tiny"
            r = c.post("/v1/completions", json={"prompt": PROMPTS[:2], "max_tokens": 12, "ignore_eos": True})
            assert r.status_code == 200, r.text
            body = r.json()
            assert [ch["token_ids"] for ch in body["choices"]] == golden[:2]
            assert body["usage"]["completion_tokens"] == 24
            # streaming: server-sent events, one token per event, then [DONE]
            toks = []
            with c.stream("POST", "/v1/completions",
                          json={"prompt": PROMPTS[2], "max_tokens": 12, "ignore_eos": True, "stream": True}) as s:
                for line in s.iter_lines():
                    if line.startswith("data: ") and line != "data: [DONE]":
                        toks += json.loads(line[6:])["choices"][0]["token_ids"]
            assert toks == golden[2]
            assert c.post("/v1/completions", json={"prompt": "text needs a tokenizer"}).status_code == 400
            assert c.post("/v1/completions", json={"prompt": []}).status_code == 400
            assert c.post("/v1/chat/completions", json={"messages": []}).status_code == 400
            m = c.get("/metrics").text
            assert "gvirt_output_tokens_total" in m and "gvirt_requests_running 0" in m
            assert "gvirt_kv_blocks_free" in m and "gvirt_prefix_cache_queries_total" in m
            st = c.get("/stats").json()
            assert st["kv_blocks_free"] == st["kv_blocks_total"]
    finally:
        eng.shutdown()


class _ToyTokenizer:
    """Token id i <-> the word "w<i>"; enough to exercise text prompts, stop strings, echo and chat."""

    def encode(self, text):
        return [int(w[1:]) for w in text.split()]

    def decode(self, ids):
        return " ".join(f"w{i}" for i in ids)

    def apply_chat_template(self, messages, add_generation_prompt=True, tokenize=True):
        ids = []
        for m in messages:
            ids += [1] + self.encode(m["content"])
        return ids + [2]


def test_http_stop_strings_n_echo_and_chat_stream(golden):
    from starlette.testclient import TestClient
    llm = _llm()
    llm.tokenizer = _ToyTokenizer()
    eng = AsyncEngine(llm)
    try:
        with TestClient(build_app(eng, "tiny")) as c:
            text_prompt = " ".join(f"w{i}" for i in PROMPTS[0])
            full = c.post("/v1/completions", json={"prompt": text_prompt, "max_tokens": 12, "ignore_eos": True}).json()
            assert full["choices"][0]["token_ids"] == golden[0]
            words = full["choices"][0]["text"].split()
            # stop string = the 5th generated word: the text ends before it and generation stops early
            stop = words[4]
            gen_text = full["choices"][0]["text"]
            cut = gen_text.find(stop)                 # substring match, like the server's
            first = len(gen_text[:cut].split())       # words wholly before the match
            r = c.post("/v1/completions", json={"prompt": text_prompt, "max_tokens": 12, "ignore_eos": True,
                                                "stop": [stop, "never-there"], "echo": True}).json()
            ch = r["choices"][0]
            assert ch["finish_reason"] == "stop"
            assert ch["text"] == text_prompt + gen_text[:cut]
            assert first + 1 <= len(ch["token_ids"]) < 12            # stopped as soon as the string appeared
            st = c.get("/stats").json()
            assert st["kv_blocks_free"] == st["kv_blocks_total"]      # the stopped request gave its blocks back
            # n choices per prompt (greedy: identical), grouped by prompt
            r = c.post("/v1/completions", json={"prompt": [PROMPTS[0], PROMPTS[1]], "n": 2, "max_tokens": 12,
                                                "ignore_eos": True}).json()
            assert [x["token_ids"] for x in r["choices"]] == [golden[0], golden[0], golden[1], golden[1]]
            assert c.post("/v1/completions", json={"prompt": PROMPTS[0], "n": 0}).status_code == 400
            # log-probabilities of the chosen token and the two most likely ones
            r = c.post("/v1/completions", json={"prompt": PROMPTS[0], "max_tokens": 5, "ignore_eos": True,
                                                "logprobs": 2}).json()
            lp = r["choices"][0]["logprobs"]
            assert r["choices"][0]["token_ids"] == golden[0][:5]
            assert lp["tokens"] == [f"w{t}" for t in golden[0][:5]] and len(lp["top_logprobs"][0]) == 2
            assert all(v <= 0 for v in lp["token_logprobs"])
            assert all(abs(max(d.values()) - v) < 1e-6 for d, v in zip(lp["top_logprobs"], lp["token_logprobs"]))
            assert c.post("/v1/completions", json={"prompt": PROMPTS[0], "logprobs": 99}).status_code == 400
            # chat: plain and streamed
            msgs = [{"role": "user", "content": "w7 w8 w9"}]
            plain = c.post("/v1/chat/completions", json={"messages": msgs, "max_tokens": 6, "ignore_eos": True}).json()
            content = plain["choices"][0]["message"]["content"]
            assert len(content.split()) == 6 and plain["usage"]["prompt_tokens"] == 5
            pieces, roles, finish = [], [], None
            with c.stream("POST", "/v1/chat/completions",
                          json={"messages": msgs, "max_tokens": 6, "ignore_eos": True, "stream": True}) as s:
                for line in s.iter_lines():
                    if line.startswith("data: ") and line != "data: [DONE]":
                        d = json.loads(line[6:])["choices"][0]
                        roles.append(d["delta"].get("role"))
                        if d["delta"].get("content"):
                            pieces.append(d["delta"]["content"])
                        finish = d["finish_reason"] or finish
            assert " ".join(pieces) == content and roles[0] == "assistant" and finish == "length"
    finally:
        eng.shutdown()
    # stop strings without a tokenizer are refused
    eng2 = AsyncEngine(_llm())
    try:
        with TestClient(build_app(eng2, "tiny")) as c:
            assert c.post("/v1/completions", json={"prompt": PROMPTS[0], "stop": "x"}).status_code == 400
    finally:
        eng2.shutdown()


def test_disaggregated_prefill_over_http(golden):
    """Prefill on one server, decode on another: the KV payload travels as bytes, the chained
    completion equals the one-engine answer, both engines end with all blocks free."""
    from starlette.testclient import TestClient
    from gvirt_b200.serve import disagg
    llm_p, llm_d = _llm(), _llm()
    llm_d.tokenizer = _ToyTokenizer()
    eng_p, eng_d = AsyncEngine(llm_p), AsyncEngine(llm_d)
    try:
        with TestClient(build_app(eng_p, "tiny")) as cp, TestClient(build_app(eng_d, "tiny")) as cd:
            def post_prefill(body):
                r = cp.post("/v1/prefill", json=body)
                assert r.status_code == 200, r.text
                return r.content

            def post_decode(blob, stop):
                r = cd.post("/v1/decode", content=blob, params=[("stop", s) for s in stop],
                            headers={"Content-Type": "application/octet-stream"})
                assert r.status_code == 200, r.text
                return r.json()

            for i in (0, 2):
                out = disagg.chain(post_prefill, post_decode, {"prompt": PROMPTS[i], "max_tokens": 12, "ignore_eos": True})
                assert out["choices"][0]["token_ids"] == golden[i]
                assert out["usage"]["prompt_tokens"] == len(PROMPTS[i])
            # the payload really carries the cache: its size grows with the prompt
            small, big = post_prefill({"prompt": PROMPTS[3], "max_tokens": 4}), post_prefill({"prompt": PROMPTS[2], "max_tokens": 4})
            assert len(big) > len(small) > 1000
            p = disagg.payload_from_bytes(big)
            assert p.prompt == PROMPTS[2] and len(p.output) == 1 and p.num_computed == len(PROMPTS[2])
            # stop strings apply on the decode side
            text = " ".join(f"w{t}" for t in golden[2])
            stop = f"w{golden[2][5]}"
            out = disagg.chain(post_prefill, post_decode, {"prompt": PROMPTS[2], "max_tokens": 12, "ignore_eos": True,
                                                           "stop": stop})
            assert out["choices"][0]["finish_reason"] == "stop" and out["choices"][0]["text"] == text[:text.find(stop)]
            assert cd.post("/v1/decode", content=b"garbage").status_code == 400
            assert cp.post("/v1/prefill", json={"prompt": [PROMPTS[0], PROMPTS[1]]}).status_code == 400
            for c in (cp, cd):
                st = c.get("/stats").json()
                assert st["kv_blocks_free"] == st["kv_blocks_total"]
    finally:
        eng_p.shutdown()
        eng_d.shutdown()


def test_queue_limit_and_request_timeout():
    """`max_pending` refuses work beyond the limit (HTTP 429) and frees the slot when a request
    ends; `timeout_s` ends a request with what it produced so far and gives its blocks back."""
    import time
    from starlette.testclient import TestClient
    from gvirt_b200.serve.async_engine import QueueFull
    eng = AsyncEngine(_llm(), max_pending=2)
    try:
        long = SamplingParams(max_tokens=80, ignore_eos=True)
        a = eng.submit(PROMPTS[0], long, timeout_s=0.15)
        b = eng.submit(PROMPTS[1], long)
        with pytest.raises(QueueFull):
            eng.submit(PROMPTS[2], long)
        with TestClient(build_app(eng, "tiny")) as c:
            assert c.post("/v1/completions", json={"prompt": PROMPTS[2], "max_tokens": 4}).status_code == 429
        ra = a.result(timeout=60)
        assert ra.finish_reason == "timeout" and 0 < len(ra.output_ids) < 100
        time.sleep(0.05)
        c3 = eng.submit(PROMPTS[3], SamplingParams(max_tokens=3, ignore_eos=True))     # the slot is free again
        assert len(c3.result(timeout=60).output_ids) == 3
        eng.cancel(b.request_id)
        assert b.result(timeout=60).finish_reason == "cancelled"
        assert eng.llm.scheduler.bm.num_free_blocks == eng.llm.num_blocks
    finally:
        eng.shutdown()


def test_bad_kv_payload_fails_its_request_not_the_engine():
    """A payload that does not fit this engine (other block size) is the sender's error: its
    future raises, the engine keeps serving and no block leaks."""
    from gvirt_b200.engine.kv_transfer import export_request
    src = _llm()
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    rid = src.add_request(PROMPTS[0], sp)
    src.step()
    payload = export_request(src, rid)
    payload.block_size = 8                      # claims another cache geometry
    eng = AsyncEngine(_llm())
    try:
        with pytest.raises(ValueError):
            eng.submit_payload(payload).result(timeout=30)
        ok = eng.submit(PROMPTS[1], sp).result(timeout=60)
        assert len(ok.output_ids) == 6 and eng.error is None
        assert eng.llm.scheduler.bm.num_free_blocks == eng.llm.num_blocks
    finally:
        eng.shutdown()


def test_truncated_kv_payload_leaks_nothing():
    """Payloads with missing layers, a wrong tensor shape, a wrong dtype or an inconsistent token
    count are refused before any block is taken: free blocks and sequence count stay as they were."""
    import copy
    from gvirt_b200.engine.kv_transfer import export_request
    src = _llm()
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    rid = src.add_request(PROMPTS[2], sp)
    src.step()
    good = export_request(src, rid)
    eng = AsyncEngine(_llm())
    try:
        bm = eng.llm.scheduler.bm
        free0 = bm.num_free_blocks
        bad = []
        p = copy.copy(good); p.layers = good.layers[:1]; bad.append(p)
        p = copy.copy(good); p.layers = [tuple(t[:, :1] for t in ts) for ts in good.layers]; bad.append(p)
        p = copy.copy(good); p.layers = [tuple(t.double() for t in ts) for ts in good.layers]; bad.append(p)
        p = copy.copy(good); p.num_computed = good.num_computed + 5; bad.append(p)
        p = copy.copy(good); p.output = [10 ** 9]; bad.append(p)
        for _ in range(3):
            for p in bad:
                with pytest.raises(ValueError):
                    eng.submit_payload(p).result(timeout=30)
        assert bm.num_free_blocks == free0 and not eng.llm.scheduler.running
        done = eng.submit_payload(good).result(timeout=60)          # the intact payload still decodes
        assert len(done.output_ids) == 6 and eng.error is None
        assert bm.num_free_blocks == eng.llm.num_blocks
    finally:
        eng.shutdown()


def test_malformed_requests_are_refused_and_the_engine_keeps_serving(golden):
    """max_tokens beyond the context window, token ids outside the vocabulary and out-of-range
    sampling parameters raise on the client side (HTTP 400); the next request is served."""
    eng = AsyncEngine(_llm())
    try:
        vocab = eng.llm.cfg.vocab_size
        ok = SamplingParams(max_tokens=12, ignore_eos=True)
        cases = [([1, 2, 3, 4, 5], SamplingParams(max_tokens=1000)),
                 ([1, vocab], ok), ([-1], ok), ([1, 2], SamplingParams(max_tokens=0)),
                 ([1, 2], SamplingParams(max_tokens=4, stop_token_ids=(vocab + 7,))),
                 ([1, 2], SamplingParams(max_tokens=4, top_p=0.0)), ([1, 2], SamplingParams(max_tokens=4, top_k=-3)),
                 ([1, 2], SamplingParams(max_tokens=4, temperature=float("nan"))),
                 ([1, 2], SamplingParams(max_tokens=4, repetition_penalty=0.0)),
                 ([1, 2], SamplingParams(max_tokens=4, presence_penalty=50.0))]
        for prompt, sp in cases:
            with pytest.raises(ValueError):
                eng.submit(prompt, sp)
        assert eng.error is None
        assert eng.submit(PROMPTS[0], ok).result(timeout=60).output_ids == golden[0]
        # a request that passes the client-side check but is refused at admission fails alone
        real_add = eng._owned.add
        def boom(gid, prompt, params):
            eng._owned.add = real_add
            raise ValueError("refused at admission")
        eng._owned.add = boom
        with pytest.raises(ValueError):
            eng.submit(PROMPTS[1], ok).result(timeout=30)
        assert eng.error is None and sum(eng._load) == 0
        assert eng.submit(PROMPTS[1], ok).result(timeout=60).output_ids == golden[1]
        from starlette.testclient import TestClient
        client = TestClient(build_app(eng, "tiny"))
        for body in ({"prompt": [1, 2, 3], "max_tokens": 1000}, {"prompt": [1, vocab + 1], "max_tokens": 4},
                     {"prompt": [1, 2], "max_tokens": "many"}, {"prompt": [1, 2], "max_tokens": 4, "top_p": 7},
                     {"prompt": [1, 2], "max_tokens": 1000, "stream": True}):
            assert client.post("/v1/completions", json=body).status_code == 400, body
        assert client.get("/health").status_code == 200
        r = client.post("/v1/completions", json={"prompt": PROMPTS[0], "max_tokens": 12, "ignore_eos": True})
        assert r.status_code == 200 and r.json()["choices"][0]["token_ids"] == golden[0]
    finally:
        eng.shutdown()
