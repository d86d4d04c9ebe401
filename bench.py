"""Headline benchmark: decode output tokens/s of Llama-3-8B (bf16, random-init weights,
synthetic token ids), 64 concurrent requests with 1024-token prompts, tensor parallel over N
GPUs of one node.

    python bench.py --gpus 1 --steps 64 --warmup 8
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 64 --warmup 8

One *step* = one decode iteration of the whole batch (64 new tokens). Two measurements:

* ``value``  — device-timed: K replays of the captured decode step (embedding -> 32 layers ->
  lm_head -> sampling) bracketed by CUDA events, max over ranks; weights (16 GB) + KV cache are
  far larger than L2, so every step streams from HBM.
* ``e2e``    — the same K steps through the public API (``LLM.step()``): per step the host
  builds the attention metadata, copies token ids + metadata from pinned memory to the device,
  replays the graph and reads the sampled tokens back; timed with the wall clock around the loop
  (barrier + synchronize on both sides), max over ranks.

``--impl reference`` would run the unmodified Ascend reference; it cannot be installed here and
prints an ``unavailable`` line. ``--impl torch`` runs the same graph with PyTorch eager ops
(cuBLAS GEMMs, SDPA attention, NCCL collectives) as the same-box floor.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

REF_UNAVAILABLE = ("refused by a safety check: offline pip install of the reference (its setup.py / CMake "
                   "build) was denied; the reference is Ascend-only (AscendC/CCE kernels, ACL, HCCL) and has "
                   "no CUDA build")


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "torch"])
    ap.add_argument("--model", default="llama-3-8b")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--out-len", type=int, default=256,
                    help="output tokens per request of the workload: the timed steps sit around its middle")
    ap.add_argument("--layers", type=int, default=0, help="debug only: override layer count (invalidates the number)")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--parallel", default="tp", choices=["tp", "ep", "dp_ep"],
                    help="tp: tensor parallel; ep: TP attention + expert-parallel MoE; "
                         "dp_ep: data-parallel attention + expert-parallel MoE")
    ap.add_argument("--quant", default="", help="override the preset's quantisation (e.g. fp8_block)")
    ap.add_argument("--router-zipf", type=float, default=0.0,
                    help="MoE: bias the router so that expert popularity follows Zipf(alpha)")
    ap.add_argument("--max-tokens", type=int, default=8192, help="max_num_batched_tokens (prefill chunk)")
    ap.add_argument("--kernel-table", default="",
                    help="after the timed regions, replay the decode step 4 more times under torch.profiler and "
                         "write rank 0's per-kernel device times to this file (diagnostic; never part of a number)")
    return ap.parse_args()


def _kernel_table(graph, path, rank, barrier, reps=4):
    """Per-kernel device time of the captured decode step on rank 0 (every rank replays)."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    barrier()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(reps):
            graph.replay()
        torch.cuda.synchronize()
    barrier()
    if rank != 0:
        return
    rows = []
    for e in prof.key_averages():
        t = getattr(e, "device_time_total", None)
        if t is None:
            t = getattr(e, "cuda_time_total", 0.0)
        if t > 0:
            rows.append((t / reps, e.count / reps, e.key))
    rows.sort(reverse=True)
    total = sum(r[0] for r in rows)
    with open(path, "w") as f:
        f.write(f"# device time per decode step by kernel, rank 0, mean of {reps} replays; sum {total:.1f} us\n")
        f.write("# us_per_step  launches_per_step  us_per_launch  kernel\n")
        for t, n, name in rows:
            f.write(f"{t:10.1f} {n:8.1f} {t / max(n, 1e-9):9.2f}  {name[:150]}\n")


class ClockSampler:
    """Samples SM clock / throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                power.append(float(f[3]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def main():
    import faulthandler
    faulthandler.enable()
    args = parse()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REF_UNAVAILABLE}))
        return 0

    import torch
    import torch.distributed as dist

    from gvirt_b200 import _native
    from gvirt_b200.engine.llm import LLM
    from gvirt_b200.engine.scheduler import SamplingParams
    from gvirt_b200.models import presets
    from gvirt_b200.parallel import state as pstate

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run "
                         f"--nproc-per-node {args.gpus}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    # parallel layouts: "tp" = everything tensor parallel; "ep" = tensor-parallel attention with
    # the experts spread over all ranks; "dp_ep" = every rank runs attention on its own requests
    # (data parallel) and the experts are spread over all ranks
    par = args.parallel
    if par == "tp":
        ctx = pstate.init_parallel(tp=world, dp=1, ep=1)
    elif par == "ep":
        ctx = pstate.init_parallel(tp=world, dp=1, ep=world, moe_tp=1)
    else:
        ctx = pstate.init_parallel(tp=1, dp=world, ep=world, moe_tp=1)
    rank = ctx.rank

    K, W, P = args.steps, max(args.warmup, 3), args.prompt_len
    B_global = args.batch
    B = B_global // ctx.dp          # requests this rank schedules
    # the timed end-to-end window is centred on the middle of the configured decode (context
    # prompt + out_len / 2); `advance` untimed steps bring the batch there after the warm-up
    advance = max(0, args.out_len // 2 - K // 2 - W)
    total_new = W + advance + K + 8
    overrides = dict(tp_size=ctx.tp, dp_size=ctx.dp, ep_size=ctx.ep, max_batch_size=B,
                     max_seq_len=P + 2 * total_new + 64, max_num_batched_tokens=args.max_tokens)
    if args.layers:
        overrides["num_layers"] = args.layers
    if args.quant:
        overrides["quant"] = args.quant
    cfg = presets.get(args.model, **overrides)
    from gvirt_b200.parallel.setup import attach_device_comm
    attach_device_comm(ctx, cfg)

    if args.impl == "torch":
        from gvirt_b200.utils.torch_floor import run_floor
        res = run_floor(cfg, ctx, B, P, K, W, advance)
        if rank == 0:
            print(json.dumps(res))
        return 0

    t_build = time.perf_counter()
    rb = None
    if args.router_zipf > 0 and cfg.is_moe:
        from gvirt_b200.models.weights import zipf_router_bias
        rb = zipf_router_bias(cfg, args.router_zipf)
    llm = LLM.from_config(cfg, ctx, seed=0, shard_from_full=False, router_bias_fn=rb,
                          use_graphs=not args.no_graph)
    runner = llm.runner
    build_s = time.perf_counter() - t_build

    # ---- warm-up of the prefill path: one untimed chunk-sized batch of requests, so that one-off
    # costs (communicator set-up of the first large collective, tensor-map encoding, kernel
    # attributes) are not billed to the first requests' time to first token
    g = torch.Generator().manual_seed(99 + ctx.dp_rank)
    n_warm = max(1, min(B, args.max_tokens // P))
    warm = torch.randint(0, cfg.vocab_size, (n_warm, P), generator=g).tolist()
    llm.generate(warm, SamplingParams(max_tokens=2, ignore_eos=True))
    torch.cuda.synchronize()
    # ---- prefill all requests through the engine (chunked), then warm-up decode steps
    g.manual_seed(1234 + ctx.dp_rank)
    prompts = torch.randint(0, cfg.vocab_size, (B, P), generator=g).tolist()
    sp = SamplingParams(max_tokens=2 * total_new + 8, ignore_eos=True)
    for p in prompts:
        llm.add_request(p, sp)
    reqs = list(llm.scheduler.waiting)
    t0 = time.perf_counter()
    while any(r.first_token_time is None for r in reqs):
        llm.step()
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0
    ttfts = sorted(r.first_token_time - r.arrival for r in reqs)
    for _ in range(W + advance):
        llm.step()
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(torch.cuda.current_device())
    # ---- (1) end to end through the public API
    h2d0, d2h0, l0 = runner.h2d_bytes, runner.d2h_bytes, runner.launch_count
    barrier()
    if rank == 0:
        sampler.start()
    n_before = [len(r.token_times) for r in reqs]
    step_ends = []
    t0 = time.perf_counter()
    for _ in range(K):
        llm.step()
        step_ends.append(time.perf_counter())
    barrier()
    e2e_s = time.perf_counter() - t0
    n_after = [len(r.token_times) for r in reqs]
    # host-side time of every step after the first (with asynchronous scheduling a step returns
    # when the previous step's tokens are in, so the differences are steady-state step times)
    step_ms = sorted((b - a) * 1e3 for a, b in zip(step_ends, step_ends[1:]))
    h2d = (runner.h2d_bytes - h2d0) / K
    d2h = (runner.d2h_bytes - d2h0) / K
    launches_e2e = runner.launch_count - l0

    # ---- (2) device-timed replays of the captured decode step
    key = runner.last_graph_key
    launches = 0
    if key is not None and not args.no_graph:
        graph = runner.graphs[key]
        for _ in range(3):
            graph.replay()
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(K):
            graph.replay()
        ev1.record()
        barrier()
        dev_ms = ev0.elapsed_time(ev1)
        launches = runner.graph_launches[key] * K
    else:
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l1 = _native.LAUNCHES
        ev0.record()
        for _ in range(K):
            llm.step()
        ev1.record()
        barrier()
        dev_ms = ev0.elapsed_time(ev1)
        launches = _native.LAUNCHES - l1
    clocks = sampler.stop() if rank == 0 else {}
    status = runner.check_status()
    if args.kernel_table and key is not None and not args.no_graph:
        _kernel_table(runner.graphs[key], args.kernel_table, rank, barrier)

    # time per output token inside the timed end-to-end window (one-off costs such as the first
    # capture of a decode graph and the wait behind other requests' prefill chunks are in TTFT)
    # only gaps between tokens that both arrived inside the window count: the barrier and the
    # start of the clock sampler in front of it are not part of any gap
    tpots = []
    for r, a, b in zip(reqs, n_before, n_after):
        if b - a >= 2:
            tpots.append((r.token_times[b - 1] - r.token_times[a]) / (b - a - 1))
    # max over ranks
    t = torch.tensor([dev_ms, e2e_s * 1e3], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = t.tolist()
    value = B_global * K / (dev_ms / 1e3)
    e2e_value = B_global * K / (e2e_ms / 1e3)
    if rank == 0:
        out = {
            "metric": "decode_output_tok_s", "value": round(value, 1), "unit": "tok/s", "n_gpus": world,
            "steps": K, "warmup": W, "ms_per_step": round(dev_ms / K, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
            "config": {"model": cfg.name, "global_batch": B_global, "seq_len": P,
                       "out_len": args.out_len, "decode_context": P + W + advance + K,
                       "e2e_context": [P + W + advance, P + W + advance + K],
                       "parallelism": {"tp": f"tp{world}", "ep": f"tp{world}_ep{world}",
                                       "dp_ep": f"dp{world}_ep{world}"}[par],
                       "quant": cfg.quant or "none", "router_zipf": args.router_zipf or None, "layers": cfg.num_layers, "kv_block": cfg.block_size,
                       "l2_policy": "inputs larger than L2 (weights + KV streamed from HBM every step)",
                       "cuda_graph": not args.no_graph},
            "e2e": {"value": round(e2e_value, 1), "unit": "tok/s", "ms_per_step": round(e2e_ms / K, 4),
                    "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                    "step_ms_p50": round(statistics.median(step_ms), 4) if step_ms else None,
                    "step_ms_max": round(step_ms[-1], 4) if step_ms else None},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "ttft_p50_s": round(statistics.median(ttfts), 4) if ttfts else None,
            "tpot_p50_s": round(statistics.median(tpots), 5) if tpots else None,
            "tpot_window": "gaps between tokens inside the timed end-to-end steps (batch in steady decode)",
            "prefill_tok_s": round(B_global * P / prefill_s, 1),
            "status_word": status, "build_s": round(build_s, 1),
        }
        print(json.dumps(out), flush=True)
    if world > 1:
        # Leave together, then skip the process-group destructor: with NCCL kernels captured in
        # CUDA graphs its teardown has been seen to block for minutes after the result was printed.
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)
    return 0


if __name__ == "__main__":
    sys.exit(main())
