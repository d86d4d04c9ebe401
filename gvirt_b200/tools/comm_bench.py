"""Device-timed micro-benchmark of the tensor-parallel building blocks on N GPUs.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m gvirt_b200.tools.comm_bench --tokens 64 --hidden 4096 --inter 14336

For each row-parallel projection of a decode step (o_proj, down_proj at the given sizes) it times,
inside one CUDA graph of `--chain` back-to-back calls and as the max over ranks:

  * ``gemm``            the local tcgen05 GEMM alone (no communication; lower bound),
  * ``gemm_ar_fused``   the fused GEMM + all-reduce kernel over peer memory,
  * ``gemm+own_ar``     GEMM followed by the stand-alone peer-memory all-reduce kernel,
  * ``gemm+nccl_ar``    GEMM followed by ``torch.distributed.all_reduce`` (the library baseline),

and prints one JSON line per case on rank 0. The role matches the reference's ``matmul_bench``
binding and swizzle sweep (xlite/xlite/_C.cpp:1001-1029, tests/performance/swizzle/
matmul_swizzle_perf.py), extended to the communication-fused kernels.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..ops import functional as F
from ..parallel import state as pstate
from ..parallel.symm import attach_symmetric_heap
from .. import _native


def _graph_time_us(fn, chain: int, reps: int) -> float:
    for _ in range(3):
        fn(0)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(chain):
            fn(i)
    g.replay()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) * 1e3 / (chain * reps)], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inter", type=int, default=14336)
    ap.add_argument("--chain", type=int, default=16)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--prefill-tokens", type=int, default=0,
                    help="also time the sequence-parallel prefill kernels at this many tokens (0 = skip)")
    ap.add_argument("--bf16-tflops", type=float, default=1396.2,
                    help="measured sustained bf16 GEMM rate used for the roofline of the prefill cases")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    ctx = pstate.init_parallel(tp=world, dp=1, ep=1, timeout_s=120)
    # sequence-parallel regions: 2 kinds x 2 parities x prefill rows x widest column count, bf16
    sp_rows = max(128, -(-args.prefill_tokens // (128 * ctx.tp)) * 128) if args.prefill_tokens > 0 else 0
    attach_symmetric_heap(ctx, nbytes=(1 << 29) + 4 * ctx.tp * sp_rows * max(args.hidden, args.inter // ctx.tp) * 2)
    if sp_rows and getattr(ctx, "symm", None) is not None:
        ctx.symm.sp_rows_cap = sp_rows
    heap, dev, rank = ctx.symm, ctx.device, ctx.rank
    M, H = args.tokens, args.hidden
    for name, N, Kfull in (("o_proj", H, H), ("down_proj", H, args.inter)):
        K = Kfull // world
        copies = max(2, int(300e6 / (N * K * 2)) + 1)            # rotate weights: stay out of L2
        ws = [(torch.randn(N, K, device=dev) * 0.02).bfloat16() for _ in range(copies)]
        x = torch.randn(M, K, device=dev).bfloat16()
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        res = {}
        res["gemm"] = _graph_time_us(lambda i: F.linear(x, ws[i % copies], out=out), args.chain, args.reps)
        if heap is not None:
            res["gemm_ar_fused"] = _graph_time_us(
                lambda i: heap.gemm_allreduce(x, ws[i % copies], out=out), args.chain, args.reps)

            xres = torch.zeros(M, N, device=dev, dtype=torch.bfloat16)
            ss = torch.zeros(128, N // 128, device=dev)
            res["gemm_ar_fused+residual+sumsq"] = _graph_time_us(
                lambda i: heap.gemm_allreduce(x, ws[i % copies], out=xres, residual=xres, ss_out=ss),
                args.chain, args.reps)

            def own(i):
                F.linear(x, ws[i % copies], out=out)
                heap.all_reduce(out)
            res["gemm+own_ar"] = _graph_time_us(own, args.chain, args.reps)

        def nccl(i):
            F.linear(x, ws[i % copies], out=out)
            dist.all_reduce(out, group=ctx.tp_group)
        res["gemm+nccl_ar"] = _graph_time_us(nccl, args.chain, args.reps)
        st = _native.read_status()
        if rank == 0:
            print(json.dumps({"case": name, "world": world, "M": M, "N": N, "K_local": K,
                              "us": {k: round(v, 2) for k, v in res.items()},
                              "msg_bytes": M * N * 2, "status_word": st}), flush=True)
        del ws
    if args.prefill_tokens > 0 and heap is not None:
        sp_cases(args, ctx, heap)
    dist.barrier()
    torch.cuda.synchronize()
    os._exit(0)


def sp_cases(args, ctx, heap) -> None:
    """Sequence-parallel prefill blocks at `--prefill-tokens` rows: the fused GEMM -> reduce-scatter
    and all-gather -> GEMM kernels against the same GEMM with the library collective. The roofline
    is the slower of the FLOPs at the measured bf16 rate and the bytes that must cross NVLink per
    rank at the measured 770 GB/s per direction."""
    world, dev, rank = ctx.tp, ctx.device, ctx.rank
    M, H = args.prefill_tokens, args.hidden
    M = M // (128 * world) * (128 * world)
    peak_tf, link = args.bf16_tflops, 770.0
    for name, N, Kfull in (("o_proj", H, H), ("down_proj", H, args.inter)):
        K = Kfull // world
        x = (torch.randn(M, K, device=dev) * 0.1).bfloat16()
        w = (torch.randn(N, K, device=dev) * 0.02).bfloat16()
        out = torch.empty(M // world, N, device=dev, dtype=torch.bfloat16)
        full = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        res = {"gemm": _graph_time_us(lambda i: F.linear(x, w, out=full), 2, args.reps)}
        if heap.can_fuse_gemm_rs(x, w):
            res["gemm_rs_fused"] = _graph_time_us(lambda i: heap.gemm_reduce_scatter(x, w, out=out), 2, args.reps)

        def lib(i):
            F.linear(x, w, out=full)
            dist.reduce_scatter_tensor(out, full, group=ctx.tp_group)
        res["gemm+nccl_rs"] = _graph_time_us(lib, 2, args.reps)
        ideal = max(2.0 * M * N * K / (peak_tf * 1e6), (world - 1) / world * M * N * 2 / (link * 1e3))
        st = _native.read_status()
        if rank == 0:
            print(json.dumps({"case": "rs:" + name, "world": world, "M": M, "N": N, "K_local": K,
                              "us": {k: round(v, 1) for k, v in res.items()}, "roofline_us": round(ideal, 1),
                              "fused_fraction_of_roofline": round(ideal / res["gemm_rs_fused"], 3)
                              if "gemm_rs_fused" in res else None, "status_word": st}), flush=True)
    for name, Nfull, K in (("qkv", H + 2 * (H // 4), H), ("gate_up", 2 * args.inter, H)):
        N = Nfull // world // 128 * 128
        xl = (torch.randn(M // world, K, device=dev) * 0.1).bfloat16()
        w = (torch.randn(N, K, device=dev) * 0.02).bfloat16()
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        xg = torch.empty(M, K, device=dev, dtype=torch.bfloat16)
        res = {"gemm": _graph_time_us(lambda i: F.linear(xg, w, out=out), 2, args.reps)}
        if heap.can_fuse_ag_gemm(xl, w):
            res["ag_gemm_fused"] = _graph_time_us(lambda i: heap.allgather_gemm(xl, w, out=out), 2, args.reps)

        def lib(i):
            dist.all_gather_into_tensor(xg, xl, group=ctx.tp_group)
            F.linear(xg, w, out=out)
        res["nccl_ag+gemm"] = _graph_time_us(lib, 2, args.reps)
        ideal = max(2.0 * M * N * K / (peak_tf * 1e6), (world - 1) / world * M * K * 2 / (link * 1e3))
        st = _native.read_status()
        if rank == 0:
            print(json.dumps({"case": "ag:" + name, "world": world, "M": M, "N_local": N, "K": K,
                              "us": {k: round(v, 1) for k, v in res.items()}, "roofline_us": round(ideal, 1),
                              "fused_fraction_of_roofline": round(ideal / res["ag_gemm_fused"], 3)
                              if "ag_gemm_fused" in res else None, "status_word": st}), flush=True)


if __name__ == "__main__":
    raise SystemExit(main())
