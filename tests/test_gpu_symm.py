"""Symmetric-heap kernels. On one GPU the heap has a single "peer" (the rank itself), which
still exercises staging, flag release/acquire, the device-side generation counter and the
rank-order reduction; with >= 2 GPUs the same kernels run across NVLink in child processes
against torch.distributed goldens."""
import pytest
import torch

from tests.gpu_util import close, status_ok

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _heap():
    from gvirt_b200.parallel.symm import SymmetricHeap
    return SymmetricHeap(None, 0, 1, torch.device("cuda", torch.cuda.current_device()), nbytes=256 << 20)


def test_collectives_single_rank_identity():
    heap = _heap()
    for dtype in (torch.float32, torch.bfloat16):
        for shape in [(1, 1), (1, 37), (8, 16), (512, 7168), (1024, 2048)]:
            x = torch.randn(shape, device=DEV).to(dtype)
            for _ in range(3):  # generations advance, parity alternates
                y = heap.all_reduce(x.clone())
                assert torch.equal(y, x)
            n = x.numel()
            if (n * x.element_size()) % 16 == 0:
                out = torch.empty(n, dtype=dtype, device=DEV)
                heap.all_gather(x.reshape(-1), out)
                assert torch.equal(out, x.reshape(-1))
                heap.reduce_scatter(x.reshape(-1), out)
                assert torch.equal(out, x.reshape(-1))
    status_ok()


def test_heap_canaries_stay_intact_and_detect_an_overrun():
    """Every region of the heap is followed by a guard; the kernels leave the guards alone and a
    write past a region's end is reported by name."""
    heap = _heap()
    x = torch.randn(64, 4096, device=DEV).bfloat16()
    w = (torch.randn(4096, 4096, device=DEV) * 0.02).bfloat16()
    for _ in range(3):
        heap.all_reduce(x.clone())
        heap.gemm_allreduce(x, w)
    big = torch.randn(1024, 2048, device=DEV)
    heap.all_reduce(big)
    torch.cuda.synchronize()
    assert len(heap._guards) >= 4
    assert heap.check_canaries() == []
    # simulate an overrun: one byte past the end of the first channel's data region
    ch = next(iter(heap.channels.values()))
    end = ch.data_off + 2 * ch.data_stride
    heap.slab[end] = 0
    bad = heap.check_canaries()
    assert bad == [f"{ch.name}/data"], bad
    status_ok()


@pytest.mark.parametrize("M,N,K", [(64, 4096, 4096), (1, 4096, 1792), (17, 1024, 512), (128, 2048, 2048),
                                   (100, 384, 256)])
def test_gemm_allreduce_single_rank(M, N, K):
    heap = _heap()
    g = torch.Generator(device=DEV).manual_seed(0)
    x = (torch.randn(M, K, device=DEV, generator=g) * 0.5).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.05).bfloat16()
    b = torch.randn(N, device=DEV, generator=g).bfloat16()
    res = torch.randn(M, N, device=DEV, generator=g).bfloat16()
    want = x.float() @ w.float().t()
    for rep in range(3):
        got = heap.gemm_allreduce(x, w)
        close(got, want, atol=4e-2, rtol=2e-2, what=f"gemm_ar rep {rep}")
    got = heap.gemm_allreduce(x, w, bias=b, residual=res)
    close(got, want + b.float() + res.float(), atol=6e-2, rtol=2e-2, what="gemm_ar + bias + residual")
    status_ok()


@pytest.mark.parametrize("M,N,K", [(64, 4096, 1024), (1, 512, 256), (100, 1024, 3584), (128, 2048, 512)])
def test_gemm_allreduce_residual_in_place_and_sumsq_single_rank(M, N, K):
    """The producer form used by the fused decode loop: the residual stream is updated in place and
    the sums of squares of the new rows are left per 128-feature tile."""
    heap = _heap()
    g = torch.Generator(device=DEV).manual_seed(1)
    x = (torch.randn(M, K, device=DEV, generator=g) * 0.5).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.05).bfloat16()
    res = torch.randn(M, N, device=DEV, generator=g).bfloat16()
    want = x.float() @ w.float().t() + res.float()
    for rep in range(2):
        xs = res.clone()
        ss = torch.full((128, N // 128), -1.0, device=DEV)
        heap.gemm_allreduce(x, w, out=xs, residual=xs, ss_out=ss)
        close(xs, want, atol=6e-2, rtol=2e-2, what=f"in-place residual rep {rep}")
        want_ss = xs.float().reshape(M, N // 128, 128).pow(2).sum(-1)
        close(ss[:M], want_ss, atol=1e-3, rtol=1e-4, what="tile sums of squares")
        assert (ss[M:] == -1).all()
    status_ok()


def test_gemm_allreduce_in_cuda_graph():
    heap = _heap()
    x = (torch.randn(32, 1024, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(512, 1024, device=DEV) * 0.05).bfloat16()
    out = torch.empty(32, 512, device=DEV, dtype=torch.bfloat16)
    heap.gemm_allreduce(x, w, out=out)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        heap.gemm_allreduce(x, w, out=out)
    for _ in range(5):  # replays advance the device-side generation
        out.zero_()
        g.replay()
        torch.cuda.synchronize()
        close(out, x.float() @ w.float().t(), atol=4e-2, what="graph replay")
    status_ok()


@pytest.mark.parametrize("fp8", [False, True])
def test_moe_a2a_single_rank(fp8):
    """Dispatch -> grouped GEMMs -> combine with the rank as its own (only) expert-parallel peer."""
    from types import SimpleNamespace
    from gvirt_b200.config import ModelConfig
    from gvirt_b200.models.weights import quantize_moe_layer_fp8
    from gvirt_b200.ops import moe_ops
    from gvirt_b200.parallel.moe_a2a import MoEA2A
    heap = _heap()
    T, H, I, E, K = 48, 512, 256, 8, 2
    cfg = ModelConfig(hidden_size=H, num_experts=E, num_experts_per_tok=K, moe_intermediate_size=I)
    a2a = MoEA2A(heap, cfg, None, tokens_cap=64, fp8=fp8)
    g = torch.Generator(device=DEV).manual_seed(3)
    L = SimpleNamespace(w13=(torch.randn(E, 2 * I, H, device=DEV, generator=g) * 0.05).bfloat16(),
                        w2=(torch.randn(E, H, I, device=DEV, generator=g) * 0.05).bfloat16())
    if fp8:
        quantize_moe_layer_fp8(L)
    for rep in range(3):  # the same regions are re-used layer after layer
        x = (torch.randn(T, H, device=DEV, generator=g) * 0.5).bfloat16()
        wts, ids = moe_ops.softmax_topk(torch.randn(T, E, device=DEV, generator=g), K, True)
        out = torch.zeros(T, H, device=DEV, dtype=torch.bfloat16)
        a2a.forward(x, wts, ids, L, out)
        want = moe_ops.experts_forward(x.cpu(), wts.cpu(), ids.cpu(), L.w13.cpu(), L.w2.cpu(), 0,
                                       w13_scale=L.w13_scale.cpu() if fp8 else None,
                                       w2_scale=L.w2_scale.cpu() if fp8 else None)
        close(out, want, atol=3e-2, rtol=5e-2, what=f"moe a2a fp8={fp8} rep {rep}")
    status_ok()


def test_gemm_sp_single_rank():
    """GEMM -> reduce-scatter and all-gather -> GEMM with one rank (staging, flags, TMA from the heap)."""
    heap = _heap()
    g = torch.Generator(device=DEV).manual_seed(5)
    for (M, N, K) in [(128, 256, 512), (512, 4096, 1024)]:
        x = (torch.randn(M, K, device=DEV, generator=g) * 0.5).bfloat16()
        w = (torch.randn(N, K, device=DEV, generator=g) * 0.05).bfloat16()
        want = x.float() @ w.float().t()
        for rep in range(3):
            close(heap.gemm_reduce_scatter(x, w), want, atol=4e-2, rtol=2e-2, what="gemm_rs")
            close(heap.allgather_gemm(x, w), want, atol=4e-2, rtol=2e-2, what="ag_gemm")
    status_ok()


def _run(mode, world):
    from tests.test_dist_cpu import run_workers
    return run_workers(mode, world, timeout=900, extra_env={"NCCL_NVLS_ENABLE": "0"})


@pytest.mark.parametrize("mode", ["collectives_gpu", "gemm_ar_gpu", "gemm_sp_gpu", "tp_model_gpu", "moe_a2a_gpu", "moe_tp_slice_gpu"])
def test_multi_gpu(mode):
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs >= 2 GPUs")
    import os
    world = int(os.environ.get("GVIRT_TEST_WORLD", "0")) or (2 if n < 4 else 4)
    _run(mode, min(world, n))


@pytest.mark.parametrize("rows", [8, 512])
def test_peer_that_never_arrives_times_out_and_context_survives(rows):
    """Failure detection on the device: a push all-reduce is told it has a peer, but nothing ever
    writes that peer's lines. The bounded poll gives up (about two seconds), the kernel returns,
    the status word carries the PEER bit, and the same context runs the next kernel normally.
    The budget is per launch: with 512 rows on one CTA every thread owns many lines, and the
    launch must still end after one wait, not one wait per line."""
    import time
    from gvirt_b200 import _native
    heap = _heap()
    status_ok()
    x = torch.randn(rows, 128, device=DEV).bfloat16()
    out = torch.empty_like(x)
    n = x.numel()
    lines = n * 2 // 8
    ch = heap.channel(f"timeout_probe_{rows}", 16 * 3 * max(lines, 1024), 1)
    fake_peers = torch.tensor([heap.slab.data_ptr(), heap.slab.data_ptr() + (128 << 20)], dtype=torch.int64,
                              device=DEV)                 # "rank 1" = an unused half of the same slab
    t0 = time.time()
    _native.call("collective", 4, 0, x, out, n, fake_peers, ch.flags_off, ch.data_off, ch.data_stride,
                 ch.state, 0, 2, 1)
    torch.cuda.synchronize()
    dt = time.time() - t0
    st = _native.read_status()
    assert st & 8, _native.describe_status(st)            # GV_ST_TIMEOUT_PEER
    assert 1.0 < dt < 6.0, dt
    _native.reset_status()
    y = heap.all_reduce(x.clone())
    assert torch.equal(y, x)
    status_ok()
