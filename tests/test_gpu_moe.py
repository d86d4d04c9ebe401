"""MoE kernels vs fp32 definitions: router top-k (softmax / sigmoid grouped; configurations of
xlite/tests/kernels/softmax_topk.py:17-49 and sigmoid_topk.py:19-87), permutation round trip
(xlite/tests/kernels/permutation.py:17-91), grouped GEMM (xlite/tests/kernels/group_matmul.py:17-73)
and the whole expert FFN."""
import pytest
import torch

from gvirt_b200.ops import moe_ops
from gvirt_b200.ops import reference as ref
from tests.gpu_util import close, status_ok

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _check_topk(w, ids, w_ref, ids_ref, what):
    # order inside the top-k set is not part of the contract: compare as sets / sorted by id
    o, o_ref = ids.long().cpu().sort(-1), ids_ref.long().cpu().sort(-1)
    assert torch.equal(o[0], o_ref[0]), f"{what}: expert sets differ"
    close(w.cpu().gather(1, o[1]), w_ref.cpu().gather(1, o_ref[1]), atol=1e-5, rtol=1e-4, what=what)


@pytest.mark.parametrize("T,E,K", [(8, 128, 8), (33, 64, 6), (5, 160, 8), (1, 8, 2)])
@pytest.mark.parametrize("renorm", [True, False])
def test_softmax_topk(T, E, K, renorm):
    logits = torch.randn(T, E, device=DEV) * 2
    w, ids = moe_ops.softmax_topk(logits, K, renorm)
    w_ref, ids_ref = ref.softmax_topk(logits.cpu(), K, renorm)
    _check_topk(w, ids, w_ref, ids_ref, "softmax_topk")


@pytest.mark.parametrize("E,G,TG,K", [(160, 1, 1, 8), (256, 8, 4, 8), (256, 1, 1, 8), (64, 4, 2, 6)])
def test_sigmoid_topk(E, G, TG, K):
    T = 9
    logits = torch.randn(T, E, device=DEV) * 2
    bias = torch.randn(E, device=DEV) * 0.5
    w, ids = moe_ops.sigmoid_topk(logits, bias, K, G, TG, True, 2.5)
    w_ref, ids_ref = ref.sigmoid_topk(logits.cpu(), bias.cpu(), K, G, TG, True, 2.5)
    _check_topk(w, ids, w_ref, ids_ref, "sigmoid_topk")


@pytest.mark.parametrize("T,H,E,K,N", [(16, 1024, 8, 2, 512), (128, 2048, 128, 8, 1536), (300, 512, 16, 4, 256),
                                       (1, 256, 4, 1, 128)])
def test_grouped_gemm_and_permutation(T, H, E, K, N):
    g = torch.Generator(device=DEV).manual_seed(0)
    x = (torch.randn(T, H, device=DEV, generator=g) * 0.5).bfloat16()
    w = (torch.randn(E, N, H, device=DEV, generator=g) * 0.05).bfloat16()
    ids = torch.stack([torch.randperm(E, device=DEV)[:K] for _ in range(T)]).to(torch.int32)
    counts = torch.zeros(E + 1, dtype=torch.int32, device=DEV)
    offsets = torch.empty(E + 1, dtype=torch.int32, device=DEV)
    row_of = torch.empty(T, K, dtype=torch.int32, device=DEV)
    xs = torch.zeros(T * K, H, dtype=torch.bfloat16, device=DEV)
    from gvirt_b200 import _native
    _native.call("moe_permute", x, ids, counts, offsets, row_of, xs, T, H, K, E, 0, T * K)
    off = offsets.cpu().tolist()
    cnt = torch.bincount(ids.flatten().long().cpu(), minlength=E).tolist()
    assert off[0] == 0 and [off[i + 1] - off[i] for i in range(E)] == cnt
    ro = row_of.cpu()
    assert sorted(ro.flatten().tolist()) == list(range(T * K))
    for t in range(min(T, 8)):
        for k in range(K):
            r = int(ro[t, k])
            assert off[int(ids[t, k])] <= r < off[int(ids[t, k]) + 1]
            assert torch.equal(xs[r], x[t])
    out = torch.zeros(T * K, N, dtype=torch.bfloat16, device=DEV)
    moe_ops.grouped_gemm(xs, w, offsets, out)
    want = torch.zeros(T * K, N)
    for e in range(E):
        a, b = off[e], off[e + 1]
        if b > a:
            want[a:b] = xs[a:b].float().cpu() @ w[e].float().cpu().t()
    close(out, want, atol=3e-2, rtol=2e-2, what="grouped gemm")
    status_ok()


@pytest.mark.parametrize("local", [(0, 8), (4, 4)])
def test_experts_forward(local):
    T, H, I, E, K = 64, 512, 256, 8, 2
    start, e_local = local
    g = torch.Generator(device=DEV).manual_seed(1)
    x = (torch.randn(T, H, device=DEV, generator=g) * 0.5).bfloat16()
    w13 = (torch.randn(E, 2 * I, H, device=DEV, generator=g) * 0.05).bfloat16()
    w2 = (torch.randn(E, H, I, device=DEV, generator=g) * 0.05).bfloat16()
    logits = torch.randn(T, E, device=DEV, generator=g)
    wts, ids = moe_ops.softmax_topk(logits, K, True)
    y = moe_ops.experts_forward(x, wts, ids, w13[start:start + e_local], w2[start:start + e_local], start)
    want = ref.moe_ffn(x.cpu(), wts.cpu(), ids.cpu(), w13[start:start + e_local].cpu(), w2[start:start + e_local].cpu(), start)
    close(y, want, atol=2e-2, rtol=3e-2, what="experts_forward")
    status_ok()


@pytest.mark.parametrize("T,H,E,K,I,clamp", [(64, 512, 8, 2, 256, 0.0), (300, 1024, 16, 4, 768, 0.0),
                                             (5, 256, 4, 1, 16, 0.0), (128, 2048, 32, 8, 176, 1.5)])
def test_grouped_gemm_swiglu_epilogue(T, H, E, K, I, clamp):
    """Gate / up rows interleaved in blocks of [16 gate | 16 up]: the grouped GEMM applies SwiGLU
    (clamped or not) in its epilogue. Compared with the fp32 definition of GEMM -> round -> SwiGLU
    and with the unfused pair of kernels; I = 16 and 176 leave partial 128-row weight tiles."""
    g = torch.Generator(device=DEV).manual_seed(2)
    x = (torch.randn(T, H, device=DEV, generator=g) * 0.5).bfloat16()
    w13 = (torch.randn(E, 2 * I, H, device=DEV, generator=g) * 0.08).bfloat16()
    w2 = (torch.randn(E, H, I, device=DEV, generator=g) * 0.05).bfloat16()
    wts, ids = moe_ops.softmax_topk(torch.randn(T, E, device=DEV, generator=g), K, True)
    w_il = moe_ops.interleave16(w13)
    assert torch.equal(moe_ops.deinterleave16(w_il), w13)
    fused = moe_ops.experts_forward(x, wts, ids, w_il, w2, 0, clamp, il16=True)
    plain = moe_ops.experts_forward(x, wts, ids, w13, w2, 0, clamp)
    want = ref.moe_ffn(x.cpu(), wts.cpu(), ids.cpu(), w13.cpu(), w2.cpu(), 0, clamp)
    close(fused, want, atol=2e-2, rtol=3e-2, what="experts_forward with the SwiGLU epilogue")
    close(fused, plain, atol=1e-2, rtol=2e-2, what="SwiGLU epilogue vs the unfused pair")
    status_ok()
