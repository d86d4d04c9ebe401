"""tcgen05 GEMM vs fp32 matmul. Shapes follow the reference's sweep (m in {1, 8}, odd k such as
7184 / 7232, n = 16128; xlite/tests/kernels/matmul.py:17-52) plus the decode / prefill shapes of
the benchmark models."""
import pytest
import torch

from gvirt_b200.ops import functional as F
from tests.gpu_util import close, status_ok

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _run(M, N, K, bias=False, splitk=0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = (torch.randn(M, K, device="cuda", generator=g) * 0.5).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).bfloat16()
    b = (torch.randn(N, device="cuda", generator=g)).bfloat16() if bias else None
    y = F.linear(x, w, b, splitk=splitk)
    want = x.float() @ w.float().t()
    if b is not None:
        want = want + b.float()
    close(y, want, atol=3e-2, rtol=2e-2, what=f"gemm M={M} N={N} K={K} bias={bias} splitk={splitk}")


def test_gemm_smallest():
    _run(8, 128, 64)
    status_ok()


@pytest.mark.parametrize("M", [1, 8, 16, 17, 64, 100, 200, 256])
def test_gemm_decode_shapes(M):
    _run(M, 4096, 4096)
    _run(M, 6144, 4096, bias=True)
    status_ok()


@pytest.mark.parametrize("splitk", [1, 2, 3, 4, 8])
def test_gemm_splitk_cluster(splitk):
    _run(64, 1024, 4096, splitk=splitk)
    _run(33, 384, 2048, bias=True, splitk=splitk)
    status_ok()


@pytest.mark.parametrize("K", [32, 128, 7168, 7184, 7232, 7296])
def test_gemm_reference_k_sweep(K):
    _run(1, 64, K)
    _run(8, 16128, K)
    status_ok()


@pytest.mark.parametrize("M,N,K", [(257, 256, 512), (300, 1000, 1024), (1024, 4096, 4096),
                                   (4096, 6144, 4096), (2050, 384, 256), (513, 72, 128)])
def test_gemm_prefill_shapes(M, N, K):
    _run(M, N, K)
    _run(M, N, K, bias=True)
    status_ok()


def test_gemm_strided_input_and_output():
    x = (torch.randn(64, 8192, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(512, 4096, device="cuda") * 0.05).bfloat16()
    out = torch.zeros(64, 1024, device="cuda", dtype=torch.bfloat16)
    F.linear(x[:, 4096:], w, out=out[:, 512:])
    close(out[:, 512:], x[:, 4096:].float() @ w.float().t(), atol=3e-2, what="strided gemm")
    assert (out[:, :512] == 0).all()
    status_ok()


@pytest.mark.parametrize("M", [1, 17, 64, 128, 200, 300, 1000])
@pytest.mark.parametrize("I,K", [(128, 256), (1792, 4096), (14336, 1024), (704, 512)])
def test_linear_swiglu_epilogue(M, I, K):
    """Gate/up GEMM with the SwiGLU in its epilogue over block-interleaved weights (weight-major
    with and without cluster split-K, token-major for M > 256) against silu(x g^T) * (x u^T)."""
    g = torch.Generator().manual_seed(M * 7 + I)
    x = (torch.randn(M, K, generator=g) * 0.5).bfloat16()
    w = (torch.randn(2 * I, K, generator=g) * 0.05).bfloat16()
    gu = (x.float() @ w.float().t()).bfloat16().float()
    want = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
    wil = F.interleave_gate_up(w).to(DEV)
    got = F.linear_swiglu(x.to(DEV), wil)
    close(got.float().cpu(), want, atol=3e-2, rtol=3e-2, what="swiglu epilogue")
    for sk in (1, 2, 4):
        if M <= 256:
            got = F.linear_swiglu(x.to(DEV), wil, splitk=sk)
            close(got.float().cpu(), want, atol=3e-2, rtol=3e-2, what=f"swiglu epilogue splitk {sk}")
    # the unfused pair over the same interleaved weights agrees as well
    gu_il = F.linear(x.to(DEV), wil)
    got2 = F.silu_and_mul(gu_il, interleaved=True)
    close(got2.float().cpu(), want, atol=3e-2, rtol=3e-2, what="interleaved silu_and_mul")
    status_ok()


@pytest.mark.parametrize("M,N,K,bias", [(1024, 512, 256, False), (1024, 256, 64, True), (1100, 384, 512, True),
                                        (2048, 6144, 4096, False), (8192, 4096, 4096, False), (4096, 1000, 1032, True)])
def test_gemm_persistent_token_major(M, N, K, bias):
    """gemm_persist.cu against fp32 matmul and against the default kernel (same accumulation order:
    bit-identical): full and ragged tiles in both dimensions, K tails, bias."""
    from gvirt_b200 import _native
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    x = (torch.randn(M, K, device="cuda", generator=g) * 0.5).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).bfloat16()
    b = torch.randn(N, device="cuda", generator=g).bfloat16() if bias else None
    y = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    for _ in range(2):      # a second launch re-uses the cached tensor maps
        _native.call("gemm_bf16_persistent", x, w, b, y, M, N, K, x.stride(0), w.stride(0), y.stride(0))
    want = x.float() @ w.float().t()
    if b is not None:
        want = want + b.float()
    close(y, want, atol=3e-2, rtol=2e-2, what=f"persistent gemm M={M} N={N} K={K}")
    assert torch.equal(y, F.linear(x, w, b))
    status_ok()
