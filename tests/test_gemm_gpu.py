"""tcgen05 GEMM against an fp32 PyTorch reference."""
import pytest
import torch

from coccl_b200.ops import gemm as G

pytestmark = pytest.mark.gpu


@pytest.fixture(params=["1cta", "2cta"], autouse=True)
def variant(request):
    G.set_variant(request.param)
    yield request.param
    G.set_variant("auto")


def _ref(a, b):
    return a.float() @ b.float().t()


def _check(c, ref, k):
    err = (c.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 2e-2 * scale + 1e-3, (err, scale)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (4096, 4096, 1024), (300, 264, 72), (2048, 1024, 4096), (8192, 256, 64), (1000, 50304 // 8, 128)])
def test_gemm_tn(cuda, M, N, K):
    torch.manual_seed(0)
    a = torch.randn(M, K, device=cuda, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=cuda, dtype=torch.bfloat16)
    c = G.gemm(a, b)
    torch.cuda.synchronize()
    G.check_errors()
    _check(c, _ref(a, b), K)


@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (True, False), (True, True)])
def test_gemm_operand_layouts(cuda, a_mn, b_mn):
    torch.manual_seed(1)
    M, N, K = 384, 512, 320
    a = torch.randn(M, K, device=cuda, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=cuda, dtype=torch.bfloat16)
    a_in = a.t().contiguous().t() if a_mn else a   # same values, M contiguous
    b_in = b.t().contiguous().t() if b_mn else b
    assert (a_in.stride(0) == 1) == a_mn and (b_in.stride(0) == 1) == b_mn
    c = G.gemm(a_in, b_in)
    torch.cuda.synchronize()
    G.check_errors()
    _check(c, _ref(a, b), K)


def test_gemm_epilogues(cuda):
    torch.manual_seed(2)
    M, N, K = 512, 768, 256
    a = torch.randn(M, K, device=cuda, dtype=torch.bfloat16) * 0.5
    b = torch.randn(N, K, device=cuda, dtype=torch.bfloat16) * 0.1
    bias = torch.randn(N, device=cuda, dtype=torch.bfloat16)
    ref = _ref(a, b) + bias.float()
    c = G.gemm(a, b, bias=bias)
    _check(c, ref, K)
    y, z = G.gemm(a, b, bias=bias, gelu=True, save_preact=True)
    _check(z, ref, K)
    _check(y, torch.nn.functional.gelu(ref, approximate="tanh"), K)
    acc = torch.ones(M, N, device=cuda, dtype=torch.float32)
    G.gemm(a, b, out=acc, accumulate=True)
    _check(acc, _ref(a, b) + 1.0, K)
    f = G.gemm(a, b, out_dtype=torch.float32)
    _check(f, _ref(a, b), K)
    torch.cuda.synchronize()
    G.check_errors()


def test_gemm_wgrad_layout_with_ragged_contraction(cuda):
    """dW = dY^T @ X with a token count that is not a multiple of 8: both operands are stored token-major, so the
    contraction length is unconstrained (rows past it read as zeros)."""
    torch.manual_seed(3)
    tokens, n_out, n_in = 97, 256, 192
    dy = torch.randn(tokens, n_out, device=cuda, dtype=torch.bfloat16)
    x = torch.randn(tokens, n_in, device=cuda, dtype=torch.bfloat16)
    dw = G.gemm(dy.t(), x.t(), out_dtype=torch.float32)
    torch.cuda.synchronize()
    G.check_errors()
    _check(dw, dy.float().t() @ x.float(), tokens)
