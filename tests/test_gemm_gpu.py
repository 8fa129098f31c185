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


def _check(c, ref, k, extra=0.0):
    """Elementwise bound by output type. The operands are bf16, so every product is exact in fp32 and an fp32 output
    differs from the fp32 reference only by the order of the sums: 1e-3 of max(|ref|, rms(ref)) per element, which a
    lost 64-wide k-block at K = 4096 (12 % of rms) fails by two orders of magnitude. A bf16 output adds its own rounding,
    half an ulp = 2^-9 relative; 2^-8 is allowed. `extra` (in units of rms) is for epilogues with device transcendentals."""
    ref = ref.float()
    rms = ref.pow(2).mean().sqrt().item()
    err = (c.float() - ref).abs()
    floor = torch.full_like(ref, rms)
    if c.dtype == torch.float32:
        bound = 1e-3 * torch.maximum(ref.abs(), floor) + extra * rms
    else:
        bound = 2.0 ** -8 * ref.abs() + (1e-3 + extra) * rms
    bad = err > bound
    assert not bad.any().item(), (c.dtype, int(bad.sum().item()), err.max().item(), rms, k)


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
    _check(y, torch.nn.functional.gelu(ref, approximate="tanh"), K, extra=2e-3)  # the device tanh is an approximation
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


@pytest.mark.parametrize("M,N,K", [(512, 512, 4096), (384, 264, 1088)])
def test_gemm_consumes_every_k_block_once(cuda, M, N, K):
    """Row m of A is non-zero only in k-block (m mod blocks), with the value (block + 1) / 64, and B is all ones: the
    exact result is C[m, :] = block + 1 for a 64-wide block. A k-block that is skipped gives 0, one that is read twice
    or from the wrong place gives another integer; every tile of the output sees every block."""
    blocks = K // 64
    a = torch.zeros(M, K, device=cuda, dtype=torch.bfloat16)
    rows = torch.arange(M, device=cuda)
    blk = rows % blocks
    cols = blk[:, None] * 64 + torch.arange(64, device=cuda)[None, :]
    a.scatter_(1, cols, ((blk + 1).float() / 64.0).to(torch.bfloat16)[:, None].expand(M, 64))
    b = torch.ones(N, K, device=cuda, dtype=torch.bfloat16)
    for dtype in (torch.float32, torch.bfloat16):
        c = G.gemm(a, b, out_dtype=dtype)
        torch.cuda.synchronize()
        G.check_errors()
        want = (blk + 1).float()[:, None].expand(M, N)
        assert torch.equal(c.float(), want), (dtype, (c.float() - want).abs().max().item())
    # and with random data a dropped block cannot hide inside the fp32 bound
    torch.manual_seed(4)
    x = torch.randn(M, K, device=cuda, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=cuda, dtype=torch.bfloat16)
    f = G.gemm(x, w, out_dtype=torch.float32)
    _check(f, _ref(x, w), K)
    lost = _ref(x[:, 64:], w[:, 64:])   # what a kernel that dropped the first block would return
    with pytest.raises(AssertionError):
        _check(lost, _ref(x, w), K)


def test_tensor_maps_of_repeated_operands_come_from_the_table(cuda):
    torch.manual_seed(6)
    a = torch.randn(512, 256, device=cuda, dtype=torch.bfloat16)
    b = torch.randn(384, 256, device=cuda, dtype=torch.bfloat16)
    out = torch.empty(512, 384, device=cuda, dtype=torch.bfloat16)
    G.gemm(a, b, out=out)
    h0, m0 = G.tensor_map_cache_stats()
    first = out.clone()
    for _ in range(5):
        G.gemm(a, b, out=out)
    h1, m1 = G.tensor_map_cache_stats()
    assert m1 == m0 and h1 >= h0 + 10      # the operand maps of every launch (and the output map where the epilogue
    # stores through TMA) come from the table, none is encoded again
    assert torch.equal(out, first)
    # same addresses, another shape: whatever the table holds, the answer belongs to the new shape
    c = G.gemm(a[:328], b)
    _check(c, _ref(a[:328], b), 256)
    torch.cuda.synchronize()
    G.check_errors()
