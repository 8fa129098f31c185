"""all-gather -> GEMM and GEMM -> FP8 reduce-scatter kernels, every rank emulated on one GPU, against fp32 PyTorch."""
import pytest
import torch

from coccl_b200.ops import codec as C
from coccl_b200.ops import tp_fused as T

pytestmark = pytest.mark.gpu


@pytest.fixture(params=["1cta", "2cta"])
def variant(request):
    """Both kernel families: single-CTA tiles, and CTA pairs (cta_group::2) where rows per rank are a multiple of 256."""
    T.set_variant("auto" if request.param == "2cta" else "1cta")
    yield request.param
    T.set_variant("auto")


@pytest.mark.parametrize("n,m,N,K,bias,gelu", [(2, 128, 256, 64, False, False), (2, 256, 520, 192, True, False),
                                               (4, 256, 512, 256, True, True), (2, 1024, 1024, 1024, False, False)])
def test_ag_gemm_emulated(cuda, variant, n, m, N, K, bias, gelu):
    torch.manual_seed(0)
    xs = [torch.randn(m, K, device=cuda, dtype=torch.bfloat16) for _ in range(n)]
    ws = [torch.randn(N, K, device=cuda, dtype=torch.bfloat16) * 0.1 for _ in range(n)]
    bs = [torch.randn(N, device=cuda, dtype=torch.bfloat16) for _ in range(n)] if bias else None
    state = {}
    for epoch in (1, 2):  # second call reuses flags and gather buffers
        outs, state = T.emulate_ag_gemm(xs, ws, bias=bs, gelu=gelu, state=state, epoch=epoch, max_ctas=148 // n)
        torch.cuda.synchronize()
        T.check_state(state)
        assert T.last_variant() == ("2cta" if variant == "2cta" and m % 256 == 0 else "1cta")
        xf = torch.cat(xs).float()
        for r in range(n):
            ref = xf @ ws[r].float().t()
            if bias:
                ref = ref + bs[r].float()
            if gelu:
                ref = torch.nn.functional.gelu(ref, approximate="tanh")
            err = (outs[r].float() - ref).abs().max().item()
            assert err <= 2e-2 * ref.abs().max().item() + 1e-3, (r, err)
        xs = [x * 0.5 for x in xs]


@pytest.mark.parametrize("n,M,N,K", [(2, 256, 256, 64), (2, 512, 512, 320), (4, 1024, 768, 256), (2, 2048, 1024, 1024), (4, 2048, 512, 2048)])
def test_gemm_rs_emulated(cuda, variant, n, M, N, K):
    torch.manual_seed(1)
    As = [torch.randn(M, K, device=cuda, dtype=torch.bfloat16) for _ in range(n)]
    Ws = [torch.randn(N, K, device=cuda, dtype=torch.bfloat16) * 0.1 for _ in range(n)]
    state = {}
    for epoch in (1, 2):
        outs, state = T.emulate_gemm_rs(As, Ws, state=state, epoch=epoch, max_ctas=148 // n)
        torch.cuda.synchronize()
        T.check_state(state)
        pair = variant == "2cta" and (M // n) % 256 == 0
        assert T.last_variant() == ("2cta" if pair else "1cta")
        parts = [As[q].float() @ Ws[q].float().t() for q in range(n)]
        exact = sum(parts)
        # oracle of the transport: every partial product goes through the MX-FP8 codec (32 columns per block)
        qparts = [C.reference_roundtrip(p.contiguous(), C.MXFP8, 1) for p in parts]
        rows = M // n
        for r in range(n):
            got = outs[r].float()
            # the pair kernel adds a rank's own partial product straight from the accumulator, unquantised
            ref_q = sum((parts[q] if (pair and q == r) else qparts[q])[r * rows:(r + 1) * rows] for q in range(n))
            ref = exact[r * rows:(r + 1) * rows]
            # the kernel's fp32 sums differ from torch's in the last bits, which can flip an E4M3 rounding
            # decision: almost every element matches the oracle, a flipped one is off by one step (<= |x|/8)
            d = (got - ref_q).abs()
            scale = ref.abs().max().item()
            assert (d > 1e-2 * scale + 1e-3).float().mean().item() < 2e-3
            assert d.max().item() <= scale / 8 + 1e-3
            rel = (got - ref).norm().item() / ref.norm().item()
            assert rel < 0.05, rel
        As = [a * 0.5 for a in As]


def test_weights_stored_contraction_major(cuda):
    """b_mn: the weight is stored [K, N] (the layout the backward passes meet); same products as with its transpose."""
    torch.manual_seed(2)
    n, m, N, K = 2, 256, 512, 320
    xs = [torch.randn(m, K, device=cuda, dtype=torch.bfloat16) for _ in range(n)]
    ws = [torch.randn(K, N, device=cuda, dtype=torch.bfloat16) * 0.1 for _ in range(n)]
    outs, st = T.emulate_ag_gemm(xs, ws, b_mn=True, max_ctas=74)
    torch.cuda.synchronize()
    T.check_state(st)
    xf = torch.cat(xs).float()
    for r in range(n):
        ref = xf @ ws[r].float()
        assert (outs[r].float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-3
    As = [torch.randn(n * m, K, device=cuda, dtype=torch.bfloat16) for _ in range(n)]
    outs, st = T.emulate_gemm_rs(As, ws, b_mn=True, max_ctas=74)
    torch.cuda.synchronize()
    T.check_state(st)
    exact = sum(As[q].float() @ ws[q].float() for q in range(n))
    for r in range(n):
        ref = exact[r * m:(r + 1) * m]
        assert ((outs[r].float() - ref).norm() / ref.norm()).item() < 0.05


@pytest.mark.parametrize("n,m,N,K,keep", [(2, 256, 512, 256, False), (4, 256, 264, 1024, True), (2, 1024, 1024, 4096, True)])
def test_ag_gemm_fp8_payload_emulated(cuda, n, m, N, K, keep):
    """Shards that cross between ranks as E4M3 + UE8M0 scales: a rank's own shard stays exact, every remote shard equals
    the MX-FP8 codec's round trip (32 columns per block), bit for bit, in the gathered copy, and the product follows."""
    T.set_variant("auto")
    torch.manual_seed(5)
    xs = [torch.randn(m, K, device=cuda, dtype=torch.bfloat16) * (0.5 + r) for r in range(n)]
    ws = [torch.randn(N, K, device=cuda, dtype=torch.bfloat16) * 0.05 for _ in range(n)]
    xq = [C.reference_roundtrip(x.float().contiguous(), C.MXFP8, 1).to(torch.bfloat16) for x in xs]
    state = {}
    for epoch in (1, 2):
        kept = [torch.zeros(m * n, K, device=cuda, dtype=torch.bfloat16) for _ in range(n)] if keep else None
        outs, state = T.emulate_ag_gemm(xs, ws, state=state, epoch=epoch, max_ctas=148 // n, payload=T.PAYLOAD_FP8, gathered=kept)
        torch.cuda.synchronize()
        T.check_state(state)
        assert T.last_variant() == "2cta"
        for r in range(n):
            seen = torch.cat([xs[q] if q == r else xq[q] for q in range(n)])   # what rank r multiplies
            if keep:
                assert torch.equal(kept[r], seen), (r, (kept[r].float() - seen.float()).abs().max().item())
            ref = seen.float() @ ws[r].float().t()
            err = (outs[r].float() - ref).abs().max().item()
            assert err <= 2e-2 * ref.abs().max().item() + 1e-3, (r, err)
            exact = torch.cat(xs).float() @ ws[r].float().t()
            assert ((outs[r].float() - exact).norm() / exact.norm()).item() < 0.05
        xs = [x * 0.5 for x in xs]
        xq = [C.reference_roundtrip(x.float().contiguous(), C.MXFP8, 1).to(torch.bfloat16) for x in xs]
