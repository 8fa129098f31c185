"""sm_100a codec kernels against the plain PyTorch fp32 oracle (coccl_b200.ops.codec.reference_roundtrip)."""
import pytest
import torch

from coccl_b200.ops import codec as C

pytestmark = pytest.mark.gpu

CFGS = [
    C.CodecConfig("sdp4bit", 4, 128, False, True),
    C.CodecConfig("sdp4bit", 4, 128, False, False),
    C.CodecConfig("sdp4bit", 8, 2048, False, False),
    C.CodecConfig("sdp4bit", 8, 512, False, True),
    C.CodecConfig("sdp4bit", 4, 64, True, False),
    C.CodecConfig("sdp4bit", 8, 128, True, True),
    C.CodecConfig("sdp4bit", 4, 32, False, True),
    C.MXFP8,
]


def _step(x, cfg):
    """Largest quantisation step of any group (bound on a single rounding flip)."""
    if cfg.kind == "mxfp8":
        return x.abs().max().item() / 8.0
    levels = (1 << (cfg.bits - 1)) - 1
    amax = x.abs().max().item() * (32 ** 0.5 * 4 if cfg.hadamard else 1.0)
    return 2.0 * amax / levels


@pytest.mark.parametrize("cfg", CFGS, ids=lambda c: f"{c.kind}{c.bits}g{c.group}{'a' if c.asym else 's'}{'h' if c.hadamard else ''}")
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("count,chunks", [(4096, 4), (1000, 3), (2048 * 5 + 136, 1), (8192 * 3 + 40, 2), (16384, 2)])
def test_roundtrip_matches_oracle(cuda, cfg, dtype, count, chunks):
    torch.manual_seed(0)
    x = (torch.randn(chunks * count, device=cuda) * 0.01).to(dtype)
    enc = C.encode(x, cfg, chunks)
    assert enc.shape == (chunks, cfg.encoded_chunk_bytes(count, dtype))
    y = C.decode(enc, cfg, count, dtype, chunks).reshape(-1).float()
    ref = C.reference_roundtrip(x, cfg, chunks).reshape(-1).to(dtype).float()
    diff = (y - ref).abs()
    # identical arithmetic up to fma contraction: almost every element matches to rounding of the
    # output type; a flipped rounding decision moves an element by at most one step
    tol = 1e-6 + 2e-3 * ref.abs().max().item()
    frac_bad = (diff > tol).float().mean().item()
    assert frac_bad < 2e-3, f"{frac_bad=} max={diff.max().item()}"
    assert diff.max().item() <= _step(x.float(), cfg) + tol


def test_encoded_sizes_match_reference_contract():
    # 1024 elements in 4 chunks, g128 q4: 544 B fp32, 576 B for 16-bit inputs
    cfg = C.CodecConfig("sdp4bit", 4, 128, False, True)
    assert 4 * cfg.encoded_chunk_bytes(256, torch.float32) == 544
    assert 4 * cfg.encoded_chunk_bytes(256, torch.bfloat16) == 576
    assert 4 * cfg.encoded_chunk_bytes(256, torch.float16) == 576


@pytest.mark.parametrize("cfg", [CFGS[0], CFGS[1], CFGS[2], CFGS[7]], ids=["q4h", "q4", "q8g2048", "mxfp8"])
def test_decode_reduce_and_drc(cuda, cfg):
    torch.manual_seed(1)
    n, count, chunks = 8, 5000, 2
    xs = [torch.randn(chunks * count, device=cuda) * 0.01 for _ in range(n)]
    enc = torch.cat([C.encode(x, cfg, chunks) for x in xs], dim=0)  # [n*chunks, B], copy i chunk j at i*chunks+j
    red = C.decode_reduce(enc, cfg, count, torch.float32, chunks, n).reshape(-1)
    ref = sum(C.reference_roundtrip(x, cfg, chunks).reshape(-1) for x in xs)
    assert torch.allclose(red, ref, atol=n * _step(xs[0], cfg) * 2e-3 + 1e-5, rtol=1e-4) or \
        ((red - ref).abs() > 1e-4).float().mean().item() < 2e-3
    # fused decode-reduce-encode == decode-reduce followed by encode without rotation; compare after decode
    drc = C.decode_reduce_encode(enc, cfg, count, torch.float32, chunks, n)
    back = C.decode(drc, cfg, count, torch.float32, chunks).reshape(-1)
    err = (back - ref).abs().max().item()
    bound = _step(ref, cfg)
    assert err <= bound, (err, bound)


def test_stochastic_rounding_is_unbiased_and_reproducible(cuda):
    cfg = C.CodecConfig("sdp4bit", 4, 128, False, False, True, seed=123)
    x = torch.full((1 << 20,), 0.3, device=cuda)
    x[::128] = 1.0  # absmax 1 -> scale 7, 0.3*7 = 2.1 -> rounds to 2 (p=.9) or 3 (p=.1)
    a = C.decode(C.encode(x, cfg), cfg, x.numel(), torch.float32).reshape(-1)
    b = C.decode(C.encode(x, cfg), cfg, x.numel(), torch.float32).reshape(-1)
    assert torch.equal(a, b)
    mask = torch.ones_like(x, dtype=torch.bool)
    mask[::128] = False
    assert abs(a[mask].mean().item() - 0.3) < 2e-3
    ref = C.reference_roundtrip(x, cfg)
    assert ((a - ref).abs() > 1e-6).float().mean().item() < 1e-3


@pytest.mark.parametrize("rate", [4, 8, 16])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("count,chunks", [(4096, 2), (1002, 3), (8192 * 2 + 36, 1)])
def test_zfp_tile_codec_is_bit_identical_to_the_cpu_coder(cuda, rate, dtype, count, chunks):
    """The tile codec writes the same stream as the CPU coder of csrc/oracle (block i at bit i * 4 * rate), and
    decodes to the same values; sums of several encoded copies equal the sum of the oracle's decodes."""
    import ctypes as CT
    from coccl_b200 import _lib
    cfg = C.CodecConfig("zfp", rate, 4, False, False)
    torch.manual_seed(11)
    x = (torch.randn(chunks * count, device=cuda) * 0.01).to(dtype)
    enc = C.encode(x, cfg, chunks)
    en = _lib.declare("cocclOracleZfpEncode", CT.c_int, [CT.c_void_p, CT.c_long, CT.c_int, CT.c_void_p])
    cb = _lib.declare("cocclOracleZfpChunkBytes", CT.c_long, [CT.c_long, CT.c_int])
    xc = x.float().cpu().reshape(chunks, count).contiguous()
    want = torch.zeros(cb(count, rate), dtype=torch.uint8)
    for ch in range(chunks):
        want.zero_()
        assert en(xc[ch].data_ptr(), count, rate, want.data_ptr()) == 0
        got = enc[ch].cpu()
        nbytes = (-(-count // 4) * 4 * rate + 7) // 8       # bits of the whole blocks, in bytes
        assert torch.equal(got[:nbytes], want[:nbytes]), (ch, (got[:nbytes] != want[:nbytes]).nonzero()[:4])
    ref = C.reference_roundtrip(x, cfg, chunks)
    y = C.decode(enc, cfg, count, dtype, chunks).reshape(-1)
    if dtype == torch.float32:
        assert torch.equal(y.cpu(), ref.cpu())
    else:
        assert ((y.float().cpu() - ref.cpu()).abs() <= ref.cpu().abs() * 2.0 ** -7 + 1e-12).all()
    if chunks > 1 and dtype == torch.float32:
        s = C.decode_reduce(enc, cfg, count, dtype, 1, chunks).reshape(-1)
        assert torch.allclose(s.cpu(), ref.cpu().reshape(chunks, count).sum(0), atol=1e-6)


@pytest.mark.parametrize("group", [32, 128, 512])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("count,chunks", [(4096, 2), (1000, 3), (8192 * 2 + 200, 1)])
def test_taco_tile_codec_matches_oracle(cuda, group, dtype, count, chunks):
    cfg = C.CodecConfig("taco", 8, group, False, False)
    torch.manual_seed(12)
    x = (torch.randn(chunks * count, device=cuda) * 0.05).to(dtype)
    enc = C.encode(x, cfg, chunks)
    assert enc.shape[1] == -(-count // group) * (group + 8)
    y = C.decode(enc, cfg, count, dtype, chunks).reshape(-1).float()
    ref = C.reference_roundtrip(x, cfg, chunks).reshape(-1).to(dtype).float()
    scale = ref.abs().max().item()
    assert ((y - ref).abs() > 2e-2 * scale).float().mean().item() < 5e-3   # a flipped FP8 rounding is spread over the group
    assert ((y - x.float()).norm() / x.float().norm()).item() < 0.05
    if chunks > 1:
        # copies with different adaptive scales add up in the rotated domain; one inverse transform serves the sum
        s = C.decode_reduce(enc, cfg, count, dtype, 1, chunks).reshape(-1).float()
        want = C.reference_roundtrip(x, cfg, chunks).reshape(chunks, count).sum(0)
        assert ((s - want).norm() / want.norm()).item() < 0.02
        drc = C.decode_reduce_encode(enc, cfg, count, dtype, 1, chunks)
        s2 = C.decode(drc, cfg, count, dtype, 1).reshape(-1).float()
        assert ((s2 - want).norm() / want.norm()).item() < 0.06
