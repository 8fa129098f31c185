"""Compressor plugins driven through the C++ compressor runtime (dlopen, parseConfig, size bound, compress,
decompress / decompressReduce) on one GPU, checked against the PyTorch fp32 oracle."""
import ctypes as C
from pathlib import Path

import pytest
import torch

from coccl_b200 import _lib
from coccl_b200.ops import codec as K

pytestmark = pytest.mark.gpu
PLUGINS = str(Path(_lib.__file__).resolve().parent / "lib" / "plugins")
NCCL_DT = {torch.float32: 7, torch.float16: 6, torch.bfloat16: 9, torch.int8: 0, torch.int32: 2}


def roundtrip(name, options, x, chunks=1, reduce=1, rounds=1):
    fn = _lib.declare("cocclApiCodecRoundTrip", C.c_int,
                      [C.c_char_p, C.c_char_p, C.c_char_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_int,
                       C.c_size_t, C.c_int, C.POINTER(C.c_size_t), C.c_void_p])
    out = torch.empty(x.numel() // reduce, dtype=x.dtype, device=x.device)
    enc = C.c_size_t(0)
    rc = fn(PLUGINS.encode(), name.encode(), options.encode(), x.data_ptr(), out.data_ptr(), x.numel(), chunks,
            NCCL_DT[x.dtype], reduce, rounds, C.byref(enc), torch.cuda.current_stream().cuda_stream)
    return rc, out, enc.value


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_sdp4bit_plugin_matches_oracle_and_reference_sizes(cuda, dtype):
    torch.manual_seed(0)
    x = (torch.randn(4 * 256, device=cuda) * 0.01).to(dtype)
    rc, y, enc = roundtrip("sdp4bit", "groupCount=128,quantBits=4,quantType=Symmetric,hadamard=true,rounding=nearest", x, chunks=4)
    assert rc == 0
    assert enc == (544 if dtype == torch.float32 else 576)   # exact encoded sizes of the reference contract
    ref = K.reference_roundtrip(x, K.CodecConfig("sdp4bit", 4, 128, False, True), 4).to(dtype)
    assert ((y.float() - ref.float()).abs() > 1e-6 + 2e-3 * ref.abs().max().item()).float().mean().item() < 5e-3
    # default options: 8 bits, groups of 2048, stochastic rounding
    x = (torch.randn(1 << 16, device=cuda)).to(dtype)
    rc, y, enc = roundtrip("sdp4bit", "", x)
    assert rc == 0 and ((y.float() - x.float()).norm() / x.float().norm()).item() < 0.02


def test_sdp4bit_plugin_fused_reduce_and_rejections(cuda):
    torch.manual_seed(1)
    x = torch.randn(8 * 5000, device=cuda) * 0.01
    rc, y, _ = roundtrip("sdp4bit", "groupCount=128,quantBits=4,hadamard=true,rounding=nearest", x, chunks=8, reduce=8)
    assert rc == 0
    ref = K.reference_roundtrip(x, K.CodecConfig("sdp4bit", 4, 128, False, True), 8).reshape(8, 5000).sum(0)
    assert torch.allclose(y, ref, atol=2e-2 * ref.abs().max().item())
    assert roundtrip("sdp4bit", "quantBits=5", x)[0] != 0
    assert roundtrip("sdp4bit", "subAdd=true,hadamard=true", x)[0] != 0
    assert roundtrip("sdp4bit", "groupCount=100", x)[0] != 0
    assert roundtrip("sdp4bit", "noSuchOption=1", x)[0] != 0


def test_sdp4bit_subadd_seeds_then_sends_deltas(cuda):
    """Stateful delta codec: the first call passes raw data through (exact) and seeds the state; later calls encode
    x - prev at 8 bits, so a value that did not change is reproduced exactly and the error shrinks."""
    torch.manual_seed(2)
    x = torch.randn(1 << 16, device=cuda, dtype=torch.bfloat16)
    rc, y1, enc1 = roundtrip("sdp4bit", "groupCount=2048,quantBits=8,subAdd=true,pipelineSize=1", x, rounds=1)
    assert rc == 0 and torch.equal(y1, x) and enc1 == x.numel() * 2      # raw pass-through
    rc, y2, enc2 = roundtrip("sdp4bit", "groupCount=2048,quantBits=8,subAdd=true,pipelineSize=1", x, rounds=3)
    assert rc == 0 and enc2 < enc1 * 0.6                                  # deltas travel encoded
    assert torch.equal(y2, x)                                             # zero delta decodes to exactly prev


def test_fp8block_plugin(cuda):
    torch.manual_seed(3)
    x = torch.randn(4 * 4096, device=cuda, dtype=torch.bfloat16)
    rc, y, enc = roundtrip("fp8block", "", x, chunks=4)
    assert rc == 0 and enc == 4 * (4096 + 128)
    ref = K.reference_roundtrip(x, K.MXFP8, 4).to(torch.bfloat16)
    assert torch.allclose(y.float(), ref.float(), atol=1e-6, rtol=1e-2)
    rc, y, _ = roundtrip("fp8block", "", x, chunks=4, reduce=4)
    assert rc == 0
    assert torch.allclose(y.float(), ref.float().reshape(4, 4096).sum(0), atol=5e-2, rtol=2e-2)
    assert roundtrip("fp8block", "blockSize=64", x)[0] != 0


def _taco_reference(x, chunks, group, target=448.0, lam=1e-6, fp8max=448.0):
    """TACO numerics in plain PyTorch (taco/taco.cu:118-218): adaptive scale, group Hadamard, FP8 E4M3."""
    n = x.numel() // chunks
    xf = x.float().reshape(chunks, n // group, group)
    h = torch.ones(1, 1, device=x.device)
    while h.shape[0] < group:
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    ada = (fp8max * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + lam)).clamp(1e-3, 1e3)
    y = (xf * ada) @ h / group ** 0.5
    qs = (y.abs().amax(-1, keepdim=True) / target).clamp(1e-12, 1e6)
    code = (y / qs).clamp(-448, 448).to(torch.float8_e4m3fn).float()
    return ((code * qs) @ h / group ** 0.5 / ada).reshape(x.shape)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("group", [32, 128, 512])
def test_taco_plugin(cuda, dtype, group):
    torch.manual_seed(3)
    x = (torch.randn(4 * 256 * 8, device=cuda) * 0.05).to(dtype)
    rc, y, enc = roundtrip("taco", f"groupSize={group}", x, chunks=4)
    assert rc == 0
    assert enc == x.numel() + (x.numel() // group) * 8  # fp8 bytes of whole groups + two floats per group
    ref = _taco_reference(x, 4, group).to(dtype).float()
    d = (y.float() - ref).abs()
    scale = ref.abs().max().item()
    assert (d > 2e-2 * scale).float().mean().item() < 5e-3  # a flipped FP8 rounding is spread over the group
    assert ((y.float() - x.float()).norm() / x.float().norm()).item() < 0.05
    if group == 128 and dtype == torch.float32:
        assert roundtrip("taco", "groupSize=128", x[:1024].contiguous(), chunks=4)[2] == 1088  # reference size contract
    assert roundtrip("taco", "groupSize=100", x)[0] != 0
    # ragged chunk: 1000 values per chunk, last group partly filled
    xr = (torch.randn(3 * 1000, device=cuda) * 0.05).to(dtype)
    rc, yr, _ = roundtrip("taco", f"groupSize={group}", xr, chunks=3)
    assert rc == 0 and ((yr.float() - xr.float()).norm() / xr.float().norm()).item() < 0.05
    rc, ye, _ = roundtrip("taco", "fp8Format=E5M2,groupSize=64", x, chunks=4)
    assert rc == 0 and ((ye.float() - x.float()).norm() / x.float().norm()).item() < 0.1


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rate", [4, 8, 11, 16])
def test_zfp_plugin_matches_cpu_oracle(cuda, dtype, rate):
    torch.manual_seed(4)
    chunks, count = 3, 4 * 1000 + 2  # ragged: the last block of a chunk is partly filled
    x = (torch.randn(chunks * count, device=cuda) * 0.01).to(dtype)
    rc, y, enc = roundtrip("zfp", f"rate={rate}", x, chunks=chunks)
    assert rc == 0
    lib = _lib.lib()
    cb = _lib.declare("cocclOracleZfpChunkBytes", C.c_long, [C.c_long, C.c_int])
    en = _lib.declare("cocclOracleZfpEncode", C.c_int, [C.c_void_p, C.c_long, C.c_int, C.c_void_p])
    de = _lib.declare("cocclOracleZfpDecode", C.c_int, [C.c_void_p, C.c_long, C.c_int, C.c_void_p])
    nbytes = cb(count, rate)
    if nbytes * chunks > x.numel() * x.element_size():
        # encoding would expand the data: the plugin passes the bytes through unchanged
        assert enc == x.numel() * x.element_size() and torch.equal(y, x)
        return
    assert enc == nbytes * chunks
    xc = x.float().cpu().reshape(chunks, count).contiguous()
    ref = torch.empty_like(xc)
    buf = torch.empty(nbytes, dtype=torch.uint8)
    for ch in range(chunks):
        assert en(xc[ch].data_ptr(), count, rate, buf.data_ptr()) == 0
        assert de(buf.data_ptr(), count, rate, ref[ch].data_ptr()) == 0
    # same coder on both sides: identical up to the rounding into the output type
    got, want = y.cpu().float().reshape(chunks, count), ref.to(dtype).float()
    if dtype == torch.float32:
        assert torch.equal(got, want)
    else:  # the last rounding into 16 bits may differ by one unit on a few values
        bad = (got != want)
        assert bad.float().mean().item() < 1e-2, bad.float().mean().item()
        assert ((got - want).abs() <= want.abs() * 2.0 ** -7 + 1e-12).all()
    if rate >= 8:
        assert ((y.float() - x.float()).abs().max() / x.float().abs().max()).item() < 2.0 ** (-(rate - 6) / 1.0) * 4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int8, torch.int32])
def test_ans_plugin_is_lossless_and_framed(cuda, dtype):
    torch.manual_seed(5)
    chunks, count = 4, 3 * 4096 + 1000
    if dtype.is_floating_point:
        x = (torch.randn(chunks * count, device=cuda) * 0.01).to(dtype)  # exponent bytes are very skewed
    elif dtype == torch.int8:
        x = (torch.randn(chunks * count, device=cuda) * 6).round().clamp(-128, 127).to(torch.int8)
    else:
        x = torch.randint(0, 100, (chunks * count,), device=cuda, dtype=torch.int32)
    for pb in (9, 10, 11):
        rc, y, enc = roundtrip("ans", f"probBits={pb}", x, chunks=chunks)
        assert rc == 0 and torch.equal(y, x)
        assert enc < x.numel() * x.element_size()
    # incompressible bytes: every frame falls back to raw and still round-trips
    u = torch.randint(-128, 128, (chunks * 8192,), device=cuda, dtype=torch.int8)
    rc, y, enc = roundtrip("ans", "", u, chunks=chunks)
    assert rc == 0 and torch.equal(y, u) and enc == u.numel()
    assert roundtrip("ans", "probBits=12", x, chunks=chunks)[0] != 0


def test_ans_plugin_frames_decode_with_cpu_oracle(cuda):
    """The GPU coder and the CPU oracle share the frame format: compare sizes on identical input."""
    torch.manual_seed(6)
    n = 5 * 4096
    x = (torch.randn(n, device=cuda) * 6).round().clamp(-128, 127).to(torch.int8)
    rc, y, enc = roundtrip("ans", "probBits=10", x, chunks=1)
    assert rc == 0 and torch.equal(y, x)
    bound = _lib.declare("cocclOracleRansFrameBound", C.c_long, [C.c_long])
    en = _lib.declare("cocclOracleRansEncode", C.c_long, [C.c_void_p, C.c_long, C.c_int, C.c_void_p])
    xc = x.cpu().view(torch.uint8).contiguous()
    frame = torch.zeros(bound(n), dtype=torch.uint8)
    assert en(xc.data_ptr(), n, 10, frame.data_ptr()) == enc
