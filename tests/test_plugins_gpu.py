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
    """Stateful delta codec: round 1 passes raw data through (exact) and seeds the state; later rounds encode
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
