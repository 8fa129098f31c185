"""CPU oracles exported by libcoccl.so against the PyTorch restatement of the same arithmetic (no GPU)."""
import ctypes as C

import pytest
import torch

from coccl_b200 import _lib
from coccl_b200.ops import codec as K


@pytest.mark.parametrize("bits,group,asym,had", [(4, 128, False, True), (8, 2048, False, False), (4, 64, True, False),
                                                 (8, 128, True, True), (4, 8, False, False)])
def test_sdp4bit_cpu_oracle_matches_pytorch(bits, group, asym, had):
    torch.manual_seed(0)
    chunks, count = 3, 5000
    x = torch.randn(chunks * count)
    fn = _lib.declare("cocclOracleSdp4bitRoundTrip", C.c_int,
                      [C.c_void_p, C.c_long, C.c_long, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p,
                       C.POINTER(C.c_double), C.POINTER(C.c_double)])
    out = torch.empty_like(x)
    mx, rms = C.c_double(), C.c_double()
    assert fn(x.data_ptr(), count, chunks, bits, group, int(asym), int(had), out.data_ptr(), C.byref(mx), C.byref(rms)) == 0
    ref = K.reference_roundtrip(x, K.CodecConfig("sdp4bit", bits, group, asym, had), chunks)
    d = (out - ref).abs()
    assert (d > 1e-6 + 1e-5 * ref.abs().max()).float().mean().item() < 1e-3  # Hadamard summation order only
    assert abs(mx.value - (out - x).abs().max().item()) < 1e-6
    assert abs(rms.value - (out - x).pow(2).mean().sqrt().item()) < 1e-6


def test_zfp_cpu_oracle_rate_and_error():
    torch.manual_seed(1)
    n = 4096
    x = torch.randn(n)
    cb = _lib.declare("cocclOracleZfpChunkBytes", C.c_long, [C.c_long, C.c_int])
    en = _lib.declare("cocclOracleZfpEncode", C.c_int, [C.c_void_p, C.c_long, C.c_int, C.c_void_p])
    de = _lib.declare("cocclOracleZfpDecode", C.c_int, [C.c_void_p, C.c_long, C.c_int, C.c_void_p])
    assert cb(n, 8) == n  # 8 bits per value: 4x for fp32, 2x for 16-bit inputs
    prev = None
    for rate in (4, 8, 12, 16, 24, 32):
        buf = torch.zeros(cb(n, rate), dtype=torch.uint8)
        y = torch.empty_like(x)
        assert en(x.data_ptr(), n, rate, buf.data_ptr()) == 0 and de(buf.data_ptr(), n, rate, y.data_ptr()) == 0
        err = (y - x).abs().max().item()
        assert prev is None or err <= prev
        prev = err
    assert prev < 1e-6  # 32 bits per value: only the rounding of the block-floating-point conversion is left
    z = torch.zeros(64)
    buf = torch.zeros(cb(64, 8), dtype=torch.uint8)
    y = torch.ones(64)
    assert en(z.data_ptr(), 64, 8, buf.data_ptr()) == 0 and de(buf.data_ptr(), 64, 8, y.data_ptr()) == 0
    assert torch.equal(y, z) and int(buf.sum()) == 0


def test_rans_cpu_oracle_roundtrip_and_ratio():
    torch.manual_seed(2)
    bound = _lib.declare("cocclOracleRansFrameBound", C.c_long, [C.c_long])
    en = _lib.declare("cocclOracleRansEncode", C.c_long, [C.c_void_p, C.c_long, C.c_int, C.c_void_p])
    de = _lib.declare("cocclOracleRansDecode", C.c_int, [C.c_void_p, C.c_long, C.c_void_p])
    n = 3 * 4096 + 1000
    # skewed bytes compress; uniform bytes do not (the coder reports 0 = store raw)
    skew = (torch.randn(n) * 6).round().clamp(-128, 127).to(torch.int8).view(torch.uint8).contiguous()
    for pb in (9, 10, 11):
        frame = torch.zeros(bound(n), dtype=torch.uint8)
        size = en(skew.data_ptr(), n, pb, frame.data_ptr())
        assert 0 < size < 0.7 * n
        out = torch.zeros(n, dtype=torch.uint8)
        assert de(frame.data_ptr(), n, out.data_ptr()) == 0
        assert torch.equal(out, skew)
    uni = torch.randint(0, 256, (n,), dtype=torch.uint8)
    frame = torch.zeros(bound(n), dtype=torch.uint8)
    assert en(uni.data_ptr(), n, 10, frame.data_ptr()) == 0
    const = torch.full((n,), 7, dtype=torch.uint8)
    size = en(const.data_ptr(), n, 10, frame.data_ptr())
    out = torch.zeros(n, dtype=torch.uint8)
    assert 0 < size < 0.1 * n and de(frame.data_ptr(), n, out.data_ptr()) == 0 and torch.equal(out, const)
