"""This library's ZFP stream against real ZFP: the reference's vendored LLNL sources, compiled unmodified for the host
(baseline/build_zfp_host.py) and run with the serial execution policy, must write the same bytes as the CPU coder that
the GPU kernels share (oracle/zfp1d.h), for one-dimensional fp32 data at fixed rate."""
import ctypes as C
import importlib.util
from pathlib import Path

import pytest
import torch

from coccl_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def zfp():
    spec = importlib.util.spec_from_file_location("build_zfp_host", ROOT / "baseline" / "build_zfp_host.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    path = mod.library() if mod.library().exists() else mod.build(quiet=True)
    if path is None:
        pytest.skip("the reference's sources are not on this machine")
    lib = C.CDLL(str(path))
    vp = C.c_void_p
    lib.zfp_stream_open.restype, lib.zfp_stream_open.argtypes = vp, [vp]
    lib.zfp_stream_close.argtypes = [vp]
    lib.zfp_stream_set_rate.restype, lib.zfp_stream_set_rate.argtypes = C.c_double, [vp, C.c_double, C.c_int, C.c_uint, C.c_int]
    lib.zfp_field_1d.restype, lib.zfp_field_1d.argtypes = vp, [vp, C.c_int, C.c_size_t]
    lib.zfp_field_free.argtypes = [vp]
    lib.zfp_stream_maximum_size.restype, lib.zfp_stream_maximum_size.argtypes = C.c_size_t, [vp, vp]
    lib.stream_open.restype, lib.stream_open.argtypes = vp, [vp, C.c_size_t]
    lib.stream_close.argtypes = [vp]
    lib.zfp_stream_set_bit_stream.argtypes = [vp, vp]
    lib.zfp_stream_rewind.argtypes = [vp]
    lib.zfp_compress.restype, lib.zfp_compress.argtypes = C.c_size_t, [vp, vp]
    lib.zfp_decompress.restype, lib.zfp_decompress.argtypes = C.c_size_t, [vp, vp]
    return lib


ZFP_TYPE_FLOAT = 3


def _reference_stream(lib, x: torch.Tensor, rate: int) -> torch.Tensor:
    stream = lib.zfp_stream_open(None)
    assert lib.zfp_stream_set_rate(stream, float(rate), ZFP_TYPE_FLOAT, 1, 0) == float(rate)
    field = lib.zfp_field_1d(x.data_ptr(), ZFP_TYPE_FLOAT, x.numel())
    cap = lib.zfp_stream_maximum_size(stream, field)
    buf = torch.zeros(cap, dtype=torch.uint8)
    bits = lib.stream_open(buf.data_ptr(), cap)
    lib.zfp_stream_set_bit_stream(stream, bits)
    lib.zfp_stream_rewind(stream)
    size = lib.zfp_compress(stream, field)
    assert size > 0
    lib.zfp_field_free(field)
    lib.zfp_stream_close(stream)
    lib.stream_close(bits)
    return buf[:size].clone()


def _inputs():
    g = torch.Generator().manual_seed(0)
    n = 4096
    yield "normal", torch.randn(n, generator=g)
    yield "small", torch.randn(n, generator=g) * 1e-2
    yield "wide range", torch.randn(n, generator=g) * torch.exp(torch.randn(n, generator=g) * 6)
    x = torch.randn(n, generator=g)
    x[128:640] = 0.0                       # whole blocks of zeros, and blocks with a few
    x[1000:1003] = 0.0
    yield "zeros inside", x
    yield "constant", torch.full((n,), 3.25)
    yield "tiny and huge", torch.cat([torch.full((2048,), 1e-38), torch.full((2048,), 1e38)]) * torch.randn(n, generator=g).sign()
    yield "ramp", torch.arange(n, dtype=torch.float32) / 7.0 - 300.0


@pytest.mark.parametrize("rate", [4, 8, 12, 16, 24, 32])
def test_stream_equals_real_zfp_bit_for_bit(zfp, rate):
    chunk_bytes = _lib.declare("cocclOracleZfpChunkBytes", C.c_long, [C.c_long, C.c_int])
    encode = _lib.declare("cocclOracleZfpEncode", C.c_int, [C.c_void_p, C.c_long, C.c_int, C.c_void_p])
    decode = _lib.declare("cocclOracleZfpDecode", C.c_int, [C.c_void_p, C.c_long, C.c_int, C.c_void_p])
    for name, x in _inputs():
        x = x.contiguous()
        want = _reference_stream(zfp, x, rate)
        mine = torch.zeros(chunk_bytes(x.numel(), rate), dtype=torch.uint8)
        assert encode(x.data_ptr(), x.numel(), rate, mine.data_ptr()) == 0
        assert mine.numel() == want.numel(), (name, rate, mine.numel(), want.numel())
        diff = (mine != want).nonzero()
        assert diff.numel() == 0, (name, rate, "first differing byte", int(diff[0]), int(mine[diff[0]]), int(want[diff[0]]))
        # and real ZFP decodes this library's stream to what this library decodes
        y = torch.empty_like(x)
        assert decode(mine.data_ptr(), x.numel(), rate, y.data_ptr()) == 0
        stream = zfp.zfp_stream_open(None)
        zfp.zfp_stream_set_rate(stream, float(rate), ZFP_TYPE_FLOAT, 1, 0)
        z = torch.empty_like(x)
        field = zfp.zfp_field_1d(z.data_ptr(), ZFP_TYPE_FLOAT, z.numel())
        bits = zfp.stream_open(mine.data_ptr(), mine.numel())
        zfp.zfp_stream_set_bit_stream(stream, bits)
        zfp.zfp_stream_rewind(stream)
        assert zfp.zfp_decompress(stream, field) > 0
        zfp.zfp_field_free(field)
        zfp.zfp_stream_close(stream)
        zfp.stream_close(bits)
        assert torch.equal(y, z), (name, rate)
