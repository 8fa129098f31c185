"""Codec front end: configuration objects, the sm_100a encode / decode(-reduce)
/ decode-reduce-encode kernels, and plain PyTorch fp32 reference
implementations of the same codecs (the oracle used by the numerics tests).

Codec semantics follow the reference plugins: SDP4Bit
(src/coccl-extend/extensions/compressor_plugin/sdp4bit/sdp4bit_quan.cu:14-109,
includes/quantization_utils.h:126-272) and, for the block-scaled FP8 codec that
the reference does not ship, TACO (taco/taco.cu:89-295) as behavioural model.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import _lib

DTYPE_CODE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
KIND_SDP4BIT, KIND_MXFP8, KIND_TACO, KIND_ZFP = 0, 1, 3, 4


@dataclass(frozen=True)
class CodecConfig:
    kind: str = "sdp4bit"          # "sdp4bit" | "mxfp8" | "taco" | "zfp"
    bits: int = 4                  # sdp4bit: 4 | 8; zfp: the rate in bits per value (4 | 8 | 16); taco: 8
    group: int = 128               # elements per quantisation group (mxfp8: 32; zfp: 4, one block; taco: 32..512)
    asym: bool = False
    hadamard: bool = True
    stochastic: bool = False
    seed: int = 0
    # taco only (reference options fp8Format, saturate, targetRange, lambda, fp8MaxValue; taco/taco.cu:16-33)
    e5m2: bool = False
    saturate: bool = True
    target_range: float = 448.0
    lam: float = 1e-6
    fp8_max: float = 0.0

    def param_bytes(self, dtype: torch.dtype) -> int:
        if self.kind == "mxfp8":
            return 1
        if self.kind == "taco":
            return 8
        if self.kind == "zfp":
            return 0
        # fp32 symmetric stores one float per group; asymmetric and all 16-bit inputs store two
        # (sdp4bit_quan.cu:63-109)
        return 4 if (dtype == torch.float32 and not self.asym) else 8

    def to_c(self, dtype: torch.dtype) -> _lib.Codec:
        if self.kind == "mxfp8":
            return _lib.Codec(KIND_MXFP8, 8, 32, 0, 0, 0, 1, self.seed & 0xFFFFFFFF)
        if self.kind == "taco":
            fmax = self.fp8_max if self.fp8_max > 0 else (57344.0 if self.e5m2 else 448.0)
            return _lib.Codec(KIND_TACO, 8, self.group, 0, 0, 0, 8, 0, int(self.e5m2) | (int(self.saturate) << 1),
                              self.target_range, self.lam, fmax)
        if self.kind == "zfp":
            return _lib.Codec(KIND_ZFP, self.bits, 4, 0, 0, 0, 0, 0)
        return _lib.Codec(KIND_SDP4BIT, self.bits, self.group, int(self.asym), int(self.hadamard),
                          int(self.stochastic), self.param_bytes(dtype), self.seed & 0xFFFFFFFF)

    def encoded_chunk_bytes(self, count: int, dtype: torch.dtype) -> int:
        g = {"mxfp8": 32, "zfp": 4}.get(self.kind, self.group)
        bits = 8 if self.kind in ("mxfp8", "taco") else self.bits
        groups = -(-count // g)
        total = groups * g * bits // 8 + groups * self.param_bytes(dtype)
        return -(-total // 4) * 4


SDP4BIT_G128 = CodecConfig("sdp4bit", 4, 128, False, True)
SDP4BIT_G128_SR = CodecConfig("sdp4bit", 4, 128, False, True, True)   # stochastic rounding, the reference's only mode
MXFP8 = CodecConfig("mxfp8", 8, 32, False, False)
TACO_G128 = CodecConfig("taco", 8, 128, False, False)
ZFP_RATE8 = CodecConfig("zfp", 8, 4, False, False)


def encode(x: torch.Tensor, cfg: CodecConfig, chunks: int = 1) -> torch.Tensor:
    """Encode `chunks` equal chunks of a contiguous tensor; returns uint8 [chunks, chunk_bytes]."""
    assert x.is_cuda and x.is_contiguous() and x.numel() % chunks == 0
    count = x.numel() // chunks
    nbytes = cfg.encoded_chunk_bytes(count, x.dtype)
    out = torch.empty((chunks, nbytes), dtype=torch.uint8, device=x.device)
    c = cfg.to_c(x.dtype)
    rc = _lib.lib().cocclkEncode(x.data_ptr(), out.data_ptr(), count, chunks, count, nbytes, DTYPE_CODE[x.dtype],
                                 c, _lib.cur_stream())
    _lib.check(rc, "cocclkEncode")
    return out


def decode_reduce(enc: torch.Tensor, cfg: CodecConfig, count: int, dtype: torch.dtype, chunks: int = 1,
                  reduce: int = 1) -> torch.Tensor:
    """out[j] = sum_i decode(enc[i*chunks + j]) for j < chunks; enc is uint8 [reduce*chunks, chunk_bytes]."""
    assert enc.is_cuda and enc.is_contiguous() and enc.shape[0] == chunks * reduce
    out = torch.empty((chunks, count), dtype=dtype, device=enc.device)
    c = cfg.to_c(dtype)
    rc = _lib.lib().cocclkDecodeReduce(enc.data_ptr(), out.data_ptr(), count, chunks, reduce, count, enc.shape[1],
                                       DTYPE_CODE[dtype], c, _lib.cur_stream())
    _lib.check(rc, "cocclkDecodeReduce")
    return out


def decode(enc, cfg, count, dtype, chunks=1):
    return decode_reduce(enc, cfg, count, dtype, chunks, 1)


def decode_reduce_encode(enc: torch.Tensor, cfg: CodecConfig, count: int, dtype: torch.dtype, chunks: int = 1,
                         reduce: int = 1) -> torch.Tensor:
    """Fused decode + sum + re-encode; `dtype` only selects the parameter layout."""
    out = torch.empty((chunks, enc.shape[1]), dtype=torch.uint8, device=enc.device)
    c = cfg.to_c(dtype)
    rc = _lib.lib().cocclkDecodeReduceEncode(enc.data_ptr(), out.data_ptr(), count, chunks, reduce, enc.shape[1],
                                             out.shape[1], c, _lib.cur_stream())
    _lib.check(rc, "cocclkDecodeReduceEncode")
    return out


# --------------------------------------------------------------------------- PyTorch fp32 oracle
def _hadamard32(x: torch.Tensor) -> torch.Tensor:
    """Unnormalised Sylvester-ordered WHT over the last dimension (size 32)."""
    n = x.shape[-1]
    h = 1
    y = x
    while h < n:
        y = y.reshape(*y.shape[:-1], n // (2 * h), 2, h)
        a, b = y[..., 0, :], y[..., 1, :]
        y = torch.stack((a + b, a - b), dim=-2).reshape(*x.shape[:-1], n)
        h *= 2
    return y


def _hash32(x: torch.Tensor) -> torch.Tensor:
    m = 0xFFFFFFFF
    x = x & m
    x = x ^ (x >> 16)
    x = (x * 0x7FEB352D) & m
    x = x ^ (x >> 15)
    x = (x * 0x846CA68B) & m
    x = x ^ (x >> 16)
    return x


def _rng_unit(seed: int, elem: torch.Tensor) -> torch.Tensor:
    """Same stream as the kernels: one hash per 4 elements, 8 bits per element."""
    quad = elem >> 2
    lo, hi = quad & 0xFFFFFFFF, quad >> 32
    inner = _hash32((seed + 0x9E3779B9 * (hi + 1)) & 0xFFFFFFFF)
    word = _hash32(lo ^ inner)
    byte = (word >> (8 * (elem & 3))) & 0xFF
    return (byte.to(torch.float32) + 0.5) / 256.0


def _zfp_oracle_roundtrip(xf: torch.Tensor, rate: int) -> torch.Tensor:
    """ZFP fixed-rate round trip of every row of xf through the CPU coder of csrc/oracle (bit-serial: no PyTorch
    restatement exists that would be more than a transliteration of it)."""
    import ctypes as C
    cb = _lib.declare("cocclOracleZfpChunkBytes", C.c_long, [C.c_long, C.c_int])
    en = _lib.declare("cocclOracleZfpEncode", C.c_int, [C.c_void_p, C.c_long, C.c_int, C.c_void_p])
    de = _lib.declare("cocclOracleZfpDecode", C.c_int, [C.c_void_p, C.c_long, C.c_int, C.c_void_p])
    xc = xf.detach().cpu().contiguous()
    out = torch.empty_like(xc)
    count = xc.shape[1]
    buf = torch.zeros(cb(count, rate), dtype=torch.uint8)
    for ch in range(xc.shape[0]):
        assert en(xc[ch].data_ptr(), count, rate, buf.data_ptr()) == 0
        assert de(buf.data_ptr(), count, rate, out[ch].data_ptr()) == 0
    return out


def reference_roundtrip(x: torch.Tensor, cfg: CodecConfig, chunks: int = 1, rng_base: int = 0) -> torch.Tensor:
    """encode->decode of every chunk in fp32 PyTorch (CPU or GPU); returns fp32 of x's shape."""
    count = x.numel() // chunks
    xf = x.detach().reshape(chunks, count).to(torch.float32)
    if cfg.kind == "zfp":
        return _zfp_oracle_roundtrip(xf, cfg.bits).reshape(x.shape).to(x.device)
    g = 32 if cfg.kind == "mxfp8" else cfg.group
    pad = (-count) % g
    if pad:
        xf = torch.cat([xf, xf.new_zeros(chunks, pad)], dim=1)
    n = xf.shape[1]
    if cfg.kind == "mxfp8":
        blk = xf.reshape(chunks, n // 32, 32)
        amax = blk.abs().amax(dim=-1, keepdim=True)
        r = amax / 448.0
        e = torch.ceil(torch.log2(torch.where(r > 0, r, torch.ones_like(r))))
        # exact power-of-two handling the way the kernel does it (exponent field, +1 if mantissa != 0)
        bits = r.view(torch.int32)
        ex = (bits >> 23) & 0xFF
        ex = ex + ((bits & 0x7FFFFF) != 0).to(torch.int32)
        ex = torch.where(amax > 0, ex.clamp(0, 254), torch.zeros_like(ex))
        scale = torch.pow(2.0, (ex - 127).to(torch.float32))
        del e
        q = (blk / scale).to(torch.float8_e4m3fn).to(torch.float32)
        out = (q * scale).reshape(chunks, n)
        return out[:, :count].reshape(x.shape)
    if cfg.kind == "taco":
        # taco/taco.cu:118-218: adaptive scale, Hadamard over the whole group, FP8 with a group scale
        grp = xf.reshape(chunks, n // g, g)
        h = torch.ones(1, 1, device=x.device)
        while h.shape[0] < g:
            h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
        fmax = cfg.fp8_max if cfg.fp8_max > 0 else (57344.0 if cfg.e5m2 else 448.0)
        ada = (fmax * torch.rsqrt((grp * grp).mean(-1, keepdim=True) + cfg.lam)).clamp(1e-3, 1e3)
        y = (grp * ada) @ h / g ** 0.5
        qs = (y.abs().amax(-1, keepdim=True) / cfg.target_range).clamp(1e-12, 1e6)
        code = (y / qs).clamp(-448, 448).to(torch.float8_e5m2 if cfg.e5m2 else torch.float8_e4m3fn).float()
        out = ((code * qs) @ h / g ** 0.5 / ada).reshape(chunks, n)
        return out[:, :count].reshape(x.shape)
    v = xf
    if cfg.hadamard:
        v = _hadamard32(v.reshape(chunks, n // 32, 32)).reshape(chunks, n)
    grp = v.reshape(chunks, n // g, g)
    qlo, qhi = -(1 << (cfg.bits - 1)), (1 << (cfg.bits - 1)) - 1
    if not cfg.asym:
        amax = grp.abs().amax(dim=-1, keepdim=True)
        scale = torch.where(amax == 0, torch.ones_like(amax), float(qhi) / amax)
        off = torch.zeros_like(amax)
    else:
        mx, mn = grp.amax(dim=-1, keepdim=True), grp.amin(dim=-1, keepdim=True)
        rng = mx - mn
        scale = torch.where(rng == 0, torch.ones_like(rng), float(1 << cfg.bits) / rng)
        off = 0.5 * (mx + mn)
    y = (grp - off) * scale
    if cfg.stochastic:
        elem = torch.arange(n, device=x.device, dtype=torch.int64).reshape(1, n) + rng_base
        ch = torch.arange(chunks, device=x.device, dtype=torch.int64).reshape(chunks, 1) << 40
        u = _rng_unit(cfg.seed, elem + ch).reshape(chunks, n // g, g)
        q = torch.floor(y + u)
    else:
        q = torch.round(y)  # half-to-even, like cvt.rni
    q = q.clamp(qlo, qhi)
    inv = 1.0 / scale
    dq = (q * inv + off).reshape(chunks, n)
    if cfg.hadamard:
        dq = _hadamard32(dq.reshape(chunks, n // 32, 32)).reshape(chunks, n) * (1.0 / 32.0)
    return dq[:, :count].reshape(x.shape)
