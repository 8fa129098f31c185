"""tcgen05 GEMM front end (csrc/kernels/gemm_kernels.cu).

`gemm(a, b, ...)` computes a @ b.T-style products without materialising
transposes: each operand is described by (tensor, contraction-major?) so the
same kernel serves forward (x @ W^T), dgrad (dy @ W) and wgrad (dy^T @ x).
"""
from __future__ import annotations

import torch

from .. import _lib

EPI_NONE, EPI_BIAS, EPI_BIAS_GELU, EPI_F32_ACC, EPI_F32 = 0, 1, 2, 3, 4

_err_words: dict[int, torch.Tensor] = {}


def _err_word(device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _err_words:
        _err_words[idx] = torch.zeros(1, dtype=torch.int32, device=device)
    return _err_words[idx]


def check_errors(device=None) -> None:
    """Raise if any GEMM launched so far gave up on a bounded wait (host sync)."""
    for idx, w in _err_words.items():
        v = int(w.item())
        if v != 0:
            w.zero_()
            raise RuntimeError(f"tcgen05 GEMM on cuda:{idx} reported error word {v & 0xFFFFFFFF:#x}")


def tensor_map_cache_stats() -> tuple[int, int]:
    """(hits, misses) of the table that returns the TMA descriptor of a repeated (address, shape, pitch) request
    without a driver call."""
    import ctypes as C
    fn = _lib.declare("cocclkTensorMapCacheStats", None, [C.POINTER(C.c_ulonglong), C.POINTER(C.c_ulonglong)])
    h, m = C.c_ulonglong(0), C.c_ulonglong(0)
    fn(C.byref(h), C.byref(m))
    return int(h.value), int(m.value)


def set_variant(name: str) -> None:
    """Pick the kernel: "auto" (by shape), "1cta" (128x256 tiles, one SM per tile) or "2cta"
    (256x256 tiles on a CTA pair with tcgen05.mma.cta_group::2)."""
    _lib.lib().cocclkGemmSetVariant({"auto": 0, "1cta": 1, "2cta": 2}[name])


def get_variant() -> str:
    return ("auto", "1cta", "2cta")[_lib.lib().cocclkGemmGetVariant()]


def _operand(t: torch.Tensor, rows: int, k: int):
    """Return (ptr tensor, ld, mn_major) for a 2-D bf16 operand of logical shape [rows, k]."""
    assert t.dtype == torch.bfloat16 and t.dim() == 2 and t.shape == (rows, k), (t.shape, rows, k)
    if t.stride(1) == 1:
        return t, t.stride(0), 0
    if t.stride(0) == 1:  # stored [k, rows]
        return t, t.stride(1), 1
    t = t.contiguous()
    return t, t.stride(0), 0


def gemm(a: torch.Tensor, b: torch.Tensor, *, bias: torch.Tensor | None = None, gelu: bool = False,
         save_preact: bool = False, out: torch.Tensor | None = None, accumulate: bool = False,
         out_dtype: torch.dtype = torch.bfloat16, max_ctas: int = 0):
    """C[M,N] = A[M,K] @ B[N,K]^T with fp32 accumulation in TMEM.

    a: [M,K] (any of the two unit-stride layouts), b: [N,K] likewise (pass W for x@W^T,
    W.t() for dy@W, ...). bias: [N] bf16 added in the epilogue; gelu: apply tanh-GELU;
    save_preact: also return the pre-activation. out fp32 + accumulate adds into `out`.
    """
    M, K = a.shape
    N, K2 = b.shape
    assert K == K2
    a_t, lda, a_mn = _operand(a, M, K)
    b_t, ldb, b_mn = _operand(b, N, K)
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    assert out.shape == (M, N) and out.stride(1) == 1
    z = None
    if out.dtype == torch.float32:
        epi = EPI_F32_ACC if accumulate else EPI_F32
        assert bias is None and not gelu
    else:
        assert out.dtype == torch.bfloat16 and not accumulate
        epi = EPI_BIAS_GELU if gelu else (EPI_BIAS if bias is not None else EPI_NONE)
        if gelu and bias is None:
            bias = torch.zeros(N, dtype=torch.bfloat16, device=a.device)
        if gelu and save_preact:
            z = torch.empty_like(out)
    err = _err_word(a.device)
    rc = _lib.lib().cocclkGemmBf16(a_t.data_ptr(), lda, a_mn, b_t.data_ptr(), ldb, b_mn, out.data_ptr(), out.stride(0),
                                   M, N, K, epi, _lib.ptr(bias), _lib.ptr(z), err.data_ptr(), max_ctas,
                                   _lib.cur_stream())
    _lib.check(rc, "cocclkGemmBf16")
    return (out, z) if save_preact else out
