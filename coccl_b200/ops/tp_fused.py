"""Tensor-parallel fusions (csrc/kernels/tp_kernels.cu): all-gather -> GEMM and GEMM -> FP8 reduce-scatter.

The emulate_* helpers play every rank on ONE GPU in a single cooperative launch (the ranks wait on one
another, so they must never be separate launches); they exist for single-GPU tests and benchmarks. The
multi-GPU entry points live on `parallel.comm.Communicator` (`ag_gemm`, `gemm_rs`).
"""
from __future__ import annotations

import torch

from .. import _lib
from .gemm import EPI_BIAS, EPI_BIAS_GELU, EPI_NONE

STATUS_BYTES = 256


def set_variant(name: str) -> None:
    """'auto' (CTA-pair kernels where rows per rank are a multiple of 256), '1cta' or '2cta' (pair kernels or an error)."""
    import ctypes as C
    _lib.declare("cocclkTpSetVariant", None, [C.c_int])({"auto": 0, "1cta": 1, "2cta": 2}[name])


def last_variant() -> str:
    """Which kernel family served the last fusion call of this process."""
    import ctypes as C
    return {0: "none", 1: "1cta", 2: "2cta"}[_lib.declare("cocclkTpLastVariant", C.c_int, [])()]


PAYLOAD_BF16, PAYLOAD_FP8 = 0, 1


def ag_ws_bytes(M: int, K: int, payload: int = PAYLOAD_BF16) -> int:
    """Workspace per rank of the all-gather fusion: the bf16 gather buffer, plus the FP8 rows and their scales when the
    shards travel as block-scaled FP8."""
    import ctypes as C
    return int(_lib.declare("cocclkAgGemmWorkspaceBytesFor", C.c_long, [C.c_int, C.c_int, C.c_int])(M, K, payload))


def rs_ws_bytes(M: int, N: int, n: int) -> int:
    return _lib.lib().cocclkGemmRsWorkspaceBytes(M, N, n)


def _state(state: dict, n: int, dev, ws_bytes: int):
    if state.get("ws_bytes", 0) < ws_bytes or state.get("n") != n:
        state["ws"] = [torch.empty(ws_bytes, dtype=torch.uint8, device=dev) for _ in range(n)]
        state["ws_bytes"], state["n"] = ws_bytes, n
    if "flags" not in state:
        state["flags"] = [torch.zeros(_lib.lib().cocclkFlagBytes() // 4, dtype=torch.int32, device=dev) for _ in range(n)]
        state["status"] = [torch.zeros(STATUS_BYTES // 4, dtype=torch.int32, device=dev) for _ in range(n)]
        state["err"] = [torch.zeros(1, dtype=torch.int32, device=dev) for _ in range(n)]
    return state


def _fill(a: _lib.TpArgs, state, n):
    for r in range(n):
        a.ws[r] = state["ws"][r].data_ptr()
        a.flags[r] = state["flags"][r].data_ptr()
        a.status[r] = state["status"][r].data_ptr()
        a.err[r] = state["err"][r].data_ptr()


def check_state(state) -> None:
    """Raise if any emulated rank recorded a wait that ran out (host sync)."""
    for r in range(state["n"]):
        code, err = int(state["status"][r][0].item()), int(state["err"][r].item())
        if code or err:
            raise RuntimeError(f"rank {r}: status {code & 0xFFFFFFFF:#x} pipeline error {err & 0xFFFFFFFF:#x}")


def emulate_ag_gemm(x_shards, w_shards, *, bias=None, gelu=False, state=None, epoch=1, max_ctas=0,
                    timeout_ms=5000.0, b_mn=False, payload=PAYLOAD_BF16, gathered=None):
    """C_r = concat(x_shards) @ w_shards[r].T (+ bias_r, GELU) for every emulated rank r (w [K, N] with b_mn).
    payload=PAYLOAD_FP8: the shards cross between the ranks as E4M3 + UE8M0 scales (CTA-pair kernel only).
    gathered: optional list of [M, K] tensors that receive each rank's gathered operand."""
    n = len(x_shards)
    m, K = x_shards[0].shape
    N = w_shards[0].shape[1] if b_mn else w_shards[0].shape[0]
    dev = x_shards[0].device
    state = _state(state if state is not None else {}, n, dev, ag_ws_bytes(m * n, K, payload))
    outs = [torch.empty(m * n, N, dtype=torch.bfloat16, device=dev) for _ in range(n)]
    a = _lib.TpArgs()
    a.nRanks, a.rankBase, a.M, a.N, a.K = n, 0, m * n, N, K
    a.epi = EPI_NONE if bias is None else (EPI_BIAS_GELU if gelu else EPI_BIAS)
    a.bMN = int(b_mn)
    a.epoch, a.timeoutNs = epoch, int(timeout_ms * 1e6)
    _fill(a, state, n)
    for r in range(n):
        assert x_shards[r].is_contiguous() and w_shards[r].is_contiguous()
        a.a[r], a.b[r], a.c[r] = x_shards[r].data_ptr(), w_shards[r].data_ptr(), outs[r].data_ptr()
        a.bias[r] = bias[r].data_ptr() if bias is not None else None
        if gathered is not None:
            a.gathered[r] = gathered[r].data_ptr()
    a.agPayload = payload
    _lib.check(_lib.lib().cocclkAgGemm(a, n, max_ctas, _lib.cur_stream()), "cocclkAgGemm")
    return outs, state


def emulate_gemm_rs(a_list, w_list, *, state=None, epoch=1, max_ctas=0, timeout_ms=5000.0, b_mn=False):
    """out_r = rows r of sum_q (a_list[q] @ w_list[q].T), the partial products sent as block-scaled FP8."""
    n = len(a_list)
    M, K = a_list[0].shape
    N = w_list[0].shape[1] if b_mn else w_list[0].shape[0]
    dev = a_list[0].device
    state = _state(state if state is not None else {}, n, dev, rs_ws_bytes(M, N, n))
    outs = [torch.empty(M // n, N, dtype=torch.bfloat16, device=dev) for _ in range(n)]
    a = _lib.TpArgs()
    a.nRanks, a.rankBase, a.M, a.N, a.K = n, 0, M, N, K
    a.epi, a.epoch, a.timeoutNs = EPI_NONE, epoch, int(timeout_ms * 1e6)
    a.bMN = int(b_mn)
    _fill(a, state, n)
    for r in range(n):
        assert a_list[r].is_contiguous() and w_list[r].is_contiguous()
        a.a[r], a.b[r], a.c[r] = a_list[r].data_ptr(), w_list[r].data_ptr(), outs[r].data_ptr()
    _lib.check(_lib.lib().cocclkGemmRs(a, n, max_ctas, _lib.cur_stream()), "cocclkGemmRs")
    return outs, state
