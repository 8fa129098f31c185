"""Tracing: NVTX ranges around every communicator call and a device-side phase trace of the fused collectives.

The reference wraps its NCCL entry points in NVTX ranges (src/collectives.cc:31-36, src/include/nvtx.h:19-32)
and has no per-phase view of a compressed collective. Here `COCCL_NVTX=1` (or `enable_nvtx()`) adds a range per
call, and `Communicator.enable_trace()` makes the fused kernels record `globaltimer` values per CTA at the
phase boundaries (kernel start, encode+push done, decode-reduce done, gather done), read back by
`Communicator.phase_times()`.
"""
from __future__ import annotations

import contextlib
import os

import torch

_nvtx = os.environ.get("COCCL_NVTX", "0") not in ("", "0")


def enable_nvtx(on: bool = True) -> None:
    global _nvtx
    _nvtx = on


@contextlib.contextmanager
def nvtx_range(name: str):
    if _nvtx and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


TRACE_MAX_CTAS = 2048


def summarise(trace: torch.Tensor) -> dict:
    """trace: int64 [TRACE_MAX_CTAS, 4] as written by one launch (zero rows = CTAs that did not run).
    Returns phase durations in microseconds over the whole grid (first start to last finish of each phase)."""
    t = trace.cpu()
    rows = t[t[:, 0] != 0]
    if rows.numel() == 0:
        return {}
    start = rows[:, 0].min().item()
    ends = [rows[:, i].max().item() for i in range(1, 4)]
    names = ["encode_push_us", "decode_reduce_us", "gather_us"]
    out, prev = {"ctas": int(rows.shape[0])}, start
    for n, e in zip(names, ends):
        out[n] = max(0, e - prev) / 1e3
        prev = max(prev, e)
    out["total_us"] = (prev - start) / 1e3
    return out
