"""Byte exchange over peer memory (csrc/kernels/exchange_kernels.cu): the transport of the staged pipeline on one
NVSwitch domain. `emulate` plays every rank on ONE GPU in a single cooperative launch (the ranks wait on one another, so
they must never be separate launches); the multi-GPU user is the C++ staged executor (csrc/runtime/peer_exchange.cc)."""
from __future__ import annotations

import ctypes as C

import torch

from .. import _lib


def pieces_for(frames: int, frame_stride: int) -> tuple[int, int]:
    pb = C.c_long(0)
    n = _lib.declare("cocclkExchangePieces", C.c_int, [C.c_int, C.c_long, C.POINTER(C.c_long)])(frames, frame_stride, C.byref(pb))
    if n < 1:
        raise ValueError(f"no piece layout for {frames} frames of {frame_stride} bytes")
    return int(n), int(pb.value)


def staging_bytes(n_ranks: int, frames: int, frame_stride: int) -> int:
    return int(_lib.declare("cocclkExchangeStagingBytes", C.c_long, [C.c_int, C.c_int, C.c_long])(n_ranks, frames, frame_stride))


def emulate(send: list[torch.Tensor], *, gather: bool, frames: int, frame_stride: int, meta: list[torch.Tensor] | None = None,
            state: dict | None = None, epoch: int = 1, max_ctas: int = 0, timeout_ms: float = 5000.0):
    """send[r]: uint8 tensor of rank r: nRanks blocks (all-to-all) or one block (all-gather) of frames * frame_stride
    bytes. meta[r]: int64 [blocks * frames, 2] = (payload bytes, encoding) per frame, or None for full frames.
    Returns (recv list [nRanks blocks each, by source], recv_meta list or None, state)."""
    n = len(send)
    dev = send[0].device
    pieces, piece_bytes = pieces_for(frames, frame_stride)
    block = frames * frame_stride
    state = state if state is not None else {}
    need = staging_bytes(n, frames, frame_stride)
    if state.get("bytes", 0) < need or state.get("n") != n:
        state["staging"] = [torch.empty(need, dtype=torch.uint8, device=dev) for _ in range(n)]
        state["bytes"], state["n"] = need, n
    if "flags" not in state:
        state["flags"] = [torch.zeros(_lib.lib().cocclkFlagBytes() // 4, dtype=torch.int32, device=dev) for _ in range(n)]
        state["status"] = [torch.zeros(64, dtype=torch.int32, device=dev) for _ in range(n)]
    recv = [torch.zeros(n * block, dtype=torch.uint8, device=dev) for _ in range(n)]
    recv_meta = [torch.zeros(n * frames, 2, dtype=torch.int64, device=dev) for _ in range(n)] if meta is not None else None
    a = _lib.ExchangeArgs()
    a.nRanks, a.rankBase, a.gather, a.frames, a.pieces = n, 0, int(gather), frames, pieces
    a.frameStride, a.pieceBytes, a.epoch, a.timeoutNs = frame_stride, piece_bytes, epoch, int(timeout_ms * 1e6)
    for r in range(n):
        assert send[r].dtype == torch.uint8 and send[r].is_contiguous() and send[r].numel() == (1 if gather else n) * block
        a.send[r], a.recv[r] = send[r].data_ptr(), recv[r].data_ptr()
        a.staging[r], a.flags[r], a.status[r] = state["staging"][r].data_ptr(), state["flags"][r].data_ptr(), state["status"][r].data_ptr()
        if meta is not None:
            assert meta[r].dtype == torch.int64 and meta[r].is_contiguous()
            a.sendMeta[r], a.recvMeta[r] = meta[r].data_ptr(), recv_meta[r].data_ptr()
    fn = _lib.declare("cocclkPeerExchange", C.c_int, [C.POINTER(_lib.ExchangeArgs), C.c_int, C.c_int, C.c_void_p])
    _lib.check(fn(C.byref(a), n, max_ctas, _lib.cur_stream()), "cocclkPeerExchange")
    return recv, recv_meta, state


def check_state(state) -> None:
    for r in range(state["n"]):
        code = int(state["status"][r][0].item())
        if code:
            raise RuntimeError(f"rank {r}: exchange status {code & 0xFFFFFFFF:#x}")
