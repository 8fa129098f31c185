"""Front end of the fused compressed collectives (csrc/kernels/collective_kernels.cuh).

Two ways to run them:
  * `emulate_collective`: every rank's buffers live on ONE GPU and a single
    cooperative launch plays all ranks (numerics tests, 1-GPU profiling);
  * `coccl_b200.parallel.comm.Communicator`: one process per GPU, peer-mapped
    symmetric workspaces, one launch per rank.
"""
from __future__ import annotations

import torch

from .. import _lib
from .codec import CodecConfig, DTYPE_CODE

OP_RS, OP_AG, OP_A2A, OP_AR1, OP_AR2, OP_AGD = 0, 1, 2, 3, 4, 5
OP_NAMES = {"reduce_scatter": OP_RS, "all_gather": OP_AG, "all_to_all": OP_A2A, "all_reduce_oneshot": OP_AR1,
            "all_reduce_twoshot": OP_AR2, "all_gather_delta": OP_AGD}


def as_c(cfg, dtype) -> _lib.Codec:
    """A CodecConfig (Python description) or an already filled cocclkCodec (from the router) as the C struct."""
    return cfg if isinstance(cfg, _lib.Codec) else cfg.to_c(dtype)


def slot_bytes(cfg, count: int, dtype) -> int:
    return _lib.lib().cocclkSlotBytes(as_c(cfg, dtype), count)


def tile_elems() -> int:
    return _lib.lib().cocclkTileElems()


def pick_slice_tiles(count: int, n_ranks: int, target_items: int = 148 * 3) -> int:
    """Tiles per slice: enough items to fill the GPU, at most 4096 slices, at most 16 tiles per slice."""
    tiles = -(-count // tile_elems())
    st = max(1, min(16, tiles * n_ranks // max(1, target_items)))
    while -(-tiles // st) > _lib.MAX_SLICES:
        st *= 2
    return st


def chunk_count(op: int, numel_in: int, n: int) -> int:
    """Elements per chunk given the per-rank INPUT size of the collective."""
    if op in (OP_RS, OP_A2A, OP_AR2):
        assert numel_in % n == 0
        return numel_in // n
    return numel_in  # all-gather shard, one-shot all-reduce vector


def workspace_bytes(op: int, cfg, count: int, dtype, n: int) -> tuple[int, int, int]:
    """(slot_bytes, region_b_offset, total) of one parity half of the workspace."""
    sb = slot_bytes(cfg, count, dtype)
    region = -(-sb * n // 256) * 256
    total = region * (2 if op == OP_AR2 else 1)
    return sb, region, total


def emulate_collective(op: str, inputs: list[torch.Tensor], cfg: CodecConfig, *, slice_tiles: int | None = None,
                       timeout_ms: float = 2000.0, max_ctas: int = 0, epoch: int = 1,
                       state: dict | None = None, slot_bytes: int | None = None) -> list[torch.Tensor]:
    """Run one fused collective for all ranks on the current GPU; inputs[r] is rank r's send buffer.
    slot_bytes: tests only: hand the kernel another slot size than the layout needs (a too small one must be refused by
    the kernel's entry check, which reports through the status words and touches nothing)."""
    opc = OP_NAMES[op]
    n = len(inputs)
    x0 = inputs[0]
    dtype, dev = x0.dtype, x0.device
    numel = x0.numel()
    count = chunk_count(opc, numel, n)
    out_numel = {OP_RS: count, OP_AG: count * n, OP_A2A: numel, OP_AR1: numel, OP_AR2: numel, OP_AGD: count * n}[opc]
    if opc == OP_AGD:
        # delta all-gather: the outputs of the previous call are the state the deltas are added to
        assert state is not None and "outs" in state, "all_gather_delta needs state['outs'] from an exact first gather"
        outs = state["outs"]
    else:
        outs = [torch.empty(out_numel, dtype=dtype, device=dev) for _ in range(n)]
    sb, region_b, total = workspace_bytes(opc, cfg, count, dtype, n)
    if state is None:
        state = {}
    if "flags" not in state:
        state["flags"] = [torch.zeros(_lib.lib().cocclkFlagBytes() // 4, dtype=torch.int32, device=dev) for _ in range(n)]
        state["status"] = [torch.zeros(4, dtype=torch.int32, device=dev) for _ in range(n)]
    if state.get("ws_bytes", 0) < total:
        state["ws"] = [torch.empty(total, dtype=torch.uint8, device=dev) for _ in range(n)]
        state["ws_bytes"] = total
    a = _lib.CollArgs()
    a.op, a.nRanks, a.rankBase, a.dtype, a.count = opc, n, 0, DTYPE_CODE[dtype], count
    a.sliceTiles = slice_tiles or pick_slice_tiles(count, n)
    a.epoch = epoch
    a.timeoutNs = int(timeout_ms * 1e6)
    a.codec = cfg.to_c(dtype)
    a.slotBytes, a.regionBOffset = (sb if slot_bytes is None else slot_bytes), region_b
    for r in range(n):
        assert inputs[r].is_contiguous() and inputs[r].numel() == numel
        a.inp[r], a.out[r] = inputs[r].data_ptr(), outs[r].data_ptr()
        a.ws[r], a.flags[r], a.status[r] = state["ws"][r].data_ptr(), state["flags"][r].data_ptr(), state["status"][r].data_ptr()
        if state.get("trace") is not None:  # list of int64 [TRACE_MAX_CTAS, 4] tensors, one per rank
            a.trace[r] = state["trace"][r].data_ptr()
    rc = _lib.lib().cocclkFusedCollective(a, n, max_ctas, _lib.cur_stream())
    _lib.check(rc, f"cocclkFusedCollective({op})")
    return outs


def status_codes(state: dict) -> list[int]:
    return [int(s[0].item()) & 0xFFFFFFFF for s in state["status"]]
