"""Expert-parallel token exchange (csrc/kernels/moe_kernels.cu).

`route_layout` ranks every (token, choice) inside its expert's queue; `emulate_dispatch` / `emulate_combine`
play all ranks on one GPU in a single cooperative launch (for tests and single-GPU benchmarks). The multi-GPU
entry points are `parallel.comm.Communicator.moe_dispatch` / `moe_combine`.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import _lib

STATUS_BYTES = 256


def route_layout(expert_ids: torch.Tensor, n_experts: int, n_ranks: int):
    """expert_ids [tokens, topk] int32 -> (pos [tokens, topk] int32, counts [n_experts] int32).
    pos = position of the entry inside the block this rank sends to the expert's rank (grouped by expert,
    token order inside an expert)."""
    ids = expert_ids.contiguous()
    assert ids.dtype == torch.int32 and n_experts % n_ranks == 0
    if not ids.is_cuda:
        return _route_layout_host(ids, n_experts, n_ranks)
    pos = torch.empty_like(ids)
    counts = torch.empty(n_experts, dtype=torch.int32, device=ids.device)
    _lib.check(_lib.lib().cocclkMoeLayout(ids.data_ptr(), ids.numel(), n_experts, n_experts // n_ranks, pos.data_ptr(),
                                          counts.data_ptr(), _lib.cur_stream()), "cocclkMoeLayout")
    return pos, counts


def _route_layout_host(ids: torch.Tensor, n_experts: int, n_ranks: int):
    """PyTorch restatement of the layout kernel for CPU tensors (the gloo tests)."""
    flat = ids.reshape(-1).long()
    counts = torch.bincount(flat, minlength=n_experts)
    order = torch.sort(flat, stable=True).indices            # by expert, then (token, choice)
    start = torch.cumsum(counts, 0) - counts
    within = torch.empty_like(flat)
    within[order] = torch.arange(flat.numel()) - start[flat[order]]
    per_rank = counts.view(n_ranks, n_experts // n_ranks)
    block_off = (torch.cumsum(per_rank, 1) - per_rank).reshape(-1)   # where an expert's queue starts inside its rank's block
    pos = (block_off[flat] + within).to(torch.int32).view_as(ids)
    return pos, counts.to(torch.int32)


def ws_bytes(n_ranks: int, capacity: int, hidden: int, local_experts: int) -> int:
    return _lib.lib().cocclkMoeWorkspaceBytes(n_ranks, capacity, hidden, local_experts)


@dataclass
class Handle:
    """What dispatch leaves for combine (per rank)."""
    expert_ids: torch.Tensor
    pos: torch.Tensor
    recv_counts: torch.Tensor    # [n_ranks, local_experts]
    recv_offsets: torch.Tensor   # [local_experts + 1]
    capacity: int
    n_experts: int


def _state(state, n, dev, nbytes):
    if state.get("ws_bytes", 0) < nbytes or state.get("n") != n:
        state["ws"] = [torch.empty(nbytes, dtype=torch.uint8, device=dev) for _ in range(n)]
        state["ws_bytes"], state["n"] = nbytes, n
    if "flags" not in state:
        state["flags"] = [torch.zeros(_lib.lib().cocclkFlagBytes() // 4, dtype=torch.int32, device=dev) for _ in range(n)]
        state["status"] = [torch.zeros(STATUS_BYTES // 4, dtype=torch.int32, device=dev) for _ in range(n)]
        state["epoch"] = 0
    return state


def check_state(state):
    for r in range(state["n"]):
        code = int(state["status"][r][0].item())
        if code:
            raise RuntimeError(f"rank {r}: status {code & 0xFFFFFFFF:#x}")


def _base_args(n, tokens, hidden, topk, n_experts, capacity, state, timeout_ms):
    a = _lib.MoeArgs()
    a.nRanks, a.rankBase, a.tokens, a.hidden, a.topk, a.experts, a.capacity = n, 0, tokens, hidden, topk, n_experts, capacity
    state["epoch"] += 1
    a.epoch, a.timeoutNs = state["epoch"], int(timeout_ms * 1e6)
    for r in range(n):
        a.ws[r], a.flags[r], a.status[r] = state["ws"][r].data_ptr(), state["flags"][r].data_ptr(), state["status"][r].data_ptr()
    return a


def emulate_dispatch(xs, ids, n_experts, *, capacity=None, state=None, max_ctas=0, timeout_ms=5000.0):
    """xs[r] [tokens, hidden] bf16, ids[r] [tokens, topk] int32 -> (recv[r] rows expert-major, handles[r], state)."""
    n = len(xs)
    tokens, hidden = xs[0].shape
    topk = ids[0].shape[1]
    dev = xs[0].device
    le = n_experts // n
    capacity = capacity or tokens * topk
    state = _state(state if state is not None else {}, n, dev, ws_bytes(n, capacity, hidden, le))
    a = _base_args(n, tokens, hidden, topk, n_experts, capacity, state, timeout_ms)
    keep, handles, recvs = [], [], []
    for r in range(n):
        pos, counts = route_layout(ids[r], n_experts, n)
        recv = torch.empty(n * capacity, hidden, dtype=torch.bfloat16, device=dev)
        roff = torch.zeros(le + 1, dtype=torch.int32, device=dev)
        rcnt = torch.zeros(n, le, dtype=torch.int32, device=dev)
        a.x[r], a.expertIds[r], a.pos[r], a.sendCounts[r] = xs[r].data_ptr(), ids[r].data_ptr(), pos.data_ptr(), counts.data_ptr()
        a.recv[r], a.recvOffsets[r], a.recvCounts[r] = recv.data_ptr(), roff.data_ptr(), rcnt.data_ptr()
        keep.append((pos, counts))
        recvs.append(recv)
        handles.append(Handle(ids[r], pos, rcnt, roff, capacity, n_experts))
    _lib.check(_lib.lib().cocclkMoeDispatch(a, n, max_ctas, _lib.cur_stream()), "cocclkMoeDispatch")
    return recvs, handles, state


def emulate_combine(ys, gates, handles, *, state, max_ctas=0, timeout_ms=5000.0):
    """ys[r]: expert outputs in recv layout; gates[r] [tokens, topk] fp32 -> out[r] [tokens, hidden] bf16."""
    n = len(ys)
    hidden = ys[0].shape[1]
    tokens, topk = gates[0].shape
    dev = ys[0].device
    h0 = handles[0]
    a = _base_args(n, tokens, hidden, topk, h0.n_experts, h0.capacity, state, timeout_ms)
    outs = []
    for r in range(n):
        out = torch.empty(tokens, hidden, dtype=torch.bfloat16, device=dev)
        h = handles[r]
        a.expertIds[r], a.pos[r], a.gates[r] = h.expert_ids.data_ptr(), h.pos.data_ptr(), gates[r].data_ptr()
        a.recvCounts[r], a.y[r], a.out[r] = h.recv_counts.data_ptr(), ys[r].data_ptr(), out.data_ptr()
        outs.append(out)
    _lib.check(_lib.lib().cocclkMoeCombine(a, n, max_ctas, _lib.cur_stream()), "cocclkMoeCombine")
    return outs
