"""Expert-parallel MoE feed-forward layer: top-k router, FP8 dispatch, per-expert MLP on the tcgen05 GEMM,
bf16 gate-weighted combine. Forward path (serving / evaluation); the token exchange kernels are in
csrc/kernels/moe_kernels.cu.

The reference has no model code; its hook for this traffic is the compressed AllToAll
(extensions/primitives/coccl_alltoall.cc:12-21) selected by the `normal.all_to_all` policy slot.
"""
from __future__ import annotations

import torch

from ..ops import gemm as G
from ..parallel.comm import Communicator


class MoELayer:
    """n_experts experts, n_experts / comm.size of them on this rank.

    Weights (bf16): router [n_experts, hidden]; per local expert w_up [ffn, hidden], b_up [ffn], w_down [hidden, ffn].
    Initialised from a seed that depends on the GLOBAL expert index, so any expert-parallel degree holds the
    same model."""

    def __init__(self, comm: Communicator, hidden: int, ffn: int, n_experts: int, topk: int = 2, seed: int = 0,
                 device=None):
        assert n_experts % comm.size == 0
        self.comm, self.hidden, self.ffn, self.n_experts, self.topk = comm, hidden, ffn, n_experts, topk
        self.local = n_experts // comm.size
        dev = device or comm.device
        g = torch.Generator(device="cpu").manual_seed(seed)
        self.router = (torch.randn(n_experts, hidden, generator=g) * 0.02).to(dev, torch.bfloat16)
        self.w_up, self.b_up, self.w_down = [], [], []
        for le in range(self.local):
            e = comm.rank * self.local + le
            ge = torch.Generator(device="cpu").manual_seed(seed * 100003 + 17 * e + 1)
            self.w_up.append((torch.randn(ffn, hidden, generator=ge) * 0.02).to(dev, torch.bfloat16))
            self.b_up.append(torch.zeros(ffn, device=dev, dtype=torch.bfloat16))
            self.w_down.append((torch.randn(hidden, ffn, generator=ge) * 0.02).to(dev, torch.bfloat16))

    def route(self, x: torch.Tensor):
        logits = G.gemm(x, self.router, out_dtype=torch.float32)
        top = logits.topk(self.topk, dim=1)
        return top.indices.to(torch.int32).contiguous(), torch.softmax(top.values, dim=1).contiguous()

    def experts(self, rows: torch.Tensor, offsets: list[int]) -> torch.Tensor:
        y = torch.empty_like(rows)
        for le in range(self.local):
            lo, hi = offsets[le], offsets[le + 1]
            if hi > lo:
                h = G.gemm(rows[lo:hi], self.w_up[le], bias=self.b_up[le], gelu=True)
                G.gemm(h, self.w_down[le], out=y[lo:hi])
        return y

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x [tokens, hidden] bf16 -> [tokens, hidden] bf16."""
        ids, gates = self.route(x)
        if self.comm.size == 1:
            return self.forward_local(x, ids, gates)
        rows, h = self.comm.moe_dispatch(x, ids, self.n_experts)
        y = self.experts(rows, h.recv_offsets.tolist())
        return self.comm.moe_combine(y, gates, h)

    def forward_local(self, x, ids, gates) -> torch.Tensor:
        """Single-rank path (all experts local): same arithmetic, plain indexing instead of the exchange."""
        out = torch.zeros(x.shape[0], self.hidden, device=x.device, dtype=torch.float32)
        for e in range(self.n_experts):
            for j in range(self.topk):
                tok = (ids[:, j] == e).nonzero()[:, 0]
                if tok.numel():
                    h = G.gemm(x[tok].contiguous(), self.w_up[e], bias=self.b_up[e], gelu=True)
                    y = G.gemm(h, self.w_down[e])
                    out[tok] += gates[tok, j:j + 1] * y.float()
        return out.to(torch.bfloat16)
