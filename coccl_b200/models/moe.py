"""Expert-parallel MoE feed-forward layer: top-k router, FP8 dispatch, per-expert MLP on the tcgen05 GEMM,
bf16 gate-weighted combine; the token exchange kernels are in csrc/kernels/moe_kernels.cu. The exchange is
differentiable: the backward of the dispatch is a combine with unit gates, the backward of the combine is a
dispatch of the output gradient scaled by the gates (FP8 on the wire) plus the gate gradients, which the combine
kernel computes as dot products on the token side.

The reference has no model code; its hook for this traffic is the compressed AllToAll
(extensions/primitives/coccl_alltoall.cc:12-21) selected by the `normal.all_to_all` policy slot.
"""
from __future__ import annotations

import torch

from ..ops import fused
from ..ops import gemm as G
from ..parallel.comm import Communicator


class _Exchange:
    """Routing of one forward pass, shared by the dispatch and the combine."""

    def __init__(self, comm, ids, n_experts):
        from ..ops import moe as M
        self.comm, self.ids, self.n_experts = comm, ids, n_experts
        self.layout = M.route_layout(ids, n_experts, comm.size)
        self.handle = None


class _Dispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, ex):
        rows, h = ex.comm.moe_dispatch(x.contiguous(), ex.ids, ex.n_experts, layout=ex.layout)
        ex.handle = h
        ctx.ex = ex
        ctx.tokens = x.shape[0]
        return rows

    @staticmethod
    def backward(ctx, d_rows):
        ex = ctx.ex
        ones = torch.ones(ctx.tokens, ex.ids.shape[1], dtype=torch.float32, device=d_rows.device)
        return ex.comm.moe_combine(d_rows.contiguous(), ones, ex.handle), None


class _Combine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, gates, ex):
        ctx.ex = ex
        ctx.save_for_backward(y, gates)
        return ex.comm.moe_combine(y.contiguous(), gates.contiguous(), ex.handle)

    @staticmethod
    def backward(ctx, d_out):
        y, gates = ctx.saved_tensors
        ex = ctx.ex
        d_out = d_out.contiguous()
        # dy[row(t, j)] = gates[t, j] * d_out[t]: the same routing, rows scaled per entry
        d_y, _ = ex.comm.moe_dispatch(d_out, ex.ids, ex.n_experts, row_scale=gates.contiguous(), layout=ex.layout)
        # d_gates[t, j] = <y[row(t, j)], d_out[t]>: send the expert outputs back once more and dot them on arrival
        _, d_g = ex.comm.moe_combine(y.contiguous(), gates.contiguous(), ex.handle, dot_with=d_out)
        return d_y, d_g, None


class _Solo:
    """Stand-in for the communicator of a group of one."""
    size, rank = 1, 0


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

    @classmethod
    def over(cls, comm, hidden: int, ffn: int, n_experts: int, topk: int, router, w_up, b_up, w_down, w_gate=None):
        """The layer over parameters that somebody else owns (a trainer's flat buffers): `w_up`, `b_up`, `w_down`
        list this rank's experts in order of their global index; comm None means every expert is local. With
        `w_gate` the experts are SwiGLU MLPs (silu(x W_gate^T) * (x W_up^T)) W_down^T without biases (the Llama / Qwen
        family); without it GELU MLPs with a bias on the first projection."""
        self = cls.__new__(cls)
        self.comm = comm if comm is not None else _Solo()
        assert n_experts % self.comm.size == 0 and len(w_up) == n_experts // self.comm.size
        self.hidden, self.ffn, self.n_experts, self.topk = hidden, ffn, n_experts, topk
        self.local = n_experts // self.comm.size
        self.router, self.w_up, self.b_up, self.w_down = router, list(w_up), list(b_up), list(w_down)
        self.w_gate = list(w_gate) if w_gate is not None else None
        return self

    def parameters(self):
        return [self.router, *self.w_up, *[b for b in self.b_up if b is not None], *self.w_down, *(self.w_gate or [])]

    def expert(self, le: int, x: torch.Tensor) -> torch.Tensor:
        """Local expert `le` on rows x."""
        gate = getattr(self, "w_gate", None)
        if gate is not None:
            h = torch.nn.functional.silu(fused.linear(x, gate[le])) * fused.linear(x, self.w_up[le])
        else:
            h = fused.linear(x, self.w_up[le], self.b_up[le], gelu=True)
        return fused.linear(h, self.w_down[le])

    def requires_grad_(self, on: bool = True):
        for p in self.parameters():
            p.requires_grad_(on)
        return self

    def route(self, x: torch.Tensor):
        if self.n_experts % 8 == 0:
            logits = fused.linear(x, self.router).float()
        else:   # narrower than the tensor-core GEMM's 8-column granule: a library matmul (its gradient arrives as
            logits = torch.nn.functional.linear(x, self.router).float()   # .grad and is folded into main_grad)
        top = logits.topk(self.topk, dim=1)
        return top.indices.to(torch.int32).contiguous(), torch.softmax(top.values, dim=1).contiguous()

    def experts(self, rows: torch.Tensor, offsets: list[int]) -> torch.Tensor:
        outs, total = [], rows.shape[0]
        for le in range(self.local):
            lo, hi = offsets[le], offsets[le + 1]
            if hi > lo:
                outs.append(self.expert(le, rows[lo:hi]))
        used = offsets[self.local]
        if used < total:  # unused tail of the receive buffer
            outs.append(rows.new_zeros(total - used, rows.shape[1]))
        return torch.cat(outs) if outs else rows.new_zeros(total, rows.shape[1])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x [tokens, hidden] bf16 -> [tokens, hidden] bf16 (differentiable)."""
        ids, gates = self.route(x)
        if self.comm.size == 1:
            return self.forward_local(x, ids, gates)
        ex = _Exchange(self.comm, ids, self.n_experts)
        rows = _Dispatch.apply(x, ex)
        y = self.experts(rows, ex.handle.recv_offsets.tolist())
        return _Combine.apply(y, gates, ex)

    def forward_local(self, x, ids, gates) -> torch.Tensor:
        """Single-rank path (all experts local): same arithmetic, plain indexing instead of the exchange."""
        out = torch.zeros(x.shape[0], self.hidden, device=x.device, dtype=torch.float32)
        for e in range(self.n_experts):
            for j in range(self.topk):
                tok = (ids[:, j] == e).nonzero()[:, 0]
                if tok.numel():
                    y = self.expert(e, x[tok].contiguous())
                    out = out.index_add(0, tok, gates[tok, j:j + 1] * y.float())
        return out.to(x.dtype)


from .gpt import TransformerLayer  # noqa: E402  (gpt.py imports this module lazily, inside the layer factory)


class MoETransformerLayer(TransformerLayer):
    """Transformer layer whose feed-forward block is a mixture of experts: attention as in the dense layer, then
    router -> FP8 dispatch over the expert-parallel group -> expert MLPs -> gate-weighted combine.

    Parameters: `router.weight` [n_experts, hidden] is replicated (main store, reduced over data parallelism like
    every dense parameter). Expert e owns `experts.e.w_up` [ffn, hidden], `experts.e.b_up` [ffn] and
    `experts.e.w_down` [hidden, ffn]; the names carry the GLOBAL expert index and the initial values are seeded by
    name, so every expert-parallel degree starts from the same model. With an expert-parallel group of more than one
    rank a rank allocates only its own experts, in `expert_store` (they are not data-parallel replicas: every token
    routed to an expert reaches its one copy, so its gradient is already complete and is never reduced)."""

    def __init__(self, cfg, idx, store, tp, ep_comm, expert_store):
        self.ep_comm, self._expert_store = ep_comm, expert_store
        super().__init__(cfg, idx, store, tp)

    def add_mlp_params(self, store, out_std):
        cfg, pre = self.cfg, self.prefix
        h, f, e_all = cfg.hidden, cfg.ffn, cfg.n_experts
        ep = self.ep_comm.size if self.ep_comm is not None else 1
        assert e_all % ep == 0, "n_experts must be a multiple of the expert-parallel size"
        local = e_all // ep
        first = (self.ep_comm.rank if self.ep_comm is not None else 0) * local
        self.expert_ids = list(range(first, first + local))
        store.add(pre + "router.weight", (e_all, h), "normal", cfg.init_std)
        target = self._expert_store if self._expert_store is not None else store
        for e in self.expert_ids:
            target.add(f"{pre}experts.{e}.w_up", (f, h), "normal", cfg.init_std)
            target.add(f"{pre}experts.{e}.b_up", (f,), "zeros")
            target.add(f"{pre}experts.{e}.w_down", (h, f), "normal", out_std)

    def bind(self, params, expert_params=None):
        for short in self.ATTENTION_PARAMS + ("router.weight",):
            self.register_parameter(short.replace(".", "_"), params[self.prefix + short])
        src = expert_params if self._expert_store is not None else params
        ups, biases, downs = [], [], []
        for e in self.expert_ids:
            for kind, bucket in (("w_up", ups), ("b_up", biases), ("w_down", downs)):
                p = src[f"{self.prefix}experts.{e}.{kind}"]
                self.register_parameter(f"experts_{e}_{kind}", p)
                bucket.append(p)
        cfg = self.cfg
        self.moe = MoELayer.over(self.ep_comm, cfg.hidden, cfg.ffn, cfg.n_experts, cfg.moe_top_k, self.router_weight,
                                 ups, biases, downs)

    def mlp(self, y):
        return self.moe.forward(y)
