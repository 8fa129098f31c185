"""The Llama / Qwen model family on the same trainer: RMSNorm, rotary positions, grouped-query attention, SwiGLU MLP,
no biases (except, optionally, on the query / key / value projections as in Qwen2.5), optional RMSNorm of queries and
keys per head (Qwen3), untied output head.

The reference trains Qwen2.5 and Qwen3 through an external Megatron trainer
(examples/training_scripts/train_qwen_coccl.sh:60-131; Qwen2.5-7B is one of its published end-to-end results,
README.md:348-354). Here the family is a layer class for the package's own trainer: `GPTConfig(arch="llama", ...)`
makes `GPTStage` build `LlamaLayer`s, and every parallel layout of the trainer (tensor + sequence, pipeline incl.
interleaved, data incl. fully sharded, context) applies unchanged, because the layer speaks the same protocol as the
GPT layer: token-major activations, `(x, delta)` between layers, column-parallel `gather_linear` and row-parallel
`linear_scatter` for the projections.

All matrix products run on the tcgen05 GEMMs (and their tensor-parallel fusions): the three attention projections
are ONE GEMM over a weight that spans `q.weight | k.weight | v.weight`, which sit back to back in the flat parameter
buffer (`ParamStore.span`), and so are the gate and up projections of the MLP. RMSNorm, the rotation of the positions
and the SwiGLU gate are written with PyTorch operations (an autograd function for the norm, so that its weight
gradient accumulates in fp32 like every other parameter's).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .gpt import TransformerLayer


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        wide = torch.promote_types(x.dtype, torch.float32)   # at least fp32
        xf = x.to(wide)
        rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
        ctx.save_for_backward(x, weight, rstd)
        return (xf * rstd * weight.to(wide)).to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        x, weight, rstd = ctx.saved_tensors
        wide = rstd.dtype
        xhat = x.to(wide) * rstd
        dyf = dy.to(wide)
        dw = (dyf * xhat).reshape(-1, x.shape[-1]).sum(0)
        g = dyf * weight.to(wide)
        dx = (rstd * (g - xhat * (g * xhat).mean(-1, keepdim=True))).to(x.dtype)
        mg = getattr(weight, "main_grad", None)
        if mg is not None:
            mg.add_(dw.to(mg.dtype))
            return dx, None, None
        return dx, dw.to(weight.dtype), None


def rms_norm(x, weight, eps: float):
    return _RMSNorm.apply(x, weight, eps)


_ROPE_CACHE: dict = {}


def _rope_tables(seq: int, dim: int, theta: float, device):
    key = (seq, dim, theta, str(device))
    t = _ROPE_CACHE.get(key)
    if t is None:
        if len(_ROPE_CACHE) > 8:
            _ROPE_CACHE.clear()
        inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32, device=device) / dim))
        ang = torch.arange(seq, dtype=torch.float32, device=device)[:, None] * inv[None, :]
        t = (torch.cat([ang.cos(), ang.cos()], -1), torch.cat([ang.sin(), ang.sin()], -1))   # [seq, dim] each
        _ROPE_CACHE[key] = t
    return t


def rotate_positions(x, theta: float):
    """Rotary position embedding on x [batch, heads, seq, dim] for positions 0 .. seq - 1 (pairs are (i, i + dim / 2))."""
    cos, sin = _rope_tables(x.shape[2], x.shape[3], theta, x.device)
    half = x.shape[3] // 2
    xf = x.float()
    rot = torch.cat([-xf[..., half:], xf[..., :half]], -1)
    return (xf * cos + rot * sin).to(x.dtype)


class LlamaLayer(TransformerLayer):
    def __init__(self, cfg, idx, store, tp):
        nn.Module.__init__(self)
        self.cfg, self.idx, self.tp, self._store = cfg, idx, tp, store
        h, f, t, d = cfg.hidden, cfg.ffn, tp.size, cfg.head_dim
        nh, nkv = cfg.n_head, cfg.kv_heads
        assert nh % t == 0 and nkv % t == 0 and f % t == 0 and nh % nkv == 0 and d % 2 == 0 and (d * nkv // t) % 8 == 0
        self.prefix = pre = f"layers.{idx}."
        out_std = cfg.init_std / math.sqrt(2.0 * cfg.n_layer)
        store.add(pre + "ln1.weight", (h,), "ones", replicated=True)
        # q | k | v and gate | up are added one after the other: each group is one GEMM over a weight that spans it
        store.add(pre + "q.weight", (nh * d // t, h), "normal", cfg.init_std)
        store.add(pre + "k.weight", (nkv * d // t, h), "normal", cfg.init_std)
        store.add(pre + "v.weight", (nkv * d // t, h), "normal", cfg.init_std)
        if cfg.qkv_bias:
            store.add(pre + "q.bias", (nh * d // t,), "zeros")
            store.add(pre + "k.bias", (nkv * d // t,), "zeros")
            store.add(pre + "v.bias", (nkv * d // t,), "zeros")
        if cfg.qk_norm:
            # one weight vector per layer, applied to every head: the ranks of a tensor-parallel group see different
            # heads, so its gradient is a partial sum like that of any replicated parameter
            store.add(pre + "q_norm.weight", (d,), "ones", replicated=True)
            store.add(pre + "k_norm.weight", (d,), "ones", replicated=True)
        store.add(pre + "o.weight", (h, nh * d // t), "normal", out_std)
        store.add(pre + "ln2.weight", (h,), "ones", replicated=True)
        self.add_mlp_params(store, out_std)

    MLP_NAMES = ("gate.weight", "up.weight", "down.weight")

    def add_mlp_params(self, store, out_std: float):
        cfg, pre, t = self.cfg, self.prefix, self.tp.size
        h, f = cfg.hidden, cfg.ffn
        store.add(pre + "gate.weight", (f // t, h), "normal", cfg.init_std)
        store.add(pre + "up.weight", (f // t, h), "normal", cfg.init_std)
        store.add(pre + "down.weight", (h, f // t), "normal", out_std)

    def names(self):
        base = ["ln1.weight", "q.weight", "k.weight", "v.weight", "o.weight", "ln2.weight", *self.MLP_NAMES]
        return (base + (["q.bias", "k.bias", "v.bias"] if self.cfg.qkv_bias else []) +
                (["q_norm.weight", "k_norm.weight"] if self.cfg.qk_norm else []))

    def bind(self, params: dict, expert_params: dict | None = None):
        pre = self.prefix
        for short in self.names():
            self.register_parameter(short.replace(".", "_"), params[pre + short])
        st = self._store
        self.wqkv = st.span([pre + "q.weight", pre + "k.weight", pre + "v.weight"])
        self.bqkv = st.span([pre + "q.bias", pre + "k.bias", pre + "v.bias"]) if self.cfg.qkv_bias else None
        self.bind_mlp(params, expert_params)

    def bind_mlp(self, params, expert_params):
        self.w_gate_up = self._store.span([self.prefix + "gate.weight", self.prefix + "up.weight"])

    def attention(self, qkv, batch, seq):
        cfg, t = self.cfg, self.tp.size
        nh, nkv, d = cfg.n_head // t, cfg.kv_heads // t, cfg.head_dim
        q, k, v = qkv.split([nh * d, nkv * d, nkv * d], dim=-1)
        q, k = q.reshape(batch, seq, nh, d), k.reshape(batch, seq, nkv, d)
        if cfg.qk_norm:
            q, k = rms_norm(q, self.q_norm_weight, cfg.eps), rms_norm(k, self.k_norm_weight, cfg.eps)
        kv = torch.stack([k, v.reshape(batch, seq, nkv, d)], 3).reshape(batch, seq, nkv, 2 * d)
        cp = getattr(self, "cp", None)
        if cp is not None:
            # context parallelism: whole sequence, a share of the heads (keys and values of a head travel together)
            assert nh % cp.size == 0 and nkv % cp.size == 0, "query and key/value heads per rank must divide by the context-parallel size"
            q, kv = cp.seq_to_heads(q.contiguous()), cp.seq_to_heads(kv)
            seq, nh, nkv = seq * cp.size, nh // cp.size, nkv // cp.size
        k, v = kv.view(batch, seq, nkv, 2, d).unbind(3)
        q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)          # [b, heads, s, d]
        q, k = rotate_positions(q, cfg.rope_theta), rotate_positions(k, cfg.rope_theta)
        if nkv != nh:   # grouped queries: every key/value head serves nh / nkv query heads
            k, v = k.repeat_interleave(nh // nkv, dim=1), v.repeat_interleave(nh // nkv, dim=1)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2)   # [b, s, heads, d]
        if cp is not None:
            o = cp.heads_to_seq(o.contiguous())
            seq, nh = seq // cp.size, nh * cp.size
        return o.reshape(batch * seq, nh * d)

    def mlp(self, y):
        z = self.tp.gather_linear(y, self.w_gate_up, None)
        gate, up = z.chunk(2, dim=-1)
        return self.tp.linear_scatter(F.silu(gate) * up, self.down_weight, None)

    def forward(self, x, delta, batch, seq):
        cfg, tp = self.cfg, self.tp
        if delta is not None:
            x = x + delta
        qkv = tp.gather_linear(rms_norm(x, self.ln1_weight, cfg.eps), self.wqkv, self.bqkv)
        x = x + tp.linear_scatter(self.attention(qkv, batch, seq), self.o_weight, None)
        return x, self.mlp(rms_norm(x, self.ln2_weight, cfg.eps))


class LlamaMoELayer(LlamaLayer):
    """The family's mixture-of-experts layer (Qwen3-MoE, Mixtral style): attention as in LlamaLayer, then a top-k router
    over `n_experts` SwiGLU experts of width `ffn`, weights = softmax over the chosen experts' logits. Tokens travel to
    the experts' ranks and back through the same exchange as the GPT mixture-of-experts layer (models/moe.py: FP8
    dispatch, bf16 combine over the expert-parallel group); with expert parallelism a rank allocates only its own
    experts, in `expert_store`."""

    MLP_NAMES = ("router.weight",)

    def __init__(self, cfg, idx, store, tp, ep_comm, expert_store):
        assert tp.size == 1, "mixture-of-experts layers are built for expert + data + pipeline parallelism (tp = 1)"
        self.ep_comm, self._expert_store = ep_comm, expert_store
        super().__init__(cfg, idx, store, tp)

    def add_mlp_params(self, store, out_std: float):
        cfg, pre = self.cfg, self.prefix
        h, f, e_all = cfg.hidden, cfg.ffn, cfg.n_experts
        ep = self.ep_comm.size if self.ep_comm is not None else 1
        assert e_all % ep == 0, "n_experts must be a multiple of the expert-parallel size"
        first = (self.ep_comm.rank if self.ep_comm is not None else 0) * (e_all // ep)
        self.expert_ids = list(range(first, first + e_all // ep))
        store.add(pre + "router.weight", (e_all, h), "normal", cfg.init_std)
        target = self._expert_store if self._expert_store is not None else store
        for e in self.expert_ids:
            target.add(f"{pre}experts.{e}.gate.weight", (f, h), "normal", cfg.init_std)
            target.add(f"{pre}experts.{e}.up.weight", (f, h), "normal", cfg.init_std)
            target.add(f"{pre}experts.{e}.down.weight", (h, f), "normal", out_std)

    def bind_mlp(self, params, expert_params):
        from .moe import MoELayer
        src = expert_params if self._expert_store is not None else params
        gates, ups, downs = [], [], []
        for e in self.expert_ids:
            for kind, bucket in (("gate", gates), ("up", ups), ("down", downs)):
                p = src[f"{self.prefix}experts.{e}.{kind}.weight"]
                self.register_parameter(f"experts_{e}_{kind}_weight", p)
                bucket.append(p)
        cfg = self.cfg
        self.moe = MoELayer.over(self.ep_comm, cfg.hidden, cfg.ffn, cfg.n_experts, cfg.moe_top_k, self.router_weight,
                                 ups, [None] * len(ups), downs, w_gate=gates)

    def mlp(self, y):
        return self.moe.forward(y)
