"""Megatron-style GPT (pre-LN, learned positions, tanh-GELU MLP) built on the
fused sm_100a ops, with tensor/sequence/pipeline-parallel hooks.

The reference ships no model code; its training launcher drives an external
Megatron trainer (examples/training_scripts/train_qwen_coccl.sh:1-131) and its
classifier only recognises DP/TP/PP traffic
(src/coccl-extend/core/training/coccl_training_classifier.cc:371-716). This
module is the framework layer that produces that traffic.

Activations are token-major [tokens, hidden] with tokens = batch*seq (batch
outermost). Under sequence parallelism the residual stream is sharded over
tokens; column-parallel linears see the all-gathered tokens and row-parallel
linears reduce-scatter their partial sums back to the shard.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import fused


@dataclass
class GPTConfig:
    n_layer: int = 32
    hidden: int = 4096
    n_head: int = 32
    ffn: int = 16384
    seq_len: int = 2048
    vocab: int = 50304
    eps: float = 1e-5
    init_std: float = 0.02
    dtype: torch.dtype = torch.bfloat16
    # Mixture-of-experts variant: with n_experts > 0 every `moe_every`-th layer (layers moe_every-1, 2*moe_every-1, ...)
    # replaces its MLP by n_experts expert MLPs of width `ffn` behind a top-`moe_top_k` router; the experts are
    # spread over the expert-parallel group (coccl_b200.models.moe.MoETransformerLayer)
    n_experts: int = 0
    moe_top_k: int = 2
    moe_every: int = 1
    # Model family. "gpt": LayerNorm, learned positions, biased linears, tanh-GELU MLP, output head tied to the word
    # embedding. "llama": the Llama / Qwen family (coccl_b200.models.llama): RMSNorm, rotary positions, grouped-query
    # attention with `n_kv_head` key/value heads, SwiGLU MLP of width `ffn`, no biases except (qkv_bias, as Qwen2.5)
    # on the query / key / value projections, untied output head unless tie_embeddings.
    arch: str = "gpt"
    n_kv_head: int = 0              # 0: as many as n_head
    kv_channels: int = 0            # width of one attention head; 0: hidden / n_head (Qwen3 sets 128 whatever the hidden size)
    rope_theta: float = 1.0e6
    qkv_bias: bool = False
    qk_norm: bool = False           # RMSNorm over the head dimension of queries and keys before the rotation (Qwen3)
    tie_embeddings: bool = True     # the llama presets set False

    @property
    def kv_heads(self) -> int:
        return self.n_kv_head or self.n_head

    def is_moe_layer(self, idx: int) -> bool:
        return self.n_experts > 0 and (idx + 1) % max(self.moe_every, 1) == 0

    @property
    def head_dim(self) -> int:
        return self.kv_channels or self.hidden // self.n_head

    def num_params(self) -> int:
        h, f = self.hidden, self.ffn
        if self.arch == "llama":
            qkv = (self.n_head + 2 * self.kv_heads) * self.head_dim
            attn = qkv * h + (qkv if self.qkv_bias else 0) + self.n_head * self.head_dim * h + 2 * h + (2 * self.head_dim if self.qk_norm else 0)
            n_moe = sum(self.is_moe_layer(i) for i in range(self.n_layer))
            mlps = (self.n_layer - n_moe) * 3 * h * f + n_moe * (self.n_experts * 3 * h * f + self.n_experts * h)
            return self.n_layer * attn + mlps + self.vocab * h * (1 if self.tie_embeddings else 2) + h
        attn = 4 * h * h + 4 * h + 4 * h           # qkv, proj, their biases, two LayerNorms
        mlp = 2 * h * f + f + h
        moe = self.n_experts * (2 * h * f + f) + self.n_experts * h        # experts (up, bias, down), router
        n_moe = sum(self.is_moe_layer(i) for i in range(self.n_layer))
        return self.n_layer * attn + (self.n_layer - n_moe) * mlp + n_moe * moe + self.vocab * h + self.seq_len * h + 2 * h

    def flops_per_token(self) -> float:
        """Training FLOPs per token (fwd+bwd = 3x fwd). Attention: QK^T and PV are 2*s*h each per token for full
        attention; a causal mask needs half of it, so 2*s*h per layer in total."""
        h, f, s = self.hidden, self.ffn, self.seq_len
        if self.arch == "llama":
            qkv = (self.n_head + 2 * self.kv_heads) * self.head_dim
            n_moe = sum(self.is_moe_layer(i) for i in range(self.n_layer))
            mlps = (self.n_layer - n_moe) * 2 * 3 * h * f + n_moe * (self.moe_top_k * 2 * 3 * h * f + 2 * h * self.n_experts)
            ao = self.n_head * self.head_dim   # width of the attention output
            return 3.0 * (self.n_layer * (2 * qkv * h + 2 * ao * h + 2 * s * ao) + mlps + 2 * h * self.vocab)
        attn = 2 * 4 * h * h + 2 * s * h
        n_moe = sum(self.is_moe_layer(i) for i in range(self.n_layer))
        dense = 2 * 2 * h * f
        moe = self.moe_top_k * 2 * 2 * h * f + 2 * h * self.n_experts   # top-k experts per token + the router
        return 3.0 * (self.n_layer * attn + (self.n_layer - n_moe) * dense + n_moe * moe + 2 * h * self.vocab)


GPT_6P7B = GPTConfig()
GPT_TINY = GPTConfig(n_layer=2, hidden=256, n_head=4, ffn=1024, seq_len=128, vocab=1024)


class NoTP:
    """Tensor-parallel context of size 1 (all hooks are identities)."""
    size, rank = 1, 0
    sequence_parallel = False

    def gather_tokens(self, x): return x
    def scatter_sum_tokens(self, x): return x
    def all_reduce_sum(self, x): return x
    def copy_to_tp(self, x): return x
    def gather_linear(self, x, w, bias=None, gelu=False): return fused.linear(x, w, bias, gelu=gelu)
    def linear_scatter(self, x, w, bias=None): return fused.linear(x, w, bias)
    def vocab_parallel_cross_entropy(self, logits, targets, scale): return fused.cross_entropy(logits, targets, scale)


class ParamStore:
    """Allocates every parameter of a pipeline stage as a view of one flat bf16 buffer,
    and every gradient as a view (`p.main_grad`) of one flat fp32 buffer, so that the
    distributed optimizer can reduce-scatter / all-gather contiguous shards."""

    def __init__(self, dtype, device, pad_to: int = 1):
        self.dtype, self.device, self.pad_to = dtype, device, pad_to
        self.specs: list[tuple[str, tuple, str, float]] = []
        self.params: dict[str, nn.Parameter] = {}
        self.replicated: dict[str, bool] = {}
        self.flat_param = None
        self.flat_grad = None

    def add(self, name, shape, init="normal", std=0.02, replicated=False):
        """replicated=True: identical on every tensor-parallel rank (its gradient is summed over the group)."""
        self.specs.append((name, tuple(shape), init, std))
        self.replicated[name] = replicated

    def materialise(self, seed=1234, tp_rank=0, grad_dtype=torch.float32):
        # replicated parameters go last, so that "everything a tensor-parallel rank other than 0 must leave out of
        # the gradient norm" is one contiguous range of the flat buffers (norm_exclude_ranges)
        self.specs.sort(key=lambda sp: self.replicated[sp[0]])
        sizes = [math.prod(s) for _, s, _, _ in self.specs]
        # every parameter starts on a 16-byte boundary of both buffers (8 elements)
        offs, total = [], 0
        for n in sizes:
            offs.append(total)
            total += -(-n // 8) * 8
        total = -(-total // self.pad_to) * self.pad_to
        self.flat_param = torch.zeros(total, dtype=self.dtype, device=self.device)
        self.flat_grad = torch.zeros(total, dtype=grad_dtype, device=self.device)
        for (name, shape, init, std), off, n in zip(self.specs, offs, sizes):
            view = self.flat_param[off:off + n].view(shape)
            if init == "normal":
                # seeded by name so that a parameter gets the same values whichever pipeline stage holds it;
                # sharded parameters fold the tensor-parallel rank in, replicated ones must not
                import zlib
                gen = torch.Generator(device=self.device)
                gen.manual_seed(seed + zlib.crc32(name.encode()) + (0 if self.replicated[name] else 7919 * tp_rank))
                view.copy_(torch.randn(shape, generator=gen, device=self.device, dtype=torch.float32) * std)
            elif init == "ones":
                view.fill_(1.0)
            p = nn.Parameter(view, requires_grad=True)
            p.main_grad = self.flat_grad[off:off + n].view(shape)
            self.params[name] = p
        self.offsets = {name: (off, n) for (name, _, _, _), off, n in zip(self.specs, offs, sizes)}
        return self

    def span(self, names):
        """One parameter over several named parameters that sit back to back in the flat buffers (same trailing shape,
        added one after the other): the fused weight of a GEMM that computes all of them at once. Returns an
        nn.Parameter whose rows are the rows of `names` in order and whose `main_grad` covers their gradients; the
        optimizer, the checkpoint and the gradient reduction keep seeing the named parameters."""
        first, last = self.offsets[names[0]], self.offsets[names[-1]]
        tail = tuple(self.params[names[0]].shape[1:])
        width = math.prod(tail) if tail else 1
        at = first[0]
        for n in names:   # back to back, whole rows
            o, cnt = self.offsets[n]
            assert o == at and cnt % 8 == 0 and tuple(self.params[n].shape[1:]) == tail, (n, "is not adjacent to its neighbours")
            at += cnt
        lo, hi = first[0], last[0] + last[1]
        p = nn.Parameter(self.flat_param[lo:hi].view((hi - lo) // width, *tail), requires_grad=True)
        p.main_grad = self.flat_grad[lo:hi].view((hi - lo) // width, *tail)
        return p

    def norm_exclude_ranges(self, tp_rank: int, drop_wte: bool):
        """[lo, hi) ranges of the flat gradient that this rank must not count in the global gradient norm because
        another rank counts the same values: parameters replicated over the tensor-parallel group hold identical
        gradients on every TP rank once they are summed (counted on TP rank 0 only), and the word embedding shared
        by the first and last pipeline stage is counted on the first stage only (`drop_wte` on the last)."""
        out = []
        if tp_rank != 0:
            rep = [self.offsets[n] for n in self.offsets if self.replicated[n]]
            if rep:
                out.append((min(o for o, _ in rep), max(o + n for o, n in rep)))
        if drop_wte and "wte" in self.offsets:
            o, n = self.offsets["wte"]
            out.append((o, o + n))
        return out


class FsdpParamStore(ParamStore):
    """Fully sharded parameters (the scheme known as FSDP / ZeRO-3) over a data-parallel communicator.

    A rank keeps 1 / R of every parameter and gradient (`flat_param_shard`, `flat_grad_shard`, R = ranks). The
    parameters of a transformer layer exist in full only while the layer runs: two buffers of the size of the largest
    layer take turns (layer k uses buffer k % 2), `gather(unit)` fills one from the shards of all ranks before the
    layer's forward and again before its backward, and `reduce_scatter_grads(unit)` sums the layer's gradients into
    the owners' shards as soon as its backward is done (GPTStage places the two calls with autograd functions around
    the layer). What does not belong to a layer (embeddings, final LayerNorm: the unit "outer") stays resident for
    the whole step; its gradients are reduced at the end. This is the traffic the reference's classifier calls
    strategy "fsdp": a steady flow of all-gathers and reduce-scatters on the data-parallel communicator
    (core/training/coccl_training_classifier.cc:555-563), served here by the same (compressed or native) collectives
    as the sharded optimizer's.

    The buffers that take turns are written through aliases with their own version counters: autograd has saved
    parameter views of several layers that share one buffer, and only the layer whose turn it is reads them."""

    OUTER = "outer"

    def __init__(self, dtype, device, comm):
        super().__init__(dtype, device, 1)
        self.comm = comm
        self.ranks = comm.size if comm is not None else 1
        self.rank = comm.rank if comm is not None else 0

    @staticmethod
    def unit_of(name: str) -> str:
        return name.split(".")[1] if name.startswith("layers.") else FsdpParamStore.OUTER

    def materialise(self, seed=1234, tp_rank=0, grad_dtype=torch.float32):
        import zlib
        R, dev = self.ranks, self.device
        units: dict[str, list] = {}
        for spec in self.specs:
            units.setdefault(self.unit_of(spec[0]), []).append(spec)
        self.unit_names = [u for u in units if u != self.OUTER]
        # layout of every unit: 8-element aligned parameters, total a multiple of 8 * R so that shards stay aligned
        self.layout, self.unit_size = {}, {}
        for u, specs in units.items():
            off = 0
            for name, shape, _, _ in specs:
                n = math.prod(shape)
                self.layout[name] = (u, off, n)
                off += -(-n // 8) * 8
            self.unit_size[u] = -(-off // (8 * R)) * (8 * R)
        biggest = max((self.unit_size[u] for u in self.unit_names), default=0)
        self.full = [torch.zeros(biggest, dtype=self.dtype, device=dev) for _ in range(2)]
        self.gfull = [torch.zeros(biggest, dtype=grad_dtype, device=dev) for _ in range(2)]
        outer = self.unit_size.get(self.OUTER, 0)
        self.outer_full = torch.zeros(outer, dtype=self.dtype, device=dev)
        self.outer_gfull = torch.zeros(outer, dtype=grad_dtype, device=dev)
        # this rank's shards of all units, back to back: what the optimizer owns
        self.shard_off, total = {}, 0
        for u in list(self.unit_names) + ([self.OUTER] if outer else []):
            self.shard_off[u] = total
            total += self.unit_size[u] // R
        self.flat_param_shard = torch.zeros(total, dtype=self.dtype, device=dev)
        self.flat_grad_shard = torch.zeros(total, dtype=grad_dtype, device=dev)
        self._scratch = torch.zeros(max([self.unit_size[u] // R for u in self.unit_size] or [0]), dtype=grad_dtype, device=dev)

        def alias(t):   # same memory, own version counter
            return torch.empty(0, dtype=t.dtype, device=t.device).set_(t.untyped_storage(), 0, t.shape)
        self._full_w = [alias(t) for t in self.full]
        self._outer_w = alias(self.outer_full)
        for u, specs in units.items():
            buf, gbuf = self._buffers(u)
            buf.zero_()
            for name, shape, init, std in specs:
                _, off, n = self.layout[name]
                view = buf[off:off + n].view(shape)
                if init == "normal":
                    gen = torch.Generator(device=dev)
                    gen.manual_seed(seed + zlib.crc32(name.encode()) + (0 if self.replicated[name] else 7919 * tp_rank))
                    view.copy_(torch.randn(shape, generator=gen, device=dev, dtype=torch.float32) * std)
                elif init == "ones":
                    view.fill_(1.0)
                prm = nn.Parameter(view, requires_grad=True)
                prm.main_grad = gbuf[off:off + n].view(shape)
                self.params[name] = prm
            self.param_shard(u).copy_(self._mine(buf, u))   # the values of the next unit overwrite the buffer
        self.gather(self.OUTER)
        return self

    def span(self, names):
        """See ParamStore.span: here the named parameters sit back to back inside their unit's buffer."""
        u, first, _ = self.layout[names[0]]
        tail = tuple(self.params[names[0]].shape[1:])
        width = math.prod(tail) if tail else 1
        at = first
        for n in names:
            un, o, cnt = self.layout[n]
            assert un == u and o == at and cnt % 8 == 0 and tuple(self.params[n].shape[1:]) == tail, (n, "is not adjacent to its neighbours")
            at += cnt
        buf, gbuf = self._buffers(u)
        p = nn.Parameter(buf[first:at].view((at - first) // width, *tail), requires_grad=True)
        p.main_grad = gbuf[first:at].view((at - first) // width, *tail)
        return p

    def _buffers(self, u):
        if u == self.OUTER:
            return self.outer_full, self.outer_gfull
        k = self.unit_names.index(u) % 2
        return self.full[k], self.gfull[k]

    def _mine(self, buf, u):
        n = self.unit_size[u] // self.ranks
        return buf[self.rank * n:(self.rank + 1) * n]

    def param_shard(self, u):
        n = self.unit_size[u] // self.ranks
        return self.flat_param_shard[self.shard_off[u]:self.shard_off[u] + n]

    def grad_shard(self, u):
        n = self.unit_size[u] // self.ranks
        return self.flat_grad_shard[self.shard_off[u]:self.shard_off[u] + n]

    def gather(self, u) -> None:
        """Bring unit `u` together from the shards of all ranks, into the buffer whose turn it is."""
        if u not in self.unit_size or self.unit_size[u] == 0:
            return
        target = self._outer_w if u == self.OUTER else self._full_w[self.unit_names.index(u) % 2]
        out = target[:self.unit_size[u]]
        with torch.no_grad():
            if self.ranks == 1:
                out.copy_(self.param_shard(u))
            else:
                self.comm.all_gather(self.param_shard(u), out)

    def zero_unit_grads(self, u) -> None:
        self._buffers(u)[1][:self.unit_size[u]].zero_()

    def reduce_scatter_grads(self, u) -> None:
        """Add the sum over all ranks of unit `u`'s gradients to the owners' shards."""
        if u not in self.unit_size or self.unit_size[u] == 0:
            return
        g = self._buffers(u)[1][:self.unit_size[u]]
        with torch.no_grad():
            if self.ranks == 1:
                self.grad_shard(u).add_(g)
            else:
                part = self._scratch[:self.unit_size[u] // self.ranks]
                self.comm.reduce_scatter(g, part)
                self.grad_shard(u).add_(part)


class _FsdpEnter(torch.autograd.Function):
    """Identity on the layer's inputs. Its backward runs when the layer's backward is complete: the layer's gradients
    go to their owners."""

    @staticmethod
    def forward(ctx, store, unit, *xs):
        ctx.store, ctx.unit = store, unit
        return tuple(x.view_as(x) for x in xs)

    @staticmethod
    def backward(ctx, *gs):
        ctx.store.reduce_scatter_grads(ctx.unit)
        return (None, None, *gs)


class _FsdpLeave(torch.autograd.Function):
    """Identity on the layer's outputs. Its backward runs before any of the layer's: the parameters come back into the
    buffer (another layer has used it since the forward) and the gradient buffer starts from zero."""

    @staticmethod
    def forward(ctx, store, unit, *xs):
        ctx.store, ctx.unit = store, unit
        return tuple(x.view_as(x) for x in xs)

    @staticmethod
    def backward(ctx, *gs):
        ctx.store.gather(ctx.unit)
        ctx.store.zero_unit_grads(ctx.unit)
        return (None, None, *gs)


class TransformerLayer(nn.Module):
    def __init__(self, cfg: GPTConfig, idx: int, store: ParamStore, tp):
        super().__init__()
        self.cfg, self.idx, self.tp = cfg, idx, tp
        h, f, t = cfg.hidden, cfg.ffn, tp.size
        assert cfg.n_head % t == 0 and f % t == 0
        self.prefix = f"layers.{idx}."
        pre = self.prefix
        out_std = cfg.init_std / math.sqrt(2.0 * cfg.n_layer)
        store.add(pre + "ln1.weight", (h,), "ones", replicated=True)
        store.add(pre + "ln1.bias", (h,), "zeros", replicated=True)
        store.add(pre + "qkv.weight", (3 * h // t, h), "normal", cfg.init_std)
        store.add(pre + "qkv.bias", (3 * h // t,), "zeros")
        store.add(pre + "proj.weight", (h, h // t), "normal", out_std)
        store.add(pre + "proj.bias", (h,), "zeros", replicated=True)
        store.add(pre + "ln2.weight", (h,), "ones", replicated=True)
        store.add(pre + "ln2.bias", (h,), "zeros", replicated=True)
        self.add_mlp_params(store, out_std)

    ATTENTION_PARAMS = ("ln1.weight", "ln1.bias", "qkv.weight", "qkv.bias", "proj.weight", "proj.bias", "ln2.weight", "ln2.bias")
    MLP_PARAMS = ("fc1.weight", "fc1.bias", "fc2.weight", "fc2.bias")

    def add_mlp_params(self, store: ParamStore, out_std: float):
        cfg, pre, t = self.cfg, self.prefix, self.tp.size
        h, f = cfg.hidden, cfg.ffn
        store.add(pre + "fc1.weight", (f // t, h), "normal", cfg.init_std)
        store.add(pre + "fc1.bias", (f // t,), "zeros")
        store.add(pre + "fc2.weight", (h, f // t), "normal", out_std)
        store.add(pre + "fc2.bias", (h,), "zeros", replicated=True)

    def bind(self, params: dict, expert_params: dict | None = None):
        for short in self.ATTENTION_PARAMS + self.MLP_PARAMS:
            self.register_parameter(short.replace(".", "_"), params[self.prefix + short])

    def mlp(self, y):
        """Feed-forward block on the normalised residual stream; returns the update that the next LayerNorm adds."""
        z = self.tp.gather_linear(y, self.fc1_weight, self.fc1_bias, gelu=True)
        return self.tp.linear_scatter(z, self.fc2_weight, self.fc2_bias)

    def attention(self, qkv, batch, seq):
        cfg, t = self.cfg, self.tp.size
        nh, d = cfg.n_head // t, cfg.head_dim
        cp = getattr(self, "cp", None)
        if cp is not None:
            # context parallelism: trade the sequence split for a head split (q, k and v of a head travel together)
            assert nh % cp.size == 0, "heads per tensor-parallel rank must divide by the context-parallel size"
            qkv = cp.seq_to_heads(qkv.view(batch, seq, nh, 3 * d))
            seq, nh = seq * cp.size, nh // cp.size
        qkv = qkv.view(batch, seq, nh, 3, d)
        # unbind: its backward is ONE stack of dq/dk/dv into the packed gradient (three selects would each
        # materialise a zero-filled copy of the whole tensor and add them up)
        q, k, v = (t.transpose(1, 2) for t in qkv.unbind(3))  # [b, heads, s, d] views
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        if cp is not None:
            o = cp.heads_to_seq(o.transpose(1, 2).contiguous())   # [b, s / cp, all local heads, d]
            seq, nh = seq // cp.size, nh * cp.size
            return o.reshape(batch * seq, nh * d)
        return o.transpose(1, 2).reshape(batch * seq, nh * d)

    def forward(self, x, delta, batch, seq):
        """x: residual stream, delta: pending update not yet added (or None). Returns (x, delta)."""
        tp = self.tp
        if delta is None:
            y = fused.layer_norm(x, self.ln1_weight, self.ln1_bias, self.cfg.eps)
        else:
            y, x = fused.layer_norm(x, self.ln1_weight, self.ln1_bias, self.cfg.eps, residual=delta)
        # column-parallel: gather the token shards (fused into the GEMM kernel when the shapes allow it)
        qkv = tp.gather_linear(y, self.qkv_weight, self.qkv_bias)
        a = self.attention(qkv, batch, seq)
        # row-parallel: partial sums are reduce-scattered over the token shards; the bias is added once
        o = tp.linear_scatter(a, self.proj_weight, self.proj_bias)
        y, x = fused.layer_norm(x, self.ln2_weight, self.ln2_bias, self.cfg.eps, residual=o)
        return x, self.mlp(y)


class GPTStage(nn.Module):
    """Layers [first, last) of the model plus the embedding (first stage) and the head (last stage).

    With `layer_ranges` the stage holds several model chunks (the virtual stages of an interleaved pipeline schedule,
    parallel/pp.py): chunk c is layers [first_c, last_c); the embedding belongs to chunk 0 and the head to the last
    chunk. All chunks share ONE parameter store, so the optimizer, the checkpoint and the gradient reduction see one
    flat buffer whatever the schedule."""

    def __init__(self, cfg: GPTConfig, device, tp=None, first_layer=0, last_layer=None, pre=True, post=True,
                 seed=1234, pad_to=1, layer_factory=None, ep_comm=None, layer_ranges=None, cp=None, fsdp_comm=None,
                 fsdp: bool = False):
        """ep_comm: communicator of the expert-parallel group for a mixture-of-experts model (None: every expert is
        local). Expert weights that differ between the ranks of that group live in a second flat buffer pair,
        `expert_store`, which data parallelism must not reduce or gather."""
        super().__init__()
        self.cfg, self.tp = cfg, tp or NoTP()
        # context parallelism (parallel.tp.CPContext or None): this rank sees positions [cp.rank * s, (cp.rank + 1) * s)
        # of every sequence, s = seq_len / cp.size
        self.cp = cp if (cp is not None and cp.size > 1) else None
        last_layer = cfg.n_layer if last_layer is None else last_layer
        self.pre, self.post = pre, post
        tp_ = self.tp
        # fsdp: parameters and gradients fully sharded over `fsdp_comm` (FsdpParamStore); a group of one still
        # runs the same gather / scatter points
        self.fsdp = bool(fsdp)
        store = FsdpParamStore(cfg.dtype, device, fsdp_comm) if self.fsdp else ParamStore(cfg.dtype, device, pad_to)
        vshard = cfg.vocab // tp_.size
        assert cfg.vocab % tp_.size == 0
        llama = cfg.arch == "llama"
        assert cfg.arch in ("gpt", "llama"), cfg.arch
        if pre or (post and cfg.tie_embeddings):
            # a tied output head shares the word embedding; under pipeline parallelism the last stage keeps
            # its own copy whose gradient is summed with the first stage's (see parallel/pp.py)
            store.add("wte", (vshard, cfg.hidden), "normal", cfg.init_std)
        if pre and not llama:
            store.add("wpe", (cfg.seq_len, cfg.hidden), "normal", cfg.init_std, replicated=True)
        self.ep_size = ep_comm.size if ep_comm is not None else 1
        # experts spread over several ranks are not replicas of one another: their own buffers. With one rank per
        # expert group they are ordinary (data-parallel replicated) parameters of the main store.
        expert_store = ParamStore(cfg.dtype, device, 8) if (cfg.n_experts > 0 and self.ep_size > 1) else None

        def default_layer(c, i, s, t):
            if llama:
                from .llama import LlamaLayer, LlamaMoELayer
                if c.is_moe_layer(i):
                    return LlamaMoELayer(c, i, s, t, ep_comm, expert_store)
                return LlamaLayer(c, i, s, t)
            if c.is_moe_layer(i):
                from .moe import MoETransformerLayer
                assert t.size == 1, "mixture-of-experts layers are built for expert + data + pipeline parallelism (tp = 1)"
                return MoETransformerLayer(c, i, s, t, ep_comm, expert_store)
            return TransformerLayer(c, i, s, t)

        make = layer_factory or default_layer
        ranges = list(layer_ranges) if layer_ranges is not None else [(first_layer, last_layer)]
        assert all(0 <= a <= b <= cfg.n_layer for a, b in ranges), ranges
        chunks = [[make(cfg, i, store, tp_) for i in range(a, b)] for a, b in ranges]
        self.layers = nn.ModuleList([layer for chunk in chunks for layer in chunk])
        self.chunks = chunks   # plain lists: the modules are registered through self.layers
        if self.cp is not None:
            for layer in self.layers:
                assert not cfg.is_moe_layer(layer.idx), "context parallelism is built for dense layers"
                layer.cp = self.cp
        if post:
            store.add("lnf.weight", (cfg.hidden,), "ones", replicated=True)
            if not llama:
                store.add("lnf.bias", (cfg.hidden,), "zeros", replicated=True)
            if not cfg.tie_embeddings:
                store.add("lm_head", (vshard, cfg.hidden), "normal", cfg.init_std)
        store.materialise(seed, tp_.rank)
        self.store = store
        self.expert_store = expert_store.materialise(seed, 0) if (expert_store is not None and expert_store.specs) else None
        for name, p in store.params.items():
            if not name.startswith("layers."):
                self.register_parameter(name.replace(".", "_"), p)
        for layer in self.layers:
            layer.bind(store.params, self.expert_store.params if self.expert_store is not None else None)

    # ---- embedding (vocab-parallel under TP)
    def embed(self, tokens):
        cfg, tp = self.cfg, self.tp
        b, s = tokens.shape
        flat = tokens.reshape(-1)
        if tp.size == 1:
            e = F.embedding(flat, self.wte)
        else:
            lo = tp.rank * (cfg.vocab // tp.size)
            local = flat - lo
            mask = (local < 0) | (local >= self.wte.shape[0])
            e = F.embedding(local.masked_fill(mask, 0), self.wte)
            e = e.masked_fill(mask[:, None], 0)
        if hasattr(self, "wpe"):
            first = self.cp.rank * s if self.cp is not None else 0   # s is this rank's part of the sequence
            pos = self.wpe[first:first + s].unsqueeze(0).expand(b, s, cfg.hidden).reshape(b * s, cfg.hidden)
        else:
            pos = None   # rotary positions are applied inside the attention
        if tp.size > 1:
            if pos is not None:
                e = e + pos / tp.size  # the position term is summed over ranks below
            e = tp.scatter_sum_tokens(e) if tp.sequence_parallel else tp.all_reduce_sum(e)
        elif pos is not None:
            e = e + pos
        return e.to(cfg.dtype)

    def chunk_is_first(self, chunk=None) -> bool:
        """Whether model chunk `chunk` (None: the whole stage) starts with the embedding."""
        return self.pre and (chunk is None or chunk == 0)

    def chunk_is_last(self, chunk=None) -> bool:
        """Whether model chunk `chunk` (None: the whole stage) ends with the head and the loss."""
        return self.post and (chunk is None or chunk == len(self.chunks) - 1)

    def forward(self, tokens_or_hidden, targets=None, loss_scale: float = 1.0, batch=None, seq=None, chunk=None):
        """First stage takes token ids [b, s]; later stages take (x, delta) from the previous stage.
        The last stage returns the scaled summed loss; others return (x, delta). `chunk` runs one model chunk of a
        stage built with `layer_ranges`; None runs all of the stage's layers in order."""
        if self.chunk_is_first(chunk):
            batch, seq = tokens_or_hidden.shape
            x, delta = self.embed(tokens_or_hidden), None
        else:
            x, delta = tokens_or_hidden
        for layer in (self.layers if chunk is None else self.chunks[chunk]):
            if self.fsdp:
                x, delta = self._sharded_layer(layer, x, delta, batch, seq)
            else:
                x, delta = layer(x, delta, batch, seq)
        if not self.chunk_is_last(chunk):
            return x, delta
        if self.cfg.arch == "llama":
            from .llama import rms_norm
            y = rms_norm(x + delta if delta is not None else x, self.lnf_weight, self.cfg.eps)
        else:
            y, _ = fused.layer_norm(x, self.lnf_weight, self.lnf_bias, self.cfg.eps, residual=delta)
        y = self.tp.gather_tokens(y)
        y = self.tp.copy_to_tp(y)
        logits = fused.linear(y, self.wte if self.cfg.tie_embeddings else self.lm_head)
        return self.tp.vocab_parallel_cross_entropy(logits, targets.reshape(-1), loss_scale)

    def _sharded_layer(self, layer, x, delta, batch, seq):
        """One layer of a fully sharded stage: gather its parameters, run it between the two autograd markers that
        place the backward's gather and reduce-scatter."""
        store, unit = self.store, str(layer.idx)
        store.gather(unit)
        if torch.is_grad_enabled():
            ins = _FsdpEnter.apply(store, unit, *((x,) if delta is None else (x, delta)))
            x, delta = ins[0], (ins[1] if len(ins) > 1 else None)
        x, delta = layer(x, delta, batch, seq)
        if torch.is_grad_enabled():
            x, delta = _FsdpLeave.apply(store, unit, x, delta)
        return x, delta

    # ---- utilities
    def zero_grad_buffer(self):
        if self.fsdp:
            self.store.flat_grad_shard.zero_()
            self.store.outer_gfull.zero_()
            return
        self.store.flat_grad.zero_()
        if self.expert_store is not None:
            self.expert_store.flat_grad.zero_()

    def post_backward_sync_autograd_grads(self):
        """Parameters touched by stock autograd ops (embeddings) receive `.grad`; fold it into main_grad."""
        for p in self.parameters():
            if p.grad is not None:
                p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                p.grad = None
