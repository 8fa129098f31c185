"""Tensor parallelism with Megatron-style sequence parallelism.

The residual stream is sharded over tokens between the tensor-parallel blocks;
a column-parallel linear consumes the all-gathered tokens and a row-parallel
linear reduce-scatters its partial sums. These are exactly the collectives the
reference's classifier expects from a TP group with `sequence_parallel=true`
(core/training/coccl_training_classifier.cc:573-581) and for which it offers the
policy slots training.tp.{all_gather,reduce_scatter,all_reduce}
(core/config/coccl_config.cc:669-695). Here they run through the fused
compressed kernels of the group's Communicator.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import fused


class _Gather(torch.autograd.Function):
    """forward: all-gather over tokens; backward: reduce-scatter."""

    @staticmethod
    def forward(ctx, x, comm):
        ctx.comm = comm
        out = torch.empty((x.shape[0] * comm.size, *x.shape[1:]), dtype=x.dtype, device=x.device)
        comm.all_gather(x.contiguous(), out, role="tp")
        return out

    @staticmethod
    def backward(ctx, dy):
        comm = ctx.comm
        out = torch.empty((dy.shape[0] // comm.size, *dy.shape[1:]), dtype=dy.dtype, device=dy.device)
        comm.reduce_scatter(dy.contiguous(), out, role="tp")
        return out, None


class _ScatterSum(torch.autograd.Function):
    """forward: reduce-scatter over tokens; backward: all-gather."""

    @staticmethod
    def forward(ctx, x, comm):
        ctx.comm = comm
        out = torch.empty((x.shape[0] // comm.size, *x.shape[1:]), dtype=x.dtype, device=x.device)
        comm.reduce_scatter(x.contiguous(), out, role="tp")
        return out

    @staticmethod
    def backward(ctx, dy):
        comm = ctx.comm
        out = torch.empty((dy.shape[0] * comm.size, *dy.shape[1:]), dtype=dy.dtype, device=dy.device)
        comm.all_gather(dy.contiguous(), out, role="tp")
        return out, None


class _AllReduce(torch.autograd.Function):
    """forward: all-reduce; backward: identity."""

    @staticmethod
    def forward(ctx, x, comm):
        y = x.contiguous().clone()
        comm.all_reduce(y, role="tp")
        return y

    @staticmethod
    def backward(ctx, dy):
        return dy, None


class _CopyToTP(torch.autograd.Function):
    """forward: identity; backward: all-reduce (input replicated over the TP group)."""

    @staticmethod
    def forward(ctx, x, comm):
        ctx.comm = comm
        return x

    @staticmethod
    def backward(ctx, dy):
        y = dy.contiguous().clone()
        ctx.comm.all_reduce(y, role="tp")
        return y, None


class _VocabParallelCE(torch.autograd.Function):
    """Cross-entropy over vocabulary shards: three small all-reduces (max, sum-exp, target logit)."""

    @staticmethod
    def forward(ctx, logits, targets, scale, comm):
        if logits.is_cuda and logits.dtype == torch.bfloat16:
            return _VocabParallelCE._forward_cuda(ctx, logits, targets, scale, comm)
        vs = logits.shape[-1]
        lo = comm.rank * vs
        lf = logits.float()
        mx = lf.amax(dim=-1)
        comm.all_reduce_small(mx, op=dist.ReduceOp.MAX)
        lf = lf - mx[:, None]
        ex = lf.exp()
        se = ex.sum(-1)
        comm.all_reduce_small(se)
        local = targets - lo
        inside = (local >= 0) & (local < vs)
        lc = local.clamp(0, vs - 1)
        tl = torch.where(inside, lf.gather(1, lc[:, None])[:, 0], torch.zeros_like(se))
        comm.all_reduce_small(tl)
        valid = targets >= 0
        loss = torch.where(valid, se.log() - tl, torch.zeros_like(se))
        p = ex / se[:, None]
        p[torch.arange(p.shape[0], device=p.device), lc] -= inside.to(p.dtype)
        p = p * (valid[:, None] * scale)
        ctx.save_for_backward(p.to(logits.dtype))
        return loss.sum() * scale

    @staticmethod
    def _forward_cuda(ctx, logits, targets, scale, comm):
        """Two kernels and one small all-gather: per-row {max, sum-exp, target logit} of this vocabulary shard, the
        exchange of those 16 bytes per row, then loss and in-place gradient (csrc/kernels/train_kernels.cu)."""
        from .. import _lib
        V = logits.shape[-1]
        lg = logits.reshape(-1, V)
        assert lg.stride(1) == 1
        tg = targets.reshape(-1).contiguous()
        M = lg.shape[0]
        dev = lg.device
        lib = _lib.lib()
        stats = torch.empty(M, 4, dtype=torch.float32, device=dev)
        _lib.check(lib.cocclkCrossEntropyStats(lg.data_ptr(), tg.data_ptr(), stats.data_ptr(), M, V, lg.stride(0),
                                               comm.rank * V, _lib.cur_stream()), "cocclkCrossEntropyStats")
        allstats = torch.empty(comm.size, M, 4, dtype=torch.float32, device=dev)
        dist.all_gather_into_tensor(allstats, stats, group=comm.group)
        loss = torch.empty(M, dtype=torch.float32, device=dev)
        _lib.check(lib.cocclkCrossEntropyFinish(lg.data_ptr(), tg.data_ptr(), allstats.data_ptr(), comm.size, loss.data_ptr(),
                                                M, V, lg.stride(0), comm.rank * V, float(scale), _lib.cur_stream()),
                   "cocclkCrossEntropyFinish")
        ctx.save_for_backward(lg)   # overwritten in place with (softmax - onehot) * scale
        ctx.shape = logits.shape
        return loss.sum() * scale

    @staticmethod
    def backward(ctx, dloss):
        (g,) = ctx.saved_tensors
        shape = getattr(ctx, "shape", None)
        return (g.reshape(shape) if shape is not None else g), None, None, None


def _gelu_bwd(dy2, z):
    from .. import _lib
    dz = torch.empty_like(dy2)
    _lib.check(_lib.lib().cocclkGeluBwd(dy2.data_ptr(), z.data_ptr(), dz.data_ptr(), dz.numel(), _lib.cur_stream()), "cocclkGeluBwd")
    return dz


def _col_sum(bias, dy2):
    from .. import _lib
    M, N = dy2.shape

    def run(out, acc):
        sc = fused.scratch(dy2.device, _lib.lib().cocclkColSumBlocks(M) * N, "colsum")
        _lib.check(_lib.lib().cocclkColSum(dy2.data_ptr(), out.data_ptr(), int(acc), sc.data_ptr(), M, N, _lib.cur_stream()),
                   "cocclkColSum")
    return fused._accum_param_grad(bias, None, run)


class _GatherLinear(torch.autograd.Function):
    """Column-parallel linear on sequence shards as ONE kernel per direction:
    forward  y = act(gather(x) @ w.T + b)      (all-gather -> GEMM, csrc/kernels/tp_kernels.cu agGemmKernel)
    backward dx = reduce_scatter(dy @ w)        (GEMM -> FP8 reduce-scatter, gemmRsKernel)."""

    @staticmethod
    def forward(ctx, x, w, bias, gelu, comm):
        m, K = x.shape
        xg = torch.empty(m * comm.size, K, dtype=x.dtype, device=x.device)
        if gelu:
            y, z = comm.ag_gemm(x.contiguous(), w, bias, True, save_preact=True, gathered=xg)
        else:
            y, z = comm.ag_gemm(x.contiguous(), w, bias, False, gathered=xg), None
        ctx.save_for_backward(xg, w, bias, z)
        ctx.comm, ctx.gelu = comm, gelu
        return y

    @staticmethod
    def backward(ctx, dy):
        xg, w, bias, z = ctx.saved_tensors
        from ..ops import gemm as G
        dy2 = dy.contiguous()
        if ctx.gelu:
            dy2 = _gelu_bwd(dy2, z)
        dx = ctx.comm.gemm_rs(dy2, w, b_mn=True) if ctx.needs_input_grad[0] else None   # w [N, K] is "[contraction, out]"
        dw = fused._accum_param_grad(w, None, lambda out, acc: G.gemm(dy2.t(), xg.t(), out=out, accumulate=acc))
        db = _col_sum(bias, dy2) if bias is not None else None
        return dx, dw, db, None, None


class _LinearScatter(torch.autograd.Function):
    """Row-parallel linear whose partial sums are reduce-scattered over the token shards, ONE kernel per direction:
    forward  o = reduce_scatter(x @ w.T) + b    (gemmRsKernel, FP8 on the wire)
    backward dx = gather(do) @ w                 (agGemmKernel)."""

    @staticmethod
    def forward(ctx, x, w, bias, comm):
        x2 = x.contiguous()
        # the bias is added once, to this rank's reduced rows (inside the kernel's epilogue); its gradient is summed
        # over the group with the other replicated parameters
        o = comm.gemm_rs(x2, w, bias=bias)
        ctx.save_for_backward(x2, w, bias)
        ctx.comm = comm
        return o

    @staticmethod
    def backward(ctx, do):
        x2, w, bias = ctx.saved_tensors
        from ..ops import gemm as G
        comm = ctx.comm
        d2 = do.contiguous()
        dg = torch.empty(d2.shape[0] * comm.size, d2.shape[1], dtype=d2.dtype, device=d2.device)
        dx = comm.ag_gemm(d2, w, b_mn=True, gathered=dg)   # w [h, f/t] is "[contraction, out]"
        dw = fused._accum_param_grad(w, None, lambda out, acc: G.gemm(dg.t(), x2.t(), out=out, accumulate=acc))
        db = _col_sum(bias, d2) if bias is not None else None
        return dx, dw, db, None


class TPContext:
    """Hooks the model calls; `comm` is the Communicator of the tensor-parallel group."""

    def __init__(self, comm, sequence_parallel: bool = True):
        self.comm = comm
        self.size, self.rank = comm.size, comm.rank
        self.sequence_parallel = sequence_parallel and comm.size > 1
        self.fuse_gemm = True   # use the one-kernel all-gather->GEMM / GEMM->reduce-scatter fusions when they apply

    def can_fuse(self, x_shard, n_out_rs=None) -> bool:
        return (self.fuse_gemm and self.sequence_parallel and x_shard.is_cuda and x_shard.dim() == 2 and
                self.comm.tp_fusable(x_shard.shape[0] * self.size, n_out_rs, x_shard.shape[1]))

    def gather_linear(self, x_shard, w, bias=None, gelu=False):
        """act(gather_tokens(x_shard) @ w.T + bias) for a column-parallel weight shard."""
        if self.can_fuse(x_shard, w.shape[1]):  # the backward reduce-scatters w.shape[1] columns
            return _GatherLinear.apply(x_shard, w, bias, gelu, self.comm)
        return fused.linear(self.gather_tokens(x_shard), w, bias, gelu=gelu)

    def linear_scatter(self, x_full, w, bias=None):
        """scatter_sum_tokens(x_full @ w.T) + bias for a row-parallel weight shard."""
        if self.size > 1 and self.fuse_gemm and self.sequence_parallel and x_full.is_cuda and x_full.dim() == 2 and \
                self.comm.tp_fusable(x_full.shape[0], w.shape[0], x_full.shape[1]):
            return _LinearScatter.apply(x_full, w, bias, self.comm)
        o = fused.linear(x_full, w, bias if self.rank == 0 else None)
        return self.scatter_sum_tokens(o)

    def gather_tokens(self, x):
        if self.size == 1:
            return x
        return _Gather.apply(x, self.comm) if self.sequence_parallel else _CopyToTP.apply(x, self.comm)

    def scatter_sum_tokens(self, x):
        if self.size == 1:
            return x
        return _ScatterSum.apply(x, self.comm) if self.sequence_parallel else _AllReduce.apply(x, self.comm)

    def all_reduce_sum(self, x):
        return x if self.size == 1 else _AllReduce.apply(x, self.comm)

    def copy_to_tp(self, x):
        # with sequence parallelism the gather's backward already reduces; otherwise the hook above did
        return x

    def vocab_parallel_cross_entropy(self, logits, targets, scale):
        if self.size == 1:
            return fused.cross_entropy(logits, targets, scale)
        return _VocabParallelCE.apply(logits, targets, scale, self.comm)


# ---------------------------------------------------------------------------- context parallelism (head exchange)
class _SeqToHeads(torch.autograd.Function):
    """[b, s / cp, heads, w] on every context-parallel rank -> [b, s, heads / cp, w]: rank j receives head group j of
    every rank's part of the sequence (one all-to-all); the backward is the opposite exchange."""

    @staticmethod
    def forward(ctx, x, comm):
        ctx.comm = comm
        return _seq_to_heads(x, comm)

    @staticmethod
    def backward(ctx, g):
        return _heads_to_seq(g.contiguous(), ctx.comm), None


class _HeadsToSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, comm):
        ctx.comm = comm
        return _heads_to_seq(x, comm)

    @staticmethod
    def backward(ctx, g):
        return _seq_to_heads(g.contiguous(), ctx.comm), None


def _seq_to_heads(x, comm):
    cp = comm.size
    b, sl, nh, w = x.shape
    send = x.view(b, sl, cp, nh // cp, w).permute(2, 0, 1, 3, 4).contiguous()      # [destination, b, s / cp, heads / cp, w]
    recv = torch.empty_like(send)
    comm.all_to_all(send.view(-1), recv.view(-1))
    return recv.permute(1, 0, 2, 3, 4).reshape(b, cp * sl, nh // cp, w)              # source rank j holds sequence part j


def _heads_to_seq(x, comm):
    cp = comm.size
    b, s, nhl, w = x.shape
    send = x.view(b, cp, s // cp, nhl, w).permute(1, 0, 2, 3, 4).contiguous()      # [destination, b, s / cp, heads / cp, w]
    recv = torch.empty_like(send)
    comm.all_to_all(send.view(-1), recv.view(-1))
    return recv.permute(1, 2, 0, 3, 4).reshape(b, s // cp, cp * nhl, w)              # source rank j holds head group j


class CPContext:
    """Context parallelism by head exchange (the scheme known as Ulysses): every rank of the group holds 1 / cp of each
    sequence for everything that works token by token; around the attention one all-to-all trades the sequence split
    for a head split, so that every rank attends over the WHOLE sequence for heads / cp heads, and a second one trades
    it back. The reference has no attention code; its launcher only forwards a context-parallel size to the external
    trainer (examples/training_scripts/train_qwen_coccl.sh:21-29)."""

    def __init__(self, comm):
        self.comm, self.size, self.rank = comm, comm.size, comm.rank

    def seq_to_heads(self, x):
        return _SeqToHeads.apply(x, self.comm)

    def heads_to_seq(self, x):
        return _HeadsToSeq.apply(x, self.comm)
