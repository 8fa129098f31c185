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
    def backward(ctx, dloss):
        (g,) = ctx.saved_tensors
        return g, None, None, None


class TPContext:
    """Hooks the model calls; `comm` is the Communicator of the tensor-parallel group."""

    def __init__(self, comm, sequence_parallel: bool = True):
        self.comm = comm
        self.size, self.rank = comm.size, comm.rank
        self.sequence_parallel = sequence_parallel and comm.size > 1

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
