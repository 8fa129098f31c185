"""Process mesh (tensor x context x data x pipeline) and the communicators of each axis; expert parallelism reuses the
data-parallel axis (each data-parallel rank holds 1/ep of the experts of a mixture-of-experts model).

Rank order follows Megatron: tp fastest, then cp, then dp, then pp:
    rank = tp_rank + tp * (cp_rank + cp * (dp_rank + dp * pp_rank))
so tensor-parallel peers are adjacent GPUs. Context-parallel ranks hold the same parameters and different parts of every
sequence, exactly like data-parallel ranks hold different sequences: gradients are reduced, and the optimizer state is
sharded, over the combined data x context group (`dp_group`, `dp_comm`), while `dp_rank` alone says which sequences a
rank reads and `cp_rank` which part of them.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .comm import NATIVE, Communicator, Policy
from .tp import TPContext


class Mesh:
    def __init__(self, tp=1, pp=1, dp=1, device=None, compress=True, policy: Policy | None = None,
                 sequence_parallel=True, ep=1, cp=1):
        world, rank = dist.get_world_size(), dist.get_rank()
        assert tp * cp * pp * dp == world, (tp, cp, pp, dp, world)
        assert ep in (1, dp), "the expert-parallel group is the data-parallel group (ep = dp) or absent (ep = 1)"
        assert ep == 1 or cp == 1, "expert parallelism and context parallelism are not combined"
        self.tp, self.pp, self.dp, self.ep, self.cp, self.device = tp, pp, dp, ep, cp, device
        self.rank = rank
        self.tp_rank = rank % tp
        self.cp_rank = (rank // tp) % cp
        self.dp_rank = (rank // (tp * cp)) % dp
        self.pp_rank = rank // (tp * cp * dp)
        pol = (policy or Policy()) if compress else NATIVE
        self.sequence_parallel = sequence_parallel

        def make(groups):
            mine = None
            for ranks in groups:
                g = dist.new_group(ranks) if len(ranks) > 1 else None
                if rank in ranks:
                    mine = (g, ranks)
            return mine

        def at(t, c, d, p):
            return t + tp * (c + cp * (d + dp * p))

        tp_groups = [[at(t, c, d, p) for t in range(tp)] for p in range(pp) for d in range(dp) for c in range(cp)]
        # gradients and optimizer shards: all replicas of a parameter, i.e. data x context
        dp_groups = [[at(t, c, d, p) for d in range(dp) for c in range(cp)] for p in range(pp) for t in range(tp)]
        pp_groups = [[at(t, c, d, p) for p in range(pp)] for d in range(dp) for c in range(cp) for t in range(tp)]
        (self.tp_group, self.tp_ranks) = make(tp_groups)
        (self.dp_group, self.dp_ranks) = make(dp_groups)
        (self.pp_group, self.pp_ranks) = make(pp_groups)
        self.cp_group, self.cp_ranks = None, [rank]
        if cp > 1:
            cp_groups = [[at(t, c, d, p) for c in range(cp)] for p in range(pp) for d in range(dp) for t in range(tp)]
            (self.cp_group, self.cp_ranks) = make(cp_groups)
        # first and last pipeline stage share the word embedding
        emb_groups = [[r[0], r[-1]] for r in pp_groups] if pp > 1 else []
        self.emb_group = None
        for ranks in emb_groups:
            g = dist.new_group(ranks)
            if rank in ranks:
                self.emb_group = g
        self.tp_comm = Communicator(self.tp_group, device, pol, "tp") if tp > 1 else None
        self.dp_comm = Communicator(self.dp_group, device, pol, "dp") if dp * cp > 1 else None
        # the head exchange of context parallelism carries attention inputs and outputs: uncompressed
        self.cp_comm = Communicator(self.cp_group, device, NATIVE, "cp") if cp > 1 else None
        self.pp_comm = Communicator(self.pp_group, device, NATIVE, "pp") if pp > 1 else None
        # token exchange of the experts: the same ranks as data parallelism, its own workspace and flags
        self.ep_comm = Communicator(self.dp_group, device, pol, "ep") if ep > 1 else None
        self.pp_prev_global = self.pp_ranks[self.pp_rank - 1] if self.pp_rank > 0 else None
        self.pp_next_global = self.pp_ranks[self.pp_rank + 1] if self.pp_rank < pp - 1 else None

    def tp_context(self):
        if self.tp_comm is None:
            return None
        return TPContext(self.tp_comm, self.sequence_parallel)

    def cp_context(self):
        if self.cp_comm is None:
            return None
        from .tp import CPContext
        return CPContext(self.cp_comm)

    def sync_shared_grads(self, stage):
        """Sum gradients of parameters that are replicated but see partial data:
        tensor-parallel replicas (LayerNorm, row-parallel biases, positions) and the word
        embedding shared by the first and last pipeline stage."""
        store = stage.store
        if self.tp_comm is not None:
            names = [n for n in store.params if store.replicated.get(n)]
            if not self.sequence_parallel:
                names = [n for n in names if not (".ln" in n or n.startswith("lnf"))]
            offsets = getattr(store, "offsets", None)
            if names and self.sequence_parallel and offsets is not None:
                # the store keeps replicated parameters together at the end of the flat buffers: one all-reduce on
                # that slice of the gradient buffer, nothing gathered or copied (the gaps between them are zero padding)
                lo = min(offsets[n][0] for n in names)
                hi = max(offsets[n][0] + offsets[n][1] for n in names)
                assert all(store.replicated[n] for n, (o, _) in offsets.items() if lo <= o < hi)
                dist.all_reduce(store.flat_grad[lo:hi], group=self.tp_group)
            elif names:
                grads = [store.params[n].main_grad for n in names]
                flat = torch.cat([g.reshape(-1) for g in grads])
                dist.all_reduce(flat, group=self.tp_group)
                off = 0
                for g in grads:
                    g.copy_(flat[off:off + g.numel()].view_as(g))
                    off += g.numel()
        if self.emb_group is not None and (stage.pre or stage.post) and stage.cfg.tie_embeddings:
            dist.all_reduce(store.params["wte"].main_grad, group=self.emb_group)

    def close(self):
        for c in (self.tp_comm, self.dp_comm, self.pp_comm, self.ep_comm, self.cp_comm):
            if c is not None:
                c.close()
