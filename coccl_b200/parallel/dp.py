"""Data parallelism with a sharded optimizer (ZeRO-1 / Megatron distributed optimizer).

Gradients live in one flat fp32 buffer per pipeline stage; each DP rank owns a
contiguous 1/dp shard of the fp32 master weights and Adam moments. A step is
  reduce-scatter(flat_grad) -> AdamW on the shard -> all-gather(bf16 params).
This is the traffic the reference's training-mode policy targets
(`training.dp.reduce_scatter` with SDP4Bit 4-bit g128 Hadamard and
`training.dp.all_gather`, examples/training_scripts/configs/training.toml:19-54;
classifier strategy "sdp", core/training/coccl_training_classifier.cc:540-571).
"""
from __future__ import annotations

import torch

from ..ops import fused


class DistributedOptimizer:
    def __init__(self, flat_param: torch.Tensor, flat_grad: torch.Tensor, dp_comm=None, *, lr=1e-4, betas=(0.9, 0.95),
                 eps=1e-8, weight_decay=0.1, clip_grad=1.0, norm_groups=(), delta_param_gather: bool | None = None,
                 norm_exclude=(), extra_sumsq=None, strategy: str = "zero1"):
        """dp_comm: communicator of the data-parallel group (None = single replica).
        norm_groups: communicators over which the squared gradient norm must be summed besides DP
        (tensor- and pipeline-parallel groups).
        norm_exclude: [lo, hi) ranges of the flat buffers whose gradients another rank of `norm_groups` already
        counts (ParamStore.norm_exclude_ranges); they are left out of this rank's sum of squares, so the clip
        coefficient equals the one of a run without tensor / pipeline parallelism.
        strategy: "zero1" (default: sharded optimizer state, reduce-scatter + all-gather) or "ddp": every rank keeps the
        whole optimizer state, the gradients are ALL-REDUCED (one- or two-shot compressed all-reduce, or native, as the
        policy's `all_reduce` slot says; the traffic the reference's classifier calls strategy "ddp",
        core/training/coccl_training_classifier.cc:544-556) and nothing is gathered afterwards.
        extra_sumsq: callable returning a device scalar that is added to this rank's sum of squared gradients before
        the sums over the groups: the squares of parameters this optimizer does not hold but the clip coefficient
        must count (the expert weights of a mixture-of-experts model, which differ per data-parallel rank).
        delta_param_gather: send the updated parameters as 8-bit deltas against what every rank already holds (the
        reference's `training.dp.all_gather` policy with subAdd, training.toml:36-54); None = follow the policy file
        (the router answers whether a delta codec is configured for this all-gather)."""
        self.flat_param, self.flat_grad, self.comm = flat_param, flat_grad, dp_comm
        self.dp = dp_comm.size if dp_comm is not None else 1
        self.rank = dp_comm.rank if dp_comm is not None else 0
        assert strategy in ("zero1", "ddp"), strategy
        self.ddp = strategy == "ddp" and self.dp > 1
        n = flat_param.numel()
        assert n % self.dp == 0, "flat buffers must be padded to a multiple of the DP size"
        self.shard = n if self.ddp else n // self.dp
        lo = 0 if self.ddp else self.rank * self.shard
        self.param_shard = flat_param[lo:lo + self.shard]
        dev = flat_param.device
        self.master = self.param_shard.float().clone()
        self.m = torch.zeros(self.shard, dtype=torch.float32, device=dev)
        self.v = torch.zeros(self.shard, dtype=torch.float32, device=dev)
        self.grad_shard = flat_grad[lo:lo + self.shard] if (self.dp == 1 or self.ddp) else torch.empty(
            self.shard, dtype=flat_grad.dtype, device=dev)
        self.lr, self.betas, self.eps, self.wd, self.clip = lr, betas, eps, weight_decay, clip_grad
        self.norm_groups = tuple(norm_groups)
        self.extra_sumsq = extra_sumsq
        # the excluded ranges, cut to this rank's shard and expressed in shard coordinates
        self._excl = [(max(a, lo) - lo, min(b, lo + self.shard) - lo) for a, b in norm_exclude
                      if max(a, lo) < min(b, lo + self.shard)]
        self._sumsq_excl = torch.zeros(1, dtype=torch.float32, device=dev)
        if delta_param_gather is None:   # follow the policy: does the router put a delta codec on this all-gather?
            delta_param_gather = bool(dp_comm is not None and hasattr(dp_comm, "uses_delta_all_gather") and
                                      dp_comm.uses_delta_all_gather(self.shard, flat_param.dtype))
        self.delta = bool(delta_param_gather) and self.dp > 1 and flat_param.is_cuda and not self.ddp
        # with deltas the optimizer must not overwrite the previous parameters before they are subtracted
        self._new_shard = torch.empty_like(self.param_shard) if self.delta else self.param_shard
        self._delta_state = None   # handle of the seeded delta all-gather (see Communicator.all_gather_delta)
        self.step_count = 0
        self._sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        self._coef = torch.ones(1, dtype=torch.float32, device=dev)
        self.grad_norm = torch.zeros(1, dtype=torch.float32, device=dev)

    def local_sum_squares(self) -> torch.Tensor:
        """Sum of squares of the whole flat gradient as it stands (no collective)."""
        fused.sum_squares(self.flat_grad, self._sumsq)
        return self._sumsq

    def step(self, grad_scale: float = 1.0, coef: torch.Tensor | None = None):
        """grad_scale multiplies every gradient before clipping (e.g. 1/dp for averaging). coef: a clip coefficient
        computed elsewhere (device scalar); the norm is then neither computed nor reduced here."""
        self.step_count += 1
        if self.ddp:
            self.comm.all_reduce(self.flat_grad)
        elif self.dp > 1:
            self.comm.reduce_scatter(self.flat_grad, self.grad_shard)
        g = self.grad_shard
        if coef is None:
            fused.sum_squares(g, self._sumsq)
            for a, b in self._excl:
                fused.sum_squares(g[a:b], self._sumsq_excl)
                self._sumsq -= self._sumsq_excl
            if self.extra_sumsq is not None:
                self._sumsq += self.extra_sumsq()
            if self.dp > 1 and not self.ddp:   # ddp: every rank already holds the whole reduced gradient
                self.comm.all_reduce_small(self._sumsq)
            for c in self.norm_groups:
                c.all_reduce_small(self._sumsq)
            fused.clip_coef(self._sumsq, self.clip, grad_scale, self._coef, self.grad_norm)
        else:
            self._coef.copy_(coef)
        fused.adam_step(self.master, self.m, self.v, g, self._new_shard, lr=self.lr, beta1=self.betas[0],
                        beta2=self.betas[1], eps=self.eps, weight_decay=self.wd, step=self.step_count,
                        grad_scale=self._coef)
        if self.delta:
            res = self.comm.all_gather(self._new_shard, self.flat_param, state=self._delta_state)
            self._delta_state = res[1] if isinstance(res, tuple) else None
        elif self.dp > 1 and not self.ddp:
            self.comm.all_gather(self.param_shard, self.flat_param)

    # ---- checkpointing (per-rank shard; see coccl_b200.utils.checkpoint)
    def state_dict(self):
        return {"master": self.master, "m": self.m, "v": self.v, "step": self.step_count}

    def load_state_dict(self, sd):
        self.master.copy_(sd["master"])
        self.m.copy_(sd["m"])
        self.v.copy_(sd["v"])
        self.step_count = int(sd["step"])
        self.param_shard.copy_(self.master)
        self._delta_state = None   # the replicas no longer match what the deltas were taken against: re-seed exactly
        if self.dp > 1 and not self.ddp:
            self.comm.all_gather(self.param_shard, self.flat_param)


class FsdpOptimizer:
    """AdamW over the shards of a fully sharded stage (models.gpt.FsdpParamStore): every rank updates the 1 / R of every
    parameter it owns, from gradients that the backward pass has already reduce-scattered layer by layer. The step
    reduces what is left (the gradients of the embeddings and the final LayerNorm, which stay resident for the whole
    step), forms the global norm from the shards, applies the update and gathers the resident parameters again; the
    layers' parameters are gathered by the next forward pass."""

    def __init__(self, store, dp_comm=None, *, lr=1e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, clip_grad=1.0):
        self.store, self.comm = store, dp_comm
        self.dp = dp_comm.size if dp_comm is not None else 1
        self.param_shard, self.grad_shard = store.flat_param_shard, store.flat_grad_shard
        dev = self.param_shard.device
        self.master = self.param_shard.float().clone()
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        self.lr, self.betas, self.eps, self.wd, self.clip = lr, betas, eps, weight_decay, clip_grad
        self.step_count = 0
        self._sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        self._coef = torch.ones(1, dtype=torch.float32, device=dev)
        self.grad_norm = torch.zeros(1, dtype=torch.float32, device=dev)
        self.ddp = False

    def step(self, grad_scale: float = 1.0, coef=None):
        self.step_count += 1
        st = self.store
        st.reduce_scatter_grads(st.OUTER)
        fused.sum_squares(self.grad_shard, self._sumsq)
        if self.dp > 1:
            self.comm.all_reduce_small(self._sumsq)   # the shards of the ranks partition every gradient
        fused.clip_coef(self._sumsq, self.clip, grad_scale, self._coef, self.grad_norm)
        fused.adam_step(self.master, self.m, self.v, self.grad_shard, self.param_shard, lr=self.lr, beta1=self.betas[0],
                        beta2=self.betas[1], eps=self.eps, weight_decay=self.wd, step=self.step_count, grad_scale=self._coef)
        st.gather(st.OUTER)

    def state_dict(self):
        return {"master": self.master, "m": self.m, "v": self.v, "step": self.step_count}

    def load_state_dict(self, sd):
        self.master.copy_(sd["master"])
        self.m.copy_(sd["m"])
        self.v.copy_(sd["v"])
        self.step_count = int(sd["step"])
        self.param_shard.copy_(self.master)
        self.store.gather(self.store.OUTER)
