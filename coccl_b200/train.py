"""Training engine: micro-batch loop, (optional) pipeline schedule, sharded optimizer.

`Trainer.train_step(tokens)` is the public entry point used by bench.py and the
examples: it takes one global-batch slice of token ids for this data-parallel
rank as a pinned host tensor [sequences, seq_len + 1], copies it to the device,
runs forward/backward over all micro-batches, reduces gradients, steps the
optimizer and returns the mean loss as a device scalar.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .models.gpt import GPTConfig, GPTStage
from .parallel.dp import DistributedOptimizer


@dataclass
class ParallelConfig:
    tp: int = 1
    pp: int = 1
    dp: int = 1
    sequence_parallel: bool = True
    # "zero1": sharded optimizer (reduce-scatter + all-gather); "ddp": gradient all-reduce; "fsdp": parameters, gradients
    # and optimizer state all sharded, a layer's parameters gathered while it runs (data parallelism only)
    dp_strategy: str = "zero1"
    ep: int = 1   # expert parallelism of a mixture-of-experts model: 1 (every rank holds all experts) or dp
    virtual_stages: int = 1   # model chunks per pipeline rank; > 1 selects the interleaved 1F1B schedule
    cp: int = 1   # context parallelism: ranks that share every sequence, each holding seq_len / cp positions of it


def split_layers(n_layer: int, stages: int) -> list[tuple[int, int]]:
    """Layer range [first, last) of each of `stages` consecutive (virtual) pipeline stages. Layers that do not divide
    evenly go to the FIRST stages: the last one also runs the final LayerNorm, the output head and the loss, which cost
    about one transformer layer (2 * hidden * vocab against 24 * hidden^2 FLOPs per token for GPT-6.7B)."""
    assert 1 <= stages <= n_layer, f"{n_layer} layers cannot fill {stages} pipeline stages"
    base, extra = divmod(n_layer, stages)
    out, first = [], 0
    for s in range(stages):
        n = base + (1 if s < extra else 0)
        out.append((first, first + n))
        first += n
    return out


class Trainer:
    def __init__(self, cfg: GPTConfig, device, *, micro_batch=2, parallel: ParallelConfig | None = None, groups=None,
                 lr=1e-4, weight_decay=0.1, clip_grad=1.0, seed=1234):
        self.cfg, self.device, self.micro_batch = cfg, device, micro_batch
        self.parallel = parallel or ParallelConfig()
        self.groups = groups  # coccl_b200.parallel.mesh.Mesh or None (single GPU)
        g = groups
        tp_ctx = g.tp_context() if g is not None else None
        pp_rank = g.pp_rank if g is not None else 0
        pp = self.parallel.pp
        chunks = self.parallel.virtual_stages if pp > 1 else 1
        assert chunks >= 1
        # virtual stage c * pp + pp_rank is this rank's chunk c (one chunk: the plain contiguous split)
        stages = split_layers(cfg.n_layer, pp * chunks)
        ranges = [stages[c * pp + pp_rank] for c in range(chunks)]
        dp = self.parallel.dp
        cp = self.parallel.cp
        assert cp == (g.cp if g is not None else 1), "ParallelConfig.cp and the mesh disagree"
        assert cfg.seq_len % cp == 0, "the sequence length must divide by the context-parallel size"
        self.cp_ctx = g.cp_context() if (g is not None and cp > 1) else None
        replicas = dp * cp   # ranks that hold the same parameters: the gradient / optimizer-shard group
        ep_comm = getattr(g, "ep_comm", None) if g is not None else None
        assert self.parallel.ep == (ep_comm.size if ep_comm is not None else 1), "ParallelConfig.ep and the mesh disagree"
        self.fsdp = self.parallel.dp_strategy == "fsdp"
        if self.fsdp:
            assert self.parallel.tp == pp == cp == self.parallel.ep == 1 and cfg.n_experts == 0, \
                "the fully sharded strategy is built for pure data parallelism of dense models"
        self.stage = GPTStage(cfg, device, tp=tp_ctx, layer_ranges=ranges, fsdp=self.fsdp,
                              fsdp_comm=(g.dp_comm if (g is not None and dp > 1) else None),
                              pre=(pp_rank == 0), post=(pp_rank == pp - 1), seed=seed, pad_to=8 * replicas * 2048,
                              ep_comm=ep_comm, cp=self.cp_ctx)
        # experts spread over the expert-parallel group: updated locally (never reduced or gathered), clipped with
        # the same coefficient as everything else; their squares enter the global norm through the main optimizer
        self.expert_opt = None
        es = self.stage.expert_store
        if es is not None:
            self.expert_opt = DistributedOptimizer(es.flat_param, es.flat_grad, None, lr=lr, weight_decay=weight_decay,
                                                   clip_grad=clip_grad)
        if self.fsdp:
            from .parallel.dp import FsdpOptimizer
            self.opt = FsdpOptimizer(self.stage.store, g.dp_comm if (g is not None and dp > 1) else None, lr=lr,
                                     weight_decay=weight_decay, clip_grad=clip_grad)
        norm_groups = []
        if g is not None:
            if g.tp_comm is not None and g.tp_comm.size > 1:
                norm_groups.append(g.tp_comm)
            if g.pp_comm is not None and g.pp_comm.size > 1:
                norm_groups.append(g.pp_comm)
        self.opt = self.opt if self.fsdp else DistributedOptimizer(self.stage.store.flat_param, self.stage.store.flat_grad,
                                        g.dp_comm if (g is not None and replicas > 1) else None, lr=lr,
                                        weight_decay=weight_decay, clip_grad=clip_grad, norm_groups=norm_groups,
                                        norm_exclude=self.stage.store.norm_exclude_ranges(
                                            g.tp_rank if g is not None else 0,
                                            drop_wte=(pp > 1 and pp_rank == pp - 1 and cfg.tie_embeddings)),
                                        extra_sumsq=(self.expert_opt.local_sum_squares if self.expert_opt is not None else None),
                                        strategy=self.parallel.dp_strategy)
        self.schedule = None
        if pp > 1:
            from .parallel.pp import InterleavedSchedule, PipelineSchedule
            self.schedule = (InterleavedSchedule(self.stage, g, cfg, micro_batch, chunks) if chunks > 1
                             else PipelineSchedule(self.stage, g, cfg, micro_batch))
        self._loss_acc = torch.zeros(1, dtype=torch.float32, device=device)
        self._dev_tokens = None

    def train_step(self, tokens: torch.Tensor) -> torch.Tensor:
        """tokens: [n_seq, seq_len+1] int64 (pinned host or device). Returns the mean token loss (device scalar); with
        context parallelism every rank of the group passes the same sequences and the returned values of the group
        add up to the mean."""
        cfg = self.cfg
        n_seq = tokens.shape[0]
        assert n_seq % self.micro_batch == 0
        n_micro = n_seq // self.micro_batch
        if tokens.device != self.device:
            if self._dev_tokens is None or self._dev_tokens.shape != tokens.shape:
                self._dev_tokens = torch.empty(tokens.shape, dtype=tokens.dtype, device=self.device)
            self._dev_tokens.copy_(tokens, non_blocking=True)
            tokens = self._dev_tokens
        if self.cp_ctx is not None:
            # this rank's part of every sequence: positions [lo, lo + s) as inputs, [lo + 1, lo + s + 1) as targets
            s_local = cfg.seq_len // self.parallel.cp
            lo = self.cp_ctx.rank * s_local
            tokens = tokens[:, lo:lo + s_local + 1]
        # health: the status words copied at the end of the previous step (no synchronisation); a wait that gave
        # up inside a fused kernel means that step's gradients or parameters are not valid
        self.check_health(wait=False)
        self.stage.zero_grad_buffer()
        self._loss_acc.zero_()
        # loss is summed over tokens of this rank's micro-batches and scaled so that the sum over
        # all data-parallel ranks is the global mean
        scale = 1.0 / (n_seq * cfg.seq_len * self.parallel.dp)
        if self.schedule is not None:
            self.schedule.run(tokens, n_micro, scale, self._loss_acc)
        else:
            for i in range(n_micro):
                mb = tokens[i * self.micro_batch:(i + 1) * self.micro_batch]
                loss = self.stage(mb[:, :-1], mb[:, 1:], scale)
                loss.backward()
                self._loss_acc += loss.detach()
        self.stage.post_backward_sync_autograd_grads()
        if self.groups is not None:
            self.groups.sync_shared_grads(self.stage)
        self.opt.step(grad_scale=1.0)
        if self.expert_opt is not None:
            self.expert_opt.step(coef=self.opt._coef)
        for c in self._comms():
            c.post_status_read()
        return self._loss_acc * self.parallel.dp  # this rank's mean loss

    @torch.no_grad()
    def eval_step(self, tokens: torch.Tensor) -> torch.Tensor:
        """Mean token loss of `tokens` [n_seq, seq_len + 1] under the current parameters: forward passes only, no
        gradient, no update. Same conventions as train_step: each data-parallel rank passes its own sequences, and
        the returned values add up over the ranks that hold a loss exactly as train_step's do."""
        cfg = self.cfg
        n_seq = tokens.shape[0]
        assert n_seq % self.micro_batch == 0
        n_micro = n_seq // self.micro_batch
        if tokens.device != self.device:
            tokens = tokens.to(self.device, non_blocking=True)
        if self.cp_ctx is not None:
            s_local = cfg.seq_len // self.parallel.cp
            lo = self.cp_ctx.rank * s_local
            tokens = tokens[:, lo:lo + s_local + 1]
        acc = torch.zeros(1, dtype=torch.float32, device=self.device)
        scale = 1.0 / (n_seq * cfg.seq_len * self.parallel.dp)
        if self.schedule is not None:
            self.schedule.run_forward_only(tokens, n_micro, scale, acc)
        else:
            for i in range(n_micro):
                mb = tokens[i * self.micro_batch:(i + 1) * self.micro_batch]
                acc += self.stage(mb[:, :-1], mb[:, 1:], scale)
        return acc * self.parallel.dp

    def _comms(self):
        g = self.groups
        return [c for c in ((g.tp_comm, g.dp_comm, g.pp_comm, getattr(g, "ep_comm", None), getattr(g, "cp_comm", None))
                            if g is not None else ())
                if c is not None]

    def check_health(self, wait: bool = True) -> None:
        """Raise coccl_b200.parallel.comm.PeerLost if a bounded wait inside a fused collective, a tensor-parallel
        fusion or the expert exchange gave up during an earlier step, and RuntimeError for a GEMM pipeline error.
        `wait=True` first waits for the copies of the status words queued by the last step."""
        for c in self._comms():
            c.poll_status(wait=wait)
        if wait:
            from .ops import gemm as G
            G.check_errors()
