"""Pipeline parallelism: non-interleaved 1F1B schedule over NCCL point-to-point.

Stage boundaries carry one activation tensor per micro-batch (the residual
stream, already summed with its pending update, token-sharded under sequence
parallelism so each tensor-parallel rank talks to its counterpart only).
The reference recognises this traffic as the PP role (a communicator of size
pipeline_parallel_size doing Send/Recv; forward iff rank<peer on send,
core/runtime/coccl_runtime.cc:83-103) and BASELINE keeps it on native NCCL p2p.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class PipelineSchedule:
    def __init__(self, stage, mesh, cfg, micro_batch: int):
        self.stage, self.mesh, self.cfg, self.mb = stage, mesh, cfg, micro_batch
        self.pp_rank, self.pp_size = mesh.pp_rank, mesh.pp
        self.prev = mesh.pp_prev_global if self.pp_rank > 0 else None
        self.next = mesh.pp_next_global if self.pp_rank < self.pp_size - 1 else None
        tokens = micro_batch * cfg.seq_len
        tp = stage.tp
        self.act_shape = (tokens // tp.size if tp.sequence_parallel else tokens, cfg.hidden)
        self.dtype = cfg.dtype
        self.group = mesh.pp_group

    # -- p2p helpers. A send and a receive that face each other across a stage boundary are
    # issued as ONE batch, so neither side can block the other (what Megatron calls
    # send_forward_recv_backward / send_backward_recv_forward).
    def _new(self):
        return torch.empty(self.act_shape, dtype=self.dtype, device=self.stage.store.flat_param.device)

    def _p2p(self, send=None, send_to=None, recv_from=None):
        ops, out = [], None
        if send is not None and send_to is not None:
            ops.append(dist.P2POp(dist.isend, send.contiguous(), send_to, self.group))
        if recv_from is not None:
            out = self._new()
            ops.append(dist.P2POp(dist.irecv, out, recv_from, self.group))
        if ops:
            for r in dist.batch_isend_irecv(ops):
                r.wait()
        return out

    def _forward(self, tokens, i, inp, scale, loss_acc):
        """Returns the stage output to send on (None on the last stage) and what backward needs."""
        mb = tokens[i * self.mb:(i + 1) * self.mb]
        b, s = self.mb, self.cfg.seq_len
        tgt = mb[:, 1:] if self.stage.post else None
        if self.stage.pre:
            out = self.stage(mb[:, :-1], tgt, scale)
        else:
            inp.requires_grad_(True)
            out = self.stage((inp, None), tgt, scale, batch=b, seq=s)
        if self.stage.post:
            loss_acc += out.detach()
            return None, (inp, out)
        x, delta = out
        y = x + delta if delta is not None else x
        return y.detach(), (inp, y)

    def _backward(self, saved, out_grad):
        inp, out = saved
        if self.stage.post:
            out.backward()
        else:
            torch.autograd.backward(out, out_grad)
        return inp.grad if inp is not None else None

    def run(self, tokens, n_micro: int, scale: float, loss_acc):
        prev, nxt = self.prev, self.next
        warm = min(self.pp_size - self.pp_rank - 1, n_micro)
        steady = n_micro - warm
        q, nf = [], 0
        for _ in range(warm):
            inp = self._p2p(recv_from=prev)
            y, saved = self._forward(tokens, nf, inp, scale, loss_acc); nf += 1
            self._p2p(send=y, send_to=nxt)
            q.append(saved)
        inp = self._p2p(recv_from=prev) if steady > 0 else None
        for k in range(steady):
            y, saved = self._forward(tokens, nf, inp, scale, loss_acc); nf += 1
            q.append(saved)
            out_grad = self._p2p(send=y, send_to=nxt, recv_from=nxt)
            in_grad = self._backward(q.pop(0), out_grad)
            last = k == steady - 1
            inp = self._p2p(send=in_grad, send_to=prev, recv_from=None if last else prev)
        for _ in range(warm):
            out_grad = self._p2p(recv_from=nxt)
            in_grad = self._backward(q.pop(0), out_grad)
            self._p2p(send=in_grad, send_to=prev)
