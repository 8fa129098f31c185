"""Pipeline parallelism over NCCL point-to-point: 1F1B (`PipelineSchedule`) and interleaved 1F1B with several model
chunks per rank (`InterleavedSchedule`).

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
        # with context parallelism a rank holds seq_len / cp positions of every sequence
        self.seq = cfg.seq_len // (stage.cp.size if getattr(stage, "cp", None) is not None else 1)
        tokens = micro_batch * self.seq
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

    def _forward(self, tokens, i, inp, scale, loss_acc, chunk=None):
        """Returns the stage output to send on (None where the model ends) and what backward needs."""
        mb = tokens[i * self.mb:(i + 1) * self.mb]
        b, s = self.mb, self.seq
        first, last = self.stage.chunk_is_first(chunk), self.stage.chunk_is_last(chunk)
        tgt = mb[:, 1:] if last else None
        if first:
            out = self.stage(mb[:, :-1], tgt, scale, chunk=chunk)
        else:
            if torch.is_grad_enabled():
                inp.requires_grad_(True)
            out = self.stage((inp, None), tgt, scale, batch=b, seq=s, chunk=chunk)
        if last:
            loss_acc += out.detach()
            return None, (inp, out)
        x, delta = out
        y = x + delta if delta is not None else x
        return y.detach(), (inp, y)

    def _backward(self, saved, out_grad, chunk=None):
        inp, out = saved
        if self.stage.chunk_is_last(chunk):
            out.backward()
        else:
            torch.autograd.backward(out, out_grad)
        return inp.grad if inp is not None else None

    def run_forward_only(self, tokens, n_micro: int, scale: float, loss_acc):
        """Evaluation: every micro-batch walks through the (virtual) stages once, no gradients, one tensor in flight
        per stage boundary. A chain of matching blocking sends and receives, so nothing can wait in a cycle."""
        chunks = len(self.stage.chunks)
        ring = list(self.mesh.pp_ranks)
        last_vs = self.pp_size * chunks - 1
        with torch.no_grad():
            for m in range(n_micro):
                for c in range(chunks):
                    vs = c * self.pp_size + self.pp_rank
                    inp = self._p2p(recv_from=ring[(self.pp_rank - 1) % self.pp_size]) if vs > 0 else None
                    y, _ = self._forward(tokens, m, inp, scale, loss_acc, chunk=c if chunks > 1 else None)
                    if vs < last_vs:
                        self._p2p(send=y, send_to=ring[(self.pp_rank + 1) % self.pp_size])

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


def interleaved_order(pp: int, rank: int, chunks: int, n_micro: int):
    """Order of the forward and backward passes of one rank under interleaved 1F1B: a list of
    (kind, chunk, micro_batch), kind 'F' or 'B'.

    Virtual stage chunk * pp + rank holds the rank's model chunk `chunk`, so a micro-batch visits every rank `chunks`
    times. Micro-batches advance in groups of `pp`: the k-th forward pass of a rank is chunk (k // pp) % chunks of
    micro-batch (k // (pp * chunks)) * pp + k % pp, and the k-th backward pass is the same micro-batch on the mirrored
    chunk. A rank runs (pp - rank - 1) * 2 + (chunks - 1) * pp forward passes ahead, then alternates, then drains.
    """
    assert n_micro % pp == 0, "interleaved 1F1B moves micro-batches in groups of the pipeline size"
    total = n_micro * chunks

    def fwd(k):
        return (k // pp) % chunks, (k // (pp * chunks)) * pp + k % pp

    def bwd(k):
        c, m = fwd(k)
        return chunks - 1 - c, m

    warm = min((pp - rank - 1) * 2 + (chunks - 1) * pp, total)
    order = [("F",) + fwd(k) for k in range(warm)]
    for k in range(total - warm):
        order.append(("F",) + fwd(warm + k))
        order.append(("B",) + bwd(k))
    order.extend(("B",) + bwd(k) for k in range(total - warm, total))
    return order


def plan_ticks(pp: int, chunks: int, n_micro: int):
    """Global plan of an interleaved step: a list of ticks, each a list with one entry per rank: the pass that rank
    runs in the tick, (kind, chunk, micro_batch), or None when its next pass still waits for a message.

    A pass may start in the tick AFTER the one that produced its input, because messages move between ticks. Every
    rank computes the same plan from (pp, chunks, n_micro), so both ends of every message agree on the tick in which
    it travels without exchanging anything.
    """
    orders = [interleaved_order(pp, r, chunks, n_micro) for r in range(pp)]
    pos, done, ticks = [0] * pp, set(), []
    last_vs = pp * chunks - 1
    while any(pos[r] < len(orders[r]) for r in range(pp)):
        row = []
        for r in range(pp):
            a = orders[r][pos[r]] if pos[r] < len(orders[r]) else None
            if a is not None:
                kind, c, m = a
                vs = c * pp + r
                if kind == "F":
                    dep = ("F", vs - 1, m) if vs > 0 else None
                else:
                    dep = ("B", vs + 1, m) if vs < last_vs else ("F", vs, m)
                if dep is not None and dep not in done:
                    a = None
            row.append(a)
        if not any(a is not None for a in row):
            raise RuntimeError(f"interleaved schedule cannot advance (pp={pp}, chunks={chunks}, micro-batches={n_micro})")
        for r, a in enumerate(row):
            if a is not None:
                pos[r] += 1
                done.add((a[0], a[1] * pp + r, a[2]))
        ticks.append(row)
    return ticks


class InterleavedSchedule(PipelineSchedule):
    """Interleaved 1F1B: every rank holds `chunks` model chunks (GPTStage built with `layer_ranges`), the pipeline has
    pp * chunks virtual stages, and the start-up and drain bubbles shrink by the factor `chunks` at the price of
    `chunks` times as many boundary messages.

    The step follows `plan_ticks`. After each tick every rank issues ONE batch of point-to-point operations: it sends
    what it produced in the tick and posts a receive for what each neighbour produced for it in the same tick. Both
    ends derive the batch from the shared plan, so the operations of every pair of ranks match in number and order
    (with two ranks the forward and the backward neighbour are the same process, which is why the order matters), and
    a batch only ever waits for batches of the same tick on other ranks. Received tensors are waited for when the pass
    that consumes them starts, not when the batch is issued.
    """

    def __init__(self, stage, mesh, cfg, micro_batch: int, chunks: int):
        super().__init__(stage, mesh, cfg, micro_batch)
        assert chunks >= 2 and len(stage.chunks) == chunks
        self.chunks = chunks
        self.ring = list(mesh.pp_ranks)   # global ranks of the pipeline group, by pipeline rank
        self._plans = {}

    def _plan(self, n_micro):
        if n_micro not in self._plans:
            self._plans[n_micro] = plan_ticks(self.pp_size, self.chunks, n_micro)
        return self._plans[n_micro]

    def _message(self, rank, action):
        """(destination pipeline rank, key of the receiving pass) of what `rank` produces with `action`, or None."""
        if action is None:
            return None
        kind, c, m = action
        vs = c * self.pp_size + rank
        if kind == "F":
            return ((rank + 1) % self.pp_size, ("F", vs + 1, m)) if vs < self.pp_size * self.chunks - 1 else None
        return ((rank - 1) % self.pp_size, ("B", vs - 1, m)) if vs > 0 else None

    def run(self, tokens, n_micro: int, scale: float, loss_acc):
        me, P = self.pp_rank, self.pp_size
        inbox, saved, pending = {}, {}, []

        def finish(batch):
            # once per request: a second wait on a completed gloo request blocks for a completion that never comes
            while batch:
                batch.pop().wait()

        def take(key):
            buf, batch = inbox.pop(key)
            finish(batch)
            return buf

        for row in self._plan(n_micro):
            produced = None
            a = row[me]
            if a is not None:
                kind, c, m = a
                vs = c * P + me
                if kind == "F":
                    inp = take(("F", vs, m)) if vs > 0 else None
                    produced, saved[(c, m)] = self._forward(tokens, m, inp, scale, loss_acc, chunk=c)
                else:
                    out_grad = take(("B", vs, m)) if vs < P * self.chunks - 1 else None
                    produced = self._backward(saved.pop((c, m)), out_grad, chunk=c)
            ops, received = [], []
            out = self._message(me, a)
            if out is not None:
                ops.append(dist.P2POp(dist.isend, produced.contiguous(), self.ring[out[0]], self.group))
            for q in range(P):
                msg = self._message(q, row[q]) if q != me else None
                if msg is not None and msg[0] == me:
                    buf = self._new()
                    ops.append(dist.P2POp(dist.irecv, buf, self.ring[q], self.group))
                    received.append((msg[1], buf))
            if ops:
                batch = list(dist.batch_isend_irecv(ops))
                for key, buf in received:
                    inbox[key] = (buf, batch)
                pending.append(batch)
                if len(pending) > 2 * P:
                    # bounds the boundary tensors kept alive for sends; a batch of tick t waits only for the peers
                    # to reach tick t, which never depends on this rank's later ticks
                    finish(pending.pop(0))
        for batch in pending:
            finish(batch)
        assert not inbox and not saved
