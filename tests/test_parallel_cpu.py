"""3-D parallel trainer on CPU ranks (gloo): every parallel layout must reproduce the single-process loss."""
import dataclasses

import pytest
import torch

from dist_utils import run_distributed


def _cfg():
    from coccl_b200.models.gpt import GPTConfig
    return GPTConfig(n_layer=4, hidden=64, n_head=4, ffn=256, seq_len=32, vocab=128, dtype=torch.float32)


def _data(cfg, n_seq):
    g = torch.Generator().manual_seed(7)
    return torch.randint(0, cfg.vocab, (n_seq, cfg.seq_len + 1), generator=g)


def _reference_losses(steps=3, n_seq=8):
    from coccl_b200.train import Trainer
    cfg = _cfg()
    tr = Trainer(cfg, torch.device("cpu"), micro_batch=2, lr=1e-2)
    tok = _data(cfg, n_seq)
    losses, norms = [], []
    for _ in range(steps):
        losses.append(tr.train_step(tok).item())
        norms.append(tr.opt.grad_norm.item())
    return tr, list(zip(losses, norms))


def _worker(rank, world, tp, pp, dp, ref_losses, ref_params, virtual_stages=1, cp=1):
    import torch.distributed as dist
    from coccl_b200.parallel.mesh import Mesh
    from coccl_b200.train import ParallelConfig, Trainer
    from coccl_b200.utils.checkpoint import shard_param
    cfg = _cfg()
    mesh = Mesh(tp=tp, pp=pp, dp=dp, cp=cp, device=torch.device("cpu"))
    tr = Trainer(cfg, torch.device("cpu"), micro_batch=2, parallel=ParallelConfig(tp, pp, dp, virtual_stages=virtual_stages, cp=cp),
                 groups=mesh, lr=1e-2)
    # load the single-process model's initial weights, re-sharded for this rank
    for name, p in tr.stage.store.params.items():
        p.data.copy_(shard_param(name, ref_params[name], mesh.tp_rank, tp))
    tr.opt.master.copy_(tr.opt.param_shard.float())
    tok = _data(cfg, 8)
    per = 8 // dp
    mine = tok[mesh.dp_rank * per:(mesh.dp_rank + 1) * per]
    for step, (ref, ref_norm) in enumerate(ref_losses):
        # evaluation (forward passes only, also through the pipeline schedules) sees the loss the training step reports
        held = tr.eval_step(mine).clone()
        dist.all_reduce(held)
        assert abs(held.item() / (tp * dp) - ref) < 2e-3 * abs(ref) + 1e-4, (step, held.item() / (tp * dp), ref)
        loss = tr.train_step(mine)
        # the global gradient norm counts every parameter once, whatever the layout: replicated parameters on one
        # tensor-parallel rank only, the shared embedding on one pipeline stage only
        norm = tr.opt.grad_norm.item()
        assert abs(norm - ref_norm) < 2e-3 * ref_norm + 1e-6, (step, norm, ref_norm)
        # mean over DP ranks of the per-rank mean == global mean; only the last stage holds the loss
        t = loss.clone()
        dist.all_reduce(t)
        total = t.item() / (tp * dp)
        assert abs(total - ref) < 2e-3 * abs(ref) + 1e-4, (step, total, ref)


@pytest.mark.parametrize("tp,pp,dp", [(2, 1, 1), (1, 2, 1), (1, 1, 2), (2, 2, 1), (2, 2, 2)])
def test_parallel_layouts_match_single_process(tp, pp, dp):
    tr, losses = _reference_losses()
    tr2, _ = _reference_losses(steps=0)
    params = {k: v.detach().clone() for k, v in tr2.stage.store.params.items()}
    run_distributed(_worker, tp * pp * dp, "gloo", (tp, pp, dp, losses, params))


@pytest.mark.parametrize("tp,pp,dp,chunks", [(1, 2, 1, 2), (2, 2, 1, 2), (1, 4, 1, 1)])
def test_interleaved_pipeline_matches_single_process(tp, pp, dp, chunks):
    """Two model chunks per pipeline rank (virtual stages c * pp + rank): same losses and gradient norms as one process."""
    tr, losses = _reference_losses()
    tr2, _ = _reference_losses(steps=0)
    params = {k: v.detach().clone() for k, v in tr2.stage.store.params.items()}
    run_distributed(_worker, tp * pp * dp, "gloo", (tp, pp, dp, losses, params, chunks))


@pytest.mark.parametrize("tp,pp,dp,cp", [(1, 1, 1, 2), (2, 1, 1, 2), (1, 2, 1, 2), (1, 1, 2, 2)])
def test_context_parallel_layouts_match_single_process(tp, pp, dp, cp):
    """Every sequence split over cp ranks, whole-sequence attention by head exchange: same losses and gradient norms."""
    tr, losses = _reference_losses()
    tr2, _ = _reference_losses(steps=0)
    params = {k: v.detach().clone() for k, v in tr2.stage.store.params.items()}
    run_distributed(_worker, tp * pp * dp * cp, "gloo", (tp, pp, dp, losses, params, 1, cp))


def _uneven_worker(rank, world, ref_losses, ref_params):
    import dataclasses as dc
    import torch.distributed as dist
    from coccl_b200.parallel.mesh import Mesh
    from coccl_b200.train import ParallelConfig, Trainer
    cfg = dc.replace(_cfg(), n_layer=3)
    mesh = Mesh(tp=1, pp=2, dp=1, device=torch.device("cpu"))
    tr = Trainer(cfg, torch.device("cpu"), micro_batch=2, parallel=ParallelConfig(1, 2, 1), groups=mesh, lr=1e-2)
    assert len(tr.stage.layers) == (2 if rank == 0 else 1)   # the stage with the head gets the smaller share
    for name, p in tr.stage.store.params.items():
        p.data.copy_(ref_params[name])
    tr.opt.master.copy_(tr.opt.param_shard.float())
    tok = _data(cfg, 8)
    for step, (ref, ref_norm) in enumerate(ref_losses):
        t = tr.train_step(tok).clone()
        dist.all_reduce(t)
        assert abs(t.item() - ref) < 2e-3 * abs(ref) + 1e-4, (step, t.item(), ref)
        assert abs(tr.opt.grad_norm.item() - ref_norm) < 2e-3 * ref_norm + 1e-6


def test_layers_that_do_not_divide_over_the_stages():
    import dataclasses as dc
    from coccl_b200.train import Trainer, split_layers
    assert split_layers(32, 2) == [(0, 16), (16, 32)]
    assert split_layers(6, 4) == [(0, 2), (2, 4), (4, 5), (5, 6)]
    assert split_layers(7, 3) == [(0, 3), (3, 5), (5, 7)]
    with pytest.raises(AssertionError):
        split_layers(2, 3)
    cfg = dc.replace(_cfg(), n_layer=3)
    tr = Trainer(cfg, torch.device("cpu"), micro_batch=2, lr=1e-2)
    params = {k: v.detach().clone() for k, v in tr.stage.store.params.items()}
    tok = _data(cfg, 8)
    ref = []
    for _ in range(3):
        loss = tr.train_step(tok).item()
        ref.append((loss, tr.opt.grad_norm.item()))
    run_distributed(_uneven_worker, 2, "gloo", (ref, params))


def test_interleaved_plan_is_complete_and_ordered():
    from coccl_b200.parallel.pp import interleaved_order, plan_ticks
    for pp, chunks, n_micro in [(2, 2, 4), (2, 2, 16), (4, 2, 8), (4, 3, 12), (8, 2, 16), (2, 4, 2)]:
        ticks = plan_ticks(pp, chunks, n_micro)
        when = {}
        for t, row in enumerate(ticks):
            for r, a in enumerate(row):
                if a is not None:
                    key = (a[0], a[1] * pp + r, a[2])
                    assert key not in when
                    when[key] = t
        last = pp * chunks - 1
        assert len(when) == 2 * n_micro * pp * chunks
        for (kind, vs, m), t in when.items():
            if kind == "F" and vs > 0:
                assert when[("F", vs - 1, m)] < t
            if kind == "B":
                assert when[("F", vs, m)] < t
                if vs < last:
                    assert when[("B", vs + 1, m)] < t
        # each rank runs its passes in its own 1F1B order, and never holds more forward passes than the warm-up allows
        for r in range(pp):
            mine = [a for row in ticks for q, a in enumerate(row) if q == r and a is not None]
            assert mine == interleaved_order(pp, r, chunks, n_micro)
            live = peak = 0
            for a in mine:
                live += 1 if a[0] == "F" else -1
                peak = max(peak, live)
            assert peak <= min((pp - r - 1) * 2 + (chunks - 1) * pp, n_micro * chunks) + 1
        # the bubble: idle ticks per rank do not grow with the number of chunks (each tick is 1/chunks as long)
        idle = sum(a is None for row in ticks for a in row) / pp
        assert idle <= 2 * (pp - 1) + 1, (pp, chunks, n_micro, idle)


# ---------------------------------------------------------------------------- mixture of experts in the trainer
def _moe_cfg():
    from coccl_b200.models.gpt import GPTConfig
    return GPTConfig(n_layer=4, hidden=64, n_head=4, ffn=128, seq_len=32, vocab=128, dtype=torch.float32,
                     n_experts=4, moe_top_k=2, moe_every=2)


def _moe_reference(steps=3):
    from coccl_b200.train import Trainer
    cfg = _moe_cfg()
    tr = Trainer(cfg, torch.device("cpu"), micro_batch=2, lr=1e-2)
    params = {k: v.detach().clone() for k, v in tr.stage.store.params.items()}
    tok = _data(cfg, 8)
    out = []
    for _ in range(steps):
        out.append((tr.train_step(tok).item(), tr.opt.grad_norm.item()))
    return params, out


def _moe_worker(rank, world, pp, dp, ref_params, ref):
    import torch.distributed as dist
    from coccl_b200.parallel.mesh import Mesh
    from coccl_b200.train import ParallelConfig, Trainer
    cfg = _moe_cfg()
    mesh = Mesh(tp=1, pp=pp, dp=dp, device=torch.device("cpu"))
    tr = Trainer(cfg, torch.device("cpu"), micro_batch=2, parallel=ParallelConfig(1, pp, dp), groups=mesh, lr=1e-2)
    assert tr.stage.expert_store is None          # ep = 1: the experts are ordinary replicated parameters
    assert any(".experts.3.w_down" in n for n in tr.stage.store.params) or pp > 1
    for name, p in tr.stage.store.params.items():
        p.data.copy_(ref_params[name])
    tr.opt.master.copy_(tr.opt.param_shard.float())
    tok = _data(cfg, 8)
    per = 8 // dp
    mine = tok[mesh.dp_rank * per:(mesh.dp_rank + 1) * per]
    for step, (ref_loss, ref_norm) in enumerate(ref):
        t = tr.train_step(mine).clone()
        dist.all_reduce(t)
        assert abs(t.item() / dp - ref_loss) < 2e-3 * abs(ref_loss) + 1e-4, (step, t.item() / dp, ref_loss)
        assert abs(tr.opt.grad_norm.item() - ref_norm) < 2e-3 * ref_norm + 1e-6, (step, tr.opt.grad_norm.item(), ref_norm)


def _moe_ep_worker(rank, world, ref_params, ref, pp=1):
    """Experts spread over the data-parallel group (ep = dp = 2): tokens travel to their experts and back, the experts
    live in their own flat buffers with their own optimizer, and the run still reproduces the single-process model."""
    import torch.distributed as dist
    from coccl_b200.parallel.mesh import Mesh
    from coccl_b200.train import ParallelConfig, Trainer
    cfg = _moe_cfg()
    mesh = Mesh(tp=1, pp=pp, dp=2, ep=2, device=torch.device("cpu"))
    tr = Trainer(cfg, torch.device("cpu"), micro_batch=2, parallel=ParallelConfig(1, pp, 2, ep=2), groups=mesh, lr=1e-2)
    es = tr.stage.expert_store
    assert es is not None and len(es.params) == (2 // pp) * 2 * 3   # MoE layers of this stage x two local experts x (up, bias, down)
    assert not any(".experts." in n for n in tr.stage.store.params)
    for store in (tr.stage.store, es):
        for name, p in store.params.items():
            p.data.copy_(ref_params[name])
    tr.opt.master.copy_(tr.opt.param_shard.float())
    tr.expert_opt.master.copy_(tr.expert_opt.param_shard.float())
    tok = _data(cfg, 8)
    mine = tok[mesh.dp_rank * 4:(mesh.dp_rank + 1) * 4]
    for step, (ref_loss, ref_norm) in enumerate(ref):
        t = tr.train_step(mine).clone()
        dist.all_reduce(t)
        assert abs(t.item() / 2 - ref_loss) < 2e-3 * abs(ref_loss) + 1e-4, (step, t.item() / 2, ref_loss)
        assert abs(tr.opt.grad_norm.item() - ref_norm) < 2e-3 * ref_norm + 1e-6, (step, tr.opt.grad_norm.item(), ref_norm)
    name = next(n for n in es.params if n.endswith("w_up"))
    assert (es.params[name].detach() - ref_params[name]).abs().max().item() > 0


@pytest.mark.parametrize("pp", [1, 2])
def test_expert_parallel_matches_single_process(pp):
    params, ref = _moe_reference()
    run_distributed(_moe_ep_worker, 2 * pp, "gloo", (params, ref, pp))


def test_moe_model_trains_and_counts_its_parameters():
    from coccl_b200.models.gpt import GPTStage
    cfg = _moe_cfg()
    assert [cfg.is_moe_layer(i) for i in range(4)] == [False, True, False, True]
    stage = GPTStage(cfg, torch.device("cpu"))
    assert sum(p.numel() for p in stage.store.params.values()) == cfg.num_params()
    _, curve = _moe_reference(steps=6)
    assert curve[-1][0] < curve[0][0] - 0.05, curve


@pytest.mark.parametrize("pp,dp", [(1, 2), (2, 1), (2, 2)])
def test_moe_layouts_match_single_process(pp, dp):
    params, ref = _moe_reference()
    run_distributed(_moe_worker, pp * dp, "gloo", (pp, dp, params, ref))


def _fsdp_worker(rank, world, ref_losses, ref_params):
    """Fully sharded: a rank holds 1 / dp of every parameter, gradient and optimizer state; layers are gathered while
    they run. Same losses and gradient norms as one process, and the shards really are shards."""
    import torch.distributed as dist
    from coccl_b200.parallel.mesh import Mesh
    from coccl_b200.train import ParallelConfig, Trainer
    cfg = _cfg()
    mesh = Mesh(tp=1, pp=1, dp=world, device=torch.device("cpu"))
    tr = Trainer(cfg, torch.device("cpu"), micro_batch=2, parallel=ParallelConfig(1, 1, world, dp_strategy="fsdp"), groups=mesh, lr=1e-2)
    st = tr.stage.store
    total = sum(st.unit_size.values())
    assert st.flat_param_shard.numel() * world == total and tr.opt.master.numel() * world == total
    assert st.full[0].numel() == max(st.unit_size[u] for u in st.unit_names) < total // 2   # two layer-sized buffers, not the model
    # load the single-process model's initial weights: unit by unit through the buffers, own shard out
    for u in list(st.unit_names) + [st.OUTER]:
        buf = st._buffers(u)[0]
        for name, (unit, off, n) in st.layout.items():
            if unit == u:
                buf[off:off + n].copy_(ref_params[name].reshape(-1))
        st.param_shard(u).copy_(st._mine(buf, u))
    st.gather(st.OUTER)
    tr.opt.master.copy_(st.flat_param_shard.float())
    tok = _data(cfg, 8)
    per = 8 // world
    mine = tok[rank * per:(rank + 1) * per]
    for step, (ref, ref_norm) in enumerate(ref_losses):
        t = tr.train_step(mine).clone()
        dist.all_reduce(t)
        assert abs(t.item() / world - ref) < 2e-3 * abs(ref) + 1e-4, (step, t.item() / world, ref)
        assert abs(tr.opt.grad_norm.item() - ref_norm) < 2e-3 * ref_norm + 1e-6, (step, tr.opt.grad_norm.item(), ref_norm)


@pytest.mark.parametrize("world", [2, 4])
def test_fully_sharded_strategy_matches_single_process(world):
    tr, losses = _reference_losses()
    tr2, _ = _reference_losses(steps=0)
    params = {k: v.detach().clone() for k, v in tr2.stage.store.params.items()}
    run_distributed(_fsdp_worker, world, "gloo", (losses, params))


def test_fully_sharded_strategy_on_one_rank_is_the_plain_trainer():
    from coccl_b200.train import ParallelConfig, Trainer
    cfg = _cfg()
    tok = _data(cfg, 8)
    plain = Trainer(cfg, torch.device("cpu"), micro_batch=2, lr=1e-2)
    shard = Trainer(cfg, torch.device("cpu"), micro_batch=2, lr=1e-2, parallel=ParallelConfig(dp_strategy="fsdp"))
    for _ in range(3):
        a, b = plain.train_step(tok).item(), shard.train_step(tok).item()
        assert abs(a - b) < 1e-5 * abs(a), (a, b)
        assert abs(plain.opt.grad_norm.item() - shard.opt.grad_norm.item()) < 1e-5 * plain.opt.grad_norm.item()


def _ddp_worker(rank, world, ref_losses, ref_params):
    import torch.distributed as dist
    from coccl_b200.parallel.mesh import Mesh
    from coccl_b200.train import ParallelConfig, Trainer
    cfg = _cfg()
    mesh = Mesh(tp=1, pp=1, dp=2, device=torch.device("cpu"))
    tr = Trainer(cfg, torch.device("cpu"), micro_batch=2, parallel=ParallelConfig(1, 1, 2, dp_strategy="ddp"), groups=mesh, lr=1e-2)
    assert tr.opt.ddp and tr.opt.master.numel() == tr.stage.store.flat_param.numel()   # whole optimizer state on every rank
    for name, p in tr.stage.store.params.items():
        p.data.copy_(ref_params[name])
    tr.opt.master.copy_(tr.opt.param_shard.float())
    tok = _data(cfg, 8)
    mine = tok[mesh.dp_rank * 4:(mesh.dp_rank + 1) * 4]
    for step, (ref, ref_norm) in enumerate(ref_losses):
        t = tr.train_step(mine).clone()
        dist.all_reduce(t)
        assert abs(t.item() / 2 - ref) < 2e-3 * abs(ref) + 1e-4, (step, t.item() / 2, ref)
        assert abs(tr.opt.grad_norm.item() - ref_norm) < 2e-3 * ref_norm + 1e-6
    # the replicas stayed identical without any parameter all-gather
    mineflat = tr.stage.store.flat_param.clone()
    other = mineflat.clone()
    dist.broadcast(other, src=0)
    assert torch.equal(mineflat, other)


def test_ddp_strategy_matches_single_process():
    tr, losses = _reference_losses()
    tr2, _ = _reference_losses(steps=0)
    params = {k: v.detach().clone() for k, v in tr2.stage.store.params.items()}
    run_distributed(_ddp_worker, 2, "gloo", (losses, params))
