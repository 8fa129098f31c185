"""The Llama / Qwen model family in the trainer (models/llama.py) on CPU: the layer against a plain PyTorch restatement,
the RMSNorm function against torch's, and every parallel layout against the single-process run."""
import dataclasses
import math

import pytest
import torch
import torch.nn.functional as F

from dist_utils import run_distributed


def _cfg(**kw):
    from coccl_b200.models.gpt import GPTConfig
    base = dict(arch="llama", n_layer=4, hidden=64, n_head=4, n_kv_head=2, ffn=128, seq_len=32, vocab=128, dtype=torch.float32,
                qkv_bias=True, qk_norm=True, tie_embeddings=False, rope_theta=10000.0)
    base.update(kw)
    return GPTConfig(**base)


def _data(cfg, n_seq):
    g = torch.Generator().manual_seed(7)
    return torch.randint(0, cfg.vocab, (n_seq, cfg.seq_len + 1), generator=g)


def test_rms_norm_function_matches_torch():
    from coccl_b200.models.llama import rms_norm
    torch.manual_seed(0)
    x = torch.randn(6, 5, 16, dtype=torch.float64, requires_grad=True)
    w = (torch.rand(16, dtype=torch.float64) + 0.5).requires_grad_(True)
    y = rms_norm(x, w, 1e-6)
    ref = F.rms_norm(x, (16,), w, 1e-6)
    assert torch.allclose(y, ref, atol=1e-12)
    g = torch.randn_like(y)
    dx, dw = torch.autograd.grad(y, (x, w), g)
    rx, rw = torch.autograd.grad(ref, (x, w), g)
    assert torch.allclose(dx, rx, atol=1e-10) and torch.allclose(dw, rw, atol=1e-10)
    # with a main_grad buffer the weight gradient accumulates there, in the buffer's precision
    w2 = w.detach().clone().requires_grad_(True)
    w2.main_grad = torch.ones(16, dtype=torch.float64)
    rms_norm(x.detach(), w2, 1e-6).backward(g)
    assert w2.grad is None and torch.allclose(w2.main_grad - 1.0, rw, atol=1e-10)


def _plain_llama_forward(cfg, p, tokens):
    """The same model written directly: complex-number rotary embedding, explicit grouped-query attention."""
    b, s = tokens.shape
    h, d, nh, nkv = cfg.hidden, cfg.head_dim, cfg.n_head, cfg.kv_heads
    x = p["wte"][tokens]                                                   # [b, s, h]
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, d, 2, dtype=torch.float64) / d))
    ang = torch.arange(s, dtype=torch.float64)[:, None] * inv[None, :]
    rot = torch.polar(torch.ones_like(ang), ang)                           # [s, d / 2]

    def rope(t):                                                           # t [b, s, heads, d]; pairs (i, i + d / 2)
        z = torch.complex(t[..., :d // 2].double(), t[..., d // 2:].double()) * rot[None, :, None, :]
        return torch.cat([z.real, z.imag], -1).to(t.dtype)

    mask = torch.full((s, s), float("-inf")).triu(1)
    for i in range(cfg.n_layer):
        pre = f"layers.{i}."
        y = F.rms_norm(x, (h,), p[pre + "ln1.weight"], cfg.eps)
        q = (y @ p[pre + "q.weight"].t() + p[pre + "q.bias"]).view(b, s, nh, d)
        k = (y @ p[pre + "k.weight"].t() + p[pre + "k.bias"]).view(b, s, nkv, d)
        v = (y @ p[pre + "v.weight"].t() + p[pre + "v.bias"]).view(b, s, nkv, d)
        if cfg.qk_norm:
            q, k = F.rms_norm(q, (d,), p[pre + "q_norm.weight"], cfg.eps), F.rms_norm(k, (d,), p[pre + "k_norm.weight"], cfg.eps)
        q, k = rope(q), rope(k)
        outs = []
        for hd in range(nh):
            kk, vv = k[:, :, hd // (nh // nkv)], v[:, :, hd // (nh // nkv)]
            att = torch.softmax(q[:, :, hd] @ kk.transpose(1, 2) / math.sqrt(d) + mask, -1)
            outs.append(att @ vv)
        x = x + torch.cat(outs, -1) @ p[pre + "o.weight"].t()
        y = F.rms_norm(x, (h,), p[pre + "ln2.weight"], cfg.eps)
        x = x + (F.silu(y @ p[pre + "gate.weight"].t()) * (y @ p[pre + "up.weight"].t())) @ p[pre + "down.weight"].t()
    logits = F.rms_norm(x, (h,), p["lnf.weight"], cfg.eps) @ p["lm_head"].t()
    return logits


def test_model_equals_a_plain_restatement():
    from coccl_b200.models.gpt import GPTStage
    cfg = _cfg()
    stage = GPTStage(cfg, torch.device("cpu"))
    p = {k: v.detach() for k, v in stage.store.params.items()}
    for name in p:     # biases and norm weights away from their trivial initial values
        if name.endswith(".bias") or ".ln" in name or name.startswith("lnf") or "_norm" in name:
            p[name].add_(torch.randn_like(p[name]) * 0.1)
    tok = _data(cfg, 2)
    inp, tgt = tok[:, :-1], tok[:, 1:]
    loss = stage(inp, tgt, 1.0)
    logits = _plain_llama_forward(cfg, p, inp)
    ref = F.cross_entropy(logits.reshape(-1, cfg.vocab), tgt.reshape(-1), reduction="sum")
    assert abs(loss.item() - ref.item()) < 1e-3 * abs(ref.item()), (loss.item(), ref.item())
    assert cfg.num_params() == sum(v.numel() for v in p.values())


def _reference(cfg, steps=3, n_seq=8):
    from coccl_b200.train import Trainer
    tr = Trainer(cfg, torch.device("cpu"), micro_batch=2, lr=1e-2)
    params = {k: v.detach().clone() for k, v in tr.stage.store.params.items()}
    tok = _data(cfg, n_seq)
    out = []
    for _ in range(steps):
        loss = tr.train_step(tok).item()
        out.append((loss, tr.opt.grad_norm.item()))
    return params, out


def _worker(rank, world, tp, pp, dp, cp, chunks, strategy, ref, ref_params):
    import torch.distributed as dist
    from coccl_b200.parallel.mesh import Mesh
    from coccl_b200.train import ParallelConfig, Trainer
    from coccl_b200.utils.checkpoint import shard_param
    cfg = _cfg()
    mesh = Mesh(tp=tp, pp=pp, dp=dp, cp=cp, device=torch.device("cpu"))
    tr = Trainer(cfg, torch.device("cpu"), micro_batch=2, groups=mesh, lr=1e-2,
                 parallel=ParallelConfig(tp, pp, dp, cp=cp, virtual_stages=chunks, dp_strategy=strategy))
    st = tr.stage.store
    if strategy == "fsdp":
        for u in list(st.unit_names) + [st.OUTER]:
            buf = st._buffers(u)[0]
            for name, (unit, off, n) in st.layout.items():
                if unit == u:
                    buf[off:off + n].copy_(ref_params[name].reshape(-1))
            st.param_shard(u).copy_(st._mine(buf, u))
        st.gather(st.OUTER)
        tr.opt.master.copy_(st.flat_param_shard.float())
    else:
        for name, p in st.params.items():
            p.data.copy_(shard_param(name, ref_params[name], mesh.tp_rank, tp))
        tr.opt.master.copy_(tr.opt.param_shard.float())
    tok = _data(cfg, 8)
    per = 8 // dp
    mine = tok[mesh.dp_rank * per:(mesh.dp_rank + 1) * per]
    for step, (ref_loss, ref_norm) in enumerate(ref):
        t = tr.train_step(mine).clone()
        dist.all_reduce(t)
        total = t.item() / (tp * dp)
        assert abs(total - ref_loss) < 2e-3 * abs(ref_loss) + 1e-4, (step, total, ref_loss)
        assert abs(tr.opt.grad_norm.item() - ref_norm) < 2e-3 * ref_norm + 1e-6, (step, tr.opt.grad_norm.item(), ref_norm)


@pytest.mark.parametrize("tp,pp,dp,cp,chunks,strategy", [
    (2, 1, 1, 1, 1, "zero1"), (1, 1, 1, 2, 1, "zero1"), (2, 2, 1, 1, 2, "zero1"), (1, 1, 2, 1, 1, "fsdp")])
def test_parallel_layouts_match_single_process(tp, pp, dp, cp, chunks, strategy):
    params, ref = _reference(_cfg())
    run_distributed(_worker, tp * pp * dp * cp, "gloo", (tp, pp, dp, cp, chunks, strategy, ref, params))


def test_training_lowers_the_loss_on_structured_tokens():
    from coccl_b200.train import Trainer
    cfg = _cfg(n_layer=2)
    tr = Trainer(cfg, torch.device("cpu"), micro_batch=2, lr=3e-3)
    ids = (torch.arange(8 * 33) * 7) % cfg.vocab
    tok = ids.view(8, 33)
    losses = [tr.train_step(tok).item() for _ in range(12)]
    assert losses[-1] < losses[0] - 0.5, losses


# ---------------------------------------------------------------------------- mixture of experts in the family
def _moe_cfg():
    return _cfg(n_layer=2, n_experts=4, moe_top_k=2, moe_every=1, qkv_bias=False)


def _moe_ep_worker(rank, world, ref, ref_params):
    import torch.distributed as dist
    from coccl_b200.parallel.mesh import Mesh
    from coccl_b200.train import ParallelConfig, Trainer
    cfg = _moe_cfg()
    mesh = Mesh(tp=1, pp=1, dp=2, ep=2, device=torch.device("cpu"))
    tr = Trainer(cfg, torch.device("cpu"), micro_batch=2, parallel=ParallelConfig(1, 1, 2, ep=2), groups=mesh, lr=1e-2)
    es = tr.stage.expert_store
    assert es is not None and len(es.params) == 2 * 2 * 3 and not any(".experts." in n for n in tr.stage.store.params)
    for store in (tr.stage.store, es):
        for name, p in store.params.items():
            p.data.copy_(ref_params[name])
    tr.opt.master.copy_(tr.opt.param_shard.float())
    tr.expert_opt.master.copy_(tr.expert_opt.param_shard.float())
    tok = _data(cfg, 8)
    mine = tok[rank * 4:(rank + 1) * 4]
    for step, (ref_loss, ref_norm) in enumerate(ref):
        t = tr.train_step(mine).clone()
        dist.all_reduce(t)
        assert abs(t.item() / 2 - ref_loss) < 2e-3 * abs(ref_loss) + 1e-4, (step, t.item() / 2, ref_loss)
        assert abs(tr.opt.grad_norm.item() - ref_norm) < 2e-3 * ref_norm + 1e-6, (step, tr.opt.grad_norm.item(), ref_norm)


def test_mixture_of_experts_with_expert_parallelism_matches_single_process():
    params, ref = _reference(_moe_cfg())
    run_distributed(_moe_ep_worker, 2, "gloo", (ref, params))
