"""The Llama / Qwen family and the fully sharded strategy on one GPU (bf16, tcgen05 GEMMs): the first loss agrees with the fp32 CPU
model built from the same parameters, and training lowers it. Runs last in the suite."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("moe", [False, True], ids=["dense", "experts"])
def test_first_loss_matches_cpu_and_training_lowers_it(moe):
    from coccl_b200.models.gpt import GPTConfig, GPTStage
    from coccl_b200.train import Trainer
    kw = dict(arch="llama", n_layer=2, hidden=512, n_head=8, n_kv_head=2, ffn=1536, seq_len=256, vocab=8192, qkv_bias=True,
              qk_norm=True, tie_embeddings=False, rope_theta=1.0e4)
    if moe:
        kw.update(ffn=512, n_experts=4, moe_top_k=2, moe_every=1, qkv_bias=False)
    dev = torch.device("cuda", 0)
    tr = Trainer(GPTConfig(**kw), dev, micro_batch=2, lr=1e-3)
    ids = (torch.arange(8 * 257) * 7) % 8192          # every id determines its successor
    tok = ids.view(8, 257).pin_memory()
    cpu = GPTStage(GPTConfig(dtype=torch.float32, **kw), torch.device("cpu"))
    for name, p in cpu.store.params.items():
        p.data.copy_(tr.stage.store.params[name].detach().float().cpu())
    with torch.no_grad():
        want = sum(cpu(tok[i:i + 2, :-1], tok[i:i + 2, 1:], 1.0 / (8 * 256)).item() for i in range(0, 8, 2))
    losses = [tr.train_step(tok).item() for _ in range(8)]
    tr.check_health()
    assert abs(losses[0] - want) < 2e-2 * want, (losses[0], want)
    assert all(l == l for l in losses) and losses[-1] < losses[0] - 1.0, losses
    held = tr.eval_step(tok).item()
    assert held < losses[0]


def test_fully_sharded_strategy_on_one_gpu_equals_the_plain_trainer():
    """One rank: the sharded store's gather / reduce-scatter points, the buffers that take turns and the sharded AdamW
    run on the GPU and must reproduce the plain trainer (same kernels, same order of operations)."""
    from coccl_b200.models.gpt import GPTConfig
    from coccl_b200.train import ParallelConfig, Trainer
    cfg = GPTConfig(n_layer=4, hidden=512, n_head=8, ffn=2048, seq_len=256, vocab=8192)
    dev = torch.device("cuda", 0)
    tok = torch.randint(0, cfg.vocab, (4, cfg.seq_len + 1), generator=torch.Generator().manual_seed(2)).pin_memory()
    plain = Trainer(cfg, dev, micro_batch=2, lr=1e-3)
    shard = Trainer(cfg, dev, micro_batch=2, lr=1e-3, parallel=ParallelConfig(dp_strategy="fsdp"))
    for step in range(4):
        a, b = plain.train_step(tok).item(), shard.train_step(tok).item()
        assert abs(a - b) < 2e-3 * abs(a), (step, a, b)
        na, nb = plain.opt.grad_norm.item(), shard.opt.grad_norm.item()
        assert abs(na - nb) < 2e-3 * na, (step, na, nb)
    plain.check_health()
