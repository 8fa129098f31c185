"""The model families against Hugging Face transformers on CPU: a randomly initialised tiny GPT2LMHeadModel, LlamaForCausalLM /
Qwen2ForCausalLM / Qwen3ForCausalLM is loaded into this package's stage through utils/hf.py, and both must give the
same loss and the same gradients."""
import pytest
import torch
import torch.nn.functional as F

transformers = pytest.importorskip("transformers")


def _hf_model(kind):
    common = dict(vocab_size=128, hidden_size=64, intermediate_size=160, num_hidden_layers=3, num_attention_heads=4,
                  num_key_value_heads=2, max_position_embeddings=64, rms_norm_eps=1e-5, tie_word_embeddings=False)
    torch.manual_seed(0)
    if kind == "llama":
        cfg = transformers.LlamaConfig(rope_theta=10000.0, attention_bias=False, **common)
        return transformers.LlamaForCausalLM(cfg)
    if kind == "qwen2":
        cfg = transformers.Qwen2Config(rope_theta=1.0e6, **common)
        return transformers.Qwen2ForCausalLM(cfg)
    cfg = transformers.Qwen3Config(rope_theta=1.0e6, head_dim=32, **common)   # heads wider than hidden / heads, as Qwen3
    return transformers.Qwen3ForCausalLM(cfg)


@pytest.mark.parametrize("kind", ["llama", "qwen2", "qwen3"])
def test_loss_and_gradients_equal_transformers(kind):
    from coccl_b200.models.gpt import GPTStage
    from coccl_b200.utils import hf
    model = _hf_model(kind).float().train()
    with torch.no_grad():   # norms and biases away from their trivial initial values
        for n, p in model.named_parameters():
            if "norm" in n or n.endswith(".bias"):
                p.add_(torch.randn_like(p) * 0.1)
    cfg = hf.config_from_hf(model.config, seq_len=32, dtype=torch.float32)
    assert cfg.qkv_bias == (kind == "qwen2") and cfg.qk_norm == (kind == "qwen3") and cfg.kv_heads == 2
    stage = GPTStage(cfg, torch.device("cpu"))
    assert hf.load_state_dict(stage, model.state_dict()) == []
    assert cfg.num_params() == sum(p.numel() for p in model.parameters())
    g = torch.Generator().manual_seed(3)
    tok = torch.randint(0, cfg.vocab, (2, cfg.seq_len + 1), generator=g)
    inp, tgt = tok[:, :-1], tok[:, 1:]
    loss = stage(inp, tgt, 1.0)
    logits = model(input_ids=inp).logits
    ref = F.cross_entropy(logits.reshape(-1, cfg.vocab), tgt.reshape(-1), reduction="sum")
    assert abs(loss.item() - ref.item()) < 2e-4 * abs(ref.item()), (loss.item(), ref.item())
    # gradients: this package accumulates them in main_grad
    stage.zero_grad_buffer()
    loss.backward()
    stage.post_backward_sync_autograd_grads()
    ref.backward()
    theirs = {hf.rename(n): p.grad for n, p in model.named_parameters()}
    for name, p in stage.store.params.items():
        a, b = p.main_grad, theirs[name]
        assert torch.allclose(a, b, atol=2e-4 * b.abs().max().item() + 1e-6), (name, (a - b).abs().max().item(), b.abs().max().item())
    # and back: the exported names load into a fresh transformers model
    fresh = _hf_model(kind).float()
    missing = fresh.load_state_dict(hf.export_state_dict([stage], cfg), strict=False)
    assert not missing.unexpected_keys and all("rotary" in k or "inv_freq" in k for k in missing.missing_keys)
    assert torch.allclose(fresh(input_ids=inp).logits, logits.detach(), atol=1e-5)


def test_tensor_parallel_slices_of_a_checkpoint():
    from coccl_b200.models.gpt import GPTStage
    from coccl_b200.utils import hf

    class TP:   # the sizes only: parameters are created per rank, nothing is exchanged
        def __init__(self, rank):
            self.size, self.rank, self.sequence_parallel = 2, rank, False

    model = _hf_model("qwen2").float()
    cfg = hf.config_from_hf(model.config, seq_len=32, dtype=torch.float32)
    sd = model.state_dict()
    stages = [GPTStage(cfg, torch.device("cpu"), tp=TP(r)) for r in range(2)]
    for r, st in enumerate(stages):
        assert hf.load_state_dict(st, sd, tp_rank=r, tp_size=2) == []
    q = torch.cat([st.store.params["layers.1.q.weight"] for st in stages], 0)
    assert torch.equal(q, sd["model.layers.1.self_attn.q_proj.weight"])
    down = torch.cat([st.store.params["layers.2.down.weight"] for st in stages], 1)
    assert torch.equal(down, sd["model.layers.2.mlp.down_proj.weight"])
    assert torch.equal(stages[1].store.params["layers.0.ln1.weight"], sd["model.layers.0.input_layernorm.weight"])
    with pytest.raises(ValueError):
        hf.load_state_dict(stages[0], sd, tp_rank=0, tp_size=1)


def test_launcher_starts_from_a_hugging_face_checkpoint(tmp_path, capsys):
    import json
    from coccl_b200.pretrain import main
    model = _hf_model("qwen2").float()
    model.save_pretrained(tmp_path / "ckpt", safe_serialization=True)
    tok = torch.randint(0, 128, (4000,), generator=torch.Generator().manual_seed(1)).numpy().astype("<u2")
    tok.tofile(tmp_path / "tokens.bin")
    main(["--hf-model", str(tmp_path / "ckpt"), "--seq-len", "32", "--device", "cpu", "--steps", "1", "--log-interval", "1",
          "--global-batch", "4", "--data", str(tmp_path / "tokens.bin"), "--lr", "0", "--min-lr", "0", "--warmup-steps", "0"])
    out = capsys.readouterr().out
    assert "loaded weights from" in out
    rec = [json.loads(l) for l in out.splitlines() if l.startswith("{") and '"step"' in l][0]
    # the first step's loss is the checkpoint's loss on that batch
    from coccl_b200.utils.data import BatchLoader, TokenFile
    loader = BatchLoader(TokenFile(str(tmp_path / "tokens.bin")), seq_len=32, global_batch=4, seed=1234, pin=False)
    batch = loader.next().clone()
    loader.close()
    logits = model(input_ids=batch[:, :-1]).logits
    ref = F.cross_entropy(logits.reshape(-1, 128), batch[:, 1:].reshape(-1)).item()
    assert abs(rec["loss"] - ref) < 1e-3 * ref, (rec, ref)


def test_gpt_equals_transformers_gpt2():
    """The benchmark's model family: this package's GPT is GPT-2's architecture, so a GPT2LMHeadModel loaded through
    utils/hf.py must give the same loss and gradients."""
    from coccl_b200.models.gpt import GPTStage
    from coccl_b200.utils import hf
    torch.manual_seed(0)
    hf_cfg = transformers.GPT2Config(vocab_size=128, n_positions=32, n_embd=64, n_layer=3, n_head=4, activation_function="gelu_new",
                                     resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
    model = transformers.GPT2LMHeadModel(hf_cfg).float().train()
    with torch.no_grad():
        for n, p in model.named_parameters():
            if "ln_" in n or n.endswith(".bias"):
                p.add_(torch.randn_like(p) * 0.1)
    cfg = hf.gpt2_config(hf_cfg, dtype=torch.float32)
    stage = GPTStage(cfg, torch.device("cpu"))
    local = hf.gpt2_to_local(model.state_dict(), cfg)
    assert hf.load_local(stage, local) == []
    assert cfg.num_params() == sum(p.numel() for p in model.parameters())
    tok = torch.randint(0, cfg.vocab, (2, cfg.seq_len + 1), generator=torch.Generator().manual_seed(3))
    inp, tgt = tok[:, :-1], tok[:, 1:]
    loss = stage(inp, tgt, 1.0)
    logits = model(input_ids=inp).logits
    ref = F.cross_entropy(logits.reshape(-1, cfg.vocab), tgt.reshape(-1), reduction="sum")
    assert abs(loss.item() - ref.item()) < 2e-4 * abs(ref.item()), (loss.item(), ref.item())
    stage.zero_grad_buffer()
    loss.backward()
    stage.post_backward_sync_autograd_grads()
    ref.backward()
    theirs = hf.gpt2_to_local({n: p.grad for n, p in model.named_parameters()} | {"lm_head.weight": None}, cfg)
    for name, p in stage.store.params.items():
        a, b = p.main_grad, theirs[name]
        assert torch.allclose(a, b, atol=2e-4 * b.abs().max().item() + 1e-6), (name, (a - b).abs().max().item())


@pytest.mark.parametrize("kind", ["qwen3_moe", "mixtral"])
def test_mixture_of_experts_equals_transformers(kind):
    from coccl_b200.models.gpt import GPTStage
    from coccl_b200.utils import hf
    torch.manual_seed(0)
    common = dict(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                  num_key_value_heads=2, max_position_embeddings=64, num_experts_per_tok=2, tie_word_embeddings=False,
                  rope_theta=1.0e6, rms_norm_eps=1e-5, router_aux_loss_coef=0.0, output_router_logits=False)
    if kind == "qwen3_moe":
        hf_cfg = transformers.Qwen3MoeConfig(moe_intermediate_size=96, head_dim=16, num_experts=4, norm_topk_prob=True,
                                             decoder_sparse_step=1, mlp_only_layers=[], **common)
        model = transformers.Qwen3MoeForCausalLM(hf_cfg)
    else:
        hf_cfg = transformers.MixtralConfig(num_local_experts=4, sliding_window=None, **common)
        model = transformers.MixtralForCausalLM(hf_cfg)
    model = model.float().train()
    with torch.no_grad():   # the expert tensors and the router start uninitialised / zero
        for n, p in model.named_parameters():
            if "experts" in n or n.endswith("mlp.gate.weight"):
                p.copy_(torch.randn_like(p) * 0.05)
            if "norm" in n:
                p.add_(torch.randn_like(p) * 0.1)
    cfg = hf.config_from_hf(hf_cfg, seq_len=32, dtype=torch.float32)
    assert (cfg.n_experts, cfg.moe_top_k, cfg.moe_every, cfg.qk_norm, cfg.ffn) == (4, 2, 1, kind == "qwen3_moe", 96)
    stage = GPTStage(cfg, torch.device("cpu"))
    assert hf.load_state_dict(stage, model.state_dict()) == []
    assert cfg.num_params() == sum(p.numel() for p in model.parameters())
    tok = torch.randint(0, cfg.vocab, (2, cfg.seq_len + 1), generator=torch.Generator().manual_seed(3))
    inp, tgt = tok[:, :-1], tok[:, 1:]
    loss = stage(inp, tgt, 1.0)
    logits = model(input_ids=inp).logits
    ref = F.cross_entropy(logits.reshape(-1, cfg.vocab), tgt.reshape(-1), reduction="sum")
    assert abs(loss.item() - ref.item()) < 2e-4 * abs(ref.item()), (loss.item(), ref.item())
    stage.zero_grad_buffer()
    loss.backward()
    stage.post_backward_sync_autograd_grads()
    ref.backward()
    theirs = {hf.rename(k): v for k, v in hf.split_experts({n: p.grad for n, p in model.named_parameters()}).items()}
    for name, p in stage.store.params.items():
        a, b = p.main_grad, theirs[name]
        assert torch.allclose(a, b, atol=3e-4 * b.abs().max().item() + 1e-6), (name, (a - b).abs().max().item(), b.abs().max().item())


@pytest.mark.parametrize("model", ["gpt-tiny", "llama-tiny"])
def test_trained_weights_leave_as_a_hugging_face_checkpoint(tmp_path, capsys, model):
    """Train a few steps here, export, load with transformers: its loss on a batch equals this package's."""
    from coccl_b200.models.gpt import GPTStage
    from coccl_b200.pretrain import main
    from coccl_b200.utils import hf
    out = tmp_path / "exported"
    main(["--model", model, "--hidden", "64", "--heads", "4", "--ffn", "128", "--seq-len", "32", "--vocab", "128", "--layers", "2",
          "--device", "cpu", "--steps", "3", "--lr", "1e-2", "--global-batch", "4", "--export-hf", str(out)] +
         (["--kv-heads", "2"] if model == "llama-tiny" else []))
    assert "exported to" in capsys.readouterr().out
    theirs = transformers.AutoModelForCausalLM.from_pretrained(out).float().eval()
    if model == "gpt-tiny":
        cfg = hf.gpt2_config(theirs.config, dtype=torch.float32)
        stage = GPTStage(cfg, torch.device("cpu"))
        assert hf.load_local(stage, hf.gpt2_to_local(theirs.state_dict(), cfg)) == []
    else:
        cfg = hf.config_from_hf(theirs.config, seq_len=32, dtype=torch.float32)
        stage = GPTStage(cfg, torch.device("cpu"))
        assert hf.load_state_dict(stage, theirs.state_dict()) == []
    tok = torch.randint(0, 128, (2, 33), generator=torch.Generator().manual_seed(5))
    ours = stage(tok[:, :-1], tok[:, 1:], 1.0).item()
    ref = F.cross_entropy(theirs(input_ids=tok[:, :-1]).logits.reshape(-1, 128), tok[:, 1:].reshape(-1), reduction="sum").item()
    assert abs(ours - ref) < 1e-3 * abs(ref), (ours, ref)
    # and the exported model is the TRAINED one, not a fresh initialisation
    fresh = GPTStage(cfg, torch.device("cpu"))
    assert (fresh.store.params["layers.0.ln1.weight"] - stage.store.params["layers.0.ln1.weight"]).abs().max().item() > 1e-4
