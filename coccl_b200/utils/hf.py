"""Bridge to Hugging Face checkpoints of the Llama / Qwen family: a model configuration from a `transformers` config,
parameter names, and loading a state dict into a (tensor- and pipeline-parallel) stage of this trainer.

The reference's launcher starts from such checkpoints (`--load` of a converted Qwen2.5 / Qwen3 model,
examples/training_scripts/train_qwen_coccl.sh:37-55, training_envs.sh:8-12). Here the names map one to one
(models/llama.py keeps q / k / v and gate / up as separate named parameters; the fused GEMM weights are views that span
them), so loading is a renaming plus the tensor-parallel slicing of utils.checkpoint.shard_param.
"""
from __future__ import annotations

import re

import torch

from ..models.gpt import GPTConfig
from .checkpoint import shard_param

_LAYER = {
    "input_layernorm.weight": "ln1.weight", "post_attention_layernorm.weight": "ln2.weight",
    "self_attn.q_proj.weight": "q.weight", "self_attn.k_proj.weight": "k.weight", "self_attn.v_proj.weight": "v.weight",
    "self_attn.q_proj.bias": "q.bias", "self_attn.k_proj.bias": "k.bias", "self_attn.v_proj.bias": "v.bias",
    "self_attn.q_norm.weight": "q_norm.weight", "self_attn.k_norm.weight": "k_norm.weight",
    "self_attn.o_proj.weight": "o.weight",
    "mlp.gate_proj.weight": "gate.weight", "mlp.up_proj.weight": "up.weight", "mlp.down_proj.weight": "down.weight",
}
_TOP = {"model.embed_tokens.weight": "wte", "model.norm.weight": "lnf.weight", "lm_head.weight": "lm_head"}


def config_from_hf(hf, *, seq_len: int | None = None, dtype=torch.bfloat16) -> GPTConfig:
    """GPTConfig(arch="llama") for a transformers LlamaConfig / Qwen2Config / Qwen3Config / Qwen3MoeConfig / MixtralConfig."""
    kind = getattr(hf, "model_type", "")
    if kind not in ("llama", "qwen2", "qwen3", "qwen3_moe", "mixtral"):
        raise ValueError(f"model type {kind!r} is not of the Llama / Qwen family")
    moe = {}
    if kind == "qwen3_moe":
        if not hf.norm_topk_prob:
            raise ValueError("the router here weighs the chosen experts by a softmax over their logits (norm_topk_prob = true)")
        if getattr(hf, "mlp_only_layers", None):
            raise ValueError("dense layers at listed positions (mlp_only_layers) are not supported; use decoder_sparse_step")
        if hf.decoder_sparse_step != 1 and hf.intermediate_size != hf.moe_intermediate_size:
            raise ValueError("dense and expert MLPs of different widths are not supported")
        moe = dict(n_experts=hf.num_experts, moe_top_k=hf.num_experts_per_tok, moe_every=hf.decoder_sparse_step)
    if kind == "mixtral":   # every layer is a mixture of experts, the chosen experts' weights are renormalised
        if getattr(hf, "sliding_window", None):
            raise ValueError("sliding-window attention is not supported")
        moe = dict(n_experts=hf.num_local_experts, moe_top_k=hf.num_experts_per_tok, moe_every=1)
    head_dim = getattr(hf, "head_dim", None) or hf.hidden_size // hf.num_attention_heads
    theta = getattr(hf, "rope_theta", None)
    rope = getattr(hf, "rope_parameters", None) or getattr(hf, "rope_scaling", None) or {}
    if theta is None:   # newer configs keep it in a dictionary
        theta = rope.get("rope_theta", 1.0e4)
    kind_of_rope = rope.get("rope_type", rope.get("type", "default")) if isinstance(rope, dict) else "default"
    if kind_of_rope not in ("default", None):
        raise ValueError(f"rotary embedding of type {kind_of_rope!r} (scaled frequencies) is not supported; plain rotary positions only")
    return GPTConfig(arch="llama", n_layer=hf.num_hidden_layers, hidden=hf.hidden_size, n_head=hf.num_attention_heads,
                     n_kv_head=getattr(hf, "num_key_value_heads", None) or hf.num_attention_heads,
                     kv_channels=0 if head_dim * hf.num_attention_heads == hf.hidden_size else head_dim,
                     ffn=hf.moe_intermediate_size if kind == "qwen3_moe" else hf.intermediate_size,
                     seq_len=seq_len or min(hf.max_position_embeddings, 2048), **moe,
                     vocab=hf.vocab_size, eps=hf.rms_norm_eps, rope_theta=float(theta),
                     qkv_bias=(kind == "qwen2") or bool(getattr(hf, "attention_bias", False)), qk_norm=kind in ("qwen3", "qwen3_moe"),
                     tie_embeddings=bool(getattr(hf, "tie_word_embeddings", False)), dtype=dtype)


def gpt2_config(hf, *, seq_len: int | None = None, dtype=torch.bfloat16) -> GPTConfig:
    """GPTConfig(arch="gpt") for a transformers GPT2Config: the same architecture as this package's GPT (pre-LayerNorm,
    learned positions, tanh-GELU MLP, tied output head)."""
    if getattr(hf, "model_type", "") != "gpt2":
        raise ValueError("not a GPT-2 configuration")
    if hf.activation_function not in ("gelu_new", "gelu_pytorch_tanh"):
        raise ValueError("this package's GPT uses the tanh form of GELU")
    return GPTConfig(n_layer=hf.n_layer, hidden=hf.n_embd, n_head=hf.n_head, ffn=hf.n_inner or 4 * hf.n_embd,
                     seq_len=seq_len or hf.n_positions, vocab=hf.vocab_size, eps=hf.layer_norm_epsilon, dtype=dtype)


def gpt2_to_local(state_dict: dict, cfg: GPTConfig) -> dict:
    """A GPT-2 state dict under this package's names and layouts. GPT-2 stores its linear layers as [in, out] and the
    fused projection as (q | k | v) x heads; here weights are [out, in] and the projection is heads x (q | k | v), so
    that a tensor-parallel rank's rows are whole heads."""
    nh, d, h = cfg.n_head, cfg.head_dim, cfg.hidden
    out = {"wte": state_dict["transformer.wte.weight"], "wpe": state_dict["transformer.wpe.weight"][:cfg.seq_len],
           "lnf.weight": state_dict["transformer.ln_f.weight"], "lnf.bias": state_dict["transformer.ln_f.bias"]}
    for i in range(cfg.n_layer):
        src, dst = f"transformer.h.{i}.", f"layers.{i}."
        for a, b in (("ln_1", "ln1"), ("ln_2", "ln2")):
            out[dst + b + ".weight"], out[dst + b + ".bias"] = state_dict[src + a + ".weight"], state_dict[src + a + ".bias"]
        w = state_dict[src + "attn.c_attn.weight"].t()                                   # [3h, h], rows (which, head, d)
        out[dst + "qkv.weight"] = w.reshape(3, nh, d, h).permute(1, 0, 2, 3).reshape(3 * h, h).contiguous()
        out[dst + "qkv.bias"] = state_dict[src + "attn.c_attn.bias"].reshape(3, nh, d).permute(1, 0, 2).reshape(3 * h).contiguous()
        out[dst + "proj.weight"] = state_dict[src + "attn.c_proj.weight"].t().contiguous()
        out[dst + "proj.bias"] = state_dict[src + "attn.c_proj.bias"]
        out[dst + "fc1.weight"] = state_dict[src + "mlp.c_fc.weight"].t().contiguous()
        out[dst + "fc1.bias"] = state_dict[src + "mlp.c_fc.bias"]
        out[dst + "fc2.weight"] = state_dict[src + "mlp.c_proj.weight"].t().contiguous()
        out[dst + "fc2.bias"] = state_dict[src + "mlp.c_proj.bias"]
    return out


def load_local(stage, local: dict, *, tp_rank: int = 0, tp_size: int = 1) -> list[str]:
    """Copy parameters given under this package's names (whole, tensor-parallel size 1) into the ones `stage` holds."""
    params, seen = stage.store.params, set()
    with torch.no_grad():
        for name, value in local.items():
            if name in params:
                piece = shard_param(name, value, tp_rank, tp_size)
                if tuple(piece.shape) != tuple(params[name].shape):
                    raise ValueError(f"{name}: shape {tuple(piece.shape)} does not fit {tuple(params[name].shape)}")
                params[name].copy_(piece.to(params[name].dtype))
                seen.add(name)
    return sorted(n for n in params if n not in seen)


def split_experts(state_dict: dict) -> dict:
    """Mixture-of-experts checkpoints keep all experts of a layer in two tensors (gate_up_proj [experts, 2 * width,
    hidden] with the gate rows first, down_proj [experts, hidden, width]); this package names every expert's three
    matrices. Returns the state dict with those tensors replaced by per-expert entries under Hugging Face style names
    that `rename` understands; the router (`mlp.gate.weight`) keeps its name."""
    out = {}
    for k, v in state_dict.items():
        m = re.match(r"(model\.layers\.\d+\.mlp\.experts)\.(gate_up_proj|down_proj)$", k)
        if not m:
            out[k] = v
            continue
        for e in range(v.shape[0]):
            if m.group(2) == "gate_up_proj":
                half = v.shape[1] // 2
                out[f"{m.group(1)}.{e}.gate_proj.weight"] = v[e, :half]
                out[f"{m.group(1)}.{e}.up_proj.weight"] = v[e, half:]
            else:
                out[f"{m.group(1)}.{e}.down_proj.weight"] = v[e]
    return out


def rename(hf_name: str) -> str | None:
    """This package's name of a Hugging Face parameter (None: a buffer that is not a parameter here)."""
    if hf_name in _TOP:
        return _TOP[hf_name]
    m = re.match(r"model\.layers\.(\d+)\.mlp\.experts\.(\d+)\.(gate|up|down)_proj\.weight$", hf_name)
    if m:
        return f"layers.{m.group(1)}.experts.{m.group(2)}.{m.group(3)}.weight"
    m = re.match(r"model\.layers\.(\d+)\.mlp\.gate\.weight$", hf_name)
    if m:
        return f"layers.{m.group(1)}.router.weight"
    m = re.match(r"model\.layers\.(\d+)\.(.+)$", hf_name)
    if m and m.group(2) in _LAYER:
        return f"layers.{m.group(1)}.{_LAYER[m.group(2)]}"
    return None


def load_state_dict(stage, state_dict: dict, *, tp_rank: int = 0, tp_size: int = 1) -> list[str]:
    """Copy a Hugging Face state dict into the parameters `stage` holds (a pipeline stage takes its own layers, a
    tensor-parallel rank its own slices). Returns the names of the stage's parameters that the state dict did not
    provide; a tensor whose shape does not fit is an error."""
    params = dict(stage.store.params)
    if getattr(stage, "expert_store", None) is not None:
        params.update(stage.expert_store.params)      # this rank's experts under expert parallelism
    seen = set()
    with torch.no_grad():
        for hf_name, value in split_experts(state_dict).items():
            name = rename(hf_name)
            if name == "lm_head" and stage.cfg.tie_embeddings:
                continue
            if name is None or name not in params:
                continue
            piece = shard_param(name, value, tp_rank, tp_size)
            if tuple(piece.shape) != tuple(params[name].shape):
                raise ValueError(f"{hf_name}: shape {tuple(piece.shape)} does not fit {name} {tuple(params[name].shape)}")
            params[name].copy_(piece.to(params[name].dtype))
            seen.add(name)
    return sorted(n for n in params if n not in seen)


def export_state_dict(stages, cfg: GPTConfig) -> dict:
    """The opposite direction for unsharded stages (tensor-parallel size 1): Hugging Face names for the parameters of
    the given pipeline stages."""
    back = {v: k for k, v in _LAYER.items()}
    top = {v: k for k, v in _TOP.items()}
    out = {}
    for stage in stages:
        for name, p in stage.store.params.items():
            m = re.match(r"layers\.(\d+)\.(.+)$", name)
            if m:
                out[f"model.layers.{m.group(1)}.{back[m.group(2)]}"] = p.detach().clone()
            elif name in top:
                out[top[name]] = p.detach().clone()
    if cfg.tie_embeddings and "model.embed_tokens.weight" in out:
        out["lm_head.weight"] = out["model.embed_tokens.weight"]
    return out


def local_to_gpt2(params: dict, cfg: GPTConfig) -> dict:
    """The opposite of gpt2_to_local: this package's GPT parameters (whole, tensor-parallel size 1) under GPT-2's names
    and layouts."""
    nh, d, h = cfg.n_head, cfg.head_dim, cfg.hidden
    out = {"transformer.wte.weight": params["wte"], "transformer.wpe.weight": params["wpe"],
           "transformer.ln_f.weight": params["lnf.weight"], "transformer.ln_f.bias": params["lnf.bias"], "lm_head.weight": params["wte"]}
    for i in range(cfg.n_layer):
        src, dst = f"layers.{i}.", f"transformer.h.{i}."
        for a, b in (("ln1", "ln_1"), ("ln2", "ln_2")):
            out[dst + b + ".weight"], out[dst + b + ".bias"] = params[src + a + ".weight"], params[src + a + ".bias"]
        w = params[src + "qkv.weight"].reshape(nh, 3, d, h).permute(1, 0, 2, 3).reshape(3 * h, h)     # rows (which, head, d)
        out[dst + "attn.c_attn.weight"] = w.t().contiguous()
        out[dst + "attn.c_attn.bias"] = params[src + "qkv.bias"].reshape(nh, 3, d).permute(1, 0, 2).reshape(3 * h).contiguous()
        out[dst + "attn.c_proj.weight"] = params[src + "proj.weight"].t().contiguous()
        out[dst + "attn.c_proj.bias"] = params[src + "proj.bias"]
        out[dst + "mlp.c_fc.weight"] = params[src + "fc1.weight"].t().contiguous()
        out[dst + "mlp.c_fc.bias"] = params[src + "fc1.bias"]
        out[dst + "mlp.c_proj.weight"] = params[src + "fc2.weight"].t().contiguous()
        out[dst + "mlp.c_proj.bias"] = params[src + "fc2.bias"]
    return {k: v.detach().clone() for k, v in out.items()}


def hf_config(cfg: GPTConfig):
    """A transformers configuration for `cfg` (dense models: GPT-2, Llama, Qwen2, Qwen3 by their distinguishing marks)."""
    import transformers
    if cfg.n_experts:
        raise ValueError("export covers dense models")
    if cfg.arch == "gpt":
        return transformers.GPT2Config(vocab_size=cfg.vocab, n_positions=cfg.seq_len, n_embd=cfg.hidden, n_layer=cfg.n_layer,
                                       n_head=cfg.n_head, n_inner=cfg.ffn, activation_function="gelu_new",
                                       layer_norm_epsilon=cfg.eps, resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
    common = dict(vocab_size=cfg.vocab, hidden_size=cfg.hidden, intermediate_size=cfg.ffn, num_hidden_layers=cfg.n_layer,
                  num_attention_heads=cfg.n_head, num_key_value_heads=cfg.kv_heads, max_position_embeddings=cfg.seq_len,
                  rms_norm_eps=cfg.eps, rope_theta=cfg.rope_theta, tie_word_embeddings=cfg.tie_embeddings)
    if cfg.qk_norm:
        return transformers.Qwen3Config(head_dim=cfg.head_dim, attention_bias=cfg.qkv_bias, **common)
    if cfg.kv_channels:
        raise ValueError("a head width other than hidden / heads needs a configuration with head_dim (Qwen3)")
    if cfg.qkv_bias:
        return transformers.Qwen2Config(**common)
    return transformers.LlamaConfig(attention_bias=False, **common)


def export_pretrained(stage, directory: str) -> None:
    """Write the parameters of an unsharded single-stage model as a Hugging Face checkpoint (`save_pretrained`)."""
    import transformers
    cfg = stage.cfg
    assert stage.pre and stage.post and stage.tp.size == 1 and not getattr(stage, "fsdp", False), \
        "export needs the whole model in one stage (tensor- and pipeline-parallel size 1)"
    conf = hf_config(cfg)
    model = transformers.AutoModelForCausalLM.from_config(conf)
    sd = local_to_gpt2(stage.store.params, cfg) if cfg.arch == "gpt" else export_state_dict([stage], cfg)
    missing = model.load_state_dict({k: v.float() for k, v in sd.items()}, strict=False)
    left = [k for k in missing.missing_keys if "inv_freq" not in k and "rotary" not in k and not k.endswith(".attn.bias")
            and not k.endswith("masked_bias")]
    if left or missing.unexpected_keys:
        raise RuntimeError(f"export does not match the transformers model: missing {left[:4]}, unexpected {missing.unexpected_keys[:4]}")
    model.to(cfg.dtype).save_pretrained(directory, safe_serialization=True)
