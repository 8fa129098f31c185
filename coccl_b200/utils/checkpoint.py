"""Checkpoint / resume and tensor-parallel re-sharding helpers.

The reference keeps no training state (its launcher only toggles the external
trainer's --save, examples/training_scripts/train_qwen_coccl.sh:37-55); the only
state inside the library is the SDP4Bit delta codec's previous parameters, which
re-seed themselves after a restart (sdp4bit_quan.cu:29-52). Here every rank saves
its own shard (bf16 params of its stage, fp32 master/Adam shard, step, RNG) plus a
small manifest; resume restores them and the loss curve continues.
"""
from __future__ import annotations

import json
import os

import torch

# GPT names, then the llama family's (models/llama.py)
COLUMN_PARALLEL = ("qkv.weight", "qkv.bias", "fc1.weight", "fc1.bias", "wte",
                   ".q.weight", ".k.weight", ".v.weight", ".q.bias", ".k.bias", ".v.bias", "gate.weight", "up.weight", "lm_head")
ROW_PARALLEL = ("proj.weight", "fc2.weight", ".o.weight", "down.weight")


def shard_param(name: str, full: torch.Tensor, tp_rank: int, tp_size: int) -> torch.Tensor:
    """Slice a full (tp=1) parameter into the shard a tensor-parallel rank holds."""
    if tp_size == 1:
        return full
    if name.endswith(COLUMN_PARALLEL):
        n = full.shape[0] // tp_size
        return full[tp_rank * n:(tp_rank + 1) * n]
    if name.endswith(ROW_PARALLEL):
        n = full.shape[1] // tp_size
        return full[:, tp_rank * n:(tp_rank + 1) * n]
    return full


def unshard_param(name: str, shards: list[torch.Tensor]) -> torch.Tensor:
    if len(shards) == 1:
        return shards[0]
    if name.endswith(COLUMN_PARALLEL):
        return torch.cat(shards, dim=0)
    if name.endswith(ROW_PARALLEL):
        return torch.cat(shards, dim=1)
    return shards[0]


def save(trainer, directory: str, step: int, rank: int = 0, world: int = 1):
    os.makedirs(directory, exist_ok=True)
    sd = {
        # a fully sharded stage keeps only this rank's shards; every other layout keeps the stage's whole flat buffer
        "flat_param": getattr(trainer.stage.store, "flat_param_shard", trainer.stage.store.flat_param).detach().cpu(),
        "optimizer": {k: (v.detach().cpu() if torch.is_tensor(v) else v) for k, v in trainer.opt.state_dict().items()},
        # experts of a mixture-of-experts model that are spread over the expert-parallel group (None otherwise)
        "expert_flat_param": (trainer.stage.expert_store.flat_param.detach().cpu()
                              if getattr(trainer.stage, "expert_store", None) is not None else None),
        "expert_optimizer": ({k: (v.detach().cpu() if torch.is_tensor(v) else v)
                              for k, v in trainer.expert_opt.state_dict().items()}
                             if getattr(trainer, "expert_opt", None) is not None else None),
        "step": step,
        "torch_rng": torch.get_rng_state(),
        "cuda_rng": torch.cuda.get_rng_state() if torch.cuda.is_available() else None,
        "codec_state_reset": True,   # stateful codecs start from a raw round after resume
    }
    tmp = os.path.join(directory, f"rank{rank:05d}.pt.tmp")
    torch.save(sd, tmp)
    os.replace(tmp, os.path.join(directory, f"rank{rank:05d}.pt"))
    if rank == 0:
        p = trainer.parallel
        with open(os.path.join(directory, "manifest.json"), "w") as f:
            json.dump({"step": step, "world": world, "tp": p.tp, "pp": p.pp, "dp": p.dp, "ep": getattr(p, "ep", 1),
                       "virtual_stages": getattr(p, "virtual_stages", 1), "cp": getattr(p, "cp", 1),
                       "model": {k: (str(v) if not isinstance(v, (int, float, bool)) else v)
                                 for k, v in vars(trainer.cfg).items()}}, f)


def load(trainer, directory: str, rank: int = 0) -> int:
    with open(os.path.join(directory, "manifest.json")) as f:
        man = json.load(f)
    p = trainer.parallel
    if (man["tp"], man["pp"], man["dp"], man.get("ep", 1)) != (p.tp, p.pp, p.dp, getattr(p, "ep", 1)):
        raise ValueError(f"checkpoint was written with tp/pp/dp/ep={man['tp']}/{man['pp']}/{man['dp']}/{man.get('ep', 1)}")
    if man.get("cp", 1) != getattr(p, "cp", 1):
        # the optimizer shards are cut over data x context ranks
        raise ValueError(f"checkpoint was written with context-parallel size {man.get('cp', 1)}")
    if man.get("virtual_stages", 1) != getattr(p, "virtual_stages", 1):
        # the layers a pipeline rank holds depend on the number of model chunks per rank
        raise ValueError(f"checkpoint was written with {man.get('virtual_stages', 1)} model chunk(s) per pipeline rank")
    sd = torch.load(os.path.join(directory, f"rank{rank:05d}.pt"), map_location="cpu", weights_only=False)
    getattr(trainer.stage.store, "flat_param_shard", trainer.stage.store.flat_param).copy_(sd["flat_param"])
    trainer.opt.load_state_dict(sd["optimizer"])
    if sd.get("expert_flat_param") is not None:
        trainer.stage.expert_store.flat_param.copy_(sd["expert_flat_param"])
        trainer.expert_opt.load_state_dict(sd["expert_optimizer"])
    torch.set_rng_state(sd["torch_rng"])
    if sd.get("cuda_rng") is not None and torch.cuda.is_available():
        torch.cuda.set_rng_state(sd["cuda_rng"])
    return int(sd["step"])
