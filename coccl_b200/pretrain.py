"""GPT pre-training launcher: the command a user runs, one process per GPU.

    python -m coccl_b200.pretrain --model gpt-tiny --steps 50                                   # one GPU
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m coccl_b200.pretrain \\
        --model gpt-6.7b --tp 2 --pp 2 --dp 2 --global-batch 128 --data tokens.bin --save ckpt --save-interval 500

The reference's counterpart is a bash launcher that exports COCCL_ENABLE / COCCL_CONFIG_FILE, preloads the library
into PyTorch and starts an external Megatron trainer with TP / PP / EP sizes, batch sizes, a learning-rate schedule and
save / load directories (examples/training_scripts/train_qwen_coccl.sh:60-131). Here the trainer is part of the
package, so the launcher is this module: the same two environment variables choose the policy (or --policy /
--no-compress), the parallel sizes are flags, and the loop adds what a long run needs: a data loader with prefetch
into pinned memory, warm-up + cosine learning-rate schedule, periodic logs (loss, gradient norm, tokens/s, model
TFLOP/s per GPU), checkpoints with resume, and the heartbeat that notices a lost rank between steps.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import time

import torch
import torch.distributed as dist

MODELS = {
    "gpt-6.7b": dict(),
    "gpt-1.3b": dict(n_layer=24, hidden=2048, n_head=16, ffn=8192),
    "gpt-2.7b": dict(n_layer=32, hidden=2560, n_head=32, ffn=10240),
    "gpt-13b": dict(n_layer=40, hidden=5120, n_head=40, ffn=20480),
    "gpt-small": dict(n_layer=4, hidden=2048, n_head=16, ffn=8192),
    "gpt-tiny": dict(n_layer=2, hidden=512, n_head=8, ffn=2048, seq_len=256, vocab=8192),
    "moe-tiny": dict(n_layer=4, hidden=512, n_head=8, ffn=1024, seq_len=256, vocab=8192, n_experts=4, moe_top_k=2, moe_every=2),
    # the Llama / Qwen family (models/llama.py): RMSNorm, rotary positions, grouped-query attention, SwiGLU, untied head
    "llama-tiny": dict(arch="llama", n_layer=2, hidden=512, n_head=8, n_kv_head=2, ffn=1536, seq_len=256, vocab=8192,
                       tie_embeddings=False, rope_theta=1.0e4),
    "llama3-8b": dict(arch="llama", n_layer=32, hidden=4096, n_head=32, n_kv_head=8, ffn=14336, seq_len=2048, vocab=128256,
                      tie_embeddings=False, rope_theta=5.0e5),
    "qwen3-moe-tiny": dict(arch="llama", n_layer=2, hidden=512, n_head=8, n_kv_head=2, ffn=512, seq_len=256, vocab=8192,
                           tie_embeddings=False, rope_theta=1.0e6, qk_norm=True, n_experts=8, moe_top_k=2, moe_every=1),
    "qwen3-30b-a3b": dict(arch="llama", n_layer=48, hidden=2048, n_head=32, n_kv_head=4, kv_channels=128, ffn=768, seq_len=2048, vocab=151936,
                          tie_embeddings=False, rope_theta=1.0e6, qk_norm=True, n_experts=128, moe_top_k=8, moe_every=1),
    "mixtral-8x7b": dict(arch="llama", n_layer=32, hidden=4096, n_head=32, n_kv_head=8, ffn=14336, seq_len=2048, vocab=32000,
                         tie_embeddings=False, rope_theta=1.0e6, n_experts=8, moe_top_k=2, moe_every=1),
    "qwen3-8b": dict(arch="llama", n_layer=36, hidden=4096, n_head=32, n_kv_head=8, ffn=12288, seq_len=2048, vocab=151936,
                     tie_embeddings=False, rope_theta=1.0e6, qk_norm=True),
    "qwen2.5-7b": dict(arch="llama", n_layer=28, hidden=3584, n_head=28, n_kv_head=4, ffn=18944, seq_len=2048, vocab=152064,
                       tie_embeddings=False, rope_theta=1.0e6, qkv_bias=True),
}


def parse(argv=None):
    ap = argparse.ArgumentParser(prog="python -m coccl_b200.pretrain", description=__doc__.split("\n\n")[0])
    m = ap.add_argument_group("model")
    m.add_argument("--model", default="gpt-tiny", choices=sorted(MODELS))
    for name, typ in (("layers", int), ("hidden", int), ("heads", int), ("kv-heads", int), ("ffn", int), ("seq-len", int),
                      ("vocab", int), ("experts", int), ("moe-top-k", int), ("moe-every", int), ("rope-theta", float)):
        m.add_argument(f"--{name}", type=typ, default=None, help="overrides the preset")
    m.add_argument("--dtype", default="bf16", choices=["bf16", "fp32"], help="fp32 is for CPU runs")
    m.add_argument("--hf-model", default=None, metavar="DIR",
                   help="start from a Hugging Face checkpoint of the Llama / Qwen family (configuration and weights; overrides --model)")
    p = ap.add_argument_group("parallelism (tp * cp * pp * dp = world size)")
    p.add_argument("--tp", type=int, default=1)
    p.add_argument("--pp", type=int, default=1)
    p.add_argument("--cp", type=int, default=1, help="context parallelism: ranks sharing every sequence (head exchange around attention)")
    p.add_argument("--dp", type=int, default=0, help="0: world size / (tp * pp * cp)")
    p.add_argument("--ep", type=int, default=1, help="expert parallelism: 1 or the data-parallel size")
    p.add_argument("--virtual-stages", type=int, default=1, help="model chunks per pipeline rank (interleaved 1F1B)")
    p.add_argument("--no-sequence-parallel", action="store_true")
    p.add_argument("--dp-strategy", default="zero1", choices=["zero1", "ddp", "fsdp"],
                   help="zero1: sharded optimizer; ddp: gradient all-reduce; fsdp: parameters, gradients and optimizer state sharded")
    c = ap.add_argument_group("collectives")
    c.add_argument("--policy", default=None, help="policy file (TOML); default: $COCCL_CONFIG_FILE, else the shipped training policy")
    c.add_argument("--no-compress", action="store_true", help="native collectives only (also COCCL_ENABLE=0)")
    t = ap.add_argument_group("training")
    t.add_argument("--steps", type=int, default=100)
    t.add_argument("--global-batch", type=int, default=0, help="sequences per step over all ranks; 0: 8 per data-parallel rank")
    t.add_argument("--micro-batch", type=int, default=2)
    t.add_argument("--lr", type=float, default=3e-4)
    t.add_argument("--min-lr", type=float, default=3e-5)
    t.add_argument("--warmup-steps", type=int, default=10)
    t.add_argument("--decay-steps", type=int, default=0, help="0: decay over --steps")
    t.add_argument("--weight-decay", type=float, default=0.1)
    t.add_argument("--clip-grad", type=float, default=1.0)
    t.add_argument("--seed", type=int, default=1234)
    d = ap.add_argument_group("data")
    d.add_argument("--data", default=None, help="flat token file (uint16 / uint32, or .npy); default: synthetic ids")
    d.add_argument("--data-dtype", default="auto", choices=["auto", "uint16", "uint32"])
    d.add_argument("--eval-data", default=None, help="held-out token file; its loss is logged as val_loss")
    d.add_argument("--eval-interval", type=int, default=0, help="steps between evaluations (0: never)")
    d.add_argument("--eval-batches", type=int, default=4, help="global batches per evaluation")
    k = ap.add_argument_group("checkpoints and logs")
    k.add_argument("--save", default=None, metavar="DIR")
    k.add_argument("--save-interval", type=int, default=0, help="0: only at the end")
    k.add_argument("--resume", action="store_true", help="continue from --save if it holds a checkpoint")
    k.add_argument("--export-hf", default=None, metavar="DIR",
                   help="write the final weights as a Hugging Face checkpoint (dense models, one rank holding the whole model)")
    k.add_argument("--log-interval", type=int, default=10)
    k.add_argument("--log-json", default=None, metavar="FILE", help="rank 0 appends one JSON line per log interval")
    k.add_argument("--heartbeat-stale-s", type=float, default=120.0, help="a peer silent for this long counts as lost; 0: off")
    ap.add_argument("--device", default="auto", choices=["auto", "cuda", "cpu"])
    return ap.parse_args(argv)


def learning_rate(step: int, *, peak: float, floor: float, warmup: int, decay: int) -> float:
    """Linear warm-up to `peak` over `warmup` steps, then a half cosine down to `floor` at step `decay`."""
    if warmup > 0 and step < warmup:
        return peak * (step + 1) / warmup
    if step >= decay:
        return floor
    frac = (step - warmup) / max(decay - warmup, 1)
    return floor + 0.5 * (peak - floor) * (1.0 + math.cos(math.pi * frac))


def model_config(args):
    from .models.gpt import GPTConfig
    if args.hf_model:
        import transformers
        from .utils import hf
        return hf.config_from_hf(transformers.AutoConfig.from_pretrained(args.hf_model), seq_len=args.seq_len,
                                 dtype=torch.bfloat16 if args.dtype == "bf16" else torch.float32)
    kw = dict(MODELS[args.model])
    for flag, field in (("layers", "n_layer"), ("hidden", "hidden"), ("heads", "n_head"), ("ffn", "ffn"), ("seq_len", "seq_len"),
                        ("vocab", "vocab"), ("experts", "n_experts"), ("moe_top_k", "moe_top_k"), ("moe_every", "moe_every"),
                        ("kv_heads", "n_kv_head"), ("rope_theta", "rope_theta")):
        v = getattr(args, flag)
        if v is not None:
            kw[field] = v
    kw["dtype"] = torch.bfloat16 if args.dtype == "bf16" else torch.float32
    return GPTConfig(**kw)


def main(argv=None) -> int:
    args = parse(argv)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    use_cuda = args.device == "cuda" or (args.device == "auto" and torch.cuda.is_available())
    dev = torch.device("cuda", local_rank) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(dev)
    dp = args.dp or world // (args.tp * args.pp * args.cp)
    if args.tp * args.pp * args.cp * dp != world:
        raise SystemExit(f"tp * cp * pp * dp = {args.tp} * {args.cp} * {args.pp} * {dp} does not equal the world size {world}")
    if not use_cuda and args.dtype == "bf16":
        args.dtype = "fp32"
    cfg = model_config(args)

    from .parallel.comm import Policy
    from .train import ParallelConfig, Trainer
    from .utils import checkpoint
    from .utils.data import BatchLoader, SyntheticTokens, TokenFile
    from .utils.health import Heartbeat, default_store

    enabled = not args.no_compress and os.environ.get("COCCL_ENABLE", "1") != "0"
    policy_file = args.policy or os.environ.get("COCCL_CONFIG_FILE")
    policy = Policy(enabled=enabled, config_file=policy_file)
    mesh = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if use_cuda:
            dist.init_process_group("nccl", device_id=dev)
        else:
            dist.init_process_group("gloo")
        from .parallel.mesh import Mesh
        mesh = Mesh(tp=args.tp, pp=args.pp, dp=dp, device=dev, compress=enabled, policy=policy,
                    sequence_parallel=not args.no_sequence_parallel, ep=args.ep, cp=args.cp)
    par = ParallelConfig(tp=args.tp, pp=args.pp, dp=dp, sequence_parallel=not args.no_sequence_parallel,
                         dp_strategy=args.dp_strategy, ep=args.ep, cp=args.cp, virtual_stages=args.virtual_stages if args.pp > 1 else 1)
    trainer = Trainer(cfg, dev, micro_batch=args.micro_batch, parallel=par, groups=mesh, lr=args.lr,
                      weight_decay=args.weight_decay, clip_grad=args.clip_grad, seed=args.seed)

    global_batch = args.global_batch or 8 * dp
    if global_batch % (dp * args.micro_batch):
        raise SystemExit("--global-batch must be a multiple of dp * micro-batch")
    if args.pp > 1 and par.virtual_stages > 1 and (global_batch // dp // args.micro_batch) % args.pp:
        raise SystemExit("interleaved 1F1B needs the micro-batches per step to be a multiple of --pp")

    start = 0
    resuming = bool(args.resume and args.save and os.path.exists(os.path.join(args.save, "manifest.json")))
    if args.hf_model and not resuming:
        import transformers
        from .utils import hf
        assert not trainer.fsdp, "--hf-model loads into whole (or tensor-parallel) parameters; the fully sharded layout is not covered"
        sd = transformers.AutoModelForCausalLM.from_pretrained(args.hf_model, torch_dtype=cfg.dtype).state_dict()
        missing = hf.load_state_dict(trainer.stage, sd, tp_rank=mesh.tp_rank if mesh else 0, tp_size=args.tp)
        if missing:
            raise SystemExit(f"{args.hf_model} does not provide {missing[:4]}{' ...' if len(missing) > 4 else ''}")
        del sd
        trainer.opt.master.copy_(trainer.opt.param_shard.float())   # the optimizer's fp32 copy follows the loaded weights
        if rank == 0:
            print(f"loaded weights from {args.hf_model}", flush=True)
    if resuming:
        start = checkpoint.load(trainer, args.save, rank=rank)
        if rank == 0:
            print(f"resumed from {args.save} at step {start}", flush=True)

    if args.data_dtype == "auto" and cfg.vocab > 65536 and not (args.data or "").endswith(".npy"):
        args.data_dtype = "uint32"   # ids of such a vocabulary do not fit 16 bits
    source = TokenFile(args.data, args.data_dtype) if args.data else SyntheticTokens(cfg.vocab, seed=args.seed)
    loader = BatchLoader(source, seq_len=cfg.seq_len, global_batch=global_batch, dp_rank=mesh.dp_rank if mesh else 0,
                         dp_size=dp, seed=args.seed, start_step=start, vocab=cfg.vocab)
    heartbeat = None
    if world > 1 and args.heartbeat_stale_s > 0 and default_store() is not None:
        heartbeat = Heartbeat(default_store(), rank, world, stale_after_s=args.heartbeat_stale_s)
        heartbeat.beat(start - 1)   # a resumed run has the steps before `start` behind it

    eval_source = None
    if args.eval_interval > 0:
        eval_source = TokenFile(args.eval_data, args.data_dtype) if args.eval_data else SyntheticTokens(cfg.vocab, seed=args.seed + 1)

    def evaluate():
        """Mean loss over the first --eval-batches global batches of the held-out stream (the same ones every time)."""
        ev = BatchLoader(eval_source, seq_len=cfg.seq_len, global_batch=global_batch, dp_rank=mesh.dp_rank if mesh else 0,
                         dp_size=dp, seed=args.seed + 1, vocab=cfg.vocab, depth=2)
        total = torch.zeros(1, dtype=torch.float32, device=dev)
        for _ in range(args.eval_batches):
            total += trainer.eval_step(ev.next())
            ev.copied()
        ev.close()
        if world > 1:
            dist.all_reduce(total)
        return total.item() / (loss_group_size * args.eval_batches)

    decay = args.decay_steps or args.steps
    tokens_per_step = global_batch * cfg.seq_len
    loss_group_size = args.tp * dp   # ranks of the last pipeline stage that hold a loss
    if rank == 0:
        print(json.dumps({"model": args.model, "params": cfg.num_params(), "world": world, "tp": args.tp, "cp": args.cp, "pp": args.pp, "dp": dp,
                          "ep": args.ep, "virtual_stages": par.virtual_stages, "global_batch": global_batch,
                          "seq_len": cfg.seq_len, "compressed_collectives": enabled and world > 1,
                          "policy": policy_file or ("shipped training policy" if enabled else "native"),
                          "data": args.data or "synthetic"}), flush=True)

    def save(step):
        if args.save:
            checkpoint.save(trainer, args.save, step, rank=rank, world=world)
            if world > 1:
                dist.barrier()
            if rank == 0:
                print(f"saved step {step} to {args.save}", flush=True)

    window_loss = torch.zeros(1, dtype=torch.float32, device=dev)
    window_steps, t_window = 0, time.time()
    last_loss = float("nan")
    try:
        for step in range(start, args.steps):
            if heartbeat is not None:
                # peers must have finished the previous step before this one's kernels launch
                heartbeat.check_peers(expect_step=step - 1, wait_s=args.heartbeat_stale_s)
            lr = learning_rate(step, peak=args.lr, floor=args.min_lr, warmup=args.warmup_steps, decay=decay)
            trainer.opt.lr = lr
            if trainer.expert_opt is not None:
                trainer.expert_opt.lr = lr
            batch = loader.next()
            loss = trainer.train_step(batch)
            loader.copied()
            window_loss += loss
            window_steps += 1
            if heartbeat is not None:
                heartbeat.beat(step)
            done = step + 1
            if done % args.log_interval == 0 or done == args.steps:
                t = window_loss.clone()
                if world > 1:
                    dist.all_reduce(t)   # only the last pipeline stage contributes; every rank takes part
                if use_cuda:
                    torch.cuda.synchronize()
                dt = time.time() - t_window
                last_loss = t.item() / (loss_group_size * window_steps)
                if rank == 0:
                    rate = tokens_per_step * window_steps / dt
                    rec = {"step": done, "loss": round(last_loss, 5), "grad_norm": round(trainer.opt.grad_norm.item(), 4),
                           "lr": lr, "tokens_per_s": round(rate, 1),
                           "model_tflops_per_gpu": round(cfg.flops_per_token() * rate / world / 1e12, 2),
                           "ms_per_step": round(1e3 * dt / window_steps, 2)}
                    print(json.dumps(rec), flush=True)
                    if args.log_json:
                        with open(args.log_json, "a") as f:
                            f.write(json.dumps(rec) + "\n")
                trainer.check_health(wait=True)
                window_loss.zero_()
                window_steps, t_window = 0, time.time()
            if eval_source is not None and (done % args.eval_interval == 0 or done == args.steps):
                val = evaluate()
                if rank == 0:
                    rec = {"step": done, "val_loss": round(val, 5)}
                    print(json.dumps(rec), flush=True)
                    if args.log_json:
                        with open(args.log_json, "a") as f:
                            f.write(json.dumps(rec) + "\n")
            if args.save_interval and done % args.save_interval == 0 and done != args.steps:
                save(done)
        save(args.steps)
        if args.export_hf:
            if args.tp * args.pp > 1 or trainer.fsdp:
                raise SystemExit("--export-hf needs the whole model on a rank (tp = pp = 1, not fully sharded)")
            if rank == 0:
                from .utils import hf
                hf.export_pretrained(trainer.stage, args.export_hf)
                print(f"exported to {args.export_hf}", flush=True)
    finally:
        loader.close()
        if heartbeat is not None:
            heartbeat.leave(args.steps)
        if mesh is not None:
            mesh.close()
        if world > 1 and dist.is_initialized():
            dist.destroy_process_group()
    if rank == 0:
        print(json.dumps({"final_loss": last_loss, "steps": args.steps}), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
