#!/usr/bin/env python
"""Headline benchmark: 3-D-parallel GPT training throughput (tokens/s) on N B200s of one node.

Model / config (the reference's GPT-6.7B end-to-end setting): GPT with 32 layers, hidden 4096, 32 heads, FFN 16384,
GELU, sequence 2048, vocabulary 50304, micro-batch 2, bf16 compute with fp32 master weights and
Adam, random-init N(0, 0.02) weights, uniform-random token ids. The 8-GPU configuration is
TP=2, PP=2, DP=2 with global batch 256; smaller N keep the per-GPU work fixed (weak scaling:
32 sequences per GPU and step) and drop parallel dimensions in the order DP, PP, TP.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 5 --warmup 3

Prints ONE JSON line on rank 0. `value` is device-timed (CUDA events around exactly K steps,
max over ranks) with the step's inputs already on the device; `e2e.value` is measured through
the public `Trainer.train_step` call with, every step, the host->device copy of the step's token
ids from pinned memory and a device->host read of the loss.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

METRIC = "gpt_train_tokens_per_s"
SEQS_PER_GPU = 32          # global batch 256 on 8 GPUs
PARALLELISM = {1: (1, 1, 1), 2: (2, 1, 1), 4: (2, 2, 1), 8: (2, 2, 2)}  # N -> (tp, pp, dp)


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, index: int, period: float = 0.2):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.nv = None

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
        }
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop_evt.wait(self.period)

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=2)
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


def reference_arm(args):
    # Two independent reasons:
    #  * the reference is a C++/CUDA fork of NCCL with no Python package and no trainer: a pip install of its source
    #    tree fails ("Neither 'setup.py' nor 'pyproject.toml' found") and its Megatron submodule is empty, so no
    #    stock code path of it produces GPT tokens/s;
    #  * built unmodified for sm_100 (baseline/build_reference.py), its NCCL 2.21.5 collective kernels fault
    #    ("an illegal memory access was encountered") or never finish on B200 (profiles/reference_collectives_2gpu.md),
    #    so even a trainer preloading it could not run. Code that faulted or hung a GPU is not started again.
    print(json.dumps({"impl": "reference", "unavailable":
                      "reference is a C++ NCCL 2.21.5 fork without setup.py/pyproject.toml (pip install fails) and ships "
                      "no trainer (empty Megatron submodule), so GPT tokens/s cannot be run from it; built for sm_100 its "
                      "own all-reduce / reduce-scatter / all-gather kernels fault or hang on B200 and are not run again"}))
    return 0


def _profile_one_step(trainer, batch, path):
    """One extra training step under torch.profiler (CUDA activities only). Writes, for this rank, the device time of
    every kernel summed over the step, its share, and the step's wall time, so that launch gaps show as the difference."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        trainer.train_step(batch)
        torch.cuda.synchronize()
    wall_ms = (time.perf_counter() - t0) * 1e3
    if path is None:
        return
    rows, tot = [], 0.0
    for e in prof.key_averages():
        t = getattr(e, "device_time_total", None)
        if t is None:
            t = e.cuda_time_total
        if t > 0:
            rows.append((t, e.count, e.key))
            tot += t
    rows.sort(reverse=True)
    with open(path, "w") as f:
        f.write(f"step wall time under the profiler {wall_ms:.1f} ms; device time summed over kernels {tot / 1e3:.1f} ms\n")
        for t, c, k in rows[:60]:
            f.write(f"{t / tot * 100:6.2f}% {t / 1e3:10.3f} ms  x{c:6d}  {k[:140]}\n")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="gpt-6.7b", choices=["gpt-6.7b", "gpt-2.7b", "gpt-13b", "gpt-small", "gpt-tiny", "qwen2.5-7b", "qwen3-8b", "llama3-8b"],
                    help="the default is the benchmark's model; the llama-family presets are extras")
    ap.add_argument("--seqs-per-gpu", type=int, default=SEQS_PER_GPU)
    ap.add_argument("--parallelism", default=None, help="override as tp,pp,dp")
    ap.add_argument("--no-compress", action="store_true", help="route collectives through NCCL only")
    ap.add_argument("--virtual-stages", type=int, default=1,
                    help="model chunks per pipeline rank (> 1: interleaved 1F1B); the default is the measured schedule")
    ap.add_argument("--profile-step", default="", metavar="FILE",
                    help="after the timed regions, run ONE more step under torch.profiler and write rank 0's per-kernel "
                         "device-time table (shares; never a bench value) to FILE")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist

    from coccl_b200 import _lib
    from coccl_b200.models.gpt import GPTConfig
    from coccl_b200.train import ParallelConfig, Trainer

    n = args.gpus
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == n, f"--gpus {n} but WORLD_SIZE={world}"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    tp, pp, dp = PARALLELISM[n] if args.parallelism is None else map(int, args.parallelism.split(","))
    assert tp * pp * dp == n

    cfg = {"gpt-6.7b": GPTConfig(),
           "gpt-2.7b": GPTConfig(n_layer=32, hidden=2560, n_head=32, ffn=10240),
           "gpt-13b": GPTConfig(n_layer=40, hidden=5120, n_head=40, ffn=20480),
           "gpt-small": GPTConfig(n_layer=4, hidden=2048, n_head=16, ffn=8192, seq_len=2048, vocab=50304),
           "gpt-tiny": GPTConfig(n_layer=2, hidden=512, n_head=8, ffn=2048, seq_len=256, vocab=8192),
           "qwen2.5-7b": GPTConfig(arch="llama", n_layer=28, hidden=3584, n_head=28, n_kv_head=4, ffn=18944, seq_len=2048,
                                   vocab=152064, tie_embeddings=False, rope_theta=1.0e6, qkv_bias=True),
           "qwen3-8b": GPTConfig(arch="llama", n_layer=36, hidden=4096, n_head=32, n_kv_head=8, ffn=12288, seq_len=2048,
                                 vocab=151936, tie_embeddings=False, rope_theta=1.0e6, qk_norm=True),
           "llama3-8b": GPTConfig(arch="llama", n_layer=32, hidden=4096, n_head=32, n_kv_head=8, ffn=14336, seq_len=2048,
                                  vocab=128256, tie_embeddings=False, rope_theta=5.0e5)}[args.model]

    mesh = None
    if n > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        from coccl_b200.parallel.mesh import Mesh
        mesh = Mesh(tp=tp, pp=pp, dp=dp, device=dev, compress=not args.no_compress)
    par = ParallelConfig(tp=tp, pp=pp, dp=dp, virtual_stages=args.virtual_stages if pp > 1 else 1)
    trainer = Trainer(cfg, dev, micro_batch=2, parallel=par, groups=mesh)

    # this DP rank's share of the global batch: seqs_per_gpu * (tp*pp) sequences per step
    seqs = args.seqs_per_gpu * tp * pp
    global_batch = seqs * dp
    gen = torch.Generator().manual_seed(1000 + (mesh.dp_rank if mesh else 0))
    host_batches = [torch.randint(0, cfg.vocab, (seqs, cfg.seq_len + 1), generator=gen).pin_memory()
                    for _ in range(2)]
    dev_batches = [b.to(dev) for b in host_batches]
    tokens_per_step = global_batch * cfg.seq_len

    def barrier():
        if n > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        trainer.train_step(dev_batches[i % 2])
    barrier()

    # ---- device-timed region: exactly K steps, inputs resident on the device
    sampler = ClockSampler(local_rank)
    sampler.start()
    launches0 = _lib.lib().cocclkLaunchCount()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(args.steps):
        loss = trainer.train_step(dev_batches[i % 2])
    e1.record()
    barrier()
    launches = _lib.lib().cocclkLaunchCount() - launches0
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop()

    # ---- end-to-end region: pinned host -> device copy of every step's tokens, loss read back every step
    barrier()
    t0 = time.perf_counter()
    last = None
    for i in range(args.steps):
        last = float(trainer.train_step(host_batches[i % 2]).item())
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    barrier()

    if args.profile_step:
        _profile_one_step(trainer, dev_batches[0], args.profile_step if rank == 0 else None)
        barrier()

    # the loss lives on the last pipeline stage: take the maximum over ranks (it is positive)
    t = torch.tensor([ms, e2e_s * 1e3, last if last is not None else 0.0], dtype=torch.float64, device=dev)
    if n > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms, last = t.tolist()
    trainer.check_health(wait=True)   # status words of every fused kernel family + GEMM pipeline errors
    if rank == 0:
        ms_per_step = ms / args.steps
        value = tokens_per_step / (ms_per_step / 1e3)
        e2e_value = tokens_per_step / (e2e_ms / args.steps / 1e3)
        out = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": n, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            # the only published GPT-6.7B figure (163.2 model TFLOP/s per GPU, reference README.md:334-340) is for
            # 32 x H800 over InfiniBand: no number exists for this hardware, so no ratio is formed
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic (uniform-random token ids, random-init weights)",
            "config": {"model": f"{args.model}: L{cfg.n_layer} h{cfg.hidden} heads{cfg.n_head} ffn{cfg.ffn} "
                                f"{'gelu' if cfg.arch == 'gpt' else f'swiglu kv{cfg.kv_heads} rope rmsnorm'} "
                                f"seq{cfg.seq_len} vocab{cfg.vocab}", "global_batch": global_batch,
                       "seq_len": cfg.seq_len, "micro_batch": 2, "parallelism": f"tp{tp}pp{pp}dp{dp}" + (f"v{par.virtual_stages}" if par.virtual_stages > 1 else ""),
                       "optimizer": "AdamW, fp32 master weights, sharded over DP",
                       "compressed_collectives": (n > 1 and not args.no_compress),
                       # hash of the effective policy (the TOML the routing session parsed) per communicator of rank 0
                       "policy_hash": {c.name: c.routing_summary().get("policy_hash", "native") for c in trainer._comms()},
                       "l2": "working set per step (>100 GB) is far larger than L2; no explicit flush"},
            "model_tflops_per_gpu": cfg.flops_per_token() * value / n / 1e12,
            "published_reference_tflops_per_gpu_32xh800": 163.2,
            "final_loss": last,
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s",
                    "h2d_bytes_per_step": int(host_batches[0].numel() * host_batches[0].element_size()),
                    "d2h_bytes_per_step": 4},
            "gpu_launches": int(launches),
            "impl": "ours",
        }
        print(json.dumps(out))
    if n > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
