"""Tensor-parallel MLP benchmark: all-gather -> GEMM (+bias, GELU) -> GEMM -> reduce-scatter.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29512 \
        -m coccl_b200.bench_tp --tokens 16384 --hidden 4096 --ffn 14336

Sequence-parallel layout: every rank holds tokens/N rows of X, ffn/N rows of W_up and ffn/N columns of W_down.
`fused` = the two one-kernel fusions (peer stores inside the tcgen05 kernels, FP8 on the reduce-scatter);
`unfused` = NCCL all_gather + the same tcgen05 GEMM + NCCL reduce_scatter (bf16), the baseline a library-only
solution gives. Timed with CUDA events, barrier before each timed iteration, L2 flushed, median of the max over
ranks. Roofline = the slower of the GEMM FLOPs at the measured cuBLAS bf16 rate and the bytes that must cross
NVLink at the measured 770 GB/s per direction.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from .ops import gemm as G
from .parallel.comm import Communicator, Policy


def _time(fn, iters, warmup, flush, dev):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    tok = torch.zeros(1, device=dev)
    evs = []
    for _ in range(iters):
        flush.zero_()
        dist.all_reduce(tok)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        evs.append((a, b))
    torch.cuda.synchronize()
    ts = torch.tensor([a.elapsed_time(b) for a, b in evs], device=dev)
    dist.all_reduce(ts, op=dist.ReduceOp.MAX)
    return float(ts.median().item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--peak-tflops", type=float, default=1645.4)
    ap.add_argument("--link-gbs", type=float, default=770.0)
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(rank)
    T, H, F = a.tokens, a.hidden, a.ffn
    f = F // world
    x = torch.randn(T // world, H, device=dev, dtype=torch.bfloat16)
    w_up = torch.randn(f, H, device=dev, dtype=torch.bfloat16) * 0.02
    b_up = torch.zeros(f, device=dev, dtype=torch.bfloat16)
    w_down = torch.randn(H, f, device=dev, dtype=torch.bfloat16) * 0.02
    comm = Communicator(None, dev, Policy(), "tp")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    xg = torch.empty(T, H, device=dev, dtype=torch.bfloat16)
    part = torch.empty(T, H, device=dev, dtype=torch.bfloat16)
    out_ref = torch.empty(T // world, H, device=dev, dtype=torch.bfloat16)

    def fused_up():   # payload as the policy says (MX-FP8 on the tensor-parallel all-gather -> FP8 on the wire)
        return comm.ag_gemm(x, w_up, bias=b_up, gelu=True)

    def fused_up_bf16():
        return comm.ag_gemm(x, w_up, bias=b_up, gelu=True, payload="bf16")

    def fused_up_fp8():
        return comm.ag_gemm(x, w_up, bias=b_up, gelu=True, payload="fp8")

    def unfused_up():
        dist.all_gather_into_tensor(xg, x)
        return G.gemm(xg, w_up, bias=b_up, gelu=True)

    h = fused_up()

    def fused_down():
        return comm.gemm_rs(h, w_down)

    def unfused_down():
        G.gemm(h, w_down, out=part)
        dist.reduce_scatter_tensor(out_ref, part)
        return out_ref

    def fused():
        return comm.gemm_rs(comm.ag_gemm(x, w_up, bias=b_up, gelu=True), w_down)

    def unfused():
        dist.all_gather_into_tensor(xg, x)
        hh = G.gemm(xg, w_up, bias=b_up, gelu=True)
        G.gemm(hh, w_down, out=part)
        dist.reduce_scatter_tensor(out_ref, part)
        return out_ref

    # numerics: fused against unfused
    y1, y0 = fused().float(), unfused().float()
    rel = ((y1 - y0).norm() / y0.norm()).item()
    res = {"what": "tp_mlp", "n_gpus": world, "tokens": T, "hidden": H, "ffn": F, "rel_diff_fused_vs_unfused": rel}
    res["ag_payload_by_policy"] = "fp8" if (comm._ag_payload_fp8(T // world, H, None) and comm._ag_payload_pays(T // world, H, f)) else "bf16"
    y8, yb = fused_up_fp8().float(), fused_up_bf16().float()
    res["rel_diff_ag_fp8_vs_bf16"] = ((y8 - yb).norm() / yb.norm()).item()
    for name, fn in (("ag_gemm_fused", fused_up), ("ag_gemm_fused_bf16", fused_up_bf16), ("ag_gemm_fused_fp8", fused_up_fp8),
                     ("ag_gemm_unfused", unfused_up), ("gemm_rs_fused", fused_down),
                     ("gemm_rs_unfused", unfused_down), ("mlp_fused", fused), ("mlp_unfused", unfused)):
        res[name + "_ms"] = _time(fn, a.iters, a.warmup, flush, dev)
    flops = 2.0 * T * H * f
    t_gemm = flops / (a.peak_tflops * 1e12) * 1e3
    ag_bytes = (world - 1) * (T // world) * H * 2
    rs_bytes = (world - 1) * (T // world) * H * (1 + 1 / 32)
    res["ag_gemm_roofline_ms"] = max(t_gemm, ag_bytes / (a.link_gbs * 1e9) * 1e3)
    res["ag_gemm_fp8_roofline_ms"] = max(t_gemm, ag_bytes * (1 + 1 / 32) / 2 / (a.link_gbs * 1e9) * 1e3)
    res["ag_gemm_fp8_frac_of_roofline"] = res["ag_gemm_fp8_roofline_ms"] / res["ag_gemm_fused_fp8_ms"]
    res["gemm_rs_roofline_ms"] = max(t_gemm, rs_bytes / (a.link_gbs * 1e9) * 1e3)
    res["ag_gemm_frac_of_roofline"] = res["ag_gemm_roofline_ms"] / res["ag_gemm_fused_bf16_ms"]
    res["gemm_rs_frac_of_roofline"] = res["gemm_rs_roofline_ms"] / res["gemm_rs_fused_ms"]
    res["tp_status"] = list(comm.tp_status())
    G.check_errors()
    if rank == 0:
        print(json.dumps(res), flush=True)
    comm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
