"""Expert-parallel all-to-all benchmark: FP8 dispatch + bf16 combine against NCCL all_to_all_single of bf16 rows.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29513 \
        -m coccl_b200.bench_moe --tokens 8192 --hidden 4096 --experts 64 --topk 2

Routing: seeded uniform-random distinct expert ids per token, softmax gates. `fused_*` = routing layout + one
kernel per direction (peer stores inside); `nccl_*` = torch index_select into a send buffer ordered by
destination + all_to_all_single with the exchanged split sizes (+ index_add for the combine). Timed with CUDA
events, barrier before each timed call, L2 flushed, median of the max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from .ops import moe as M
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
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--topk", type=int, default=2)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(1000 + rank)
    T, H, E, k = a.tokens, a.hidden, a.experts, a.topk
    le = E // world
    x = torch.randn(T, H, device=dev, dtype=torch.bfloat16)
    top = torch.rand(T, E, device=dev).topk(k, dim=1)
    ids = top.indices.to(torch.int32).contiguous()
    gates = torch.softmax(top.values, dim=1).float().contiguous()
    comm = Communicator(None, dev, Policy(), "ep")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    state = {}

    def fused_dispatch():
        state["rows"], state["h"] = comm.moe_dispatch(x, ids, E)

    def fused_combine():
        return comm.moe_combine(state["rows"], gates, state["h"])

    # NCCL baseline: bf16 rows ordered by destination rank
    flat = ids.reshape(-1).long()
    order = torch.sort(flat, stable=True).indices
    tok_of = order // k
    send_counts = torch.bincount(flat // le, minlength=world)
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts)
    in_split, out_split = send_counts.tolist(), recv_counts.tolist()
    recv_buf = torch.empty(sum(out_split), H, device=dev, dtype=torch.bfloat16)
    back_buf = torch.empty(T * k, H, device=dev, dtype=torch.bfloat16)

    def nccl_dispatch():
        send = x.index_select(0, tok_of)
        dist.all_to_all_single(recv_buf, send, out_split, in_split)

    def nccl_combine():
        dist.all_to_all_single(back_buf, recv_buf, in_split, out_split)
        out = torch.zeros(T, H, device=dev, dtype=torch.float32)
        out.index_add_(0, tok_of, back_buf.float() * gates.reshape(-1)[order].unsqueeze(1))
        return out.to(torch.bfloat16)

    fused_dispatch()
    y_f = fused_combine().float()
    nccl_dispatch()
    y_n = nccl_combine().float()
    rel = ((y_f - y_n).norm() / y_n.norm()).item()  # identity experts: fused differs by the FP8 rounding only
    res = {"what": "moe_all_to_all", "n_gpus": world, "tokens_per_rank": T, "hidden": H, "experts": E, "topk": k,
           "rel_diff_fused_vs_nccl": rel}
    for name, fn in (("fused_dispatch", fused_dispatch), ("fused_combine", fused_combine),
                     ("nccl_dispatch", nccl_dispatch), ("nccl_combine", nccl_combine)):
        res[name + "_ms"] = _time(fn, a.iters, a.warmup, flush, dev)
    raw = T * k * H * 2
    res["dispatch_effective_gbs_fused"] = raw / res["fused_dispatch_ms"] / 1e6
    res["dispatch_effective_gbs_nccl"] = raw / res["nccl_dispatch_ms"] / 1e6
    res["combine_effective_gbs_fused"] = raw / res["fused_combine_ms"] / 1e6
    res["combine_effective_gbs_nccl"] = raw / res["nccl_combine_ms"] / 1e6
    res["status"] = comm.moe_status()
    if rank == 0:
        print(json.dumps(res), flush=True)
    comm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
