"""Micro-benchmarks of single kernels (device-timed with CUDA events, L2 flushed between iterations).

    python -m coccl_b200.bench_kernels gemm --m 4096 --n 4096 --k 4096 [--iters 20]
    python -m coccl_b200.bench_kernels codec --codec sdp4bit --dtype fp32 --mib 1024
    python -m coccl_b200.bench_kernels collective --op reduce_scatter --ranks 8 --mib 256   (ranks emulated on one GPU)
    python -m coccl_b200.bench_kernels tp --ranks 2 --m 4096 --k 4096 --n 2048 [--tp-variant 1cta]   (emulated ranks)
    python -m coccl_b200.bench_kernels moe --ranks 4 --tokens 4096 --hidden 4096 --experts 32     (emulated ranks)

Also the small, self-ending workloads used for ncu captures (see profiles/).
"""
from __future__ import annotations

import argparse
import json

import torch

from .ops import codec as C
from .ops import collective as K
from .ops import gemm as G


def timed(fn, iters=20, warmup=5, flush_mib=256):
    dev = torch.device("cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    flush = torch.empty(flush_mib << 20, dtype=torch.uint8, device=dev)
    ts = []
    for _ in range(iters):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "codec", "collective", "tp", "moe", "train", "exchange"])
    ap.add_argument("--tp-variant", default="auto", choices=["auto", "1cta", "2cta"])
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--experts", type=int, default=32)
    ap.add_argument("--topk", type=int, default=2)
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--layout", default="tn", choices=["tn", "nn", "nt"])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--codec", default="sdp4bit", choices=["sdp4bit", "sdp4bit_sr", "mxfp8", "sdp8", "taco", "zfp4", "zfp8", "zfp16"])
    ap.add_argument("--dtype", default="fp32", choices=["fp32", "bf16"])
    ap.add_argument("--mib", type=int, default=256)
    ap.add_argument("--op", default="reduce_scatter")
    ap.add_argument("--ranks", type=int, default=8)
    ap.add_argument("--variant", default="auto", choices=["auto", "1cta", "2cta"])
    ap.add_argument("--cublas", action="store_true", help="time torch.matmul (cuBLAS) instead")
    a = ap.parse_args()
    dev = torch.device("cuda")
    dt = torch.float32 if a.dtype == "fp32" else torch.bfloat16
    cfgs = {"sdp4bit": C.SDP4BIT_G128, "sdp4bit_sr": C.CodecConfig("sdp4bit", 4, 128, False, True, True),
            "mxfp8": C.MXFP8, "sdp8": C.CodecConfig("sdp4bit", 8, 2048, False, False), "taco": C.TACO_G128,
            "zfp4": C.CodecConfig("zfp", 4, 4, False, False), "zfp8": C.ZFP_RATE8,
            "zfp16": C.CodecConfig("zfp", 16, 4, False, False)}
    out = {"what": a.what}
    if a.what == "gemm":
        G.set_variant(a.variant)
        x = torch.randn(a.m, a.k, device=dev, dtype=torch.bfloat16)
        w = torch.randn(a.n, a.k, device=dev, dtype=torch.bfloat16)
        if a.layout == "nn":      # dgrad-like: B stored [K, N]
            w = w.t().contiguous().t()
        if a.layout == "nt":      # wgrad-like: both operands stored with the contraction dimension outermost
            x = x.t().contiguous().t()
            w = w.t().contiguous().t()
        fn = (lambda: x @ w.t()) if a.cublas else (lambda: G.gemm(x, w))
        ms = timed(fn, a.iters, a.warmup)
        G.check_errors()
        out.update(m=a.m, n=a.n, k=a.k, layout=a.layout, impl="cublas" if a.cublas else "tcgen05-" + a.variant, ms=ms,
                   tflops=2 * a.m * a.n * a.k / ms / 1e9)
    elif a.what == "codec":
        cfg = cfgs[a.codec]
        n = (a.mib << 20) // (4 if dt == torch.float32 else 2)
        x = (torch.randn(n, device=dev) * 0.01).to(dt)
        enc = C.encode(x, cfg, 8)
        t_enc = timed(lambda: C.encode(x, cfg, 8), a.iters, a.warmup)
        t_dec = timed(lambda: C.decode(enc, cfg, n // 8, dt, 8), a.iters, a.warmup)
        t_red = timed(lambda: C.decode_reduce(enc, cfg, n // 8, dt, 1, 8), a.iters, a.warmup)
        raw = x.numel() * x.element_size()
        out.update(codec=a.codec, dtype=a.dtype, raw_mib=a.mib, encoded_bytes=enc.numel(),
                   encode_ms=t_enc, encode_gbs_traffic=(raw + enc.numel()) / t_enc / 1e6,
                   decode_ms=t_dec, decode_gbs_traffic=(raw + enc.numel()) / t_dec / 1e6,
                   decode_reduce8_ms=t_red, decode_reduce8_gbs_traffic=(raw / 8 + enc.numel()) / t_red / 1e6)
    elif a.what == "tp":
        # all-gather -> GEMM then GEMM -> FP8 reduce-scatter with every rank emulated on this GPU in one launch each
        # (each rank owns 1/ranks of the SMs, "peer" memory is local): per rank X shard [m, k], W_up [n, k], W_down [k, n]
        from .ops import tp_fused as T
        T.set_variant(a.tp_variant)
        n = a.ranks
        xs = [torch.randn(a.m, a.k, device=dev, dtype=torch.bfloat16) for _ in range(n)]
        ws = [torch.randn(a.n, a.k, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(n)]
        w2 = [torch.randn(a.k, a.n, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(n)]
        s1, s2, ep = {}, {}, [1]   # epochs must increase per workspace: the flags carry them
        ys, s1 = T.emulate_ag_gemm(xs, ws, state=s1, epoch=1, max_ctas=148 // n)
        torch.cuda.synchronize()

        def ag():
            ep[0] += 1
            T.emulate_ag_gemm(xs, ws, state=s1, epoch=ep[0], max_ctas=148 // n)

        def rs():
            ep[0] += 1
            T.emulate_gemm_rs(ys, w2, state=s2, epoch=ep[0], max_ctas=148 // n)
        t_ag = timed(ag, a.iters, a.warmup)
        var_ag = T.last_variant()
        t_rs = timed(rs, a.iters, a.warmup)
        T.check_state(s1)
        T.check_state(s2)
        fl = 2.0 * n * (a.m * n) * a.n * a.k
        out.update(ranks=n, m=a.m, n=a.n, k=a.k, variant=var_ag, ag_gemm_ms=t_ag, ag_gemm_tflops_all_ranks=fl / t_ag / 1e9,
                   gemm_rs_ms=t_rs, gemm_rs_tflops_all_ranks=fl / t_rs / 1e9,
                   note="all ranks emulated on one GPU: TFLOP/s over the whole device, no NVLink involved")
    elif a.what == "train":
        # the trainer's own kernels on one transformer layer's shapes: LayerNorm forward + backward (with the column sums of
        # the gamma / beta gradients), bias-gradient column sums (inside the linear's backward), cross-entropy forward +
        # backward, AdamW with fp32 master weights
        from .ops import fused as F_
        T_, H_ = a.tokens, a.hidden
        x = torch.randn(T_, H_, device=dev, dtype=torch.bfloat16, requires_grad=True)
        g = torch.ones(H_, device=dev, dtype=torch.bfloat16, requires_grad=True)
        b = torch.zeros(H_, device=dev, dtype=torch.bfloat16, requires_grad=True)
        dy = torch.randn(T_, H_, device=dev, dtype=torch.bfloat16)

        def ln():
            y = F_.layer_norm(x, g, b)
            y.backward(dy)
            x.grad = g.grad = b.grad = None
        w = torch.randn(a.n, H_, device=dev, dtype=torch.bfloat16, requires_grad=True) * 0.02
        w = w.detach().requires_grad_(True)
        wb = torch.zeros(a.n, device=dev, dtype=torch.bfloat16, requires_grad=True)
        xin = torch.randn(T_, H_, device=dev, dtype=torch.bfloat16)
        dz = torch.randn(T_, a.n, device=dev, dtype=torch.bfloat16)

        def lin():   # forward GEMM, then wgrad GEMM + bias-gradient column sum (no dgrad: the input needs no gradient)
            z = F_.linear(xin, w, wb)
            z.backward(dz)
            w.grad = wb.grad = None
        V_ = 50304
        logits = torch.randn(T_, V_, device=dev, dtype=torch.bfloat16, requires_grad=True)
        tgt = torch.randint(0, V_, (T_,), device=dev)

        def ce():
            loss = F_.cross_entropy(logits, tgt, 1.0 / T_)
            loss.backward()
            logits.grad = None
        np_ = 64 << 20
        master = torch.randn(np_, device=dev)
        m1, v1 = torch.zeros_like(master), torch.zeros_like(master)
        gr = torch.randn(np_, device=dev) * 1e-3
        pb = torch.empty(np_, device=dev, dtype=torch.bfloat16)
        step = [0]

        def adam():
            step[0] += 1
            F_.adam_step(master, m1, v1, gr, pb, lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step[0])
        t_ln, t_lin, t_ce, t_adam = (timed(f, a.iters, a.warmup) for f in (ln, lin, ce, adam))
        out.update(tokens=T_, hidden=H_, layer_norm_fwd_bwd_ms=t_ln, ln_gbs=(5 * T_ * H_ * 2) / t_ln / 1e6,
                   linear_fwd_wgrad_bias_ms=t_lin, cross_entropy_fwd_bwd_ms=t_ce, ce_gbs=(3 * T_ * V_ * 2) / t_ce / 1e6,
                   adam_64mi_params_ms=t_adam, adam_gbs=(np_ * (4 * 4 + 3 * 4 + 2)) / t_adam / 1e6,
                   note="GB/s = algorithmic bytes (LN: x, dy read twice + y, dx written; CE: logits read twice + gradient "
                        "written; Adam: master, m, v read and written, gradient read, bf16 parameter written)")
    elif a.what == "exchange":
        # peer-memory byte exchange of the staged pipeline, all ranks emulated on this GPU
        from .ops import exchange as X_
        n = a.ranks
        block = (a.mib << 20) // n // 16 * 16
        send = [torch.randint(0, 256, (n * block,), dtype=torch.uint8, device=dev) for _ in range(n)]
        st_, ep = {}, [0]

        def ex():
            ep[0] += 1
            X_.emulate(send, gather=False, frames=1, frame_stride=block, state=st_, epoch=ep[0], max_ctas=max(1, 296 // n))
        ms = timed(ex, a.iters, a.warmup)
        X_.check_state(st_)
        out.update(ranks=n, per_rank_mib=a.mib, ms=ms, copy_gbs_all_ranks=(2.0 * n * n * block * 2) / ms / 1e6,
                   note="all-to-all of per_rank_mib from every rank; every byte is stored into staging and copied out "
                        "(2 reads + 2 writes per byte), all ranks on one GPU, so GB/s is HBM traffic of the whole device")
    elif a.what == "moe":
        from .ops import moe as M
        n = a.ranks
        xs = [torch.randn(a.tokens, a.hidden, device=dev, dtype=torch.bfloat16) for _ in range(n)]
        ids, gates = [], []
        for r in range(n):
            top = torch.rand(a.tokens, a.experts, device=dev).topk(a.topk, dim=1)
            ids.append(top.indices.to(torch.int32).contiguous())
            gates.append(torch.softmax(top.values, dim=1).float().contiguous())
        state = {}
        recvs, hs, state = M.emulate_dispatch(xs, ids, a.experts, state=state)
        torch.cuda.synchronize()
        t_d = timed(lambda: M.emulate_dispatch(xs, ids, a.experts, state=state), a.iters, a.warmup)
        t_c = timed(lambda: M.emulate_combine(recvs, gates, hs, state=state), a.iters, a.warmup)
        M.check_state(state)
        rows = n * a.tokens * a.topk
        out.update(ranks=n, tokens=a.tokens, hidden=a.hidden, experts=a.experts, topk=a.topk, dispatch_ms=t_d,
                   combine_ms=t_c, dispatch_rows_gbs=rows * a.hidden * 2 / t_d / 1e6, combine_rows_gbs=rows * a.hidden * 2 / t_c / 1e6,
                   note="all ranks emulated on one GPU; GB/s = bf16 bytes of the routed rows over the time")
    else:
        cfg = cfgs[a.codec]
        n = a.ranks
        numel = (a.mib << 20) // (4 if dt == torch.float32 else 2)
        if a.op == "all_gather":
            numel //= n
        numel = numel // (n * 2048) * (n * 2048)
        xs = [(torch.randn(numel, device=dev) * 0.01).to(dt) for _ in range(n)]
        st, ep = {}, [0]

        def fn():
            ep[0] += 1
            K.emulate_collective(a.op, xs, cfg, state=st, epoch=ep[0])
        ms = timed(fn, a.iters, a.warmup)
        out.update(op=a.op, ranks=n, codec=a.codec, dtype=a.dtype, per_rank_input_mib=numel * xs[0].element_size() / 2**20,
                   ms=ms, status=K.status_codes(st),
                   note="all ranks emulated on one GPU: time covers the work of all ranks, HBM traffic only")
    print(json.dumps(out))


if __name__ == "__main__":
    main()
