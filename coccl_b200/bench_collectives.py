"""Compressed-collective sweep: effective GB/s against message size, fused kernels vs native NCCL.

Launch with one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29511 \
        -m coccl_b200.bench_collectives --min-mib 1 --max-mib 1024 --out sweep.json

Bandwidth follows the reference harness (tests/coccl-tests/doc/PERFORMANCE.md:16-145,
tests/coccl-tests/src/all_reduce_comp_twoshot.cu:42-48, all_gather_comp.cu:62-68, alltoall_comp.cu:60-66): it is
computed on UNCOMPRESSED logical bytes, algbw = S / t, busbw = algbw * 2(N-1)/N for all-reduce and
algbw * (N-1)/N for reduce-scatter / all-gather / all-to-all, with S the all-reduce buffer or the N-rank total.
Unlike the reference harness (host wall clock) every call is timed with CUDA events on the launching stream;
a barrier precedes each timed call, L2 is flushed between calls, and the reported time is the median over
iterations of the maximum over ranks.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from .parallel.comm import NATIVE, Communicator, Policy

# name -> (compressor plugin, its options): what a user would write in the policy file. sdp4bit rounds to nearest,
# sdp4bit_sr stochastically (the reference's SDP4Bit has only the stochastic mode).
_SDP = {"groupCount": 128, "quantBits": 4, "quantType": "Symmetric", "hadamard": True}
CODECS = {"sdp4bit": ("sdp4bit", dict(_SDP, rounding="nearest")), "sdp4bit_sr": ("sdp4bit", dict(_SDP, rounding="stochastic")),
          "mxfp8": ("fp8block", {}), "taco": ("taco", {"fp8Format": "E4M3", "groupSize": 128}), "zfp8": ("zfp", {"rate": 8})}
OPS = ("all_reduce", "reduce_scatter", "all_gather", "all_to_all")


def _policy(codec, threshold: int, autotune: bool) -> Policy:
    """A normal-mode policy file with this codec on every collective; the all-reduce algorithm is left to the selector,
    which (with autotune) is fed one-shot / two-shot timings of this group at the first call."""
    name, options = codec
    return Policy.normal(name, options, threshold_bytes=threshold, autotune=autotune)


def _buffers(op: str, total_bytes: int, dtype, n: int, dev):
    """(input, output) for a call whose logical size S is `total_bytes`."""
    es = torch.empty(0, dtype=dtype).element_size()
    unit = n * 2048
    if op == "all_reduce":
        numel = max(unit, total_bytes // es // unit * unit)
        x = (torch.randn(numel, device=dev) * 1e-2).to(dtype)
        return x, x
    per = max(2048, total_bytes // es // n // 2048 * 2048)
    if op == "reduce_scatter":
        return (torch.randn(per * n, device=dev) * 1e-2).to(dtype), torch.empty(per, device=dev, dtype=dtype)
    if op == "all_gather":
        return (torch.randn(per, device=dev) * 1e-2).to(dtype), torch.empty(per * n, device=dev, dtype=dtype)
    return (torch.randn(per * n, device=dev) * 1e-2).to(dtype), torch.empty(per * n, device=dev, dtype=dtype)


def _call(comm: Communicator, op: str, inp, out):
    if op == "all_reduce":
        comm.all_reduce(inp)
    elif op == "reduce_scatter":
        comm.reduce_scatter(inp, out)
    elif op == "all_gather":
        comm.all_gather(inp, out)
    else:
        comm.all_to_all(inp, out)


def _time(comm: Communicator, op: str, inp, out, iters: int, warmup: int, flush) -> float:
    for _ in range(warmup):
        _call(comm, op, inp, out)
    torch.cuda.synchronize()
    tok = torch.zeros(1, device=inp.device)
    ts = torch.zeros(iters, device=inp.device)
    evs = []
    for _ in range(iters):
        flush.zero_()
        dist.all_reduce(tok)  # lines the ranks up; not timed
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        _call(comm, op, inp, out)
        b.record()
        evs.append((a, b))
    torch.cuda.synchronize()
    for i, (a, b) in enumerate(evs):
        ts[i] = a.elapsed_time(b)
    dist.all_reduce(ts, op=dist.ReduceOp.MAX)
    return float(ts.median().item())


def _reference(a) -> None:
    """The stock binaries of the reference, built by baseline/build_reference.py, with the same sizes, dtypes and
    bandwidth convention. Cases whose programs faulted or hung on this hardware print an `unavailable` line."""
    import subprocess
    import sys
    from pathlib import Path
    runner = Path(__file__).resolve().parent.parent / "baseline" / "run_reference.py"
    if not runner.exists():
        print(json.dumps({"impl": "reference", "unavailable": "baseline/run_reference.py is not in this checkout"}))
        return
    def size(mib):
        return f"{int(mib * 1024)}K" if mib < 1 else (f"{int(mib)}M" if mib < 1024 else f"{int(mib // 1024)}G")
    cmd = [sys.executable, str(runner), "--gpus", str(a.gpus), "--min", size(a.min_mib), "--max", size(a.max_mib),
           "--ops", a.ops, "--dtypes", a.dtypes, "--warmup", str(max(a.warmup, 5)), "--iters", str(max(a.iters, 20))]
    if a.out:
        cmd += ["--out", a.out]
    subprocess.run(cmd, check=False)


def table(path: str, min_mib: float) -> None:
    """Markdown table of a sweep written with --out: time per codec, speed-up over NCCL and bus bandwidth."""
    with open(path) as f:
        d = json.load(f)
    names = [k[:-3] for k in d["rows"][0] if k.endswith("_ms") and k != "native_ms"]
    head = ["op", "dtype", "MiB", "native ms"] + [f"{n} ms" for n in names] + [f"{n} x" for n in names] + \
           ["native busbw"] + [f"{n} busbw" for n in names]
    print("| " + " | ".join(head) + " |")
    print("|" + "---|" * len(head))
    for r in d["rows"]:
        mib = r["bytes"] / (1 << 20)
        if mib < min_mib:
            continue
        cells = [r["op"], r["dtype"], f"{mib:g}", f"{r['native_ms']:.3f}"]
        cells += [f"{r[n + '_ms']:.3f}" for n in names]
        cells += [f"{r['native_ms'] / r[n + '_ms']:.2f}" for n in names]
        cells += [f"{r['native_busbw_gbs']:.0f}"] + [f"{r[n + '_busbw_gbs']:.0f}" for n in names]
        print("| " + " | ".join(cells) + " |")
    for name, info in d.get("routing", {}).items():
        log = info.get("measured") if isinstance(info, dict) else None
        if log:
            print(f"\nselector input measured by communicator '{name}' (policy {info.get('policy_hash')}):")
            for m in log:
                times = ", ".join(f"{k[:-3]} {v:.1f} us" for k, v in m.items() if k.endswith("_us"))
                print(f"  {m['what']} {m['dtype'].replace('torch.', '')} {m['bytes'] / (1 << 20):g} MiB: {times}")
            break


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--min-mib", type=float, default=1)
    ap.add_argument("--max-mib", type=float, default=1024)
    ap.add_argument("--ops", default=",".join(OPS))
    ap.add_argument("--codecs", default="sdp4bit,mxfp8")
    ap.add_argument("--dtypes", default="fp32,bf16")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--out", default="")
    ap.add_argument("--threshold", type=int, default=0, help="compression_threshold_bytes of the policy (0: every size compressed)")
    ap.add_argument("--no-autotune", action="store_true", help="selector heuristics instead of measured one-/two-shot times")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"],
                    help="reference: run the reference's own stock *_perf binaries (baseline/run_reference.py), "
                         "nothing of this library; launch WITHOUT torchrun, with --gpus N")
    ap.add_argument("--gpus", type=int, default=2, help="--impl reference only: ranks of the single-process run")
    ap.add_argument("--table", default="", metavar="JSON", help="print the markdown table of an earlier --out file and exit")
    ap.add_argument("--table-min-mib", type=float, default=16)
    a = ap.parse_args()
    if a.table:
        return table(a.table, a.table_min_mib)
    if a.impl == "reference":
        return _reference(a)

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(1234 + rank)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    comms = {"native": Communicator(None, dev, NATIVE, "native")}
    for c in a.codecs.split(","):
        comms[c] = Communicator(None, dev, _policy(CODECS[c], a.threshold, not a.no_autotune), c)
    dts = {"fp32": torch.float32, "bf16": torch.bfloat16}
    rows = []
    size = a.min_mib
    sizes = []
    while size <= a.max_mib:
        sizes.append(int(size * (1 << 20)))
        size *= 2
    for op in a.ops.split(","):
        bus = (2.0 * (world - 1) / world) if op == "all_reduce" else ((world - 1) / world)
        for dn in a.dtypes.split(","):
            for S in sizes:
                inp, out = _buffers(op, S, dts[dn], world, dev)
                logical = (inp.numel() if op != "all_gather" else out.numel()) * inp.element_size()
                row = {"op": op, "dtype": dn, "bytes": logical, "n_gpus": world}
                for name, comm in comms.items():
                    ms = _time(comm, op, inp, out, a.iters, a.warmup, flush)
                    row[name + "_ms"] = ms
                    row[name + "_algbw_gbs"] = logical / ms / 1e6
                    row[name + "_busbw_gbs"] = logical / ms / 1e6 * bus
                for name in comms:
                    if name != "native":
                        row[name + "_speedup"] = row["native_ms"] / row[name + "_ms"]
                        st = comms[name].status()
                        if st:
                            row[name + "_status"] = st
                rows.append(row)
                if rank == 0:
                    print(json.dumps(row), flush=True)
                del inp, out
    if rank == 0 and a.out:
        with open(a.out, "w") as f:
            json.dump({"n_gpus": world, "timing": "cuda events, max over ranks, median of %d, L2 flushed" % a.iters,
                       "routing": {name: c.routing_summary() for name, c in comms.items()},
                       "rows": rows}, f, indent=1)
    for c in comms.values():
        c.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
