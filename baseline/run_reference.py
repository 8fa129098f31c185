"""Drive the reference's own stock benchmark binaries (built by baseline/build_reference.py) and collect their tables.

What runs is exactly what examples/benchmarks_scripts/communication_benchmarks.sh of the reference runs on one
node (`run_case`, lines 57-90): the nccl-tests style `*_perf` programs in single-process mode (`-t N -g 1`),
`-c 0` (no data check, the codecs are lossy), `-f 2` size steps, NCCL_BUFFSIZE=16 MiB, autotune off, first with
COCCL_ENABLE=0 (native NCCL 2.21.5 of the reference) and then with COCCL_ENABLE=1 and a policy file per codec.
Nothing of this repository's kernels or runtime is on that path: the binaries link the reference's libnccl.so.2
and dlopen the reference's plugins.

Policies follow the benchmark configuration this repository is measured on: SDP4Bit 4 bit, groups of 128,
symmetric, Hadamard rotation (the all-reduce uses hadamard=false, as the reference's own benchmark policy does,
examples/benchmarks_scripts/configs/sdp4bit.toml:27-49: its fused decompress-reduce-compress kernel has no
rotated variant, sdp4bit_quan.cu:265-268); ZFP fixed rate 8; TACO E4M3 groups of 128 as the reference's FP8
codec; threshold 8 MiB; pipeline.depth 4 (which the reference forces to 1 on one node for unframed codecs,
coccl_pipeline_execute.cc:545-550).

Output: one JSON line per (op, codec, dtype, size) on stdout and, with --out, one JSON file:
  {"op", "impl": "reference", "codec": "native" | "sdp4bit" | "zfp" | "taco", "dtype", "n_gpus", "bytes",
   "ms", "algbw_gbs", "busbw_gbs", "timing": "host wall clock / iterations, max over ranks (-a 3)"}
A binary that exits non-zero or runs into its time limit is recorded as {"unavailable": reason} for that case
and is not started again.

Observed on 2 x B200 (driver 580, CUDA 12.9; log kept in profiles/reference_collectives_2gpu.md): the reference's
NCCL 2.21.5 core predates this architecture and its own collective kernels do not run here. Native
`all_reduce_perf` and `reduce_scatter_perf` stop with "an illegal memory access was encountered", native
`all_gather_perf` and the compressed reduce-scatter / all-to-all / all-reduce programs never finish, the compressed
all-gather faults like the native one. Only the send/receive based `alltoall_p2p_perf` completes. Code that
faulted or hung a GPU is not started again: CLOSED below turns those cases into `unavailable` lines without
launching anything, and the compressed programs that were not reached before the call ended are closed with
them because they drive the same NCCL kernels.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent
BUILD = HERE / "_ref" / "build"
PLUGINS = BUILD / "obj" / "coccl-extend" / "compressor_plugin" / "libcompress"
TESTS = BUILD / "tests"

NATIVE_BIN = {"all_reduce": "all_reduce_perf", "reduce_scatter": "reduce_scatter_perf", "all_gather": "all_gather_perf",
              "all_to_all": "alltoall_p2p_perf"}
COMP_BIN = {"all_reduce": "all_reduce_comp_twoshot_perf", "reduce_scatter": "reduce_scatter_comp_oneshot_perf",
            "all_gather": "all_gather_comp_perf", "all_to_all": "alltoall_comp_perf",
            "all_reduce_oneshot": "all_reduce_comp_oneshot_perf"}
TOML_OP = {"all_reduce": "all_reduce", "reduce_scatter": "reduce_scatter", "all_gather": "all_gather",
           "all_to_all": "all_to_all"}
DTYPE_FLAG = {"fp32": "float", "bf16": "bfloat16", "fp16": "half"}

_ILLEGAL = "reference NCCL 2.21.5 kernel faults on B200: 'an illegal memory access was encountered' (common.cu:304)"
_HANG = "reference program did not finish within 120 s on B200 (1 MiB - 64 MiB, 2 GPUs)"
_SAME = "not started: it drives the same reference NCCL kernels and runtime that faulted or hung on B200"
# (codec or "*" for every compressed codec, op) -> why the case is closed on B200
CLOSED = {
    ("native", "all_reduce"): _ILLEGAL, ("native", "reduce_scatter"): _ILLEGAL, ("native", "all_gather"): _HANG,
    ("sdp4bit", "all_reduce"): "reference all_reduce_comp_twoshot_perf exited 2 before its first table row on B200",
    ("sdp4bit", "reduce_scatter"): _HANG, ("sdp4bit", "all_gather"): _ILLEGAL, ("sdp4bit", "all_to_all"): _HANG,
    ("zfp", "all_reduce"): _HANG,
    ("*", "all_reduce"): _SAME, ("*", "reduce_scatter"): _SAME, ("*", "all_gather"): _SAME, ("*", "all_to_all"): _SAME,
}


def closed_reason(codec: str, op: str):
    if (codec, op) in CLOSED:
        return CLOSED[(codec, op)]
    if codec != "native" and ("*", op) in CLOSED:
        return CLOSED[("*", op)]
    return None


def codec_options(codec: str, op: str, stochastic_note: list) -> dict:
    if codec == "sdp4bit":
        # the reference always rounds stochastically (quantization_utils.h:153-174); there is no switch
        return {"groupCount": 128, "quantBits": 4, "quantType": '"Symmetric"',
                "hadamard": "false" if op == "all_reduce" else "true"}
    if codec == "zfp":
        return {"rate": 8}
    if codec == "taco":
        return {"fp8Format": '"E4M3"', "groupSize": 128}
    if codec == "dietgpu":
        return {"probBits": 10}
    raise ValueError(codec)


def write_policy(path: Path, codec: str, threshold: int, depth: int) -> None:
    lines = ["[runtime]", 'mode = "normal"', f"compression_threshold_bytes = {threshold}", "",
             "[compressor_plugins]", f'compressors = ["{codec}"]', f'library_path = "{PLUGINS}"', "",
             "[pipeline]", f"depth = {depth}", "", "[autotune]", "enabled = false", ""]
    for op in ("all_to_all", "all_gather", "all_reduce", "reduce_scatter"):
        scopes = ("default",) if op in ("all_to_all", "all_gather") else ("default", "intra", "inter")
        for scope in scopes:
            lines += [f"[normal.{op}.{scope}]", f'compressor = "{codec}"', "", f"[normal.{op}.{scope}.config]"]
            lines += [f"{k} = {v}" for k, v in codec_options(codec, op, []).items()]
            lines.append("")
    path.write_text("\n".join(lines))


def parse_table(text: str):
    """Rows of the nccl-tests table: size count type redop root | time algbw busbw #wrong | (in place) ..."""
    rows = []
    for ln in text.splitlines():
        f = ln.split()
        if len(f) < 9 or ln.lstrip().startswith("#"):
            continue
        try:
            size, t_us, algbw, busbw = int(f[0]), float(f[5]), float(f[6]), float(f[7])
        except ValueError:
            continue
        rows.append((size, t_us, algbw, busbw))
    return rows


def run_case(binary: str, n: int, dtype: str, lo: str, hi: str, warmup: int, iters: int, env: dict, limit_s: int):
    cmd = [str(TESTS / binary), "-b", lo, "-e", hi, "-f", "2", "-g", "1", "-t", str(n), "-w", str(warmup), "-n", str(iters),
           "-c", "0", "-a", "3", "-d", DTYPE_FLAG[dtype]]
    t0 = time.time()
    try:
        r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=limit_s)
    except subprocess.TimeoutExpired as e:
        return None, f"{binary} did not finish within {limit_s} s", (e.stdout or "")[-2000:] if isinstance(e.stdout, str) else ""
    out = r.stdout + "\n" + r.stderr
    if r.returncode != 0:
        return None, f"{binary} exited {r.returncode}", out[-2000:]
    rows = parse_table(r.stdout)
    if not rows:
        return None, f"{binary} printed no table", out[-2000:]
    return rows, f"{time.time() - t0:.0f} s", out[-400:]


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=2)
    ap.add_argument("--min", default="1M")
    ap.add_argument("--max", default="1G")
    ap.add_argument("--ops", default="all_reduce,reduce_scatter,all_gather,all_to_all")
    ap.add_argument("--codecs", default="native,sdp4bit,zfp,taco")
    ap.add_argument("--dtypes", default="fp32,bf16")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--depth", type=int, default=4)
    ap.add_argument("--threshold", type=int, default=8 << 20)
    ap.add_argument("--case-limit-s", type=int, default=240)
    ap.add_argument("--time-limit-s", type=int, default=1500, help="stop starting new cases after this many seconds")
    ap.add_argument("--out", default="")
    ap.add_argument("--log", default="")
    a = ap.parse_args()

    if not (TESTS / "all_reduce_perf").exists():
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not built (python baseline/build_reference.py)"}))
        return 0
    base_env = dict(os.environ)
    base_env["LD_LIBRARY_PATH"] = f"{BUILD / 'lib'}:/usr/local/cuda/lib64:" + base_env.get("LD_LIBRARY_PATH", "")
    base_env.setdefault("NCCL_DEBUG", "WARN")
    base_env.setdefault("NCCL_BUFFSIZE", str(16 << 20))
    tmp = Path(tempfile.mkdtemp(prefix="coccl_ref_cfg_"))
    rows, dead = [], {}
    t_start = time.time()
    logf = open(a.log, "a") if a.log else None
    for codec in a.codecs.split(","):
        env = dict(base_env)
        if codec == "native":
            env["COCCL_ENABLE"] = "0"
            env.pop("COCCL_CONFIG_FILE", None)
        else:
            cfg = tmp / f"{codec}-d{a.depth}.toml"
            write_policy(cfg, codec, a.threshold, a.depth)
            env["COCCL_ENABLE"] = "1"
            env["COCCL_CONFIG_FILE"] = str(cfg)
        for op in a.ops.split(","):
            binary = (NATIVE_BIN if codec == "native" else COMP_BIN)[op]
            for dt in a.dtypes.split(","):
                key = (codec, op)
                if closed_reason(codec, op) is not None:
                    reason, res, tail = closed_reason(codec, op), None, ""
                elif time.time() - t_start > a.time_limit_s:
                    reason = "not run: the time limit of this call was reached"
                    res, tail = None, ""
                elif key in dead:
                    reason, res, tail = dead[key], None, ""
                else:
                    res, reason, tail = run_case(binary, a.gpus, dt, a.min, a.max, a.warmup, a.iters, env, a.case_limit_s)
                    if res is None:
                        dead[key] = reason + " (not started again)"
                if logf:
                    logf.write(f"=== {codec} {op} {dt} n={a.gpus}: {reason}\n{tail}\n")
                    logf.flush()
                if res is None:
                    row = {"op": op, "impl": "reference", "codec": codec, "dtype": dt, "n_gpus": a.gpus, "unavailable": reason}
                    rows.append(row)
                    print(json.dumps(row), flush=True)
                    continue
                for size, t_us, algbw, busbw in res:
                    row = {"op": op, "impl": "reference", "codec": codec, "dtype": dt, "n_gpus": a.gpus, "bytes": size,
                           "ms": t_us / 1e3, "algbw_gbs": algbw, "busbw_gbs": busbw}
                    rows.append(row)
                    print(json.dumps(row), flush=True)
    if a.out:
        with open(a.out, "w") as f:
            json.dump({"impl": "reference", "n_gpus": a.gpus,
                       "timing": "reference harness: host wall clock over iterations (enqueue + stream sync), max over ranks (-a 3)",
                       "protocol": {"warmup": a.warmup, "iters": a.iters, "depth": a.depth, "threshold": a.threshold,
                                    "NCCL_BUFFSIZE": base_env["NCCL_BUFFSIZE"]},
                       "rows": rows}, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
