"""Codec error and throughput, this library's plugins next to the reference's own plugin binaries.

Both sets of `lib<name>.so` are loaded by the SAME host code: this library's compressor runtime
(csrc/compression/compressor_runtime.cc) through `cocclApiCodecRoundTrip`. The plugin ABI is the reference's
(include/compressor_plugin/detail/coccl_compressor_abi.h, version 8), so the reference's binaries, built unmodified
by baseline/build_reference.py, load as they are. Inputs are seeded and identical for both sides:

  * 4,194,304 fp32 values ~N(0,1), seed 0, one chunk (the CPU-slice configuration),
  * 64 Mi values ~N(0,1e-2) in fp32 and bf16, eight chunks (the collective sweep's data).

Per case: encoded bytes, max and RMS error of decode(encode(x)) against x, RMS relative to the RMS of x, and the
time of one compress+decompress round trip (host wall clock around n in-stream round trips between two device
synchronisations, minus the same call with one round, divided by n-1: allocation and set-up cancel; n is chosen
so that the measured call runs about 50 ms).

    python -m coccl_b200.bench_codec_parity [--reference-plugins baseline/_ref/build/obj/coccl-extend/compressor_plugin/libcompress]
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import time
from pathlib import Path

import torch

from . import _lib

NCCL_DT = {torch.float32: 7, torch.float16: 6, torch.bfloat16: 9}
ROOT = Path(__file__).resolve().parent
OURS = ROOT / "lib" / "plugins"
REF_DEFAULT = ROOT.parent / "baseline" / "_ref" / "build" / "obj" / "coccl-extend" / "compressor_plugin" / "libcompress"

# (label, ours: (plugin, options), reference: (plugin, options)); the reference's SDP4Bit always rounds
# stochastically, so this library's plugin is asked for the same
CASES = [
    ("sdp4bit q4 g128 hadamard (stochastic)",
     ("sdp4bit", "groupCount=128,quantBits=4,quantType=Symmetric,hadamard=true,rounding=stochastic"),
     ("sdp4bit", "groupCount=128,quantBits=4,quantType=Symmetric,hadamard=true")),
    ("sdp4bit q4 g128 hadamard (nearest, ours only)",
     ("sdp4bit", "groupCount=128,quantBits=4,quantType=Symmetric,hadamard=true,rounding=nearest"), None),
    ("sdp4bit q8 g2048", ("sdp4bit", "groupCount=2048,quantBits=8,quantType=Symmetric,rounding=stochastic"),
     ("sdp4bit", "groupCount=2048,quantBits=8,quantType=Symmetric")),
    ("taco e4m3 g128", ("taco", "fp8Format=E4M3,groupSize=128"), ("taco", "fp8Format=E4M3,groupSize=128")),
    ("fp8block (mx-fp8, ours only)", ("fp8block", ""), None),
    ("zfp rate 8", ("zfp", "rate=8"), ("zfp", "rate=8")),
    ("zfp rate 16", ("zfp", "rate=16"), ("zfp", "rate=16")),
    ("rANS probBits 10 (lossless)", ("ans", "probBits=10"), ("dietgpu", "probBits=10")),
]


def roundtrip(plugin_dir, name, options, x, chunks, rounds):
    fn = _lib.declare("cocclApiCodecRoundTrip", C.c_int,
                      [C.c_char_p, C.c_char_p, C.c_char_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_int,
                       C.c_size_t, C.c_int, C.POINTER(C.c_size_t), C.c_void_p])
    out = torch.empty_like(x)
    enc = C.c_size_t(0)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    rc = fn(str(plugin_dir).encode(), name.encode(), options.encode(), x.data_ptr(), out.data_ptr(), x.numel(), chunks,
            NCCL_DT[x.dtype], 1, rounds, C.byref(enc), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return rc, out, enc.value, time.perf_counter() - t0


def measure(plugin_dir, spec, x, chunks, rounds):
    name, options = spec
    rc, y, enc, t1 = roundtrip(plugin_dir, name, options, x, chunks, 1)
    if rc != 0:
        return {"error": f"round trip returned {rc}"}
    # a first estimate sizes the measured run to about 50 ms of round trips, so that the allocation and plugin
    # set-up inside the harness call (cancelled by the subtraction) do not drown a microsecond-scale kernel pair
    t1 = min(roundtrip(plugin_dir, name, options, x, chunks, 1)[3] for _ in range(3))
    tr = roundtrip(plugin_dir, name, options, x, chunks, rounds)[3]
    est = max((tr - t1) / (rounds - 1), 2e-6)
    n = int(min(max(0.05 / est, rounds), 2000))
    tn = min(roundtrip(plugin_dir, name, options, x, chunks, n)[3] for _ in range(2))
    d = (y.float() - x.float())
    rms_x = x.float().pow(2).mean().sqrt().item()
    per = max((tn - t1) / (n - 1), 1e-9)
    raw = x.numel() * x.element_size()
    return {"encoded_bytes": int(enc), "ratio": raw / max(enc, 1), "max_err": d.abs().max().item(),
            "rms_err": d.pow(2).mean().sqrt().item(), "rel_rms": d.pow(2).mean().sqrt().item() / rms_x,
            "roundtrip_ms": per * 1e3, "roundtrip_gbs": raw / per / 1e9}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference-plugins", default=str(REF_DEFAULT))
    ap.add_argument("--rounds", type=int, default=6)
    ap.add_argument("--big-elems", type=int, default=64 << 20)
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    dev = torch.device("cuda")
    ref_dir = Path(a.reference_plugins)
    have_ref = ref_dir.is_dir()
    g = torch.Generator(device=dev).manual_seed(0)
    inputs = [("fp32 4Mi N(0,1) 1 chunk", torch.randn(4194304, generator=g, device=dev), 1),
              ("fp32 N(0,1e-2) 8 chunks", torch.randn(a.big_elems, generator=g, device=dev) * 1e-2, 8)]
    inputs.append(("bf16 N(0,1e-2) 8 chunks", inputs[1][1].to(torch.bfloat16), 8))
    rows = []
    for label, ours, ref in CASES:
        for iname, x, chunks in inputs:
            row = {"codec": label, "input": iname, "ours": measure(OURS, ours, x, chunks, a.rounds)}
            if ref is not None:
                row["reference"] = measure(ref_dir, ref, x, chunks, a.rounds) if have_ref else {"error": "reference plugins not built"}
            rows.append(row)
            print(json.dumps(row), flush=True)
    if a.out:
        with open(a.out, "w") as f:
            json.dump({"rows": rows, "reference_plugins": str(ref_dir) if have_ref else None}, f, indent=1)


if __name__ == "__main__":
    main()
