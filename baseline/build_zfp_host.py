"""Build the reference's own ZFP (the LLNL library it vendors) for the HOST into baseline/_ref/zfp_host/libzfp.so.

The reference's ZFP plugin configures the library for one dimension and a fixed rate
(zfp/coccl_interface/zfp_plugin.cc:26-33: zfp_stream_set_rate(stream, rate, type, 1, false)) and runs its CUDA
execution policy; the same library's serial policy (zfp/src/zfp.c:1116-1135, template/encode1.c) writes the same
stream on the CPU. This script compiles those sources unmodified, without the CUDA back end, so that a CPU test can
demand that this library's ZFP stream equals real ZFP's bit for bit (tests/test_zfp_reference_stream_cpu.py).

Nothing is written next to the sources: one compiler command, objects in the compiler's temporary directory.

Usage:  python baseline/build_zfp_host.py [--src <reference checkout>]
(--src defaults to the directory `reference` beside this repository, or $COCCL_REFERENCE_SRC)
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref" / "zfp_host"
ZFP_SUBDIR = Path("src") / "coccl-extend" / "extensions" / "compressor_plugin" / "zfp"


def reference_dir(explicit: str | None = None) -> Path:
    return Path(explicit or os.environ.get("COCCL_REFERENCE_SRC") or HERE.parent.parent / "reference")


def library() -> Path:
    return OUT / "libzfp.so"


def build(src: Path | None = None, quiet: bool = False) -> Path | None:
    """Returns the library's path, or None when the reference's sources are not there."""
    zfp = (src or reference_dir()) / ZFP_SUBDIR
    sources = sorted((zfp / "src").glob("*.c"))
    if not sources:
        return None
    OUT.mkdir(parents=True, exist_ok=True)
    tmp = OUT / "libzfp.so.tmp"
    cmd = [os.environ.get("CC", "gcc"), "-std=c99", "-O2", "-fPIC", "-shared", f"-I{zfp / 'include'}", *map(str, sources),
           "-o", str(tmp), "-lm"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("building the reference's ZFP for the host failed:\n" + r.stderr[-4000:])
    os.replace(tmp, library())
    if not quiet:
        print(library())
    return library()


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--src", default=None)
    args = ap.parse_args()
    out = build(reference_dir(args.src))
    if out is None:
        print("reference sources not found", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
