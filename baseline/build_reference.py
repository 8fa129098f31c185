"""Build the unmodified reference (hpdps-group/COCCL) for sm_100 into baseline/_ref.

The reference is a C++/CUDA fork of NCCL 2.21.5 with no Python package, so it
cannot be pip-installed; its own make targets are driven here instead, the same
ones as examples/build_scripts/build.sh:33-45 of the reference:

  make src.build                       libnccl.so.2 with the COCCL runtime + the four codec plugins
  make -f src/coccl-extend/Makefile coccl-config-check
  make -C tests/coccl-tests            the nccl-tests style *_perf binaries (MPI=0: single process, -t N -g 1)

The sources are copied to a scratch directory first because the reference's
make writes generated files next to some sources; nothing in the copy is
edited.  Two settings differ from build.sh, both only a target architecture:
NVCC_GENCODE is compute_100/sm_100 (the library's default list stops at
compute_90, makefiles/common.mk:30-57), and the dietGPU plugin's cmake runs
through baseline/cmake_sm100.sh (make variable CMAKE), which swaps the
hard-coded COCCL_CUDA_ARCHITECTURES=80 of dietgpu/Makefile:30 for 100 and adds
the policy flag the vendored glog needs under a current CMake.

Usage:  python baseline/build_reference.py [--jobs N] [--src <reference checkout>] [--scratch /tmp/coccl_ref_src]
(--src defaults to the directory `reference` beside this repository, or $COCCL_REFERENCE_SRC)
Outputs under baseline/_ref/build: lib/libnccl.so.2, bin/coccl-config-check,
obj/coccl-extend/compressor_plugin/libcompress/lib{sdp4bit,taco,zfp,dietgpu}.so, tests/*_perf.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref" / "build"
GENCODE = "-gencode=arch=compute_100,code=sm_100"


def run(cmd, cwd=None, env=None, log=None):
    print("+", " ".join(map(str, cmd)), flush=True)
    t0 = time.time()
    r = subprocess.run(list(map(str, cmd)), cwd=cwd, env=env, stdout=log, stderr=subprocess.STDOUT)
    print(f"  exit {r.returncode} after {time.time() - t0:.0f} s", flush=True)
    return r.returncode


def prune() -> None:
    """Drop what only the build needed (objects, the static library): the tree travels to the GPU box with every run."""
    for p in list((OUT / "obj").rglob("*")):
        if p.is_file() and p.parent.name != "libcompress":
            p.unlink()
    for p in list((OUT / "tests").rglob("*.o")) + [OUT / "lib" / "libnccl_static.a"]:
        if p.exists():
            p.unlink()


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--jobs", type=int, default=os.cpu_count() or 4)
    ap.add_argument("--src", default=os.environ.get("COCCL_REFERENCE_SRC", str(Path(__file__).resolve().parents[2] / "reference")))
    ap.add_argument("--scratch", default="/tmp/coccl_ref_src")
    ap.add_argument("--cuda-home", default=os.environ.get("CUDA_HOME", "/usr/local/cuda"))
    a = ap.parse_args()

    scratch = Path(a.scratch)
    if not scratch.exists():
        shutil.copytree(a.src, scratch, symlinks=True, ignore=shutil.ignore_patterns(".git"))
    OUT.mkdir(parents=True, exist_ok=True)
    env = dict(os.environ, CUDA_HOME=a.cuda_home, NCCL_HOME=str(OUT))
    env["PATH"] = f"{a.cuda_home}/bin:" + env.get("PATH", "")
    logf = open(HERE / "_ref" / "build.log", "a")
    status = {}

    status["libnccl"] = run(["make", "-C", scratch, "-j", a.jobs, "src.build", "DEBUG=0", f"CUDA_HOME={a.cuda_home}",
                             f"BUILDDIR={OUT}", f"NVCC_GENCODE={GENCODE}", f"CMAKE={HERE / 'cmake_sm100.sh'}"], env=env, log=logf)

    status["config_check"] = run(["make", "-C", scratch, "-f", "src/coccl-extend/Makefile", "coccl-config-check",
                                  f"BUILDDIR={OUT}", f"NCCLDIR={scratch}", "COCCL_ROOT=src/coccl-extend",
                                  f"CUDA_HOME={a.cuda_home}"], env=env, log=logf)

    status["perf_tests"] = run(["make", "-C", scratch / "tests/coccl-tests", "-j", a.jobs, "DEBUG=0", "MPI=0",
                                f"CUDA_HOME={a.cuda_home}", f"NCCL_HOME={OUT}", f"BUILDDIR={OUT / 'tests'}",
                                f"NVCC_GENCODE={GENCODE}"], env=env, log=logf)
    if all(v == 0 for v in status.values()):
        prune()
    print(status)
    (HERE / "_ref" / "build_status.txt").write_text("".join(f"{k}={v}\n" for k, v in status.items()))
    return 0 if all(v == 0 for v in status.values()) else 1


if __name__ == "__main__":
    sys.exit(main())
