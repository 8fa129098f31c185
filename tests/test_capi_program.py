"""A C program that knows only the NCCL API, linked against libcoccl_nccl.so: the drop-in surface
(32 nccl* names + their p-prefixed aliases, src/nccl.h.in:84-486 of the reference)."""
import os
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
LIB = ROOT / "coccl_b200" / "lib"
SRC = ROOT / "tests" / "capi" / "nccl_program.c"
CUDA = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))

NAMES = """AllGather AllReduce AllToAll Bcast Broadcast CommAbort CommCount CommCuDevice CommDeregister CommDestroy CommFinalize
CommGetAsyncError CommInitAll CommInitRank CommInitRankConfig CommRegister CommSplit CommUserRank GetErrorString GetLastError
GetUniqueId GetVersion GroupEnd GroupStart MemAlloc MemFree Recv RedOpCreatePreMulSum RedOpDestroy Reduce ReduceScatter Send""".split()


def _build(tmp_path):
    from coccl_b200 import _lib
    _lib.lib()   # builds the libraries if they are missing
    exe = tmp_path / "nccl_program"
    cmd = ["gcc", "-O1", str(SRC), "-o", str(exe), f"-I{CUDA}/include", f"-L{LIB}", "-lcoccl_nccl", f"-L{CUDA}/lib64", "-lcudart",
           "-lm", "-lpthread", f"-Wl,-rpath,{LIB}", f"-Wl,-rpath,{CUDA}/lib64"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def test_drop_in_library_exports_the_whole_nccl_surface():
    from coccl_b200 import _lib
    _lib.lib()
    out = subprocess.run(["nm", "-D", "--defined-only", str(LIB / "libcoccl_nccl.so")], capture_output=True, text=True).stdout
    have = {ln.split()[-1] for ln in out.splitlines() if ln.strip()}
    missing = [p + n for n in NAMES for p in ("nccl", "pnccl") if p + n not in have]
    assert not missing, missing
    for name in ("AllReduceCompOneShot", "AllReduceCompTwoShot", "AllReduceCompTripleShot", "ReduceScatterCompOneShot",
                 "ReduceScatterCompTwoShot", "AllGatherComp", "AllToAllComp", "SendComp", "RecvDecomp"):
        assert "pcoccl" + name in have


def test_c_program_links_and_answers_without_a_gpu(tmp_path):
    exe = _build(tmp_path)
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "version" in r.stdout


@pytest.mark.gpu
@pytest.mark.parametrize("enabled", [False, True])
def test_c_program_runs_collectives_through_the_drop_in_library(tmp_path, enabled):
    import torch
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs 2 GPUs")
    exe = _build(tmp_path)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", NCCL_DEBUG="WARN")
    if enabled:
        env.update(COCCL_ENABLE="1", COCCL_CONFIG_FILE=str(ROOT / "coccl_b200" / "configs" / "normal-sdp4bit.toml"))
    else:
        env.pop("COCCL_ENABLE", None)
    r = subprocess.run([str(exe), "run", "2"], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stdout + r.stderr
