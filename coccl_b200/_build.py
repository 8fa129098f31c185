"""In-tree build of the native parts of coccl_b200.

Produces, next to the sources (nothing goes to a JIT cache):
  coccl_b200/lib/libcoccl.so          host runtime (C++17) + sm_100a kernels, C ABI
  coccl_b200/lib/plugins/lib<name>.so  compressor plugins (one shared library per codec)
  coccl_b200/lib/coccl-config-check    TOML policy checker CLI
  coccl_b200/lib/coccl-perf            collective benchmark through the C API (one process, one thread per GPU)
  coccl_b200/lib/coccl_host_tests      host-only unit-test runner for the C++ runtime
  coccl_b200/_pg.so                    torch.distributed backend (built on demand, needs torch headers)

The reference builds the same split with make: COCCL host sources into
libnccl.so (src/Makefile:14-20, src/coccl-extend/Makefile:11-29), plugins and
coccl-config-check as separate targets (src/coccl-extend/Makefile:36-90).
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = ROOT / "lib"
OBJ = ROOT.parent / "build" / "obj"

NVCC = os.environ.get("NVCC", shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc")
CXX = os.environ.get("CXX", "g++")
CUDA_HOME = os.environ.get("CUDA_HOME", str(Path(NVCC).resolve().parent.parent))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--extended-lambda",
    "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function", "-I", str(CSRC), "-I", str(CSRC / "include"),
]
CXX_FLAGS = ["-O2", "-g", "-std=c++17", "-fPIC", "-Wall", "-Wno-unused-function", "-I", str(CSRC),
             "-I", str(CSRC / "include"), "-I", f"{CUDA_HOME}/include"]


def _newest_header_mtime() -> float:
    m = 0.0
    for pat in ("*.h", "*.cuh", "*.hpp"):
        for p in CSRC.rglob(pat):
            m = max(m, p.stat().st_mtime)
    return m


def _needs(src: Path, out: Path, hdr_mtime: float) -> bool:
    if not out.exists():
        return True
    t = out.stat().st_mtime
    return src.stat().st_mtime > t or hdr_mtime > t


def _link(cmd_before_out, out: Path, cmd_after_out, verbose):
    """Link into a temporary name and rename: a reader (a loader, a snapshot of the tree) never sees a half-written file."""
    tmp = out.with_name(out.name + ".tmp")
    _run([*cmd_before_out, tmp, *cmd_after_out], verbose)
    os.replace(tmp, out)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(map(str, cmd)), flush=True)
    r = subprocess.run(list(map(str, cmd)), capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"build step failed: {' '.join(map(str, cmd))}\n{r.stdout}\n{r.stderr}")
    return r


def _compile(src: Path, verbose: bool, hdr_mtime: float, extra=(), tag: str = "") -> Path:
    rel = src.relative_to(CSRC)
    out = OBJ / rel.with_suffix(rel.suffix + tag + ".o")
    out.parent.mkdir(parents=True, exist_ok=True)
    if _needs(src, out, hdr_mtime):
        if src.suffix == ".cu":
            _run([NVCC, *NVCC_FLAGS, *extra, "-c", src, "-o", out], verbose)
        else:
            _run([CXX, *CXX_FLAGS, *extra, "-c", src, "-o", out], verbose)
    return out


# Sources of libcoccl.so: every .cu under kernels/ and every .cc of the host runtime.
LIB_DIRS = ["kernels", "config", "runtime", "training", "tuning", "pipeline", "memory", "compression", "symm",
            "api", "oracle"]
PLUGIN_DIR = CSRC / "codecs"
TOOLS_DIR = CSRC / "tools"
TESTS_DIR = CSRC / "tests"


def _lib_sources():
    srcs = []
    for d in LIB_DIRS:
        p = CSRC / d
        if p.is_dir():
            srcs += sorted(p.glob("*.cu")) + sorted(p.glob("*.cc"))
    return srcs


def build(verbose: bool = False, jobs: int | None = None) -> Path:
    """Compile everything that is out of date; returns the path of libcoccl.so."""
    LIB.mkdir(exist_ok=True)
    (LIB / "plugins").mkdir(exist_ok=True)
    hdr = _newest_header_mtime()
    jobs = jobs or max(1, (os.cpu_count() or 2))
    srcs = _lib_sources()
    with cf.ThreadPoolExecutor(jobs) as ex:
        objs = list(ex.map(lambda s: _compile(s, verbose, hdr), srcs))
    so = LIB / "libcoccl.so"
    if not so.exists() or any(o.stat().st_mtime > so.stat().st_mtime for o in objs):
        _link([NVCC, "-shared", "-o"], so, [*objs, "-ldl", "-lpthread", "-Xlinker", "--no-undefined"], verbose)

    # bounds-checked twin (COCCL_CHECKED_KERNELS=1 makes the Python layer load it): the same objects, except that the
    # translation units with the codec accesses are compiled with -DCOCCL_BOUNDS_CHECK
    checked_units = {CSRC / "kernels" / "collective_kernels.cu", CSRC / "kernels" / "codec_kernels.cu"}
    with cf.ThreadPoolExecutor(jobs) as ex:
        cobjs = list(ex.map(lambda s: _compile(s, verbose, hdr, ("-DCOCCL_BOUNDS_CHECK",), ".checked"), sorted(checked_units)))
    cso = LIB / "libcoccl_checked.so"
    rest = [o for s_, o in zip(srcs, objs) if s_ not in checked_units]
    if not cso.exists() or any(o.stat().st_mtime > cso.stat().st_mtime for o in cobjs + rest):
        _link([NVCC, "-shared", "-o"], cso, [*cobjs, *rest, "-ldl", "-lpthread", "-Xlinker", "--no-undefined"], verbose)

    # plugins: one shared library per codec source
    if PLUGIN_DIR.is_dir():
        def plug(src: Path):
            name = src.stem.replace("_plugin", "")
            out = LIB / "plugins" / f"lib{name}.so"
            if _needs(src, out, hdr):
                _link([NVCC, *NVCC_FLAGS, "-shared", src, "-o"], out, [f"-L{LIB}", "-lcoccl",
                      "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/.."], verbose)
            return out
        with cf.ThreadPoolExecutor(jobs) as ex:
            list(ex.map(plug, sorted(PLUGIN_DIR.glob("*_plugin.cu"))))

    # tools and the host-test runner link against libcoccl.so
    rpath = ["-Wl,-rpath,$ORIGIN", f"-L{LIB}", "-lcoccl"]
    shim = CSRC / "shim" / "nccl_shim.cc"
    if shim.exists():
        out = LIB / "libcoccl_nccl.so"
        if _needs(shim, out, hdr) or so.stat().st_mtime > out.stat().st_mtime:
            _link([CXX, *CXX_FLAGS, "-shared", shim, "-o"], out, rpath, verbose)
    if TOOLS_DIR.is_dir():
        for src in sorted(TOOLS_DIR.glob("*.cc")):
            out = LIB / src.stem.replace("_", "-")
            if _needs(src, out, hdr) or so.stat().st_mtime > out.stat().st_mtime:
                _link([CXX, *CXX_FLAGS, src, "-o"], out, [*rpath, f"-L{CUDA_HOME}/lib64", "-lcudart", "-ldl", "-lpthread",
                                                         f"-Wl,-rpath,{CUDA_HOME}/lib64"], verbose)
    if TESTS_DIR.is_dir():
        tsrcs = sorted(TESTS_DIR.glob("*.cc"))
        if tsrcs:
            out = LIB / "coccl_host_tests"
            if any(_needs(s, out, hdr) for s in tsrcs) or so.stat().st_mtime > out.stat().st_mtime:
                _link([CXX, *CXX_FLAGS, *tsrcs, "-o"], out, [*rpath, "-ldl", "-lpthread"], verbose)
    return so


def build_torch_backend(verbose: bool = False) -> Path | None:
    """Compile the c10d backend (csrc/torch/*.cpp) against the installed torch headers."""
    tdir = CSRC / "torch"
    srcs = sorted(tdir.glob("*.cpp")) if tdir.is_dir() else []
    if not srcs:
        return None
    import sysconfig
    import torch
    from torch.utils import cpp_extension as ce

    out = ROOT / "_pg.so"
    hdr = _newest_header_mtime()
    so = LIB / "libcoccl.so"
    if not any(_needs(s, out, hdr) for s in srcs) and out.stat().st_mtime >= so.stat().st_mtime:
        return out
    inc = []
    for p in ce.include_paths():
        inc += ["-I", p]
    inc += ["-I", sysconfig.get_paths()["include"], "-I", f"{CUDA_HOME}/include"]
    tlib = str(Path(torch.__file__).parent / "lib")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = [CXX, "-O2", "-std=c++17", "-fPIC", "-shared", f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DTORCH_EXTENSION_NAME=_pg",
           "-DUSE_C10D_NCCL", "-DUSE_CUDA", "-I", str(CSRC), "-I", str(CSRC / "include"), *inc, *srcs, "-o", out,
           f"-L{tlib}", "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_python", "-ltorch_cuda", "-lc10_cuda",
           f"-L{LIB}", "-lcoccl", f"-Wl,-rpath,{tlib}", "-Wl,-rpath,$ORIGIN/lib"]
    _run(cmd, verbose)
    return out


if __name__ == "__main__":
    v = "-v" in sys.argv
    print(build(verbose=v))
    if "--torch" in sys.argv:
        print(build_torch_backend(verbose=v))
