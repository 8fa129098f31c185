"""C++ host runtime: runs the host-only unit-test binary (config, SDK, router, group, planner, frame
exchange, buffer manager with fake CUDA, autotune, training classifier) and the coccl-config-check CLI
on the shipped policy files. No GPU needed."""
import os
import re
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
LIB = ROOT / "coccl_b200" / "lib"


@pytest.fixture(scope="module")
def built():
    from coccl_b200 import _build
    _build.build()
    return LIB


def _run_host_tests(built):
    r = subprocess.run([str(built / "coccl_host_tests")], capture_output=True, text=True, timeout=300)
    return r, re.findall(r"^\[( OK |FAIL)\] (\S+)$", r.stdout, flags=re.M)


def test_host_unit_tests_all_pass(built):
    r, cases = _run_host_tests(built)
    failed = [name for status, name in cases if status == "FAIL"]
    assert r.returncode == 0 and not failed, f"failed: {failed}\n{r.stdout[-3000:]}\n{r.stderr[-3000:]}"
    assert len(cases) >= 40


@pytest.mark.parametrize("name", ["normal-sdp4bit.toml", "normal-fp8block.toml", "normal-mixed.toml", "training.toml",
                                  "normal-zfp-sdp4bit.toml", "normal-taco-ans.toml"])
def test_config_check_accepts_shipped_configs(built, name):
    r = subprocess.run([str(built / "coccl-config-check"), str(ROOT / "coccl_b200" / "configs" / name)],
                       capture_output=True, text=True, timeout=60)
    assert r.returncode == 0, r.stderr
    assert "# OK (2 nodes x 8 devices)" in r.stdout
    assert "runtime.mode = " in r.stdout


def test_config_check_exit_codes(built, tmp_path):
    exe = str(built / "coccl-config-check")
    assert subprocess.run([exe], capture_output=True).returncode == 2
    assert subprocess.run([exe, "--nodes"], capture_output=True).returncode == 2
    bad = tmp_path / "bad.toml"
    bad.write_text('[runtime]\nmode = "normal"\n[pipeline]\ndepth = 99\n')
    r = subprocess.run([exe, str(bad)], capture_output=True, text=True)
    assert r.returncode == 1 and "pipeline.depth" in r.stderr
    # options a codec does not know are rejected when the plugin parses them
    plug = tmp_path / "p.toml"
    plug.write_text('[runtime]\nmode = "normal"\n[compressor_plugins]\ncompressors = ["sdp4bit"]\n'
                    f'library_path = "{LIB / "plugins"}"\n[normal.all_reduce.default]\ncompressor = "sdp4bit"\n'
                    '[normal.all_reduce.default.config]\nquantBitz = 4\n')
    r = subprocess.run([exe, "--nodes", "1", "--devices-per-node", "8", str(plug)], capture_output=True, text=True)
    assert r.returncode == 1 and "quantBitz" in r.stderr
    plug.write_text(plug.read_text().replace("quantBitz = 4", "subAdd = true\nhadamard = true"))
    r = subprocess.run([exe, str(plug)], capture_output=True, text=True)
    assert r.returncode == 1 and "subAdd" in r.stderr


def test_baseline_config_one_cpu_slice(built):
    """CPU-only slice: coccl-config-check parses a normal-mode policy (threshold 1 MiB, depth 4, all_reduce ->
    zfp rate 8, reduce_scatter -> sdp4bit) and the SDP4Bit CPU reference round trip runs on a seed-0 fp32 tensor
    of 4,194,304 N(0,1) values (group 128, 4 bits, symmetric, Hadamard); report max / RMS error."""
    import ctypes as C
    import torch
    from coccl_b200 import _lib
    from coccl_b200.ops.codec import CodecConfig, reference_roundtrip
    r = subprocess.run([str(built / "coccl-config-check"), "--nodes", "1", "--devices-per-node", "8",
                        str(ROOT / "coccl_b200" / "configs" / "normal-zfp-sdp4bit.toml")], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    for needle in ("compression_threshold_bytes = 1048576", "pipeline.depth = 4", "zfp", "rate", "sdp4bit", "hadamard"):
        assert needle in r.stdout, needle
    g = torch.Generator().manual_seed(0)
    x = torch.randn(4_194_304, generator=g)
    # the C++ oracle of libcoccl.so and the PyTorch restatement agree
    fn = _lib.declare("cocclOracleSdp4bitRoundTrip", C.c_int,
                      [C.c_void_p, C.c_long, C.c_long, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p,
                       C.POINTER(C.c_double), C.POINTER(C.c_double)])
    yc = torch.empty_like(x)
    mx, rm = C.c_double(), C.c_double()
    assert fn(x.data_ptr(), x.numel(), 1, 4, 128, 0, 1, yc.data_ptr(), C.byref(mx), C.byref(rm)) == 0
    cfg = CodecConfig("sdp4bit", 4, 128, False, True, stochastic=False)
    y = reference_roundtrip(x, cfg)
    err = (y - x)
    max_err, rms = err.abs().max().item(), err.pow(2).mean().sqrt().item()
    # one quantisation step in the rotated domain is absmax/7; after the inverse rotation the error of an
    # element is an average of 32 such errors: RMS ~ step/sqrt(12)
    assert rms < 0.2 and max_err < 1.0, (max_err, rms)
    sr = reference_roundtrip(x, CodecConfig("sdp4bit", 4, 128, False, True, stochastic=True, seed=0))
    assert abs((sr - x).mean().item()) < 2e-3  # stochastic rounding is unbiased
    assert abs(mx.value - max_err) < 1e-3 and abs(rm.value - rms) < 1e-5
    assert ((yc - y).abs() > 1e-5).float().mean().item() < 1e-3
    print(f"sdp4bit g128 q4 hadamard: max_err={max_err:.4f} rms={rms:.4f} (C++ oracle {mx.value:.4f} / {rm.value:.4f})")
