"""The third-party codec under examples/plugin: built against the SDK headers only, accepted by the policy checker
(CPU), and driven through the compressor runtime on a GPU."""
import ctypes as C
import os
import shutil
import subprocess
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
EX = ROOT / "examples" / "plugin"


@pytest.fixture(scope="module")
def built(tmp_path_factory):
    if shutil.which("nvcc") is None:
        pytest.skip("nvcc not on PATH")
    from coccl_b200 import _lib
    _lib.lib()   # builds coccl-config-check if it is missing
    out = tmp_path_factory.mktemp("bf16cast")
    r = subprocess.run(["bash", str(EX / "build.sh"), str(out)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    return out, r.stdout


def test_example_plugin_builds_and_passes_the_policy_check(built):
    out, log = built
    assert (out / "libbf16cast.so").exists()
    assert "plugin bf16cast: ABI v8, capabilities 0x7" in log and "# OK" in log
    assert "normal.all_to_all.default.config.rounding = truncate" in log
    # a value the codec refuses is reported by the checker, with the key
    bad = out / "bad.toml"
    bad.write_text((out / "bf16cast.toml").read_text().replace('rounding = "nearest"', 'rounding = "up"'))
    r = subprocess.run([str(ROOT / "coccl_b200" / "lib" / "coccl-config-check"), str(bad)], capture_output=True, text=True)
    assert r.returncode != 0 and "rounding" in (r.stdout + r.stderr)
    # so is a key the codec does not know
    bad.write_text((out / "bf16cast.toml").read_text().replace('rounding = "nearest"', 'rounding = "nearest"\nbits = 8'))
    r = subprocess.run([str(ROOT / "coccl_b200" / "lib" / "coccl-config-check"), str(bad)], capture_output=True, text=True)
    assert r.returncode != 0 and "bits" in (r.stdout + r.stderr)


@pytest.mark.gpu
def test_example_plugin_round_trip_and_fused_reduction(built):
    from coccl_b200 import _lib
    out, _ = built
    dev = torch.device("cuda", 0)
    fn = _lib.declare("cocclApiCodecRoundTrip", C.c_int,
                      [C.c_char_p, C.c_char_p, C.c_char_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_int,
                       C.c_size_t, C.c_int, C.POINTER(C.c_size_t), C.c_void_p])

    def roundtrip(options, x, chunks=1, reduce=1, dtype_code=7):
        y = torch.empty(x.numel() // reduce, dtype=x.dtype, device=dev)
        enc = C.c_size_t(0)
        rc = fn(str(out).encode(), b"bf16cast", options.encode(), x.data_ptr(), y.data_ptr(), x.numel(), chunks, dtype_code,
                reduce, 1, C.byref(enc), torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        return rc, y, enc.value

    torch.manual_seed(3)
    x = torch.randn(4 * 4096, device=dev)
    rc, y, enc = roundtrip("", x, chunks=4)
    assert rc == 0 and enc == x.numel() * 2
    assert torch.equal(y, x.bfloat16().float())                     # round to nearest even, as torch does
    rc, y, _ = roundtrip("rounding=truncate", x, chunks=4)
    assert rc == 0 and torch.equal(y.view(torch.int32), x.view(torch.int32) & ~0xFFFF)
    # four encoded copies summed while decoding: chunk r * 2 + c is copy r of output chunk c
    rc, y, _ = roundtrip("", x, chunks=8, reduce=4)
    assert rc == 0
    want = x.bfloat16().float().view(4, 2, 2048).sum(0).reshape(-1)
    assert torch.allclose(y, want, rtol=1e-6, atol=1e-6)
    assert roundtrip("rounding=up", x)[0] != 0
