"""The bounds-checked twin of the kernel library (libcoccl_checked.so, -DCOCCL_BOUNDS_CHECK) and the slot-geometry check
that every build makes at kernel entry."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def test_codec_and_collective_suites_pass_with_range_checked_accesses(cuda):
    """The emulated-rank collective tests and the codec tests once more, through the library whose every codec access
    is preceded by a range check (conftest asserts after each test that the error word stayed clear): all codecs, odd
    counts, tails, both all-reduce algorithms, the delta all-gather."""
    env = dict(os.environ, COCCL_CHECKED_KERNELS="1")
    r = subprocess.run([sys.executable, "-m", "pytest", "tests/test_collective_emulated_gpu.py", "tests/test_codec_gpu.py",
                        "-q", "-x", "-m", "gpu", "-p", "no:cacheprovider"], cwd=ROOT, env=env, capture_output=True, text=True,
                       timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert " passed" in r.stdout and "failed" not in r.stdout.splitlines()[-1]


def test_checked_library_reports_itself(cuda):
    env = dict(os.environ, COCCL_CHECKED_KERNELS="1")
    code = "from coccl_b200 import _lib; c, w = _lib.bounds_word(); print(int(c), w[0])"
    r = subprocess.run([sys.executable, "-c", code], cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.split()[-2:] == ["1", "0"], r.stdout + r.stderr
    from coccl_b200 import _lib
    assert _lib.bounds_word()[0] is (os.environ.get("COCCL_CHECKED_KERNELS", "") not in ("", "0"))


@pytest.mark.parametrize("op", ["reduce_scatter", "all_reduce_twoshot"])
def test_slot_smaller_than_the_chunk_is_refused_at_kernel_entry(cuda, op):
    """A slot size from the host that cannot hold an encoded chunk would make ranks write over each other's slots. The
    kernel checks the geometry before it touches anything: every rank reports phase 0xB in its status word, the
    workspace keeps its canary bytes, nothing is written, nothing faults."""
    from coccl_b200.ops import codec as C
    from coccl_b200.ops import collective as K
    n, numel = 4, 4 * 8192 * 3
    xs = [torch.randn(numel, device=cuda) * 0.01 for _ in range(n)]
    state = {}
    K.emulate_collective(op, xs, C.SDP4BIT_G128, state=state, epoch=1)        # sizes the workspace
    torch.cuda.synchronize()
    assert K.status_codes(state) == [0] * n
    sb, _, _ = K.workspace_bytes(K.OP_NAMES[op], C.SDP4BIT_G128, K.chunk_count(K.OP_NAMES[op], numel, n), xs[0].dtype, n)
    for w in state["ws"]:
        w.fill_(0xA5)
    outs = K.emulate_collective(op, xs, C.SDP4BIT_G128, state=state, epoch=2, slot_bytes=sb - 16)
    torch.cuda.synchronize()
    codes = K.status_codes(state)
    assert all(c & 0x80000000 and ((c >> 23) & 0xff) == 0xB for c in codes), [hex(c) for c in codes]
    assert all(int(w.min().item()) == 0xA5 and int(w.max().item()) == 0xA5 for w in state["ws"])
    del outs
