"""bench.py contract pieces that need no GPU."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_reference_arm_reports_unavailable():
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "1",
                        "--warmup", "1"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and line["unavailable"]


def test_collective_reference_runner_closes_what_faulted():
    """The reference's NCCL 2.21.5 all-reduce / reduce-scatter / all-gather kernels faulted or hung on B200: the
    runner must answer those cases without starting anything (it also answers like this where baseline/_ref is
    not built)."""
    r = subprocess.run([sys.executable, "-m", "coccl_b200.bench_collectives", "--impl", "reference", "--gpus", "2",
                        "--ops", "all_reduce,reduce_scatter,all_gather", "--codecs", "native,sdp4bit", "--dtypes", "fp32",
                        "--min-mib", "1", "--max-mib", "2"], capture_output=True, text=True, timeout=300, cwd=str(ROOT))
    assert r.returncode == 0, r.stderr
    lines = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert lines and all(l["impl"] == "reference" and l["unavailable"] for l in lines)
