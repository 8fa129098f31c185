"""The pre-training launcher and its data loader on CPU: schedule, data determinism, resume, a two-rank run."""
import json
import os
import socket
import subprocess
import sys

import numpy as np
import pytest
import torch

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TINY = ["--model", "gpt-tiny", "--layers", "2", "--hidden", "64", "--heads", "4", "--ffn", "128", "--seq-len", "32",
        "--vocab", "128", "--device", "cpu", "--log-interval", "1", "--warmup-steps", "2", "--lr", "1e-2"]


def _token_file(tmp_path, n=6000, vocab=128):
    # a stream with structure (each id determines the next one most of the time), so that a few steps lower the loss
    rng = np.random.default_rng(5)
    path = str(tmp_path / "tokens.bin")
    ids = (np.arange(n) * 7) % vocab
    noise = rng.random(n) < 0.1
    ids[noise] = rng.integers(0, vocab, int(noise.sum()))
    ids.astype("<u2").tofile(path)
    return path


def _records(text):
    return [json.loads(l) for l in text.splitlines() if l.startswith("{")]


def test_learning_rate_schedule():
    from coccl_b200.pretrain import learning_rate
    kw = dict(peak=1.0, floor=0.1, warmup=4, decay=20)
    assert [round(learning_rate(s, **kw), 3) for s in range(4)] == [0.25, 0.5, 0.75, 1.0]
    assert learning_rate(4, **kw) == pytest.approx(1.0)
    assert learning_rate(12, **kw) == pytest.approx(0.55)
    assert learning_rate(20, **kw) == learning_rate(500, **kw) == 0.1
    vals = [learning_rate(s, **kw) for s in range(4, 21)]
    assert all(a >= b for a, b in zip(vals, vals[1:]))


def test_loader_is_a_pure_function_of_seed_step_and_rank(tmp_path):
    from coccl_b200.utils.data import BatchLoader, SyntheticTokens, TokenFile, sequence_starts
    path = _token_file(tmp_path)
    src = TokenFile(path)
    raw = np.fromfile(path, dtype="<u2").astype(np.int64)
    kw = dict(seq_len=32, global_batch=8, seed=3, vocab=128, pin=False)
    whole = BatchLoader(src, dp_rank=0, dp_size=1, **kw)
    halves = [BatchLoader(src, dp_rank=r, dp_size=2, **kw) for r in range(2)]
    seen = []
    for step in range(30):   # 6000 tokens = 187 windows: crosses an epoch boundary at step 23
        b = whole.next()
        assert torch.equal(b, torch.cat([h.next() for h in halves]))
        starts = sequence_starts(src.length, 32, 3, step, 8)
        for row, s in zip(b, starts):
            assert np.array_equal(row.numpy(), raw[s:s + 33])
        seen.extend(int(s) for s in starts)
    windows = (6000 - 1) // 32
    assert sorted(seen[:windows]) == [w * 32 for w in range(windows)]   # one epoch visits every window exactly once
    resumed = BatchLoader(src, dp_rank=1, dp_size=2, start_step=30, **kw)
    assert torch.equal(resumed.next(), halves[1].next())
    for l in [whole, resumed] + halves:
        l.close()
    syn = SyntheticTokens(1000, seed=9)
    assert np.array_equal(syn.tokens(4000, 300)[90:110], syn.tokens(4090, 20))
    with pytest.raises(RuntimeError):
        bad = BatchLoader(src, dp_rank=0, dp_size=1, seq_len=32, global_batch=8, seed=3, vocab=64, pin=False)
        try:
            bad.next()
        finally:
            bad.close()


def test_resume_continues_the_uninterrupted_run(tmp_path, capsys):
    from coccl_b200.pretrain import main
    data = _token_file(tmp_path)
    common = TINY + ["--data", data, "--global-batch", "4", "--decay-steps", "8"]
    main(common + ["--steps", "8"])
    full = _records(capsys.readouterr().out)
    ck = str(tmp_path / "ck")
    main(common + ["--steps", "4", "--save", ck])
    capsys.readouterr()
    main(common + ["--steps", "8", "--save", ck, "--resume"])
    tail = _records(capsys.readouterr().out)
    want = {r["step"]: r["loss"] for r in full if "step" in r}
    got = {r["step"]: r["loss"] for r in tail if "step" in r}
    assert sorted(got) == [5, 6, 7, 8]
    for s in got:
        assert got[s] == pytest.approx(want[s], rel=1e-5), (s, got, want)
    assert want[8] < want[1]


def test_two_rank_launch_matches_one_process(tmp_path, capsys):
    """The command a user runs: torch.distributed.run, two gloo ranks, pipeline-parallel with two chunks per rank."""
    from coccl_b200.pretrain import main
    data = _token_file(tmp_path)
    common = TINY + ["--data", data, "--global-batch", "8", "--steps", "3", "--layers", "4"]
    main(common)
    one = {r["step"]: r["loss"] for r in _records(capsys.readouterr().out) if "step" in r}
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, PYTHONPATH=REPO + os.pathsep + os.environ.get("PYTHONPATH", ""), OMP_NUM_THREADS="2")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", str(port), "-m", "coccl_b200.pretrain"] + common +
                         ["--pp", "2", "--virtual-stages", "2", "--log-json", str(tmp_path / "log.jsonl")],
                         env=env, cwd=REPO, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    two = {r["step"]: r["loss"] for r in _records(open(tmp_path / "log.jsonl").read())}
    assert sorted(two) == [1, 2, 3]
    for s in two:
        assert two[s] == pytest.approx(one[s], rel=2e-3), (two, one)


def test_validation_loss_is_logged_and_falls(tmp_path, capsys):
    from coccl_b200.pretrain import main
    data = _token_file(tmp_path)
    common = TINY + ["--data", data, "--eval-data", data, "--global-batch", "4", "--eval-interval", "4", "--eval-batches", "2"]
    main(common + ["--steps", "12", "--decay-steps", "12"])
    vals = [r["val_loss"] for r in _records(capsys.readouterr().out) if "val_loss" in r]
    assert len(vals) == 3 and vals[-1] < vals[0] - 0.2, vals
    # without updates the held-out batches give the same loss every time
    main(common + ["--steps", "8", "--lr", "0", "--min-lr", "0", "--warmup-steps", "0"])
    vals = [r["val_loss"] for r in _records(capsys.readouterr().out) if "val_loss" in r]
    assert len(vals) == 2 and vals[0] == vals[1], vals


def _launch(argv, tmp_path, nproc=2):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, PYTHONPATH=REPO + os.pathsep + os.environ.get("PYTHONPATH", ""), OMP_NUM_THREADS="2")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc),
                          "--master-addr", "127.0.0.1", "--master-port", str(port), "-m", "coccl_b200.pretrain"] + argv,
                         env=env, cwd=REPO, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    return out.stdout


def test_expert_parallel_launch_saves_and_resumes(tmp_path):
    """Mixture-of-experts model, experts over the two data-parallel ranks: the checkpoint carries the expert buffers of
    each rank, and the resumed run (whose peers start with the earlier steps behind them) reproduces the full run."""
    data = _token_file(tmp_path)
    common = ["--model", "moe-tiny", "--hidden", "64", "--heads", "4", "--ffn", "128", "--seq-len", "32", "--vocab", "128",
              "--device", "cpu", "--ep", "2", "--data", data, "--global-batch", "8", "--log-interval", "1", "--lr", "1e-2",
              "--warmup-steps", "2", "--decay-steps", "6", "--heartbeat-stale-s", "20"]
    full = {r["step"]: r["loss"] for r in _records(_launch(common + ["--steps", "6"], tmp_path)) if "step" in r}
    ck = str(tmp_path / "ck")
    _launch(common + ["--steps", "3", "--save", ck], tmp_path)
    assert sorted(os.listdir(ck)) == ["manifest.json", "rank00000.pt", "rank00001.pt"]
    tail = {r["step"]: r["loss"] for r in _records(_launch(common + ["--steps", "6", "--save", ck, "--resume"], tmp_path)) if "step" in r}
    assert sorted(tail) == [4, 5, 6]
    for s in tail:
        assert tail[s] == pytest.approx(full[s], rel=1e-4), (tail, full)


def test_fully_sharded_launch_saves_and_resumes(tmp_path):
    """--dp-strategy fsdp on two ranks: each rank's checkpoint holds its shards only, and the resumed run continues
    the uninterrupted one."""
    data = _token_file(tmp_path)
    common = TINY + ["--data", data, "--global-batch", "8", "--dp-strategy", "fsdp", "--decay-steps", "6", "--heartbeat-stale-s", "20"]
    full = {r["step"]: r["loss"] for r in _records(_launch(common + ["--steps", "6"], tmp_path)) if "step" in r}
    ck = str(tmp_path / "ck")
    _launch(common + ["--steps", "3", "--save", ck], tmp_path)
    shard = torch.load(os.path.join(ck, "rank00001.pt"), map_location="cpu", weights_only=False)
    tail = {r["step"]: r["loss"] for r in _records(_launch(common + ["--steps", "6", "--save", ck, "--resume"], tmp_path)) if "step" in r}
    assert sorted(tail) == [4, 5, 6]
    for s in tail:
        assert tail[s] == pytest.approx(full[s], rel=1e-4), (tail, full)
    assert full[6] < full[1]
    # half of the model per rank (two ranks), not the model
    from coccl_b200.models.gpt import GPTConfig
    n = GPTConfig(n_layer=2, hidden=64, n_head=4, ffn=128, seq_len=32, vocab=128).num_params()
    assert 0.45 * n < shard["flat_param"].numel() < 0.6 * n


def test_example_launchers_parse_and_name_existing_modules():
    """The shell launchers under examples/ are syntactically valid and call modules and files that exist."""
    import importlib.util
    import re
    ex = os.path.join(REPO, "examples")
    scripts = sorted(f for f in os.listdir(ex) if f.endswith(".sh"))
    assert scripts == ["build.sh", "communication_benchmarks.sh", "preload.sh", "train_gpt.sh"]
    for name in scripts:
        path = os.path.join(ex, name)
        assert os.access(path, os.X_OK), name
        out = subprocess.run(["bash", "-n", path], capture_output=True, text=True)
        assert out.returncode == 0, out.stderr
        text = open(path).read()
        for mod in re.findall(r"-m (coccl_b200[\w.]*)", text):
            assert importlib.util.find_spec(mod) is not None, (name, mod)
        for rel in re.findall(r"\$root/(coccl_b200/configs/[\w.-]+\.toml)", text):
            assert os.path.exists(os.path.join(REPO, rel)), (name, rel)
