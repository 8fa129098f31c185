"""The pre-training launcher on one GPU: pinned batches handed to the device asynchronously, bf16 kernels, a checkpoint
that the second call resumes."""
import json

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _records(text):
    return [json.loads(l) for l in text.splitlines() if l.startswith("{")]


def test_launcher_trains_saves_and_resumes_on_a_gpu(tmp_path, capsys):
    from coccl_b200.pretrain import main
    vocab, n = 8192, 400_000
    ids = (np.arange(n) * 7) % vocab           # every id determines its successor: a few steps lower the loss
    path = str(tmp_path / "tokens.bin")
    ids.astype("<u2").tofile(path)
    common = ["--model", "gpt-tiny", "--data", path, "--global-batch", "8", "--log-interval", "2", "--lr", "1e-3",
              "--warmup-steps", "2", "--decay-steps", "12"]
    main(common + ["--steps", "12"])
    full = {r["step"]: r for r in _records(capsys.readouterr().out) if "step" in r}
    assert full[12]["loss"] < full[2]["loss"] - 0.5 and full[12]["tokens_per_s"] > 0
    ck = str(tmp_path / "ck")
    main(common + ["--steps", "6", "--save", ck])
    capsys.readouterr()
    main(common + ["--steps", "12", "--save", ck, "--resume"])
    tail = {r["step"]: r for r in _records(capsys.readouterr().out) if "step" in r}
    assert sorted(tail) == [8, 10, 12]
    for s in tail:
        assert tail[s]["loss"] == pytest.approx(full[s]["loss"], rel=2e-2), (s, tail[s], full[s])
    torch.cuda.synchronize()
