"""Checkpoint / resume: an interrupted run continues on the same loss curve (single process, CPU)."""
import torch

from coccl_b200.models.gpt import GPTConfig
from coccl_b200.train import Trainer
from coccl_b200.utils import checkpoint as ck


def _batches(cfg, n, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg.vocab, (4, cfg.seq_len + 1), generator=g) for _ in range(n)]


def test_resume_continues_the_loss_curve(tmp_path):
    cfg = GPTConfig(n_layer=2, hidden=64, n_head=4, ffn=128, seq_len=32, vocab=128)
    data = _batches(cfg, 5)
    ref = Trainer(cfg, torch.device("cpu"), micro_batch=2, lr=1e-2, seed=7)
    ref_losses = [ref.train_step(b).item() for b in data]
    a = Trainer(cfg, torch.device("cpu"), micro_batch=2, lr=1e-2, seed=7)
    first = [a.train_step(b).item() for b in data[:3]]
    ck.save(a, str(tmp_path / "ckpt"), step=3)
    b = Trainer(cfg, torch.device("cpu"), micro_batch=2, lr=1e-2, seed=999)  # different init: must be overwritten
    assert ck.load(b, str(tmp_path / "ckpt")) == 3
    rest = [b.train_step(x).item() for x in data[3:]]
    assert first == ref_losses[:3]
    assert all(abs(x - y) < 1e-5 for x, y in zip(rest, ref_losses[3:])), (rest, ref_losses[3:])
