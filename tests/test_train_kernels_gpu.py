"""Trainer kernels against PyTorch fp32 references."""
import dataclasses

import pytest
import torch
import torch.nn.functional as F

from coccl_b200.ops import fused

pytestmark = pytest.mark.gpu


def test_layernorm_fwd_bwd(cuda):
    torch.manual_seed(0)
    M, H = 300, 1024
    x = torch.randn(M, H, device=cuda, dtype=torch.bfloat16, requires_grad=True)
    r = torch.randn(M, H, device=cuda, dtype=torch.bfloat16, requires_grad=True)
    g = (1 + 0.1 * torch.randn(H, device=cuda)).to(torch.bfloat16).requires_grad_(True)
    b = (0.1 * torch.randn(H, device=cuda)).to(torch.bfloat16).requires_grad_(True)
    y, xs = fused.layer_norm(x, g, b, 1e-5, residual=r)
    dy = torch.randn_like(y)
    dxs = torch.randn_like(xs)
    (y.float() * dy.float()).sum().add((xs.float() * dxs.float()).sum()).backward()
    xr, rr, gr, br = (t.detach().float().requires_grad_(True) for t in (x, r, g, b))
    xsr = (xr + rr).detach().to(torch.bfloat16).float() + (xr + rr) - (xr + rr).detach()
    yr = F.layer_norm(xsr, (H,), gr, br, 1e-5)
    ((yr * dy.float()).sum() + (xsr * dxs.float()).sum()).backward()
    assert torch.allclose(y.float(), yr, atol=3e-2, rtol=2e-2)
    assert torch.allclose(x.grad.float(), xr.grad, atol=5e-2, rtol=3e-2)
    assert torch.allclose(r.grad.float(), rr.grad, atol=5e-2, rtol=3e-2)
    assert torch.allclose(g.grad.float(), gr.grad, atol=0.5, rtol=3e-2)
    assert torch.allclose(b.grad.float(), br.grad, atol=0.5, rtol=3e-2)


def test_linear_gelu_fwd_bwd_with_main_grad(cuda):
    torch.manual_seed(1)
    M, K, N = 512, 256, 768
    x = (torch.randn(M, K, device=cuda) * 0.5).to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(N, K, device=cuda) * 0.05).to(torch.bfloat16).requires_grad_(True)
    bias = (torch.randn(N, device=cuda) * 0.1).to(torch.bfloat16).requires_grad_(True)
    w.main_grad = torch.zeros(N, K, device=cuda)
    bias.main_grad = torch.zeros(N, device=cuda)
    y = fused.linear(x, w, bias, gelu=True)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr, wr, br = (t.detach().float().requires_grad_(True) for t in (x, w, bias))
    yr = F.gelu(F.linear(xr, wr, br), approximate="tanh")
    yr.backward(dy.float())
    assert torch.allclose(y.float(), yr, atol=2e-2, rtol=2e-2)
    assert torch.allclose(x.grad.float(), xr.grad, atol=3e-2, rtol=3e-2)
    assert torch.allclose(w.main_grad, wr.grad, atol=0.3, rtol=3e-2)
    assert torch.allclose(bias.main_grad, br.grad, atol=0.3, rtol=3e-2)
    assert w.grad is None and bias.grad is None


def test_cross_entropy(cuda):
    torch.manual_seed(2)
    M, V = 257, 50304
    logits = (torch.randn(M, V, device=cuda) * 2).to(torch.bfloat16)
    tgt = torch.randint(0, V, (M,), device=cuda)
    tgt[5] = -1
    ref_in = logits.float().requires_grad_(True)
    ref = F.cross_entropy(ref_in, tgt, ignore_index=-1, reduction="sum") * 0.01
    ref.backward()
    lg = logits.clone().requires_grad_(True)
    loss = fused.cross_entropy(lg, tgt, 0.01)
    loss.backward()
    assert abs(loss.item() - ref.item()) < 2e-3 * abs(ref.item())
    assert torch.allclose(lg.grad.float(), ref_in.grad, atol=2e-4, rtol=2e-2)


def test_adam_and_norm(cuda):
    torch.manual_seed(3)
    n = 100003
    master = torch.randn(n, device=cuda)
    m = torch.zeros(n, device=cuda)
    v = torch.zeros(n, device=cuda)
    g = torch.randn(n, device=cuda)
    p = torch.empty(n, device=cuda, dtype=torch.bfloat16)
    ref = master.clone().requires_grad_(True)
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    ss = torch.zeros(1, device=cuda)
    coef = torch.ones(1, device=cuda)
    norm = torch.zeros(1, device=cuda)
    for step in range(1, 4):
        fused.sum_squares(g, ss)
        fused.clip_coef(ss, 1.0, 1.0, coef, norm)
        assert abs(norm.item() - g.norm().item()) < 1e-3 * g.norm().item()
        fused.adam_step(master, m, v, g, p, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step,
                        grad_scale=coef)
        ref.grad = g * min(1.0, 1.0 / (g.norm().item() + 1e-6))
        opt.step()
    assert torch.allclose(master, ref.detach(), atol=1e-5, rtol=1e-4)
    assert torch.allclose(p.float(), master, atol=1e-2, rtol=1e-2)


def test_gpt_step_matches_cpu_reference(cuda):
    """Tiny GPT: loss and gradients of the CUDA kernels path vs the fp32 CPU restatement of the same model."""
    from coccl_b200.models.gpt import GPTConfig, GPTStage
    cfg = GPTConfig(n_layer=2, hidden=256, n_head=4, ffn=1024, seq_len=128, vocab=1024)
    gpu = GPTStage(cfg, cuda, seed=5)
    cpu = GPTStage(dataclasses.replace(cfg, dtype=torch.float32), torch.device("cpu"), seed=5)
    cpu.store.flat_param.copy_(gpu.store.flat_param.float().cpu())
    torch.manual_seed(0)
    tok = torch.randint(0, cfg.vocab, (2, cfg.seq_len + 1))
    scale = 1.0 / (2 * cfg.seq_len)
    lg = gpu(tok[:, :-1].to(cuda), tok[:, 1:].to(cuda), scale)
    lg.backward()
    gpu.post_backward_sync_autograd_grads()
    lc = cpu(tok[:, :-1], tok[:, 1:], scale)
    lc.backward()
    cpu.post_backward_sync_autograd_grads()
    assert abs(lg.item() - lc.item()) < 2e-2
    a, b = gpu.store.flat_grad.cpu(), cpu.store.flat_grad
    rel = (a - b).norm() / b.norm()
    assert rel < 5e-2, rel.item()


@pytest.mark.parametrize("tp,M,V", [(2, 300, 1024), (4, 64, 25152)])
def test_vocab_parallel_cross_entropy_kernels(cuda, tp, M, V):
    """Two-pass cross-entropy over a vocabulary split into `tp` shards (all shards on this GPU): the combined loss and
    the in-place gradients equal the fp32 reference over the whole vocabulary."""
    import ctypes as C
    from coccl_b200 import _lib
    torch.manual_seed(21)
    full = (torch.randn(M, tp * V, device=cuda) * 3).to(torch.bfloat16)
    tgt = torch.randint(0, tp * V, (M,), device=cuda)
    tgt[::7] = -1   # ignored rows
    scale = 0.37
    shards = [full[:, r * V:(r + 1) * V].contiguous() for r in range(tp)]
    lib = _lib.lib()
    stats = torch.empty(tp, M, 4, dtype=torch.float32, device=cuda)
    for r in range(tp):
        _lib.check(lib.cocclkCrossEntropyStats(shards[r].data_ptr(), tgt.data_ptr(), stats[r].data_ptr(), M, V, V, r * V,
                                               _lib.cur_stream()), "stats")
    losses = []
    for r in range(tp):
        loss = torch.empty(M, dtype=torch.float32, device=cuda)
        _lib.check(lib.cocclkCrossEntropyFinish(shards[r].data_ptr(), tgt.data_ptr(), stats.data_ptr(), tp, loss.data_ptr(), M, V, V,
                                                r * V, scale, _lib.cur_stream()), "finish")
        losses.append(loss)
    lf = full.float()
    valid = tgt >= 0
    ref_loss = torch.where(valid, torch.logsumexp(lf, -1) - lf.gather(1, tgt.clamp(min=0)[:, None])[:, 0], torch.zeros(M, device=cuda))
    p = torch.softmax(lf, -1)
    p[torch.arange(M, device=cuda), tgt.clamp(min=0)] -= 1.0
    ref_grad = p * valid[:, None] * scale
    for r in range(tp):
        assert torch.allclose(losses[r], ref_loss, atol=2e-3, rtol=2e-3)
        assert torch.equal(losses[r], losses[0])   # every rank computes the same loss
        got = shards[r].float()
        want = ref_grad[:, r * V:(r + 1) * V]
        assert (got - want).abs().max().item() <= 4e-3 * scale + 1e-6


@pytest.mark.parametrize("M,N", [(4096, 4096), (100, 264), (2048, 6144), (33, 8)])
def test_column_sum(cuda, M, N):
    """Bias-gradient column sum (two kernels, fixed summation order) against fp32 torch, overwrite and accumulate."""
    import ctypes as C
    from coccl_b200 import _lib
    torch.manual_seed(22)
    x = torch.randn(M, N, device=cuda).to(torch.bfloat16)
    lib = _lib.lib()
    sc = torch.empty(lib.cocclkColSumBlocks(M) * N, dtype=torch.float32, device=cuda)
    out = torch.full((N,), 5.0, device=cuda)
    _lib.check(lib.cocclkColSum(x.data_ptr(), out.data_ptr(), 0, sc.data_ptr(), M, N, _lib.cur_stream()), "colsum")
    ref = x.float().sum(0)
    assert torch.allclose(out, ref, atol=1e-3 * M ** 0.5, rtol=1e-5)
    first = out.clone()
    _lib.check(lib.cocclkColSum(x.data_ptr(), out.data_ptr(), 1, sc.data_ptr(), M, N, _lib.cur_stream()), "colsum")
    assert torch.allclose(out, 2 * first, atol=1e-5, rtol=1e-6)   # same partial sums in the same order, added once more
