"""MoE routing layout, FP8 dispatch and bf16 combine, every rank emulated on one GPU, against plain PyTorch."""
import pytest
import torch

from coccl_b200.ops import codec as C
from coccl_b200.ops import moe as M

pytestmark = pytest.mark.gpu


def test_route_layout_is_a_stable_sort(cuda):
    torch.manual_seed(0)
    n_experts, n_ranks = 16, 4
    ids = torch.randint(0, n_experts, (1000, 2), device=cuda, dtype=torch.int32)
    pos, counts = M.route_layout(ids, n_experts, n_ranks)
    flat = ids.reshape(-1).long()
    assert torch.equal(counts.long(), torch.bincount(flat, minlength=n_experts))
    le = n_experts // n_ranks
    # reference: stable sort by expert; position inside the destination rank's block
    order = torch.sort(flat, stable=True).indices
    ref = torch.empty_like(flat)
    cum = torch.cumsum(counts.long(), 0) - counts.long()
    rank_base = cum[(torch.arange(n_experts, device=cuda) // le) * le]
    sorted_e = flat[order]
    ref[order] = torch.arange(flat.numel(), device=cuda) - rank_base[sorted_e]
    assert torch.equal(pos.reshape(-1).long(), ref)


@pytest.mark.parametrize("n,tokens,hidden,topk,n_experts", [(2, 64, 256, 2, 4), (4, 300, 512, 2, 16), (2, 1024, 1024, 1, 8)])
def test_dispatch_and_combine_emulated(cuda, n, tokens, hidden, topk, n_experts):
    torch.manual_seed(1)
    le = n_experts // n
    xs = [torch.randn(tokens, hidden, device=cuda, dtype=torch.bfloat16) for _ in range(n)]
    ids, gates = [], []
    for r in range(n):
        # distinct experts per token
        sc = torch.rand(tokens, n_experts, device=cuda)
        top = sc.topk(topk, dim=1)
        ids.append(top.indices.to(torch.int32).contiguous())
        gates.append(torch.softmax(top.values, dim=1).float().contiguous())
    state = {}
    for _ in range(2):
        recvs, handles, state = M.emulate_dispatch(xs, ids, n_experts, state=state)
        torch.cuda.synchronize()
        M.check_state(state)
        # oracle: rows of expert e on rank d = for src in ranks: tokens of src routed to e, in token order
        xq = [C.reference_roundtrip(x.float().contiguous(), C.MXFP8, 1).to(torch.bfloat16) for x in xs]
        for d in range(n):
            rows, offs = [], [0]
            for e_local in range(le):
                e = d * le + e_local
                for s in range(n):
                    tok = (ids[s] == e).nonzero()[:, 0]  # a token picks an expert at most once
                    rows.append(xq[s][tok])
                offs.append(offs[-1] + sum((ids[s] == e).sum().item() for s in range(n)))
            ref = torch.cat(rows)
            assert handles[d].recv_offsets.tolist() == offs
            got = recvs[d][:ref.shape[0]]
            assert torch.equal(got, ref), (d, (got.float() - ref.float()).abs().max().item())
        # experts: y = 2 * x + (global expert index); combine = sum_j gate_j * y_j
        ys = []
        for d in range(n):
            y = recvs[d].float() * 2.0
            offs = handles[d].recv_offsets.tolist()
            for e_local in range(le):
                y[offs[e_local]:offs[e_local + 1]] += float(d * le + e_local)
            ys.append(y.to(torch.bfloat16))
        outs = M.emulate_combine(ys, gates, handles, state=state)
        torch.cuda.synchronize()
        M.check_state(state)
        for s in range(n):
            ref = torch.zeros(tokens, hidden, device=cuda)
            for j in range(topk):
                yj = (xq[s].float() * 2.0 + ids[s][:, j:j + 1].float()).to(torch.bfloat16).float()
                ref += gates[s][:, j:j + 1] * yj
            assert torch.allclose(outs[s].float(), ref, atol=2e-2 * ref.abs().max().item(), rtol=0)
