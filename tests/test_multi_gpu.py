"""Fused compressed collectives and the parallel trainer on real peer GPUs (one process per GPU, NCCL plumbing).
Skipped when fewer than two GPUs are visible."""
import pytest
import torch

from dist_utils import run_distributed

pytestmark = pytest.mark.gpu


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _collectives_worker(rank, world):
    import torch.distributed as dist
    from coccl_b200.ops import codec as C
    from coccl_b200.parallel.comm import Communicator, Policy
    dev = torch.device("cuda", rank)
    # normal-mode policy files: SDP4Bit on every collective, threshold 0; one forces the one-shot all-reduce, one the
    # two-shot (the selector's choice between them is covered by the autotune test)
    comm = Communicator(None, dev, Policy.normal("sdp4bit", threshold_bytes=0, all_reduce_algorithm="twoshot"), "default")
    comm1 = Communicator(None, dev, Policy.normal("sdp4bit", threshold_bytes=0, all_reduce_algorithm="oneshot"), "oneshot")
    for dtype in (torch.float32, torch.bfloat16):
        for numel in (world * 4096, world * 300000):
            torch.manual_seed(100 + rank)
            x = (torch.randn(numel, device=dev) * 0.01).to(dtype)
            xs = [torch.empty_like(x) for _ in range(world)]
            dist.all_gather(xs, x)
            cfg = C.SDP4BIT_G128
            c = numel // world
            # reduce-scatter
            out = torch.empty(c, dtype=dtype, device=dev)
            comm.reduce_scatter(x, out)
            ref = sum(C.reference_roundtrip(xq, cfg, world).reshape(world, c)[rank] for xq in xs)
            bad = ((out.float() - ref.to(dtype).float()).abs() > 1e-5 + 2e-2 * ref.abs().max()).float().mean().item()
            assert bad < 5e-3, ("rs", dtype, numel, bad)
            # all-gather
            out = torch.empty(numel * world, dtype=dtype, device=dev)
            comm.all_gather(x, out)
            ref = torch.cat([C.reference_roundtrip(xq, cfg, 1) for xq in xs])
            bad = ((out.float() - ref.to(dtype).float()).abs() > 1e-5 + 2e-2 * ref.abs().max()).float().mean().item()
            assert bad < 5e-3, ("ag", dtype, numel, bad)
            # all-to-all
            out = torch.empty(numel, dtype=dtype, device=dev)
            comm.all_to_all(x, out)
            ref = torch.cat([C.reference_roundtrip(xq, cfg, world).reshape(world, c)[rank] for xq in xs])
            bad = ((out.float() - ref.to(dtype).float()).abs() > 1e-5 + 2e-2 * ref.abs().max()).float().mean().item()
            assert bad < 5e-3, ("a2a", dtype, numel, bad)
            # all-reduce, both algorithms
            exact = sum(xq.float() for xq in xs)
            for cm, twoshot in ((comm, True), (comm1, False)):
                y = x.clone()
                cm.all_reduce(y)
                rel = ((y.float() - exact).norm() / exact.norm()).item()
                assert rel < 0.3, ("ar", dtype, numel, twoshot, rel)
                if twoshot:  # every rank decodes the same re-encoded bytes
                    ys = [torch.empty_like(y) for _ in range(world)]
                    dist.all_gather(ys, y)
                    assert all(torch.equal(ys[0], t) for t in ys)
    assert comm.stats["compressed_calls"] == 16 and comm.stats["native_calls"] == 0
    assert comm1.stats["compressed_calls"] == 4 and comm1.stats["native_calls"] == 0
    assert comm.status() == 0 and comm1.status() == 0
    comm.close()
    comm1.close()


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_fused_collectives_over_peer_memory():
    run_distributed(_collectives_worker, min(_ngpu(), 8) if _ngpu() in (2, 4, 8) else 2, "nccl")


def _trainer_worker(rank, world, tp, pp, dp, compress, delta=False):
    import torch.distributed as dist
    from coccl_b200.models.gpt import GPTConfig
    from coccl_b200.parallel.mesh import Mesh
    from coccl_b200.parallel.comm import Policy
    from coccl_b200.train import ParallelConfig, Trainer
    dev = torch.device("cuda", rank)
    cfg = GPTConfig(n_layer=4, hidden=512, n_head=8, ffn=2048, seq_len=256, vocab=8192)
    mesh = Mesh(tp=tp, pp=pp, dp=dp, device=dev, compress=compress,
                policy=Policy.training(threshold_bytes=0, dp_delta=delta))
    tr = Trainer(cfg, dev, micro_batch=2, parallel=ParallelConfig(tp, pp, dp), groups=mesh, lr=3e-4)
    g = torch.Generator().manual_seed(5 + mesh.dp_rank)
    tok = torch.randint(0, cfg.vocab, (8, cfg.seq_len + 1), generator=g).pin_memory()
    losses = []
    for _ in range(6):
        t = tr.train_step(tok).clone()
        dist.all_reduce(t)
        losses.append(t.item() / (tp * dp))
    assert losses[-1] < losses[0] - 0.2, losses
    assert all(l == l for l in losses)
    if delta:
        # every replica holds the same parameters after the delta all-gathers, and they track the fp32 master weights
        assert tr.opt.delta
        fp = tr.stage.store.flat_param
        ref = fp.clone()
        dist.broadcast(ref, src=0, group=mesh.dp_comm.group)
        assert torch.equal(fp, ref)
        lo = tr.opt.rank * tr.opt.shard
        own = fp[lo:lo + tr.opt.shard].float()
        assert (own - tr.opt.master).abs().max().item() < 2e-2 * tr.opt.master.abs().max().item() + 1e-3
    for c in (mesh.tp_comm, mesh.dp_comm):
        if c is not None:
            assert c.status() == 0
            if compress:
                assert c.stats["compressed_calls"] > 0
    mesh.close()


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("layout", ["tp2", "dp2", "pp2"])
def test_trainer_two_gpus_compressed(layout):
    tp, pp, dp = {"tp2": (2, 1, 1), "dp2": (1, 1, 2), "pp2": (1, 2, 1)}[layout]
    run_distributed(_trainer_worker, 2, "nccl", (tp, pp, dp, True))


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_trainer_dp2_delta_parameter_gather():
    run_distributed(_trainer_worker, 2, "nccl", (1, 1, 2, True, True))


@pytest.mark.skipif(_ngpu() < 8, reason="needs 8 GPUs")
def test_trainer_3d_eight_gpus():
    run_distributed(_trainer_worker, 8, "nccl", (2, 2, 2, True))


def _tp_fused_worker(rank, world):
    import torch.distributed as dist
    from coccl_b200.ops import codec as C
    from coccl_b200.parallel.comm import Communicator, Policy
    dev = torch.device("cuda", rank)
    comm = Communicator(None, dev, Policy(), "tp")
    m, K, N = 256, 512, 768
    for it in range(3):  # several calls: parity halves of the workspace and epochs are reused
        torch.manual_seed(7 + rank + 10 * it)
        x = torch.randn(m, K, device=dev, dtype=torch.bfloat16)
        w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.1
        b = torch.randn(N, device=dev, dtype=torch.bfloat16)
        xs = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(xs, x)
        y = comm.ag_gemm(x, w, bias=b, gelu=True, payload="bf16")
        ref = torch.nn.functional.gelu(torch.cat(xs).float() @ w.float().t() + b.float(), approximate="tanh")
        assert (y.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-3
        # the same product with the shards on the wire as block-scaled FP8: remote shards equal the codec's round trip
        kept = torch.empty(m * world, K, device=dev, dtype=torch.bfloat16)
        y8 = comm.ag_gemm(x, w, bias=b, gelu=True, payload="fp8", gathered=kept)
        from coccl_b200.ops import tp_fused as T8
        if T8.last_variant() == "2cta":
            seen = torch.cat([xs[q] if q == rank else C.reference_roundtrip(xs[q].float().contiguous(), C.MXFP8, 1).to(torch.bfloat16)
                              for q in range(world)])
            assert torch.equal(kept, seen)
            ref8 = torch.nn.functional.gelu(seen.float() @ w.float().t() + b.float(), approximate="tanh")
            assert (y8.float() - ref8).abs().max().item() <= 2e-2 * ref8.abs().max().item() + 1e-3
        assert ((y8.float() - ref).norm() / ref.norm()).item() < 0.05
        # second half of the MLP: y [M, N] @ w2[N2, N]^T, partial sums reduce-scattered as FP8
        w2 = torch.randn(512, N, device=dev, dtype=torch.bfloat16) * 0.05
        out = comm.gemm_rs(y, w2)
        part = y.float() @ w2.float().t()
        q = C.reference_roundtrip(part.contiguous(), C.MXFP8, 1)
        parts = [torch.empty_like(q) for _ in range(world)]
        dist.all_gather(parts, q)
        rows = m  # M / world
        # the CTA-pair kernel (rows per rank a multiple of 256) adds a rank's own partial product straight from the
        # accumulator; only what crosses the link is quantised
        from coccl_b200.ops import tp_fused as T
        if T.last_variant() == "2cta":
            parts[rank] = part
        refq = sum(parts)[rank * rows:(rank + 1) * rows]
        d = (out.float() - refq).abs()
        scale = refq.abs().max().item()
        assert (d > 1e-2 * scale + 1e-3).float().mean().item() < 2e-3 and d.max().item() <= scale / 8 + 1e-3
    assert comm.tp_status() == (0, 0)
    comm.close()


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_tp_fusions_over_peer_memory():
    run_distributed(_tp_fused_worker, min(_ngpu(), 8) if _ngpu() in (2, 4, 8) else 2, "nccl")


def _moe_worker(rank, world):
    import torch.distributed as dist
    from coccl_b200.models.moe import MoELayer
    from coccl_b200.parallel.comm import NATIVE, Communicator, Policy
    dev = torch.device("cuda", rank)
    comm = Communicator(None, dev, Policy(), "ep")
    layer = MoELayer(comm, hidden=512, ffn=1024, n_experts=4 * world, topk=2, seed=3)
    # the same model with every expert on one rank
    solo = Communicator.__new__(Communicator)
    solo.size, solo.rank, solo.device = 1, 0, dev
    ref_layer = MoELayer(solo, hidden=512, ffn=1024, n_experts=4 * world, topk=2, seed=3, device=dev)
    for it in range(2):
        torch.manual_seed(50 + rank + it)
        x = torch.randn(384, 512, device=dev, dtype=torch.bfloat16)
        y = layer.forward(x)
        ids, gates = layer.route(x)
        ref = ref_layer.forward_local(x, ids, gates)
        rel = ((y.float() - ref.float()).norm() / ref.float().norm()).item()
        assert rel < 0.06, rel  # FP8 on the dispatched activations
    # training: gradients through the exchange (dispatch <-> combine are each other's backward) against the local model
    layer.requires_grad_(True)
    ref_layer.requires_grad_(True)
    torch.manual_seed(90 + rank)
    x = torch.randn(384, 512, device=dev, dtype=torch.bfloat16)
    probe = torch.randn(384, 512, device=dev)
    xa = x.clone().requires_grad_(True)
    (layer.forward(xa).float() * probe).sum().backward()
    xb = x.clone().requires_grad_(True)
    ids, _ = ref_layer.route(x)
    logits = torch.nn.functional.linear(xb, ref_layer.router).float()
    gates = torch.softmax(logits.gather(1, ids.long()), dim=1)
    (ref_layer.forward_local(xb, ids, gates).float() * probe).sum().backward()
    rel = ((xa.grad.float() - xb.grad.float()).norm() / xb.grad.float().norm()).item()
    assert rel < 0.12, ("dx", rel)
    le = layer.local
    for k in range(le):
        e = rank * le + k
        # an expert's weight gradient collects the tokens of every rank
        gref = ref_layer.w_up[e].grad.float().clone() if ref_layer.w_up[e].grad is not None else torch.zeros_like(ref_layer.w_up[e]).float()
        for other in range(world):
            for kk in range(le):
                ee = other * le + kk
                g = ref_layer.w_up[ee].grad
                buf = g.float().clone() if g is not None else torch.zeros(ref_layer.w_up[ee].shape, device=dev)
                dist.all_reduce(buf)
                if ee == e:
                    gref = buf
        got = layer.w_up[k].grad.float()
        rel = ((got - gref).norm() / (gref.norm() + 1e-6)).item()
        assert rel < 0.15, ("dw_up", e, rel)
    rr = ((layer.router.grad.float() - ref_layer.router.grad.float()).norm() / (ref_layer.router.grad.float().norm() + 1e-6)).item()
    assert rr < 0.2, ("drouter", rr)
    assert comm.moe_status() == 0
    comm.close()


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_moe_layer_expert_parallel():
    run_distributed(_moe_worker, min(_ngpu(), 8) if _ngpu() in (2, 4, 8) else 2, "nccl")


def _nvls_worker(rank, world):
    import torch.distributed as dist
    from coccl_b200.parallel.comm import Communicator, Policy
    dev = torch.device("cuda", rank)
    # a policy whose threshold keeps every call uncompressed, autotune on: the first all-reduce of a datatype times
    # NCCL against the multimem kernel and the router picks per size from those numbers
    comm = Communicator(None, dev, Policy.normal("sdp4bit", threshold_bytes=1 << 30, autotune=True), "nvls")
    used, bad = 0, []
    # the kernel itself, whatever the selector prefers: when the fabric offers multicast it must serve the call
    torch.manual_seed(3 + rank)
    x = torch.randn(1 << 18, device=dev)
    ref = x.clone()
    dist.all_reduce(ref)
    served = comm.all_reduce_nvls(x)
    have_mc = comm._nvls is not None and comm._nvls["mc"] != 0
    assert served == have_mc
    if served:
        assert torch.allclose(x, ref, atol=1e-5 * ref.abs().max().item(), rtol=0)
        assert comm.stats["nvls_calls"] == 1
    for dtype, n in ((torch.float32, 4096 * world), (torch.bfloat16, 1 << 20), (torch.float32, (1 << 22) + 64 * world)):
        for it in range(2):
            torch.manual_seed(11 + rank + it)
            x = torch.randn(n, device=dev).to(dtype)
            ref = x.clone()
            dist.all_reduce(ref)
            comm.all_reduce(x)  # below the threshold: multimem path when the fabric offers multicast, else NCCL
            tol = 1e-5 if dtype == torch.float32 else 3e-2
            if not torch.allclose(x.float(), ref.float(), atol=tol * ref.float().abs().max().item(), rtol=0):
                bad.append((str(dtype), n, it))
    # a tensor that lives in the symmetric buffer is reduced in place: no staging copies
    sym = comm.symmetric_tensor(1 << 20, torch.float32)
    assert (sym is not None) == have_mc
    if sym is not None:
        torch.manual_seed(21 + rank)
        sym.copy_(torch.randn(1 << 20, device=dev))
        ref = sym.clone()
        dist.all_reduce(ref)
        copies, calls = comm.stats.get("nvls_staged_copies", 0), comm.stats["nvls_calls"]
        assert comm.all_reduce_nvls(sym)
        assert comm.stats["nvls_calls"] == calls + 1 and comm.stats.get("nvls_staged_copies", 0) == copies
        assert torch.allclose(sym, ref, atol=1e-5 * ref.abs().max().item(), rtol=0)
        # ordinary tensors still work afterwards (staged behind the handed-out tensor)
        y = torch.randn(1 << 16, device=dev)
        ref = y.clone()
        dist.all_reduce(ref)
        assert comm.all_reduce_nvls(y) and torch.allclose(y, ref, atol=1e-5 * ref.abs().max().item(), rtol=0)
    used = comm.stats.get("nvls_calls", 0)
    if have_mc:
        assert used > 0
    if rank == 0:
        print(f"multicast available: {have_mc}; nvls_calls={used}; measured: {comm.routing_summary().get('measured')}")
    if have_mc:   # the measurements were taken and handed to the router
        assert any(r["what"] == "all_reduce_uncompressed" for r in comm.routing_summary()["measured"])
    # leave in order before judging the result: no rank exits while its memory is still bound to the multicast object
    torch.cuda.synchronize()
    dist.barrier()
    comm.close()
    comm._nvls = None
    torch.cuda.synchronize()
    dist.barrier()
    assert not bad, bad


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_nvls_all_reduce_or_native_fallback():
    run_distributed(_nvls_worker, min(_ngpu(), 8) if _ngpu() in (2, 4, 8) else 2, "nccl")


def _lost_peer_worker(rank, world):
    """Rank 1 never launches its side of an all-reduce: rank 0's bounded waits run out (50 ms), the kernel returns,
    and the status word copied after the call makes poll_status raise PeerLost with the phase and peer. Nothing
    traps or hangs; rank 1 has no kernel in flight."""
    import torch.distributed as dist
    from coccl_b200.parallel.comm import Communicator, PeerLost, Policy
    dev = torch.device("cuda", rank)
    comm = Communicator(None, dev, Policy.normal("sdp4bit", threshold_bytes=0, all_reduce_algorithm="twoshot", timeout_ms=50.0), "default")
    x = torch.randn(world * 65536, device=dev)
    comm.all_reduce(x.clone())          # both ranks: maps the peer memory, epoch 1
    comm.post_status_read()
    comm.poll_status(wait=True)         # healthy
    dist.barrier()
    raised = False
    if rank == 0:
        comm.all_reduce(x.clone())      # epoch 2 on rank 0 only
        comm.post_status_read()
        try:
            comm.poll_status(wait=True)
        except PeerLost as e:
            raised = True
            assert e.family == "collective" and e.where["phase"] in (2, 3) and e.where["peer"] < world, e.where
        assert raised
    torch.cuda.synchronize()
    dist.barrier()
    comm.close()


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_lost_peer_raises_on_the_host():
    run_distributed(_lost_peer_worker, 2, "nccl")
