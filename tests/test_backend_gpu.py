"""torch.distributed backend "coccl" on 2 GPUs: collectives above the threshold run compressed, small and
unsupported ones natively, and the rest of the c10d surface is served by the inner NCCL group."""
import os
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      COCCL_ENABLE="1", COCCL_CONFIG_FILE=str(ROOT / "coccl_b200" / "configs" / "normal-sdp4bit.toml"))
    import sys
    sys.path.insert(0, str(ROOT))
    torch.cuda.set_device(rank)
    import coccl_b200.parallel.backend  # noqa: F401  (registers "coccl")
    dist.init_process_group("coccl", rank=rank, world_size=world)
    dev = torch.device("cuda", rank)
    torch.manual_seed(rank)
    n = world * (3 << 20)   # 24 MiB of fp32 per rank: above the 8 MiB threshold
    x = torch.randn(n, device=dev) * 0.01
    ref = x.clone()
    xs = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(xs, ref)                     # list form -> inner NCCL, exact
    exact = sum(xs)
    y = x.clone()
    dist.all_reduce(y)
    rel = ((y - exact).norm() / exact.norm()).item()
    assert 1e-4 < rel < 0.3, rel                 # lossy: it did go through the 4-bit codec
    small = x[:1024].clone()
    dist.all_reduce(small)
    assert torch.allclose(small, exact[:1024], atol=1e-6)   # below the threshold: native and exact
    out = torch.empty(n // world, device=dev)
    dist.reduce_scatter_tensor(out, x)
    c = n // world
    assert ((out - exact[rank * c:(rank + 1) * c]).norm() / exact.norm()).item() < 0.3
    full = torch.empty(n * world, device=dev)
    dist.all_gather_into_tensor(full, x)
    assert ((full - torch.cat(xs)).norm() / torch.cat(xs).norm()).item() < 0.2
    o2 = torch.empty_like(x)
    dist.all_to_all_single(o2, x)
    want = torch.cat([t[rank * c:(rank + 1) * c] for t in xs])
    assert ((o2 - want).norm() / want.norm()).item() < 0.2
    imax = torch.tensor([rank + 1], device=dev)
    dist.all_reduce(imax, op=dist.ReduceOp.MAX)   # not a sum: native
    assert imax.item() == world
    dist.barrier()
    objs = [None] * world
    dist.all_gather_object(objs, {"rank": rank})
    assert [o["rank"] for o in objs] == list(range(world))
    pg = dist.distributed_c10d._get_default_group()._get_backend(dev)
    native, compressed, deferred, lookups, fused, staged = pg.stats()
    assert compressed >= 4 and fused >= 4 and native >= 2, pg.stats()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_coccl_backend_two_gpus():
    import torch.multiprocessing as mp
    from dist_utils import _free_port
    port = _free_port()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_worker, args=(r, 2, port)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
