"""Failure detection without any GPU fault: failures are made on the host (a rank that leaves between steps, a
rank that never joins, a rank that raises), and the survivors learn of them from the store or from a short
process-group timeout. gloo ranks on CPU."""
import datetime
import os
import socket
import time

import pytest
import torch
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _leave_worker(rank, world, port, q):
    import torch.distributed as dist
    from coccl_b200.utils.health import Heartbeat, PeerLost
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=30))
    dist.init_process_group("gloo", store=store, rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    hb = Heartbeat(store, rank, world, stale_after_s=2.0)
    x = torch.ones(4)
    result = "finished"
    try:
        for step in range(4):
            hb.check_peers(expect_step=step - 1, wait_s=5.0)   # before launching anything of this step
            dist.all_reduce(x)
            hb.beat(step)
            if rank == world - 1 and step == 1:
                hb.leave(step)  # orderly: between steps, nothing in flight
                result = "left"
                break
    except PeerLost as e:
        result = f"lost:{e.rank}:{step}"
    q.put((rank, result))
    if result == "left":
        time.sleep(1.0)  # keep the sockets open while the others read the store
    os._exit(0)  # no collective teardown with a missing peer


def test_rank_leaving_between_steps_is_seen_on_the_host():
    world, port = 3, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    ps = [ctx.Process(target=_leave_worker, args=(r, world, port, q)) for r in range(world)]
    for p in ps:
        p.start()
    for p in ps:
        p.join(60)
    res = dict(q.get() for _ in range(world))
    assert res[2] == "left"
    assert res[0] == "lost:2:2" and res[1] == "lost:2:2", res  # noticed before step 2 launched


def _absent_worker(rank, world, port, q):
    import torch.distributed as dist
    from coccl_b200.utils.health import Heartbeat, PeerLost
    if rank == world - 1:
        q.put((rank, "absent"))
        return  # never joins
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), wait_for_workers=False,
                          timeout=datetime.timedelta(seconds=5))
    hb = Heartbeat(store, rank, world, stale_after_s=1.0)
    try:
        hb.check_peers(expect_step=-1, wait_s=1.5)
        q.put((rank, "ok"))
    except PeerLost as e:
        q.put((rank, f"lost:{e.rank}:{e.reason}"))
    time.sleep(0.5)


def test_rank_that_never_joins_is_reported():
    world, port = 3, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    ps = [ctx.Process(target=_absent_worker, args=(r, world, port, q)) for r in range(world)]
    for p in ps:
        p.start()
    for p in ps:
        p.join(60)
    res = dict(q.get() for _ in range(world))
    assert res[0].startswith("lost:2:never registered") and res[1].startswith("lost:2:never registered"), res


def _raise_worker(rank, world, port, q):
    import torch.distributed as dist
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=30))
    dist.init_process_group("gloo", store=store, rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    x = torch.ones(4)
    dist.all_reduce(x)
    if rank == 1:
        q.put((rank, "raised"))
        os._exit(1)  # dies between steps without telling anyone
    try:
        dist.all_reduce(x)  # the short process-group timeout ends this collective with an error
        q.put((rank, "no error"))
    except Exception as e:  # noqa: BLE001
        q.put((rank, "error:" + type(e).__name__))
    os._exit(0)


def test_short_process_group_timeout_ends_a_collective_with_a_dead_peer():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    ps = [ctx.Process(target=_raise_worker, args=(r, world, port, q)) for r in range(world)]
    for p in ps:
        p.start()
    for p in ps:
        p.join(60)
    res = dict(q.get() for _ in range(world))
    assert res[1] == "raised" and res[0].startswith("error:"), res


def test_plugin_load_failure_degrades_to_an_error_not_a_crash(tmp_path):
    """Host-side fault injection: a policy that names a plugin that cannot be loaded is rejected at load time."""
    import subprocess
    from pathlib import Path
    from coccl_b200 import _build
    _build.build()
    lib = Path(_build.__file__).resolve().parent / "lib"
    bad = tmp_path / "bad.toml"
    bad.write_text('[runtime]\nmode = "normal"\n[compressor_plugins]\ncompressors = ["nosuchcodec"]\n'
                   f'library_path = "{lib / "plugins"}"\n[normal.all_reduce.default]\ncompressor = "nosuchcodec"\n')
    r = subprocess.run([str(lib / "coccl-config-check"), str(bad)], capture_output=True, text=True)
    assert r.returncode == 1 and "nosuchcodec" in r.stderr
