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


def test_status_word_raises_peer_lost_with_decoded_fields():
    """poll_status turns a non-zero status word (as a bounded wait writes it: 0x80000000 | phase << 23 | peer << 15 |
    slice) into PeerLost; a pending copy whose event has not completed is left for the next poll."""
    import torch
    from coccl_b200.parallel.comm import Communicator, PeerLost

    class Ev:
        def __init__(self, done): self.done = done
        def query(self): return self.done
        def synchronize(self): self.done = True

    c = Communicator(None, None, None, "dp")
    word = 0x80000000 | (2 << 23) | (5 << 15) | 77
    host = torch.zeros(16, dtype=torch.int32)
    host[1] = word - (1 << 32)
    c._health = {"host": host, "event": Ev(False), "families": ["collective", "tensor-parallel fusion"], "pending": True}
    c.poll_status(wait=False)            # copy still in flight: nothing raised, still pending
    assert c._health["pending"]
    try:
        c.poll_status(wait=True)
    except PeerLost as e:
        assert e.family == "tensor-parallel fusion" and e.where == {"phase": 2, "peer": 5, "slice": 77}
    else:
        raise AssertionError("PeerLost not raised")
    assert not c._health["pending"]
    c.poll_status(wait=True)             # consumed: a second poll is quiet


def test_tp_fusion_follows_the_policy():
    """The one-kernel TP fusions quantise to FP8: they are taken only when the router, reading the policy file, answers
    "compressed" for the tensor-parallel all-gather and names the MX-FP8 codec for the tensor-parallel reduce-scatter,
    i.e. also only above the threshold."""
    from coccl_b200.parallel.comm import NATIVE, Communicator, Policy, Router

    def fusable(policy, rows=4096, n=1024, width=1024):
        c = Communicator(None, None, policy, "tp")
        c.cuda, c.size, c._tp_sig = True, 2, object()   # pretend: CUDA group of two with its signal region open
        c.router = Router.of(policy, 2)
        return c.tp_fusable(rows, n, width)

    base = Policy.training(threshold_bytes=0)
    assert fusable(base)
    rs = '[training.tp.reduce_scatter.default]\ncompressor = "fp8block"\n'
    ag = '[training.tp.all_gather.default]\ncompressor = "fp8block"\n'
    assert rs in base.toml and ag in base.toml
    assert not fusable(Policy(toml=base.toml.replace(rs, "")))          # no codec on the reduce-scatter
    assert not fusable(Policy(toml=base.toml.replace(ag, "")))          # no codec on the all-gather
    sdp = rs.replace('"fp8block"', '"sdp4bit"')
    assert not fusable(Policy(toml=base.toml.replace(rs, sdp)))         # another codec: the unfused path serves it
    assert not fusable(Policy.training(threshold_bytes=4096 * 1024 * 2))      # bytes <= threshold stays native
    assert fusable(Policy.training(threshold_bytes=4096 * 1024 * 2 - 1))
    assert not fusable(NATIVE)
