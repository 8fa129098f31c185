"""The NCCL-compatible C API end to end on 2 GPUs: communicator init over the system NCCL, TOML policy from
COCCL_CONFIG_FILE, router, fused executor over peer memory, staged pipeline for a codec that cannot run
fused (the stateful delta codec), grouped compressed send/recv, explicit coccl*Comp* calls and statistics."""
import ctypes as C
import os
from pathlib import Path

import pytest
import torch

from dist_utils import run_distributed

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
PLUGINS = ROOT / "coccl_b200" / "lib" / "plugins"

CONFIG = f"""
[runtime]
mode = "normal"
compression_threshold_bytes = 65536
[compressor_plugins]
compressors = ["sdp4bit", "fp8block"]
library_path = "{PLUGINS}"
[autotune]
enabled = false
[normal.all_reduce.default]
compressor = "sdp4bit"
[normal.all_reduce.default.config]
groupCount = 128
quantBits = 4
hadamard = true
rounding = "nearest"
[normal.reduce_scatter.default]
compressor = "sdp4bit"
[normal.reduce_scatter.default.config]
groupCount = 128
quantBits = 4
hadamard = true
rounding = "nearest"
[normal.all_to_all.default]
compressor = "fp8block"
[normal.all_gather.default]
compressor = "sdp4bit"
[normal.all_gather.default.config]
groupCount = 2048
quantBits = 8
subAdd = true
[normal.sendrecv.default]
compressor = "fp8block"
"""


class UniqueId(C.Structure):
    _fields_ = [("internal", C.c_char * 128)]  # passed BY VALUE to CommInitRank, hence a struct


class Stats(C.Structure):
    _fields_ = [(n, C.c_ulonglong) for n in ("native", "compressed", "deferred", "lookups", "fused", "staged")]


def _worker(rank, world, cfg_path):
    import torch.distributed as dist
    os.environ["COCCL_ENABLE"] = "1"
    os.environ["COCCL_CONFIG_FILE"] = cfg_path
    from coccl_b200 import _lib
    from coccl_b200.ops import codec as K
    lib = _lib.lib()
    dev = torch.device("cuda", rank)
    vp, sz, i32 = C.c_void_p, C.c_size_t, C.c_int
    uid = UniqueId()
    if rank == 0:
        assert _lib.declare("cocclApiGetUniqueId", i32, [C.POINTER(UniqueId)])(C.byref(uid)) == 0
    box = [bytes(uid)]
    dist.broadcast_object_list(box, src=0)
    uid = UniqueId.from_buffer_copy(box[0])
    comm = vp()
    init = _lib.declare("cocclApiCommInitRank", i32, [C.POINTER(vp), i32, UniqueId, i32])
    assert init(C.byref(comm), world, uid, rank) == 0
    st = torch.cuda.current_stream().cuda_stream
    F32 = 7
    ar = _lib.declare("cocclApiAllReduce", i32, [vp, vp, sz, i32, i32, vp, vp])
    rs = _lib.declare("cocclApiReduceScatter", i32, [vp, vp, sz, i32, i32, vp, vp])
    ag = _lib.declare("cocclApiAllGather", i32, [vp, vp, sz, i32, vp, vp])
    a2a = _lib.declare("cocclApiAllToAll", i32, [vp, vp, sz, i32, vp, vp])
    send = _lib.declare("cocclApiSend", i32, [vp, sz, i32, i32, vp, vp])
    recv = _lib.declare("cocclApiRecv", i32, [vp, sz, i32, i32, vp, vp])
    gstart = _lib.declare("cocclApiGroupStart", i32, [])
    gend = _lib.declare("cocclApiGroupEnd", i32, [])
    stats_fn = _lib.declare("cocclApiGetStats", None, [C.POINTER(Stats)])

    def stats():
        s = Stats()
        stats_fn(C.byref(s))
        return s

    torch.manual_seed(10 + rank)
    n = world * 100000
    x = torch.randn(n, device=dev) * 0.01
    xs = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(xs, x)
    exact = sum(xs)
    # all-reduce (two-shot by heuristic) through the fused kernel
    y = x.clone()
    assert ar(y.data_ptr(), y.data_ptr(), n, F32, 0, comm, st) == 0
    torch.cuda.synchronize()
    assert ((y - exact).norm() / exact.norm()).item() < 0.25
    s = stats()
    assert s.fused == 1 and s.compressed == 1
    # below the threshold: native, exact
    small = x[:1000].clone()
    assert ar(small.data_ptr(), small.data_ptr(), 1000, F32, 0, comm, st) == 0
    torch.cuda.synchronize()
    assert torch.allclose(small, exact[:1000], atol=1e-6)
    assert stats().native >= 1
    # reduce-scatter vs oracle
    out = torch.empty(n // world, device=dev)
    assert rs(x.data_ptr(), out.data_ptr(), n // world, F32, 0, comm, st) == 0
    torch.cuda.synchronize()
    cfg = K.CodecConfig("sdp4bit", 4, 128, False, True)
    ref = sum(K.reference_roundtrip(t, cfg, world).reshape(world, -1)[rank] for t in xs)
    assert ((out - ref).abs() > 2e-2 * ref.abs().max()).float().mean().item() < 5e-3
    # all-to-all through fp8block (fused)
    o2 = torch.empty_like(x)
    assert a2a(x.data_ptr(), o2.data_ptr(), n // world, F32, comm, st) == 0
    torch.cuda.synchronize()
    ref = torch.cat([K.reference_roundtrip(t, K.MXFP8, world).reshape(world, -1)[rank] for t in xs])
    assert torch.allclose(o2, ref, atol=1e-6, rtol=1e-2)
    fused_before = stats().fused
    # all-gather with the stateful delta codec: staged pipeline; the first call is raw (exact), the second sends deltas
    full = torch.empty(n * world, device=dev)
    for rnd in range(2):
        assert ag(x.data_ptr(), full.data_ptr(), n, F32, comm, st) == 0
        torch.cuda.synchronize()
        assert torch.equal(full, torch.cat(xs)), rnd
    s = stats()
    assert s.staged >= 2 and s.fused == fused_before
    # grouped compressed send/recv: one batch
    peer = 1 - rank
    rbuf = torch.empty_like(x)
    assert gstart() == 0
    assert send(x.data_ptr(), n, F32, peer, comm, st) == 0
    assert recv(rbuf.data_ptr(), n, F32, peer, comm, st) == 0
    assert gend() == 0
    torch.cuda.synchronize()
    ref = K.reference_roundtrip(xs[peer], K.MXFP8, 1)
    assert torch.allclose(rbuf, ref, atol=1e-6, rtol=1e-2)
    # explicit call ignores the threshold
    tiny = x[:4096].clone()
    comp = _lib.declare("cocclAllReduceCompOneShot", i32, [vp, vp, sz, i32, i32, vp, vp])
    before = stats().compressed
    assert comp(tiny.data_ptr(), tiny.data_ptr(), 4096, F32, 0, comm, st) == 0
    torch.cuda.synchronize()
    assert stats().compressed == before + 1
    assert ((tiny - exact[:4096]).norm() / exact[:4096].norm()).item() < 0.3
    assert _lib.declare("cocclApiCommDestroy", i32, [vp])(comm) == 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_c_api_two_gpus(tmp_path):
    p = tmp_path / "policy.toml"
    p.write_text(CONFIG)
    run_distributed(_worker, 2, "nccl", (str(p),))


STAGED_CONFIG = f"""
[runtime]
mode = "normal"
compression_threshold_bytes = 65536
[compressor_plugins]
compressors = ["ans", "zfp"]
library_path = "{PLUGINS}"
[autotune]
enabled = false
[pipeline]
depth = 2
[normal.all_gather.default]
compressor = "ans"
[normal.all_gather.default.config]
probBits = 10
[normal.all_to_all.default]
compressor = "ans"
[normal.all_to_all.default.config]
probBits = 10
[normal.all_reduce.default]
compressor = "ans"
[normal.all_reduce.default.config]
probBits = 10
[normal.reduce_scatter.default]
compressor = "zfp"
[normal.reduce_scatter.default.config]
rate = 12
"""


def _staged_worker(rank, world, cfg_path, transport):
    """Codecs that have no fused kernel form (rANS with its variable-size frames, ZFP at a rate without a tile codec)
    run through the staged pipeline; on one node their encoded bytes must travel through this library's own
    peer-memory exchange kernel, not through a library collective, and give the same answers either way."""
    import torch.distributed as dist
    os.environ["COCCL_ENABLE"] = "1"
    os.environ["COCCL_CONFIG_FILE"] = cfg_path
    if transport:
        os.environ["COCCL_STAGED_TRANSPORT"] = transport
    from coccl_b200 import _lib
    dev = torch.device("cuda", rank)
    vp, sz, i32 = C.c_void_p, C.c_size_t, C.c_int
    uid = UniqueId()
    if rank == 0:
        assert _lib.declare("cocclApiGetUniqueId", i32, [C.POINTER(UniqueId)])(C.byref(uid)) == 0
    box = [bytes(uid)]
    dist.broadcast_object_list(box, src=0)
    uid = UniqueId.from_buffer_copy(box[0])
    comm = vp()
    assert _lib.declare("cocclApiCommInitRank", i32, [C.POINTER(vp), i32, UniqueId, i32])(C.byref(comm), world, uid, rank) == 0
    st = torch.cuda.current_stream().cuda_stream
    F32 = 7
    ar = _lib.declare("cocclApiAllReduce", i32, [vp, vp, sz, i32, i32, vp, vp])
    rs = _lib.declare("cocclApiReduceScatter", i32, [vp, vp, sz, i32, i32, vp, vp])
    ag = _lib.declare("cocclApiAllGather", i32, [vp, vp, sz, i32, vp, vp])
    a2a = _lib.declare("cocclApiAllToAll", i32, [vp, vp, sz, i32, vp, vp])
    peer_calls = _lib.declare("cocclApiPeerExchangeCalls", C.c_ulonglong, [])
    stats_fn = _lib.declare("cocclApiGetStats", None, [C.POINTER(Stats)])
    torch.manual_seed(40 + rank)
    n = world * (1 << 18)
    # values with few distinct bytes, so that the entropy coder really shortens the frames (and a constant block,
    # whose frames come out tiny, next to a noisy one that stays raw)
    x = (torch.randint(-8, 8, (n,), device=dev).float() * 0.125)
    x[: n // 4] = 1.0
    x[n // 2: n // 2 + 65536] = torch.randn(65536, device=dev)
    xs = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(xs, x)
    for rnd in range(2):   # the second round reuses staging halves and flags
        full = torch.empty(n * world, device=dev)
        assert ag(x.data_ptr(), full.data_ptr(), n, F32, comm, st) == 0
        torch.cuda.synchronize()
        assert torch.equal(full, torch.cat(xs)), ("all_gather", rnd)          # lossless
        o = torch.empty_like(x)
        assert a2a(x.data_ptr(), o.data_ptr(), n // world, F32, comm, st) == 0
        torch.cuda.synchronize()
        per = n // world
        assert torch.equal(o, torch.cat([t[rank * per:(rank + 1) * per] for t in xs])), ("all_to_all", rnd)
        y = x.clone()
        assert ar(y.data_ptr(), y.data_ptr(), n, F32, 0, comm, st) == 0
        torch.cuda.synchronize()
        assert torch.allclose(y, sum(xs), atol=1e-5), ("all_reduce", rnd)
        out = torch.empty(per, device=dev)
        assert rs(x.data_ptr(), out.data_ptr(), per, F32, 0, comm, st) == 0
        torch.cuda.synchronize()
        exact = sum(xs)[rank * per:(rank + 1) * per]
        assert ((out - exact).norm() / exact.norm()).item() < 2e-2, ("reduce_scatter zfp rate 12", rnd)
    s = Stats()
    stats_fn(C.byref(s))
    assert s.staged >= 8 and s.fused == 0
    calls = int(peer_calls())
    if transport == "nccl":
        assert calls == 0
    else:
        assert calls >= 8, calls     # every exchange of every staged call went through the peer-memory kernel
    err = C.c_int(0)
    assert _lib.declare("cocclApiCommGetAsyncError", i32, [vp, C.POINTER(C.c_int)])(comm, C.byref(err)) == 0 and err.value == 0
    assert _lib.declare("cocclApiCommDestroy", i32, [vp])(comm) == 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("transport", ["", "nccl"], ids=["peer-memory", "nccl"])
def test_staged_codecs_travel_over_peer_memory(tmp_path, transport):
    p = tmp_path / "staged.toml"
    p.write_text(STAGED_CONFIG)
    run_distributed(_staged_worker, 2, "nccl", (str(p), transport), timeout=300)


# ---------------------------------------------------------------------------- selection from measured times
def _measured_worker(rank, world, cfg_path):
    """[autotune] enabled: the first all-reduce of a size bucket times the one-shot and the two-shot fused kernel in
    place of guessing; the user's buffers are untouched by the trial runs, the result is the compressed sum, and later
    calls of the bucket are not timed again."""
    import torch.distributed as dist
    os.environ["COCCL_ENABLE"] = "1"
    os.environ["COCCL_CONFIG_FILE"] = cfg_path
    from coccl_b200 import _lib
    dev = torch.device("cuda", rank)
    vp, sz, i32 = C.c_void_p, C.c_size_t, C.c_int
    uid = UniqueId()
    if rank == 0:
        assert _lib.declare("cocclApiGetUniqueId", i32, [C.POINTER(UniqueId)])(C.byref(uid)) == 0
    box = [bytes(uid)]
    dist.broadcast_object_list(box, src=0)
    uid = UniqueId.from_buffer_copy(box[0])
    comm = vp()
    assert _lib.declare("cocclApiCommInitRank", i32, [C.POINTER(vp), i32, UniqueId, i32])(C.byref(comm), world, uid, rank) == 0
    ar = _lib.declare("cocclApiAllReduce", i32, [vp, vp, sz, i32, i32, vp, vp])
    measured = _lib.declare("cocclApiMeasuredSelection", None, [C.POINTER(C.c_ulonglong), C.POINTER(C.c_ulonglong)])
    stats_fn = _lib.declare("cocclApiGetStats", None, [C.POINTER(Stats)])

    def table():
        a, b = C.c_ulonglong(), C.c_ulonglong()
        measured(C.byref(a), C.byref(b))
        return a.value, b.value

    st = torch.cuda.current_stream().cuda_stream
    F32, SUM = 7, 0
    torch.manual_seed(20 + rank)
    seen = []
    for n in (1 << 18, 1 << 18, 1 << 22, (1 << 18) + 1024 * world):   # 1 MiB twice, 16 MiB, 1 MiB again (same bucket)
        x = torch.randn(n, device=dev) * 0.01
        keep = x.clone()
        xs = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(xs, x)
        exact = torch.stack(xs).sum(0)
        y = torch.full_like(x, float("nan"))
        assert ar(x.data_ptr(), y.data_ptr(), n, F32, SUM, comm, st) == 0
        torch.cuda.synchronize()
        assert torch.equal(x, keep), "the trial runs must not write the send buffer"
        rel = ((y - exact).float().norm() / exact.float().norm()).item()
        assert 1e-4 < rel < 0.3, (n, rel)
        seen.append(table())
    assert seen[0] == (1, 1) and seen[1] == (1, 1) and seen[2] == (2, 2) and seen[3] == (2, 2), seen
    s = Stats()
    stats_fn(C.byref(s))
    # four real calls plus (1 warm-up + 3 timed) x 2 algorithms x 2 buckets, all through the fused kernels
    assert s.fused == 4 + 16 and s.staged == 0, (s.fused, s.staged)
    err = i32(-1)
    assert _lib.declare("cocclApiCommGetAsyncError", i32, [vp, C.POINTER(i32)])(comm, C.byref(err)) == 0 and err.value == 0
    dist.barrier()
    assert _lib.declare("cocclApiCommDestroy", i32, [vp])(comm) == 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_all_reduce_algorithm_from_measured_times(tmp_path):
    p = tmp_path / "policy.toml"
    p.write_text(CONFIG.replace("[autotune]\nenabled = false", "[autotune]\nenabled = true"))
    assert "enabled = true" in p.read_text()
    run_distributed(_measured_worker, 2, "nccl", (str(p),), timeout=300)
