"""Training mode and the explicit calls of the C API on real GPUs.

Two programs, after tests/coccl-tests/src/coccl_training_known_roles.cc:36-160 and
tests/coccl-tests/src/coccl_collective_correctness.cu:355-408 of the reference:

  * known roles: the world is split into a data-, a tensor- and a pipeline-parallel communicator of the SAME size, so
    that only the traffic can tell them apart; after the observation window each must carry its role, route by the
    role's policy from a common call on, and a communicator that appears later with one constant collective must
    stay unknown and native;
  * correctness: every explicit coccl*Comp* entry point is called once next to the native collective on the same
    input, and the mean relative error is reported and bounded. With four GPUs the run also pretends to be two
    nodes of two ranks (COCCL_LOCAL_RANKS=2), which makes the two-level recipes real.
"""
import ctypes as C
import json
import os
import time
from pathlib import Path

import pytest
import torch

from dist_utils import run_distributed

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
PLUGINS = ROOT / "coccl_b200" / "lib" / "plugins"

SDP4 = 'groupCount = 128\nquantBits = 4\nquantType = "Symmetric"\nhadamard = true\nrounding = "nearest"\n'
SDP8 = 'groupCount = 2048\nquantBits = 8\nquantType = "Symmetric"\n'

TRAINING = f"""
[runtime]
mode = "training"
compression_threshold_bytes = 65536
[compressor_plugins]
compressors = ["sdp4bit", "fp8block"]
library_path = "{PLUGINS}"
[training]
observation_iterations = 5
[training.classifier]
data_parallel_size = 2
tensor_parallel_size = 2
pipeline_parallel_size = 2
dp_strategy = "sdp"
sequence_parallel = true
[training.dp.reduce_scatter.default]
compressor = "sdp4bit"
[training.dp.reduce_scatter.default.config]
{SDP4}
[training.dp.all_gather.default]
compressor = "sdp4bit"
[training.dp.all_gather.default.config]
{SDP8}
[training.tp.all_reduce.default]
compressor = "fp8block"
[autotune]
enabled = false
"""


def _scoped(op: str, codec: str, options: str) -> str:
    out = ""
    for scope in ("default", "intra", "inter"):
        out += f"[normal.{op}.{scope}]\ncompressor = \"{codec}\"\n"
        if options:
            out += f"[normal.{op}.{scope}.config]\n{options}"
    return out


NORMAL = f"""
[runtime]
mode = "normal"
compression_threshold_bytes = 1073741824
[compressor_plugins]
compressors = ["sdp4bit", "fp8block"]
library_path = "{PLUGINS}"
[autotune]
enabled = false
{_scoped("all_reduce", "sdp4bit", SDP4)}
{_scoped("reduce_scatter", "sdp4bit", SDP4)}
[normal.all_gather.default]
compressor = "sdp4bit"
[normal.all_gather.default.config]
{SDP8}
[normal.all_to_all.default]
compressor = "fp8block"
[normal.sendrecv.default]
compressor = "fp8block"
"""


class UniqueId(C.Structure):
    _fields_ = [("internal", C.c_char * 128)]


class Stats(C.Structure):
    _fields_ = [(n, C.c_ulonglong) for n in ("native", "compressed", "deferred", "lookups", "fused", "staged")]


class TrainingRole(C.Structure):
    _fields_ = [("role", C.c_int), ("candidate", C.c_int), ("committed", C.c_int), ("active", C.c_int),
                ("confidence", C.c_double), ("calls_per_iteration", C.c_double), ("ag_to_rs", C.c_double),
                ("observed", C.c_ulonglong), ("activation", C.c_ulonglong)]


DP, TP, PP, UNKNOWN = 1, 2, 3, 4
F32 = 7


class Api:
    def __init__(self, rank, world, cfg_path, local_ranks=None):
        import torch.distributed as dist
        os.environ["COCCL_ENABLE"] = "1"
        os.environ["COCCL_CONFIG_FILE"] = cfg_path
        if local_ranks:
            os.environ["COCCL_LOCAL_RANKS"] = str(local_ranks)
        from coccl_b200 import _lib
        self.L = _lib
        vp, sz, i32 = C.c_void_p, C.c_size_t, C.c_int
        self.vp = vp
        uid = UniqueId()
        if rank == 0:
            assert _lib.declare("cocclApiGetUniqueId", i32, [C.POINTER(UniqueId)])(C.byref(uid)) == 0
        box = [bytes(uid)]
        dist.broadcast_object_list(box, src=0)
        uid = UniqueId.from_buffer_copy(box[0])
        self.world = vp()
        assert _lib.declare("cocclApiCommInitRank", i32, [C.POINTER(vp), i32, UniqueId, i32])(C.byref(self.world), world, uid, rank) == 0
        red = [vp, vp, sz, i32, i32, vp, vp]
        plain = [vp, vp, sz, i32, vp, vp]
        p2p = [vp, sz, i32, i32, vp, vp]
        self.fn = {}
        for name, sig in (("cocclApiAllReduce", red), ("cocclApiReduceScatter", red), ("cocclApiAllGather", plain),
                          ("cocclApiAllToAll", plain), ("cocclApiSend", p2p), ("cocclApiRecv", p2p),
                          ("cocclAllReduceCompOneShot", red), ("cocclAllReduceCompTwoShot", red),
                          ("cocclAllReduceCompTripleShot", red), ("cocclReduceScatterCompOneShot", red),
                          ("cocclReduceScatterCompTwoShot", red), ("cocclAllGatherComp", plain), ("cocclAllToAllComp", plain),
                          ("cocclSendComp", p2p), ("cocclRecvDecomp", p2p)):
            self.fn[name] = _lib.declare(name, i32, sig)
        self.group_start = _lib.declare("cocclApiGroupStart", i32, [])
        self.group_end = _lib.declare("cocclApiGroupEnd", i32, [])
        self._split = _lib.declare("cocclApiCommSplit", i32, [vp, i32, i32, C.POINTER(vp), vp])
        self._stats = _lib.declare("cocclApiGetStats", None, [C.POINTER(Stats)])
        self._role = _lib.declare("cocclApiCommTrainingRole", i32, [vp, C.POINTER(TrainingRole)])
        self._destroy = _lib.declare("cocclApiCommDestroy", i32, [vp])

    def split(self, color, key):
        child = self.vp()
        assert self._split(self.world, color, key, C.byref(child), None) == 0
        return child

    def stats(self):
        s = Stats()
        self._stats(C.byref(s))
        return s

    def role(self, comm):
        r = TrainingRole()
        assert self._role(comm, C.byref(r)) == 0
        return r

    def destroy(self, *comms):
        for c in comms:
            assert self._destroy(c) == 0


def _known_roles(rank, world, cfg_path):
    import torch.distributed as dist
    api = Api(rank, world, cfg_path)
    dev = torch.device("cuda", rank)
    st = torch.cuda.current_stream().cuda_stream
    dp, tp, pp = api.split(0, rank), api.split(0, rank), api.split(0, rank)
    n = 1 << 18  # 1 MiB of fp32: the smallest call the classifier takes as evidence
    torch.manual_seed(5 + rank)
    send = torch.randn(2 * n, device=dev) * 0.01
    recv = torch.empty(2 * n, device=dev)
    f = api.fn
    peer = 1 - rank

    def cycle():
        assert f["cocclApiAllGather"](send.data_ptr(), recv.data_ptr(), n // 2, F32, dp, st) == 0        # bf16-like parameters
        for _ in range(6):
            assert f["cocclApiAllReduce"](send.data_ptr(), recv.data_ptr(), n, F32, 0, tp, st) == 0
        assert api.group_start() == 0
        for _ in range(4):
            if rank == 0:
                assert f["cocclApiSend"](send.data_ptr(), n, F32, peer, pp, st) == 0
                assert f["cocclApiRecv"](recv.data_ptr(), n, F32, peer, pp, st) == 0
            else:
                assert f["cocclApiRecv"](recv.data_ptr(), n, F32, peer, pp, st) == 0
                assert f["cocclApiSend"](send.data_ptr(), n, F32, peer, pp, st) == 0
        assert api.group_end() == 0
        assert f["cocclApiReduceScatter"](send.data_ptr(), recv.data_ptr(), n, F32, 0, dp, st) == 0      # fp32 gradients: 2x the gather
        torch.cuda.synchronize()
        time.sleep(0.005)  # the optimizer step: the pause that marks an iteration

    for _ in range(5):
        cycle()
    # inside the window everything is native and nothing is active yet
    assert api.stats().compressed == 0
    for c in (dp, tp):
        assert api.role(c).active == 0
    assert api.role(pp).role == PP   # point-to-point traffic on a communicator of the pipeline size: decided by size at once
    for _ in range(11):
        cycle()
    roles = {"dp": api.role(dp), "tp": api.role(tp), "pp": api.role(pp)}
    assert (roles["dp"].role, roles["tp"].role, roles["pp"].role) == (DP, TP, PP), {k: v.role for k, v in roles.items()}
    for r in roles.values():
        assert r.committed == 1 and r.active == 1 and r.confidence >= 0.6
    assert abs(roles["dp"].ag_to_rs - 0.5) < 0.05
    assert roles["tp"].calls_per_iteration == 6.0 and roles["dp"].calls_per_iteration == 2.0
    # both ranks switched at the same call: the activation call numbers agree
    acts = [None, None]
    dist.all_gather_object(acts, [roles[k].activation for k in ("dp", "tp", "pp")])
    assert acts[0] == acts[1], acts
    assert api.stats().compressed > 0

    # routed by role: the DP reduce-scatter is now SDP4Bit, the TP all-reduce block-scaled FP8, PP stays native
    xs = [torch.empty_like(send) for _ in range(world)]
    dist.all_gather(xs, send)
    before = api.stats()
    out = torch.empty(n, device=dev)
    assert f["cocclApiReduceScatter"](send.data_ptr(), out.data_ptr(), n, F32, 0, dp, st) == 0
    y = send[:n].clone()
    assert f["cocclApiAllReduce"](y.data_ptr(), y.data_ptr(), n, F32, 0, tp, st) == 0
    torch.cuda.synchronize()
    after = api.stats()
    assert after.compressed == before.compressed + 2
    exact_rs = sum(t[rank * n:(rank + 1) * n] for t in xs)
    exact_ar = sum(t[:n] for t in xs)
    e_rs = ((out - exact_rs).abs().mean() / exact_rs.abs().mean()).item()
    e_ar = ((y - exact_ar).abs().mean() / exact_ar.abs().mean()).item()
    assert 1e-4 < e_rs < 0.3 and 1e-5 < e_ar < 0.08, (e_rs, e_ar)   # lossy, so not exactly zero either
    native_before = api.stats().native
    assert api.group_start() == 0
    if rank == 0:
        assert f["cocclApiSend"](send.data_ptr(), n, F32, peer, pp, st) == 0
    else:
        assert f["cocclApiRecv"](recv.data_ptr(), n, F32, peer, pp, st) == 0
    assert api.group_end() == 0
    torch.cuda.synchronize()
    if rank == 1:
        assert torch.equal(recv[:n], xs[0][:n])   # no pipeline policy: exact
    assert api.stats().native > native_before
    # a role without a policy for the operation stays native (DP all-reduce has none)
    z = send[:n].clone()
    assert f["cocclApiAllReduce"](z.data_ptr(), z.data_ptr(), n, F32, 0, dp, st) == 0
    torch.cuda.synchronize()
    assert torch.allclose(z, exact_ar, atol=1e-6)

    # a communicator that shows up after the roles are fixed, with one constant collective: unknown, native
    late = api.split(0, rank)
    for _ in range(16):
        w = send[:n].clone()
        assert f["cocclApiAllReduce"](w.data_ptr(), w.data_ptr(), n, F32, 0, late, st) == 0
        torch.cuda.synchronize()
        time.sleep(0.002)
    r = api.role(late)
    assert r.active == 0 and (r.committed == 0 or r.role == UNKNOWN)
    assert torch.allclose(w, exact_ar, atol=1e-6)
    api.destroy(late, dp, tp, pp, api.world)


def _mre(got, exact):
    return ((got - exact).abs().mean() / exact.abs().mean()).item()


def _correctness(rank, world, cfg_path, local_ranks, report_path):
    import torch.distributed as dist
    api = Api(rank, world, cfg_path, local_ranks)
    dev = torch.device("cuda", rank)
    st = torch.cuda.current_stream().cuda_stream
    comm, f = api.world, api.fn
    torch.manual_seed(77 + rank)
    per = 1 << 18
    n = world * per
    x = torch.randn(n, device=dev) * 0.01
    xs = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(xs, x)
    exact_sum = sum(xs)
    rows = {}

    def run_ar(name):
        y = x.clone()
        assert f[name](y.data_ptr(), y.data_ptr(), n, F32, 0, comm, st) == 0, name
        torch.cuda.synchronize()
        rows[name] = _mre(y, exact_sum)

    def run_rs(name):
        out = torch.empty(per, device=dev)
        assert f[name](x.data_ptr(), out.data_ptr(), per, F32, 0, comm, st) == 0, name
        torch.cuda.synchronize()
        rows[name] = _mre(out, exact_sum[rank * per:(rank + 1) * per])

    before = api.stats().compressed
    # the threshold of this policy is 1 GiB: automatic routing would leave every call native
    y = x.clone()
    assert f["cocclApiAllReduce"](y.data_ptr(), y.data_ptr(), n, F32, 0, comm, st) == 0
    torch.cuda.synchronize()
    rows["native all_reduce"] = _mre(y, exact_sum)
    assert api.stats().compressed == before
    run_ar("cocclAllReduceCompOneShot")
    run_ar("cocclAllReduceCompTwoShot")
    run_ar("cocclAllReduceCompTripleShot")
    run_rs("cocclReduceScatterCompOneShot")
    run_rs("cocclReduceScatterCompTwoShot")
    full = torch.empty(n * world, device=dev)
    assert f["cocclAllGatherComp"](x.data_ptr(), full.data_ptr(), n, F32, comm, st) == 0
    torch.cuda.synchronize()
    rows["cocclAllGatherComp"] = _mre(full, torch.cat(xs))
    o = torch.empty_like(x)
    assert f["cocclAllToAllComp"](x.data_ptr(), o.data_ptr(), per, F32, comm, st) == 0
    torch.cuda.synchronize()
    rows["cocclAllToAllComp"] = _mre(o, torch.cat([t[rank * per:(rank + 1) * per] for t in xs]))
    peer = rank ^ 1
    r = torch.empty_like(x)
    assert api.group_start() == 0
    assert f["cocclSendComp"](x.data_ptr(), n, F32, peer, comm, st) == 0
    assert f["cocclRecvDecomp"](r.data_ptr(), n, F32, peer, comm, st) == 0
    assert api.group_end() == 0
    torch.cuda.synchronize()
    rows["cocclSendComp/cocclRecvDecomp"] = _mre(r, xs[peer])
    assert api.stats().compressed >= before + 8
    # bounds: exact for native; 4-bit groups of 128 land near 0.17 per encode (two or three encodes on the longer
    # recipes), 8-bit groups of 2048 near 0.01, block-scaled FP8 near 0.03
    assert rows["native all_reduce"] < 1e-6
    limits = {"cocclAllReduceCompOneShot": 0.25, "cocclAllReduceCompTwoShot": 0.35, "cocclAllReduceCompTripleShot": 0.45,
              "cocclReduceScatterCompOneShot": 0.25, "cocclReduceScatterCompTwoShot": 0.35, "cocclAllGatherComp": 0.02,
              "cocclAllToAllComp": 0.05, "cocclSendComp/cocclRecvDecomp": 0.05}
    for k, lim in limits.items():
        assert 1e-5 < rows[k] < lim, (k, rows[k], lim)
    if rank == 0:
        s = api.stats()
        report = {"n_gpus": world, "local_ranks": local_ranks or world, "elements": n, "mean_relative_error": rows,
                  "fused_calls": int(s.fused), "staged_calls": int(s.staged)}
        print("CAPI_CORRECTNESS " + json.dumps(report), flush=True)
        if report_path:
            Path(report_path).parent.mkdir(parents=True, exist_ok=True)
            with open(report_path, "a") as fh:
                fh.write(json.dumps(report) + "\n")
    api.destroy(api.world)


def _report_path():
    return os.environ.get("COCCL_TEST_REPORT", "")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_known_roles_two_gpus(tmp_path):
    p = tmp_path / "training.toml"
    p.write_text(TRAINING)
    run_distributed(_known_roles, 2, "nccl", (str(p),), timeout=300)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_explicit_calls_mean_relative_error_two_gpus(tmp_path):
    p = tmp_path / "normal.toml"
    p.write_text(NORMAL)
    run_distributed(_correctness, 2, "nccl", (str(p), None, _report_path()), timeout=300)


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_explicit_calls_two_level_on_four_gpus(tmp_path):
    """Four GPUs of one box declared as two nodes of two ranks: the reduce-scatter two-shot and the all-reduce
    triple-shot run their intra-node and inter-node levels on different communicators."""
    p = tmp_path / "normal.toml"
    p.write_text(NORMAL)
    run_distributed(_correctness, 4, "nccl", (str(p), 2, _report_path()), timeout=300)
