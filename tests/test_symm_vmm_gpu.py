"""cuMem VMM backend of the symmetric memory (csrc/symm/symm_vmm.cc): physical chunks exported as file descriptors,
growth in place, and the fused collectives running over it; plus the NVSwitch multicast binding the multimem
all-reduce uses when the fabric has one."""
import ctypes as C
import os

import pytest
import torch

from dist_utils import run_distributed

pytestmark = pytest.mark.gpu


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _api():
    from coccl_b200 import _lib
    vp, sz, i32 = C.c_void_p, C.c_size_t, C.c_int
    d = _lib.declare
    return {"set": d("cocclSymmSetBackend", i32, [i32]), "get": d("cocclSymmGetBackend", i32, []),
            "alloc": d("cocclSymmAlloc", i32, [sz, C.POINTER(vp)]), "grow": d("cocclSymmGrow", i32, [vp, sz]),
            "local": d("cocclSymmLocalPtr", vp, [vp]), "bytes": d("cocclSymmBytes", sz, [vp]),
            "free": d("cocclSymmFree", i32, [vp]), "export": d("cocclSymmExport", i32, [vp, vp]),
            "import": d("cocclSymmImport", i32, [vp, i32, vp, C.POINTER(vp)]),
            "hbytes": d("cocclSymmHandleBytes", i32, [])}


def test_vmm_buffer_grows_where_it_is(cuda):
    from coccl_b200 import _lib
    a = _api()
    before = a["get"]()
    if a["set"](1) != 0:
        pytest.skip("cuMem VMM with POSIX descriptors is not available on this device")
    try:
        h = C.c_void_p()
        assert a["alloc"](3 << 20, C.byref(h)) == 0
        base, size = a["local"](h), a["bytes"](h)
        assert size >= 3 << 20 and size % (2 << 20) == 0
        t = _lib.tensor_from_ptr(base, size, cuda)
        assert int(t.sum().item()) == 0          # zero-initialised
        t.fill_(7)
        assert a["grow"](h, 40 << 20) == 0
        assert a["local"](h) == base and a["bytes"](h) >= 40 << 20
        big = _lib.tensor_from_ptr(base, a["bytes"](h), cuda)
        assert int(big[:size].min().item()) == 7 and int(big[size:].max().item()) == 0   # old part kept, new part zero
        big[size:].fill_(9)
        torch.cuda.synchronize()
        assert int(big[-1].item()) == 9
        assert a["grow"](h, 1 << 20) == 0          # never shrinks, never fails for a smaller request
        # an IPC buffer cannot grow in place and says so
        a["set"](0)
        g = C.c_void_p()
        assert a["alloc"](1 << 20, C.byref(g)) == 0 and a["grow"](g, 8 << 20) != 0
        del t, big
        assert a["free"](g) == 0 and a["free"](h) == 0
    finally:
        a["set"](before)


def _collectives_over_vmm(rank, world):
    import torch.distributed as dist
    from coccl_b200.parallel.comm import Communicator, Policy
    dev = torch.device("cuda", rank)
    comm = Communicator(None, dev, Policy.normal("sdp4bit", {"groupCount": 128, "quantBits": 4, "quantType": "Symmetric",
                                                             "hadamard": True}, threshold_bytes=0), "vmm")
    ptrs = None
    for numel in (1 << 18, 1 << 22, 1 << 25):        # the workspace grows twice
        torch.manual_seed(numel + rank)
        x = torch.randn(numel, device=dev) * 0.01
        exact = x.clone()
        dist.all_reduce(exact)
        y = x.clone()
        comm.all_reduce(y)
        assert ((y - exact).norm() / exact.norm()).item() < 0.3
        assert comm._ws is not None and comm._ws.backend == 1
        if ptrs is None:
            ptrs = list(comm._ws.ptrs)
        assert list(comm._ws.ptrs) == ptrs, "growth moved a mapping"
        out = torch.empty(numel // world, device=dev)
        comm.reduce_scatter(x, out)
        chunk = exact.view(world, -1)[rank]
        assert ((out - chunk).norm() / chunk.norm()).item() < 0.3
    assert comm.status() == 0 and comm.stats["compressed_calls"] == 6
    comm.close()


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_fused_collectives_over_vmm_regions(monkeypatch):
    monkeypatch.setenv("COCCL_SYMM_BACKEND", "vmm")
    run_distributed(_collectives_over_vmm, 2, "nccl", timeout=300)


def _own_multicast(rank, world):
    import torch.distributed as dist
    from coccl_b200 import _lib
    from coccl_b200.parallel.comm import Communicator, Policy
    dev = torch.device("cuda", rank)
    comm = Communicator(None, dev, Policy.normal("sdp4bit", threshold_bytes=1 << 30, autotune=False), "nvls")
    supported = _lib.declare("cocclSymmMulticastSupported", C.c_int, [])() == 1
    sym = comm.symmetric_tensor(1 << 20, torch.float32)
    own = comm._nvls is not None and comm._nvls.get("h") is not None and type(comm._nvls["h"]).__name__ == "_Symm"
    if rank == 0:
        print(f"multicast supported by the driver: {supported}; own binding in use: {own}; "
              f"multicast address: {comm._nvls['mc'] if comm._nvls else 0:#x}")
    # failures are collected and judged only after the orderly teardown: no rank leaves while its memory is still bound
    # to the multicast object
    bad = []
    if supported and not (own and sym is not None):
        bad.append("the library's own multicast binding must serve where the device supports it")
    if sym is not None:
        for it in range(3):
            torch.manual_seed(31 + rank + it)
            sym.copy_(torch.randn(1 << 20, device=dev))
            ref = sym.clone()
            dist.all_reduce(ref)
            if not comm.all_reduce_nvls(sym):
                bad.append(f"call {it} not served")
            elif not torch.allclose(sym, ref, atol=1e-5 * ref.abs().max().item(), rtol=0):
                bad.append(f"call {it} wrong by {(sym - ref).abs().max().item()}")
        if comm.stats.get("nvls_staged_copies", 0) != 0:
            bad.append("in-place call staged copies")
    torch.cuda.synchronize()
    dist.barrier()
    comm.close()      # unbinds while every rank is alive, then unmaps, then frees
    torch.cuda.synchronize()
    dist.barrier()
    assert not bad, bad


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_multimem_all_reduce_over_own_multicast_binding(monkeypatch):
    monkeypatch.setenv("COCCL_NVLS_BACKEND", "own")
    run_distributed(_own_multicast, min(_ngpu(), 8) if _ngpu() in (2, 4, 8) else 2, "nccl", timeout=300)
