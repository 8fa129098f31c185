"""Communicator: one per process group; routes every collective either to a fused
compressed kernel over peer-mapped symmetric memory or to torch.distributed
(NCCL on GPUs, gloo on CPU).

Routing mirrors the reference router (src/coccl-extend/core/runtime/coccl_runtime.cc:181-229):
compression must be enabled, a codec must be configured for (role, operation), the
datatype must be one the codec handles, the reduction must be a sum, an all-reduce
must be divisible by the group size, and the message must be LARGER than the
threshold (`bytes <= threshold` stays native). Total bytes are scaled by the number
of ranks for all-gather / reduce-scatter / all-to-all (coccl_runtime.cc:57-76).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from .. import _lib
from ..ops import collective as K
from ..ops.codec import MXFP8, SDP4BIT_G128, CodecConfig, DTYPE_CODE


@dataclass
class Policy:
    """Per (role, operation) codec selection; None = native."""
    enabled: bool = True
    threshold_bytes: int = 8 << 20
    codecs: dict = field(default_factory=lambda: {
        ("dp", "reduce_scatter"): SDP4BIT_G128,
        ("dp", "all_reduce"): SDP4BIT_G128,
        ("dp", "all_gather"): None,            # parameters: kept exact (no delta codec state yet)
        ("tp", "all_gather"): MXFP8,
        ("tp", "reduce_scatter"): MXFP8,
        ("tp", "all_reduce"): MXFP8,
        ("ep", "all_to_all"): MXFP8,
        ("default", "reduce_scatter"): SDP4BIT_G128,
        ("default", "all_gather"): SDP4BIT_G128,
        ("default", "all_reduce"): SDP4BIT_G128,
        ("default", "all_to_all"): SDP4BIT_G128,
    })
    all_reduce_oneshot_max_bytes: int = 1 << 20
    timeout_ms: float = 20000.0
    max_ctas: int = 0

    def codec_for(self, role: str, op: str) -> CodecConfig | None:
        if not self.enabled:
            return None
        return self.codecs.get((role, op), None)


NATIVE = Policy(enabled=False)


class _Symm:
    """A symmetric buffer: local allocation + mapped peers."""

    def __init__(self, comm: "Communicator", nbytes: int):
        lib = _lib.lib()
        self._alloc = _lib.declare("cocclSymmAlloc", C.c_int, [C.c_size_t, C.POINTER(C.c_void_p)])
        self._export = _lib.declare("cocclSymmExport", C.c_int, [C.c_void_p, C.c_void_p])
        self._import = _lib.declare("cocclSymmImport", C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.POINTER(C.c_void_p)])
        self._local = _lib.declare("cocclSymmLocalPtr", C.c_void_p, [C.c_void_p])
        self._free = _lib.declare("cocclSymmFree", C.c_int, [C.c_void_p])
        h = C.c_void_p()
        _lib.check(self._alloc(nbytes, C.byref(h)), "cocclSymmAlloc")
        self.handle, self.nbytes = h, nbytes
        buf = C.create_string_buffer(64)
        _lib.check(self._export(h, buf), "cocclSymmExport")
        handles = [None] * comm.size
        dist.all_gather_object(handles, bytes(buf.raw), group=comm.group)
        self.ptrs = []
        for p in range(comm.size):
            if p == comm.rank:
                self.ptrs.append(self._local(h))
            else:
                m = C.c_void_p()
                hb = C.create_string_buffer(handles[p], 64)
                _lib.check(self._import(h, p, hb, C.byref(m)), "cocclSymmImport")
                self.ptrs.append(m.value)

    def free(self):
        if self.handle is not None:
            self._free(self.handle)
            self.handle = None


class Communicator:
    def __init__(self, group=None, device=None, policy: Policy | None = None, name: str = "default"):
        self.group = group
        self.size = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = device
        self.policy = policy or Policy()
        self.name = name
        self.cuda = device is not None and torch.device(device).type == "cuda"
        self.epoch = 0
        self._ws: _Symm | None = None
        self._ws_half = 0
        self._sig: _Symm | None = None
        self.stats = {"compressed_calls": 0, "native_calls": 0, "compressed_raw_bytes": 0, "native_bytes": 0}
        if self.size > _lib.MAX_RANKS:
            self.policy = NATIVE  # fused kernels cover one NVSwitch domain of up to 8 ranks

    # ------------------------------------------------------------------ symmetric state
    def _ensure(self, half_bytes: int):
        if self._sig is None:
            flag_bytes = _lib.lib().cocclkFlagBytes()
            self._flag_bytes = flag_bytes
            self._sig = _Symm(self, flag_bytes + 256)
        if self._ws is None or self._ws_half < half_bytes:
            if self._ws is not None:
                torch.cuda.synchronize()
                dist.barrier(group=self.group)
                self._ws.free()
            half = -(-max(half_bytes, 1 << 20) // (1 << 20)) * (1 << 20)
            self._ws = _Symm(self, 2 * half)
            self._ws_half = half
            dist.barrier(group=self.group)

    def _fused(self, opc: int, inp: torch.Tensor, out: torch.Tensor, cfg: CodecConfig):
        n = self.size
        count = K.chunk_count(opc, inp.numel(), n)
        sb, region_b, total = K.workspace_bytes(opc, cfg, count, inp.dtype, n)
        self._ensure(total)
        self.epoch += 1
        parity = self.epoch & 1
        a = _lib.CollArgs()
        a.op, a.nRanks, a.rankBase, a.dtype, a.count = opc, n, self.rank, DTYPE_CODE[inp.dtype], count
        a.sliceTiles = K.pick_slice_tiles(count, n)
        a.epoch = self.epoch & 0x7FFFFFFF
        a.timeoutNs = int(self.policy.timeout_ms * 1e6)
        a.codec = cfg.to_c(inp.dtype)
        a.slotBytes, a.regionBOffset = sb, region_b
        a.inp[self.rank], a.out[self.rank] = inp.data_ptr(), out.data_ptr()
        for p in range(n):
            a.ws[p] = self._ws.ptrs[p] + parity * self._ws_half
            a.flags[p] = self._sig.ptrs[p]
            a.status[p] = self._sig.ptrs[p] + self._flag_bytes
        rc = _lib.lib().cocclkFusedCollective(a, 1, self.policy.max_ctas, _lib.cur_stream())
        _lib.check(rc, "cocclkFusedCollective")
        self.stats["compressed_calls"] += 1
        self.stats["compressed_raw_bytes"] += inp.numel() * inp.element_size()

    def status(self) -> int:
        """Error word written by bounded waits (0 = ok). Synchronises the device."""
        if self._sig is None:
            return 0
        torch.cuda.synchronize()
        w = (C.c_uint * 1)()
        cudart_memcpy = _lib.declare("cocclHostRead32", C.c_int, [C.c_void_p, C.POINTER(C.c_uint)])
        _lib.check(cudart_memcpy(self._sig.ptrs[self.rank] + self._flag_bytes, w), "cocclHostRead32")
        return int(w[0])

    def _route(self, role: str, op: str, inp: torch.Tensor, total_bytes: int, divisible: bool = True):
        if self.size == 1 or not self.cuda or not inp.is_cuda:
            return None
        cfg = self.policy.codec_for(role, op) or self.policy.codec_for("default", op) if self.policy.enabled else None
        if cfg is None or inp.dtype not in DTYPE_CODE or not divisible:
            return None
        if total_bytes <= self.policy.threshold_bytes:
            return None
        if not (inp.is_contiguous() and inp.data_ptr() % 4 == 0):
            return None
        return cfg

    def _native(self, nbytes):
        self.stats["native_calls"] += 1
        self.stats["native_bytes"] += nbytes

    # ------------------------------------------------------------------ collectives
    def reduce_scatter(self, inp: torch.Tensor, out: torch.Tensor, role: str = "default"):
        """out = sum over ranks of inp[rank chunk]; inp has size*out.numel() elements."""
        if self.size == 1:
            out.copy_(inp.reshape(out.shape))
            return out
        nbytes = inp.numel() * inp.element_size()
        cfg = self._route(role, "reduce_scatter", inp, nbytes)
        if cfg is not None:
            self._fused(K.OP_RS, inp, out, cfg)
        else:
            self._native(nbytes)
            dist.reduce_scatter_tensor(out, inp, group=self.group)
        return out

    def all_gather(self, inp: torch.Tensor, out: torch.Tensor, role: str = "default"):
        if self.size == 1:
            out.copy_(inp.reshape(out.shape))
            return out
        nbytes = out.numel() * out.element_size()
        cfg = self._route(role, "all_gather", inp, nbytes)
        if cfg is not None:
            self._fused(K.OP_AG, inp, out, cfg)
        else:
            self._native(nbytes)
            dist.all_gather_into_tensor(out, inp, group=self.group)
        return out

    def all_reduce(self, x: torch.Tensor, role: str = "default"):
        if self.size == 1:
            return x
        nbytes = x.numel() * x.element_size()
        cfg = self._route(role, "all_reduce", x, nbytes, divisible=(x.numel() % self.size == 0))
        if cfg is not None:
            op = K.OP_AR1 if nbytes <= self.policy.all_reduce_oneshot_max_bytes else K.OP_AR2
            self._fused(op, x, x, cfg)
        else:
            self._native(nbytes)
            dist.all_reduce(x, group=self.group)
        return x

    def all_to_all(self, inp: torch.Tensor, out: torch.Tensor, role: str = "default"):
        if self.size == 1:
            out.copy_(inp)
            return out
        nbytes = inp.numel() * inp.element_size()
        cfg = self._route(role, "all_to_all", inp, nbytes, divisible=(inp.numel() % self.size == 0))
        if cfg is not None:
            self._fused(K.OP_A2A, inp, out, cfg)
        else:
            self._native(nbytes)
            dist.all_to_all_single(out, inp, group=self.group)
        return out

    def all_reduce_small(self, t: torch.Tensor, op=dist.ReduceOp.SUM):
        if self.size > 1:
            dist.all_reduce(t, op=op, group=self.group)
        return t

    def barrier(self):
        if self.size > 1:
            dist.barrier(group=self.group)

    def global_rank(self, group_rank: int) -> int:
        return dist.get_global_rank(self.group, group_rank) if self.group is not None else group_rank

    def close(self):
        if self._ws is not None or self._sig is not None:
            torch.cuda.synchronize()
            if self.size > 1:
                dist.barrier(group=self.group)
        for s in (self._ws, self._sig):
            if s is not None:
                s.free()
        self._ws = self._sig = None
