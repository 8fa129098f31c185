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
from ..utils.trace import nvtx_range

K_NAMES = {0: "reduce_scatter", 1: "all_gather", 2: "all_to_all", 3: "all_reduce_oneshot", 4: "all_reduce_twoshot",
           5: "all_gather_delta"}


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
    dp_param_delta: bool = False    # ZeRO-1 parameter all-gather as 8-bit deltas (subAdd); exact first round
    nvls_all_reduce: bool = False   # uncompressed all-reduce below the threshold through multimem instead of NCCL
    timeout_ms: float = 20000.0
    max_ctas: int = 0

    def codec_for(self, role: str, op: str) -> CodecConfig | None:
        if not self.enabled:
            return None
        return self.codecs.get((role, op), None)


NATIVE = Policy(enabled=False)


class PeerLost(RuntimeError):
    """A bounded wait inside a fused kernel ran out: a peer did not deliver. `where` decodes the status word."""

    def __init__(self, family: str, word: int, err: int = 0):
        self.family, self.word, self.err = family, word, err
        self.where = {"phase": (word >> 23) & 0xFF, "peer": (word >> 15) & 0xFF, "slice": word & 0x7FFF}
        super().__init__(f"{family}: a wait on a peer gave up (status 0x{word:08x} = {self.where}, pipeline error 0x{err:08x}); "
                         "the outputs of that call are not valid")


class SymmUnavailable(RuntimeError):
    """Peer-mapped memory could not be set up on at least one rank of the group (agreed by all ranks)."""


class _Symm:
    """A symmetric buffer: local allocation + mapped peers.

    Opening and replacing one is collective and follows the protocol of csrc/runtime/symm_workspace.h: a rank
    frees its allocation only after every peer has unmapped it, and a failure on one rank makes every rank raise
    SymmUnavailable, so that all of them leave the fused path at the same call."""

    def __init__(self, comm: "Communicator", nbytes: int, replaces: "_Symm | None" = None):
        lib = _lib.lib()
        self._alloc = _lib.declare("cocclSymmAlloc", C.c_int, [C.c_size_t, C.POINTER(C.c_void_p)])
        self._export = _lib.declare("cocclSymmExport", C.c_int, [C.c_void_p, C.c_void_p])
        self._import = _lib.declare("cocclSymmImport", C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.POINTER(C.c_void_p)])
        self._local = _lib.declare("cocclSymmLocalPtr", C.c_void_p, [C.c_void_p])
        self._close = _lib.declare("cocclSymmCloseImports", C.c_int, [C.c_void_p])
        self._free = _lib.declare("cocclSymmFree", C.c_int, [C.c_void_p])
        self.handle, self.nbytes, self.ptrs = None, nbytes, []
        if replaces is not None:
            # nobody's kernels use the old mapping any more, then nobody maps it, then it is freed
            torch.cuda.synchronize()
            dist.barrier(group=comm.group)
            replaces.close_imports()
            dist.barrier(group=comm.group)
            replaces.free()
        h = C.c_void_p()
        buf = C.create_string_buffer(64)
        ok = self._alloc(nbytes, C.byref(h)) == 0 and self._export(h, buf) == 0
        self.handle = h if h.value else None
        offers = [None] * comm.size
        dist.all_gather_object(offers, (ok, bytes(buf.raw)), group=comm.group)
        ok = all(o[0] for o in offers)
        if ok:
            for p in range(comm.size):
                if p == comm.rank:
                    self.ptrs.append(self._local(h))
                    continue
                m = C.c_void_p()
                hb = C.create_string_buffer(offers[p][1], 64)
                if self._import(h, p, hb, C.byref(m)) != 0:
                    ok = False
                    break
                self.ptrs.append(m.value)
        outcome = [None] * comm.size
        dist.all_gather_object(outcome, ok, group=comm.group)
        if not all(outcome):
            self.close_imports()
            dist.barrier(group=comm.group)
            self.free()
            raise SymmUnavailable(f"peer memory of group '{comm.name}' could not be mapped on ranks "
                                  f"{[i for i, o in enumerate(outcome) if not o]}")

    def close_imports(self):
        if self.handle is not None:
            self._close(self.handle)

    def free(self):
        if self.handle is not None:
            self._free(self.handle)
            self.handle = None


class _Arena:
    """Parity-double-buffered symmetric workspace + flag/status block + epoch counter of one kernel family."""

    def __init__(self, comm: "Communicator", name: str = "moe"):
        self.comm, self.name = comm, name
        self.flag_bytes = _lib.lib().cocclkFlagBytes()
        self.sig = _Symm(comm, self.flag_bytes + 256)
        self.ws: _Symm | None = None
        self.half = 0
        self.epoch = 0

    def ensure(self, half_bytes: int):
        if self.ws is None or self.half < half_bytes:
            half = -(-max(half_bytes, 1 << 20) // (1 << 20)) * (1 << 20)
            old, self.ws, self.half = self.ws, None, 0
            self.ws = _Symm(self.comm, 2 * half, replaces=old)
            self.half = half

    def next(self):
        """(epoch, [workspace half of every rank], [flags], [status])"""
        self.epoch += 1
        off = (self.epoch & 1) * self.half
        n = self.comm.size
        return (self.epoch & 0xFFFFFFFF, [self.ws.ptrs[p] + off for p in range(n)], list(self.sig.ptrs),
                [self.sig.ptrs[p] + self.flag_bytes for p in range(n)])

    def status_ptr(self) -> int:
        return self.sig.ptrs[self.comm.rank] + self.flag_bytes

    def status(self) -> int:
        torch.cuda.synchronize()
        w = (C.c_uint * 1)()
        rd = _lib.declare("cocclHostRead32", C.c_int, [C.c_void_p, C.POINTER(C.c_uint)])
        _lib.check(rd(self.status_ptr(), w), "cocclHostRead32")
        return int(w[0])

    def close_imports(self):
        for s in (self.ws, self.sig):
            if s is not None:
                s.close_imports()

    def free(self):
        for s in (self.ws, self.sig):
            if s is not None:
                s.free()
        self.ws = self.sig = None


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
        self._tp_ws: _Symm | None = None
        self._tp_sig: _Symm | None = None
        self._tp_half = 0
        self._tp_epoch = 0
        self._moe: _Arena | None = None
        self._nvls: dict | None = None
        self._trace: torch.Tensor | None = None
        self._health: dict | None = None
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
            half = -(-max(half_bytes, 1 << 20) // (1 << 20)) * (1 << 20)
            old, self._ws, self._ws_half = self._ws, None, 0
            self._ws = _Symm(self, 2 * half, replaces=old)
            self._ws_half = half

    def _leave_fused_path(self, why: Exception) -> None:
        import warnings
        warnings.warn(f"coccl_b200: group '{self.name}' falls back to native collectives on every rank: {why}")
        self.policy = NATIVE

    def _fused(self, opc: int, inp: torch.Tensor, out: torch.Tensor, cfg: CodecConfig) -> bool:
        """Launch the fused kernel; False (nothing launched, on any rank) when peer memory cannot be mapped."""
        n = self.size
        count = K.chunk_count(opc, inp.numel(), n)
        sb, region_b, total = K.workspace_bytes(opc, cfg, count, inp.dtype, n)
        try:
            self._ensure(total)
        except SymmUnavailable as e:
            self._leave_fused_path(e)
            return False
        self.epoch += 1
        parity = self.epoch & 1
        a = _lib.CollArgs()
        a.op, a.nRanks, a.rankBase, a.dtype, a.count = opc, n, self.rank, DTYPE_CODE[inp.dtype], count
        a.sliceTiles = K.pick_slice_tiles(count, n)
        a.epoch = self.epoch & 0xFFFFFFFF
        a.timeoutNs = int(self.policy.timeout_ms * 1e6)
        a.codec = cfg.to_c(inp.dtype)
        a.slotBytes, a.regionBOffset = sb, region_b
        a.inp[self.rank], a.out[self.rank] = inp.data_ptr(), out.data_ptr()
        for p in range(n):
            a.ws[p] = self._ws.ptrs[p] + parity * self._ws_half
            a.flags[p] = self._sig.ptrs[p]
            a.status[p] = self._sig.ptrs[p] + self._flag_bytes
        if self._trace is not None:
            self._trace.zero_()
            a.trace[self.rank] = self._trace.data_ptr()
        with nvtx_range(f"coccl.fused.{K_NAMES.get(opc, opc)}.{cfg.kind}"):
            rc = _lib.lib().cocclkFusedCollective(a, 1, self.policy.max_ctas, _lib.cur_stream())
        _lib.check(rc, "cocclkFusedCollective")
        self.stats["compressed_calls"] += 1
        self.stats["compressed_raw_bytes"] += inp.numel() * inp.element_size()
        return True

    def enable_trace(self, on: bool = True) -> None:
        """Record per-CTA phase timestamps of every following fused collective (see utils.trace)."""
        from ..utils.trace import TRACE_MAX_CTAS
        self._trace = torch.zeros(TRACE_MAX_CTAS, 4, dtype=torch.int64, device=self.device) if on else None

    def phase_times(self) -> dict:
        """Phase durations (us) of the last fused collective on this rank; synchronises the device."""
        from ..utils.trace import summarise
        if self._trace is None:
            return {}
        torch.cuda.synchronize()
        return summarise(self._trace)

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
        if cfg is None or not self._fused(K.OP_RS, inp, out, cfg):
            self._native(nbytes)
            with nvtx_range("coccl.native.reduce_scatter"):
                dist.reduce_scatter_tensor(out, inp, group=self.group)
        return out

    def all_gather(self, inp: torch.Tensor, out: torch.Tensor, role: str = "default"):
        if self.size == 1:
            out.copy_(inp.reshape(out.shape))
            return out
        nbytes = out.numel() * out.element_size()
        cfg = self._route(role, "all_gather", inp, nbytes)
        if cfg is None or not self._fused(K.OP_AG, inp, out, cfg):
            self._native(nbytes)
            with nvtx_range("coccl.native.all_gather"):
                dist.all_gather_into_tensor(out, inp, group=self.group)
        return out

    # ------------------------------------------------------------------ NVSwitch (multimem) all-reduce
    def _ensure_nvls(self, nbytes: int) -> bool:
        """Symmetric buffer bound to a multicast object (torch symmetric memory does the allocation and the
        binding; the reduction kernel is csrc/kernels/nvls_kernels.cu). False when the fabric has no multicast."""
        if self._nvls is not None and self._nvls["bytes"] >= nbytes:
            return self._nvls["mc"] != 0
        if self._nvls is not None and self._nvls["mc"] == 0:
            return False
        import torch.distributed._symmetric_memory as symm_mem
        size = max(nbytes, 64 << 20)
        try:
            t = symm_mem.empty(size, dtype=torch.uint8, device=self.device)
            h = symm_mem.rendezvous(t, (self.group or dist.group.WORLD).group_name)
            mc = int(h.multicast_ptr or 0)
        except Exception:  # noqa: BLE001 - no symmetric memory support in this build / on this fabric
            t, h, mc = None, None, 0
        ok = torch.tensor([1 if mc else 0], device=self.device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
        if int(ok.item()) == 0:
            mc = 0
        flags = self._nvls["flags"] if self._nvls is not None else _Symm(self, _lib.lib().cocclkNvlsFlagBytes() + 256)
        epoch = self._nvls["epoch"] if self._nvls is not None else 0
        self._nvls = {"t": t, "h": h, "mc": mc, "bytes": size, "flags": flags, "epoch": epoch}
        return mc != 0

    def all_reduce_nvls(self, x: torch.Tensor) -> bool:
        """In-place sum over ranks through the switch. Returns False (x untouched) when multicast is unavailable or
        the size does not split into 16-byte vectors per rank."""
        nbytes = x.numel() * x.element_size()
        if x.dtype not in DTYPE_CODE or nbytes % (16 * self.size) != 0 or not x.is_contiguous():
            return False
        if not self._ensure_nvls(nbytes):
            return False
        st = self._nvls
        buf = st["t"][:nbytes].view(x.dtype)
        buf.copy_(x.view(-1))
        st["epoch"] += 1
        fl = (C.c_void_p * self.size)(*[st["flags"].ptrs[p] for p in range(self.size)])
        status = st["flags"].ptrs[self.rank] + _lib.lib().cocclkNvlsFlagBytes()
        with nvtx_range("coccl.nvls.all_reduce"):
            rc = _lib.lib().cocclkNvlsAllReduce(st["mc"], x.numel(), DTYPE_CODE[x.dtype], self.size, self.rank, fl, status,
                                                st["epoch"] & 0xFFFFFFFF, int(self.policy.timeout_ms * 1e6),
                                                self.policy.max_ctas, _lib.cur_stream())
        _lib.check(rc, "cocclkNvlsAllReduce")
        x.view(-1).copy_(buf)
        self.stats["nvls_calls"] = self.stats.get("nvls_calls", 0) + 1
        return True

    def all_reduce(self, x: torch.Tensor, role: str = "default"):
        if self.size == 1:
            return x
        nbytes = x.numel() * x.element_size()
        cfg = self._route(role, "all_reduce", x, nbytes, divisible=(x.numel() % self.size == 0))
        if cfg is None and self.policy.nvls_all_reduce and self.cuda and x.is_cuda and self.all_reduce_nvls(x):
            return x
        op = K.OP_AR1 if nbytes <= self.policy.all_reduce_oneshot_max_bytes else K.OP_AR2
        if cfg is None or not self._fused(op, x, x, cfg):
            self._native(nbytes)
            with nvtx_range("coccl.native.all_reduce"):
                dist.all_reduce(x, group=self.group)
        return x

    def all_to_all(self, inp: torch.Tensor, out: torch.Tensor, role: str = "default"):
        if self.size == 1:
            out.copy_(inp)
            return out
        nbytes = inp.numel() * inp.element_size()
        cfg = self._route(role, "all_to_all", inp, nbytes, divisible=(inp.numel() % self.size == 0))
        if cfg is None or not self._fused(K.OP_A2A, inp, out, cfg):
            self._native(nbytes)
            with nvtx_range("coccl.native.all_to_all"):
                dist.all_to_all_single(out, inp, group=self.group)
        return out

    # ------------------------------------------------------------------ tensor-parallel fusions
    def _ensure_tp(self, half_bytes: int):
        if self._tp_sig is None:
            self._tp_flag_bytes = _lib.lib().cocclkFlagBytes()
            self._tp_sig = _Symm(self, self._tp_flag_bytes + 256)
            self._tp_err = torch.zeros(1, dtype=torch.int32, device=self.device)
        if self._tp_ws is None or self._tp_half < half_bytes:
            half = -(-max(half_bytes, 1 << 20) // (1 << 20)) * (1 << 20)
            old, self._tp_ws, self._tp_half = self._tp_ws, None, 0
            self._tp_ws = _Symm(self, 2 * half, replaces=old)
            self._tp_half = half

    def _tp_args(self, M: int, N: int, K: int):
        self._tp_epoch += 1
        parity = self._tp_epoch & 1
        a = _lib.TpArgs()
        a.nRanks, a.rankBase, a.M, a.N, a.K = self.size, self.rank, M, N, K
        a.epoch = self._tp_epoch & 0xFFFFFFFF
        a.timeoutNs = int(self.policy.timeout_ms * 1e6)
        for p in range(self.size):
            a.ws[p] = self._tp_ws.ptrs[p] + parity * self._tp_half
            a.flags[p] = self._tp_sig.ptrs[p]
            a.status[p] = self._tp_sig.ptrs[p] + self._tp_flag_bytes
        a.err[self.rank] = self._tp_err.data_ptr()
        return a

    def ag_gemm(self, x_local: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, gelu: bool = False,
                out: torch.Tensor | None = None, *, b_mn: bool = False, save_preact: bool = False,
                gathered: torch.Tensor | None = None):
        """concat_over_ranks(x_local) @ w.T (+ bias, GELU) in ONE kernel: the shards travel over peer memory
        while the tensor cores already work on the local shard. x_local [m, K] bf16; w [N, K], or [K, N] with
        b_mn=True (then the product is gather(x) @ w). save_preact: also return the pre-activation (GELU only).
        gathered: optional [M, K] tensor that receives the gathered input (for a later weight gradient)."""
        from ..ops import tp_fused as T
        m, K = x_local.shape
        N = w.shape[1] if b_mn else w.shape[0]
        M = m * self.size
        assert x_local.is_contiguous() and w.is_contiguous() and x_local.dtype == torch.bfloat16
        if out is None:
            out = torch.empty(M, N, dtype=torch.bfloat16, device=x_local.device)
        self._ensure_tp(T.ag_ws_bytes(M, K))
        a = self._tp_args(M, N, K)
        a.epi = T.EPI_NONE if bias is None else (T.EPI_BIAS_GELU if gelu else T.EPI_BIAS)
        a.bMN = int(b_mn)
        a.a[self.rank], a.b[self.rank], a.c[self.rank] = x_local.data_ptr(), w.data_ptr(), out.data_ptr()
        a.bias[self.rank] = bias.data_ptr() if bias is not None else None
        z = None
        if save_preact and gelu and bias is not None:
            z = torch.empty_like(out)
            a.z[self.rank] = z.data_ptr()
        if gathered is not None:
            assert gathered.is_contiguous() and gathered.shape == (M, K) and gathered.dtype == torch.bfloat16
            a.gathered[self.rank] = gathered.data_ptr()   # the CTA-pair kernel copies the operand out itself
        with nvtx_range("coccl.fused.ag_gemm"):
            _lib.check(_lib.lib().cocclkAgGemm(a, 1, self.policy.max_ctas, _lib.cur_stream()), "cocclkAgGemm")
        self.stats["compressed_calls"] += 1
        if gathered is not None and _lib.lib().cocclkTpLastVariant() != 2:
            # the peers' shards are in this call's half of the workspace, the own shard never left x_local
            cp = _lib.declare("cocclDeviceCopy", C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p])
            row = K * 2
            ws, r, st = a.ws[self.rank], self.rank, _lib.cur_stream()
            if r > 0:
                _lib.check(cp(gathered.data_ptr(), ws, r * m * row, st), "cocclDeviceCopy")
            if r + 1 < self.size:
                off = (r + 1) * m * row
                _lib.check(cp(gathered.data_ptr() + off, ws + off, (self.size - r - 1) * m * row, st), "cocclDeviceCopy")
            gathered[r * m:(r + 1) * m].copy_(x_local)
        return (out, z) if save_preact else out

    def gemm_rs(self, a_mat: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None, *, b_mn: bool = False,
                bias: torch.Tensor | None = None) -> torch.Tensor:
        """reduce_scatter over ranks of (a_mat @ w.T) along the rows, in ONE kernel: the partial products leave
        the GEMM epilogue as block-scaled FP8 straight into the destination ranks' memory. a_mat [M, K]; w [N, K],
        or [K, N] with b_mn=True (then the product is a_mat @ w). bias [N] bf16 is added once to the reduced rows."""
        from ..ops import tp_fused as T
        M, K = a_mat.shape
        N = w.shape[1] if b_mn else w.shape[0]
        assert a_mat.is_contiguous() and w.is_contiguous() and a_mat.dtype == torch.bfloat16
        if out is None:
            out = torch.empty(M // self.size, N, dtype=torch.bfloat16, device=a_mat.device)
        self._ensure_tp(T.rs_ws_bytes(M, N, self.size))
        a = self._tp_args(M, N, K)
        a.epi = T.EPI_NONE
        a.bMN = int(b_mn)
        a.a[self.rank], a.b[self.rank], a.c[self.rank] = a_mat.data_ptr(), w.data_ptr(), out.data_ptr()
        if bias is not None:
            assert bias.dtype == torch.bfloat16 and bias.is_contiguous() and bias.numel() == N
            a.bias[self.rank] = bias.data_ptr()
        with nvtx_range("coccl.fused.gemm_rs"):
            _lib.check(_lib.lib().cocclkGemmRs(a, 1, self.policy.max_ctas, _lib.cur_stream()), "cocclkGemmRs")
        if bias is not None and _lib.lib().cocclkTpLastVariant() != 2:
            out += bias   # the single-CTA kernel's reducer has no bias operand
        self.stats["compressed_calls"] += 1
        self.stats["compressed_raw_bytes"] += M * N * 2
        return out

    def tp_fusable(self, rows_total: int, n_out_rs: int | None = None, width: int | None = None) -> bool:
        """Whether the one-kernel TP fusions serve a problem with `rows_total` gathered rows (and, for gemm_rs,
        `n_out_rs` output columns). The fusions quantise the reduce-scattered partial sums to block-scaled FP8, so
        they apply only where the policy asks for exactly that: an MX-FP8 codec on ('tp', 'reduce_scatter'), a
        codec on ('tp', 'all_gather'), and a message above the threshold (`width` = columns of the gathered
        operand; the router's `bytes <= threshold` rule, coccl_runtime.cc:214). Otherwise the caller takes the
        unfused path, whose collectives are routed one by one."""
        if not (self.cuda and self.policy.enabled and 1 < self.size <= _lib.MAX_RANKS):
            return False
        rs = self.policy.codec_for("tp", "reduce_scatter")
        ag = self.policy.codec_for("tp", "all_gather")
        if rs is None or ag is None or rs.kind != "mxfp8":
            return False
        cols = max(width or 0, n_out_rs or 0)
        if cols and rows_total * cols * 2 <= self.policy.threshold_bytes:
            return False
        if rows_total % (self.size * 128) != 0:
            return False
        if n_out_rs is not None and n_out_rs % 256 != 0:
            return False
        if self._tp_sig is None:
            try:
                self._ensure_tp(1 << 20)   # collective: every rank of the group asks this at the same call
            except SymmUnavailable as e:
                self._leave_fused_path(e)
                return False
        return True

    def tp_status(self) -> tuple[int, int]:
        """(status word, pipeline error word) of the tensor-parallel fusions; synchronises the device."""
        if self._tp_sig is None:
            return 0, 0
        torch.cuda.synchronize()
        w = (C.c_uint * 1)()
        rd = _lib.declare("cocclHostRead32", C.c_int, [C.c_void_p, C.POINTER(C.c_uint)])
        _lib.check(rd(self._tp_sig.ptrs[self.rank] + self._tp_flag_bytes, w), "cocclHostRead32")
        return int(w[0]), int(self._tp_err.item())

    # ------------------------------------------------------------------ expert parallelism
    def _moe_args(self, tokens, hidden, topk, n_experts, capacity):
        from ..ops import moe as M
        if self._moe is None:
            self._moe = _Arena(self)
        self._moe.ensure(M.ws_bytes(self.size, capacity, hidden, n_experts // self.size))
        epoch, ws, flags, status = self._moe.next()
        a = _lib.MoeArgs()
        a.nRanks, a.rankBase, a.tokens, a.hidden, a.topk = self.size, self.rank, tokens, hidden, topk
        a.experts, a.capacity, a.epoch, a.timeoutNs = n_experts, capacity, epoch, int(self.policy.timeout_ms * 1e6)
        for p in range(self.size):
            a.ws[p], a.flags[p], a.status[p] = ws[p], flags[p], status[p]
        return a

    def moe_dispatch(self, x: torch.Tensor, expert_ids: torch.Tensor, n_experts: int, capacity: int | None = None,
                     row_scale: torch.Tensor | None = None, layout=None):
        """Send every token to the ranks of its top-k experts as block-scaled FP8 (one kernel: gather, quantise,
        peer stores, dequantise on arrival). Returns (rows [R, hidden] bf16 grouped by local expert, handle);
        handle.recv_offsets[e] .. [e+1] are the rows of local expert e."""
        from ..ops import moe as M
        tokens, hidden = x.shape
        topk = expert_ids.shape[1]
        capacity = capacity or tokens * topk
        le = n_experts // self.size
        pos, counts = layout if layout is not None else M.route_layout(expert_ids, n_experts, self.size)
        recv = torch.empty(self.size * capacity, hidden, dtype=torch.bfloat16, device=x.device)
        roff = torch.zeros(le + 1, dtype=torch.int32, device=x.device)
        rcnt = torch.zeros(self.size, le, dtype=torch.int32, device=x.device)
        a = self._moe_args(tokens, hidden, topk, n_experts, capacity)
        r = self.rank
        a.x[r], a.expertIds[r], a.pos[r], a.sendCounts[r] = x.data_ptr(), expert_ids.data_ptr(), pos.data_ptr(), counts.data_ptr()
        a.recv[r], a.recvOffsets[r], a.recvCounts[r] = recv.data_ptr(), roff.data_ptr(), rcnt.data_ptr()
        if row_scale is not None:
            assert row_scale.dtype == torch.float32 and row_scale.is_contiguous() and row_scale.shape == expert_ids.shape
            a.rowScale[r] = row_scale.data_ptr()
        _lib.check(_lib.lib().cocclkMoeDispatch(a, 1, self.policy.max_ctas, _lib.cur_stream()), "cocclkMoeDispatch")
        self.stats["compressed_calls"] += 1
        self.stats["compressed_raw_bytes"] += tokens * topk * hidden * 2
        h = M.Handle(expert_ids, pos, rcnt, roff, capacity, n_experts)
        h.keep = (counts, x, row_scale)
        h.counts = counts
        return recv, h

    def moe_combine(self, y: torch.Tensor, gates: torch.Tensor, handle, dot_with: torch.Tensor | None = None):
        """Return the expert outputs (same row layout as moe_dispatch's result) to the token owners as bf16 and
        form out[t] = sum_j gates[t, j] * y_j in one kernel. With dot_with [tokens, hidden] the kernel also returns
        dots[t, j] = <y_j, dot_with[t]> (the gate gradients when dot_with is the output gradient)."""
        tokens, topk = gates.shape
        hidden = y.shape[1]
        out = torch.empty(tokens, hidden, dtype=torch.bfloat16, device=y.device)
        a = self._moe_args(tokens, hidden, topk, handle.n_experts, handle.capacity)
        r = self.rank
        a.expertIds[r], a.pos[r], a.gates[r] = handle.expert_ids.data_ptr(), handle.pos.data_ptr(), gates.data_ptr()
        a.recvCounts[r], a.y[r], a.out[r] = handle.recv_counts.data_ptr(), y.data_ptr(), out.data_ptr()
        dots = None
        if dot_with is not None:
            assert dot_with.dtype == torch.bfloat16 and dot_with.is_contiguous() and dot_with.shape == (tokens, hidden)
            dots = torch.empty(tokens, topk, dtype=torch.float32, device=y.device)
            a.dotWith[r], a.dotOut[r] = dot_with.data_ptr(), dots.data_ptr()
        _lib.check(_lib.lib().cocclkMoeCombine(a, 1, self.policy.max_ctas, _lib.cur_stream()), "cocclkMoeCombine")
        return out if dot_with is None else (out, dots)

    def moe_status(self) -> int:
        return 0 if self._moe is None else self._moe.status()

    def all_gather_delta(self, inp: torch.Tensor, out: torch.Tensor, cfg: CodecConfig | None = None, state=None):
        """All-gather that sends the CHANGE of `inp` since the previous call (parameters after an optimizer step move
        little, so 8 bits of a small delta carry far more precision than 8 bits of the value). `out` itself is the
        codec state: every rank adds the same decoded deltas to it. The caller owns the state handle: pass None
        for the first call (an exact native all-gather that seeds `out`, as the reference's subAdd codec does with
        its raw first round, sdp4bit_quan.cu:286-353) and afterwards the handle that the previous call returned.
        Between calls `out` must not be written by anyone else (load a checkpoint into it -> pass None again);
        the handle also pins `out`'s storage, so a recycled address cannot be mistaken for seeded state.
        Returns the handle (None when the delta path is not usable and the call ran exact)."""
        if self.size == 1:
            out.copy_(inp.reshape(out.shape))
            return None
        cfg = cfg or CodecConfig("sdp4bit", 8, 2048, False, False)
        usable = self.cuda and inp.is_cuda and inp.dtype in DTYPE_CODE and inp.is_contiguous() and out.is_contiguous()
        seeded = (state is not None and state.get("out") is out and state.get("numel") == out.numel()
                  and state.get("version") == out._version)
        if not usable or not seeded or not self._fused(K.OP_AGD, inp, out, cfg):
            self._native(out.numel() * out.element_size())
            dist.all_gather_into_tensor(out, inp, group=self.group)
        if not usable or not self.policy.enabled:
            return None
        # the kernel and the native call write `out` behind autograd's back; record the version counter after
        # our own write so that a later in-place write by anyone else is noticed
        return {"out": out, "numel": out.numel(), "version": out._version}

    def all_reduce_small(self, t: torch.Tensor, op=dist.ReduceOp.SUM):
        if self.size > 1:
            dist.all_reduce(t, op=op, group=self.group)
        return t

    def barrier(self):
        if self.size > 1:
            dist.barrier(group=self.group)

    def global_rank(self, group_rank: int) -> int:
        return dist.get_global_rank(self.group, group_rank) if self.group is not None else group_rank

    # ------------------------------------------------------------------ health
    def post_status_read(self) -> None:
        """Queue a copy of every status / error word of this communicator's fused kernels into pinned host memory
        behind the work already on the current stream. Costs a few 4-byte copies and one event, no synchronisation;
        `poll_status` looks at the result later (the trainer does both once per step)."""
        if not self.cuda:
            return
        words = []  # (family, device address)
        if self._sig is not None:
            words.append(("collective", self._sig.ptrs[self.rank] + self._flag_bytes))
        if self._tp_sig is not None:
            words.append(("tensor-parallel fusion", self._tp_sig.ptrs[self.rank] + self._tp_flag_bytes))
            words.append(("tensor-parallel pipeline", self._tp_err.data_ptr()))
        if self._moe is not None:
            words.append(("expert all-to-all", self._moe.status_ptr()))
        if self._nvls is not None and self._nvls.get("flags") is not None:
            words.append(("multimem all-reduce", self._nvls["flags"].ptrs[self.rank] + _lib.lib().cocclkNvlsFlagBytes()))
        if not words:
            return
        if self._health is None:
            self._health = {"host": torch.zeros(16, dtype=torch.int32).pin_memory(), "event": torch.cuda.Event(),
                            "families": [], "pending": False}
        rd = _lib.declare("cocclAsyncRead32", C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p])
        h = self._health
        for i, (_, addr) in enumerate(words):
            _lib.check(rd(h["host"].data_ptr() + 4 * i, addr, 1, _lib.cur_stream()), "cocclAsyncRead32")
        h["families"] = [f for f, _ in words]
        h["event"].record()
        h["pending"] = True

    def poll_status(self, wait: bool = False) -> None:
        """Raise PeerLost if the words copied by the last `post_status_read` show that a wait gave up. Without
        `wait` a copy that has not finished yet is simply looked at on the next call."""
        h = self._health
        if h is None or not h["pending"]:
            return
        if wait:
            h["event"].synchronize()
        elif not h["event"].query():
            return
        h["pending"] = False
        vals = [int(v) & 0xFFFFFFFF for v in h["host"][:len(h["families"])].tolist()]
        for fam, v in zip(h["families"], vals):
            if v != 0:
                if fam == "tensor-parallel pipeline":
                    raise PeerLost(fam, 0, v)
                raise PeerLost(fam, v)

    def close(self):
        arenas = [self._ws, self._sig, self._tp_ws, self._tp_sig, self._moe, self._nvls["flags"] if self._nvls else None]
        if any(x is not None for x in arenas):
            torch.cuda.synchronize()
            if self.size > 1:
                dist.barrier(group=self.group)
            for x in arenas:
                if x is not None:
                    x.close_imports()
            if self.size > 1:
                dist.barrier(group=self.group)
        for x in arenas:
            if x is not None:
                x.free()
        self._ws = self._sig = self._tp_ws = self._tp_sig = self._moe = None
