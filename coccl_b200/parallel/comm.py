"""Communicator: one per process group; runs every collective either as a fused compressed kernel over peer-mapped
symmetric memory or on torch.distributed (NCCL on GPUs, gloo on CPU).

WHICH of the two is not decided here. Every call is described to a routing session of the native runtime
(csrc/api/router_api.cc), which runs the same code as the C API: the rule order of the reference router
(src/coccl-extend/core/runtime/coccl_runtime.cc:181-229: enabled, sum only, divisibility, role known in training
mode, a codec configured for the scope, `bytes <= threshold` stays native, algorithm selection), on the policy model
of its TOML files (COCCL_CONFIG_FILE schema: normal / training mode, per-operation default/intra/inter scopes,
thresholds, autotune section). This module turns the decision into a kernel launch, owns the symmetric memory, and
feeds the selector with measurements of the kernels that actually serve the calls.
"""
from __future__ import annotations

import ctypes as C
import hashlib
import os
import tempfile
from dataclasses import dataclass
from pathlib import Path

import torch
import torch.distributed as dist

from .. import _lib
from ..ops import collective as K
from ..ops.codec import DTYPE_CODE
from ..utils.trace import nvtx_range

K_NAMES = {0: "reduce_scatter", 1: "all_gather", 2: "all_to_all", 3: "all_reduce_oneshot", 4: "all_reduce_twoshot",
           5: "all_gather_delta"}
CONFIG_DIR = Path(__file__).resolve().parent.parent / "configs"
PLUGIN_DIR = Path(__file__).resolve().parent.parent / "lib" / "plugins"
NCCL_DTYPE = {torch.float32: 7, torch.float16: 6, torch.bfloat16: 9, torch.int8: 0, torch.int32: 2, torch.int64: 4}
ROLE = {"dp": 1, "tp": 2, "pp": 3}                       # communicator name -> COCCL_ROLE_*; anything else: normal
OP = {"all_gather": 0, "reduce_scatter": 1, "all_reduce": 2, "all_to_all": 3, "sendrecv": 4}   # COCCL_OP_*
ALGO_AR_ONESHOT, ALGO_AR_TWOSHOT = 3, 4


class Decision(C.Structure):
    """Mirror of cocclRouteDecision (csrc/include/coccl/router.h)."""
    _fields_ = [("compressed", C.c_int), ("algorithm", C.c_int), ("fusable", C.c_int), ("delta", C.c_int),
                ("native_variant", C.c_int), ("role", C.c_int), ("threshold_bytes", C.c_size_t), ("total_bytes", C.c_size_t),
                ("codec", _lib.Codec), ("compressor", C.c_char * 32)]


@dataclass
class Policy:
    """Where the routing rules come from: a policy file in the reference's TOML schema (or its text), read by the native
    router. `Policy()` is the shipped training policy (configs/training.toml: SDP4Bit on the data-parallel gradient
    reduce-scatter, 8-bit deltas on the parameter all-gather, block-scaled FP8 on tensor-parallel traffic, threshold
    8 MiB). The remaining fields are launch knobs of this layer, not routing rules."""
    enabled: bool = True
    config_file: str | None = None   # default: configs/training.toml
    toml: str | None = None          # inline policy text instead of a file
    timeout_ms: float = 20000.0      # bound of every device-side wait
    max_ctas: int = 0                # CTAs a fused kernel may occupy (0 = all it can keep resident)
    measure: bool = True             # time one-shot / two-shot (and multimem) at first use where [autotune] enabled = true
    nvls: bool = True                # the multimem all-reduce is a candidate for uncompressed calls below the threshold

    def text(self) -> str | None:
        if not self.enabled:
            return None
        if self.toml is not None:
            return self.toml
        return Path(self.config_file or CONFIG_DIR / "training.toml").read_text()

    def base_dir(self) -> Path:
        return Path(self.config_file).resolve().parent if (self.toml is None and self.config_file) else CONFIG_DIR

    @staticmethod
    def normal(compressor: str = "sdp4bit", options: dict | None = None, *, threshold_bytes: int = 8 << 20,
               autotune: bool = False, all_reduce_algorithm: str = "auto", per_op: dict | None = None, **kw) -> "Policy":
        """A normal-mode policy with one codec on every collective (per_op: {operation: (compressor, options)}
        overrides single operations). The text is what a user would put in COCCL_CONFIG_FILE."""
        if options is None:
            options = {"sdp4bit": {"groupCount": 128, "quantBits": 4, "quantType": "Symmetric", "hadamard": True,
                                   "rounding": "nearest"}}.get(compressor, {})
        per_op = dict(per_op or {})
        names = sorted({compressor} | {c for c, _ in per_op.values()})

        def val(v):
            return ("true" if v else "false") if isinstance(v, bool) else (f'"{v}"' if isinstance(v, str) else str(v))
        lines = ["[runtime]", 'mode = "normal"', f"compression_threshold_bytes = {threshold_bytes}", "",
                 "[compressor_plugins]", "compressors = [" + ", ".join(f'"{n}"' for n in names) + "]",
                 f'library_path = "{PLUGIN_DIR}"', "", "[autotune]", f"enabled = {val(autotune)}",
                 f'all_reduce_algorithm = "{all_reduce_algorithm}"', ""]
        for op in ("all_gather", "reduce_scatter", "all_reduce", "all_to_all", "sendrecv"):
            c, o = per_op.get(op, (compressor, options))
            lines += [f"[normal.{op}.default]", f'compressor = "{c}"']
            if o:
                lines += [f"[normal.{op}.default.config]"] + [f"{k} = {val(v)}" for k, v in o.items()]
            lines.append("")
        return Policy(toml="\n".join(lines), **kw)

    @staticmethod
    def training(*, threshold_bytes: int = 8 << 20, dp_delta: bool = True, autotune: bool = True, **kw) -> "Policy":
        """The shipped training policy with the threshold replaced (tests and small models use 0) and, with
        dp_delta=False, without the delta codec on the parameter all-gather (it then stays native)."""
        text = (CONFIG_DIR / "training.toml").read_text()
        text = text.replace("compression_threshold_bytes = 8388608", f"compression_threshold_bytes = {threshold_bytes}")
        text = text.replace('library_path = "../lib/plugins"', f'library_path = "{PLUGIN_DIR}"')
        if not autotune:
            text = text.replace("[autotune]\nenabled = true", "[autotune]\nenabled = false")
        if not dp_delta:
            a = text.index("[training.dp.all_gather.default]")
            b = text.index("[training.tp.all_gather.default]")
            text = text[:a] + text[b:]
        return Policy(toml=text, **kw)


NATIVE = Policy(enabled=False)


class Router:
    """One routing session of the native runtime per distinct policy text (process-wide cache)."""
    _cache: dict = {}

    def __init__(self, policy: Policy, devices_per_node: int):
        self._open = _lib.declare("cocclRouterOpen", C.c_int, [C.c_char_p, C.c_int, C.c_int, C.POINTER(C.c_void_p), C.c_char_p, C.c_size_t])
        self._decide = _lib.declare("cocclRouterDecide", C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_size_t, C.c_int, C.c_int,
                                                                   C.c_int, C.c_int, C.c_int, C.POINTER(Decision)])
        self._eff = _lib.declare("cocclRouterEffectiveConfig", C.c_char_p, [C.c_void_p])
        self._hash = _lib.declare("cocclRouterConfigHash", C.c_uint64, [C.c_void_p])
        self._training = _lib.declare("cocclRouterTrainingMode", C.c_int, [C.c_void_p])
        try:
            self._max_ctas = _lib.declare("cocclRouterFusedMaxCtas", C.c_int, [C.c_void_p])
        except AttributeError:   # a library built before the key existed
            self._max_ctas = None
        self._set = _lib.declare("cocclRouterSetMeasured", C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_double])
        self._set_native = _lib.declare("cocclRouterSetMeasuredNative", C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_double])
        self._stats = _lib.declare("cocclRouterStats", None, [C.c_void_p, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)])
        text = policy.text()
        path = None
        if text is not None:
            # the parser resolves library_path against the file's directory: keep inline text next to the shipped files' plugins
            tmp = Path(tempfile.gettempdir()) / f"coccl_policy_{os.getpid()}_{hashlib.sha1(text.encode()).hexdigest()[:12]}.toml"
            fixed = text.replace('library_path = "../lib/plugins"', f'library_path = "{PLUGIN_DIR}"')
            tmp.write_text(fixed)
            path = str(tmp).encode()
        h, err = C.c_void_p(), C.create_string_buffer(1024)
        rc = self._open(path, 1, max(1, devices_per_node), C.byref(h), err, 1024)
        if rc != 0:
            raise RuntimeError(f"policy rejected by the router: {err.value.decode() or rc}")
        self.handle = h
        self.measured: set = set()     # (kind, dtype, nranks) already timed
        self.tuning_log: list = []     # rows of what was timed and fed to the selector
        self.autotune = "autotune.enabled = true" in self.effective_config()

    @classmethod
    def of(cls, policy: Policy, devices_per_node: int) -> "Router | None":
        text = policy.text()
        if text is None:
            return None
        key = (text, devices_per_node)
        if key not in cls._cache:
            cls._cache[key] = Router(policy, devices_per_node)
        return cls._cache[key]

    def decide(self, role: int, op: str, dtype: torch.dtype, count: int, n_ranks: int, rank: int, explicit: int = -1) -> Decision:
        d = Decision()
        rc = self._decide(self.handle, role, OP[op], NCCL_DTYPE.get(dtype, 1), count, n_ranks, 1, rank, 0, explicit, C.byref(d))
        if rc != 0:
            raise RuntimeError(f"cocclRouterDecide failed with {rc}")
        return d

    def effective_config(self) -> str:
        return self._eff(self.handle).decode()

    def fused_max_ctas(self) -> int:
        """[runtime] fused_kernel_max_ctas of the policy file (0 = no limit)."""
        return int(self._max_ctas(self.handle)) if self._max_ctas is not None else 0

    def config_hash(self) -> str:
        return f"{int(self._hash(self.handle)):016x}"

    def training_mode(self) -> bool:
        return bool(self._training(self.handle))

    def set_measured(self, op: str, dtype, n_ranks: int, log2_bytes: int, algorithm: int, seconds: float):
        self._set(self.handle, OP[op], NCCL_DTYPE[dtype], n_ranks, log2_bytes, algorithm, seconds)

    def set_measured_native(self, dtype, n_ranks: int, log2_bytes: int, variant: int, seconds: float):
        self._set_native(self.handle, NCCL_DTYPE[dtype], n_ranks, log2_bytes, variant, seconds)

    def stats(self) -> dict:
        a, b, c = C.c_uint64(), C.c_uint64(), C.c_uint64()
        self._stats(self.handle, C.byref(a), C.byref(b), C.byref(c))
        return {"native": a.value, "compressed": b.value, "policy_lookups": c.value}


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

    def __init__(self, comm: "Communicator", nbytes: int, replaces: "_Symm | None" = None, backend: int | None = None):
        """backend: None = the process default (COCCL_SYMM_BACKEND), 0 = CUDA IPC, 1 = cuMem VMM for this region only."""
        lib = _lib.lib()
        self._alloc = _lib.declare("cocclSymmAlloc", C.c_int, [C.c_size_t, C.POINTER(C.c_void_p)])
        self._export = _lib.declare("cocclSymmExport", C.c_int, [C.c_void_p, C.c_void_p])
        self._import = _lib.declare("cocclSymmImport", C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.POINTER(C.c_void_p)])
        self._local = _lib.declare("cocclSymmLocalPtr", C.c_void_p, [C.c_void_p])
        self._close = _lib.declare("cocclSymmCloseImports", C.c_int, [C.c_void_p])
        self._free = _lib.declare("cocclSymmFree", C.c_int, [C.c_void_p])
        self._grow = _lib.declare("cocclSymmGrow", C.c_int, [C.c_void_p, C.c_size_t])
        get_backend = _lib.declare("cocclSymmGetBackend", C.c_int, [])
        set_backend = _lib.declare("cocclSymmSetBackend", C.c_int, [C.c_int])
        default_backend = int(get_backend())
        self.backend = default_backend if backend is None else backend   # 0: CUDA IPC, 1: cuMem VMM
        self.handle, self.nbytes, self.ptrs = None, nbytes, []
        if replaces is not None:
            # nobody's kernels use the old mapping any more, then nobody maps it, then it is freed
            torch.cuda.synchronize()
            dist.barrier(group=comm.group)
            replaces.close_imports()
            dist.barrier(group=comm.group)
            replaces.free()
        h = C.c_void_p()
        hbytes = int(_lib.declare("cocclSymmHandleBytes", C.c_int, [])())
        buf = C.create_string_buffer(hbytes)
        ok = self.backend == default_backend or set_backend(self.backend) == 0
        ok = ok and self._alloc(nbytes, C.byref(h)) == 0 and self._export(h, buf) == 0
        set_backend(default_backend)
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
                hb = C.create_string_buffer(offers[p][1], hbytes)
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

    @classmethod
    def resized(cls, comm: "Communicator", old: "_Symm | None", nbytes: int) -> "_Symm":
        """Collective: a region of at least `nbytes` in place of `old`. A cuMem VMM region grows where it is (no pointer
        on any rank changes, nothing is unmapped); otherwise, or when that fails on some rank, the old region is closed
        and a new one opened by the protocol of __init__."""
        if old is not None and old.backend == 1 and old.grow(comm, nbytes):
            return old
        return cls(comm, nbytes, replaces=old)

    def grow(self, comm: "Communicator", nbytes: int) -> bool:
        """Collective, VMM regions only: every rank adds physical chunks behind its buffer, the new export handles are
        exchanged and every rank maps the new chunks of every peer behind the old ones. True only if every rank
        managed and every pointer is what it was."""
        torch.cuda.synchronize()
        dist.barrier(group=comm.group)   # nobody's kernels still use the old extent (callers re-split the region)
        hbytes = int(_lib.declare("cocclSymmHandleBytes", C.c_int, [])())
        buf = C.create_string_buffer(hbytes)
        ok = self._grow(self.handle, nbytes) == 0 and self._export(self.handle, buf) == 0
        offers = [None] * comm.size
        dist.all_gather_object(offers, (ok, bytes(buf.raw)), group=comm.group)
        ok = all(o[0] for o in offers)
        if ok:
            for p in range(comm.size):
                if p == comm.rank:
                    continue
                m = C.c_void_p()
                hb = C.create_string_buffer(offers[p][1], hbytes)
                if self._import(self.handle, p, hb, C.byref(m)) != 0 or m.value != self.ptrs[p]:
                    ok = False
                    break
        outcome = [None] * comm.size
        dist.all_gather_object(outcome, ok, group=comm.group)
        if all(outcome):
            self.nbytes = nbytes
            return True
        return False

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
            self.ws = _Symm.resized(self.comm, old, 2 * half)
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
        self.stats = {"compressed_calls": 0, "native_calls": 0, "compressed_raw_bytes": 0, "native_bytes": 0,
                      "unfused_codec_calls": 0, "nvls_calls": 0}
        self.role = ROLE.get(name, 0)
        self._last: Decision | None = None
        self._decisions: dict = {}
        if self.size > _lib.MAX_RANKS:
            self.policy = NATIVE  # fused kernels cover one NVSwitch domain of up to 8 ranks
        self.router = Router.of(self.policy, self.size) if (self.cuda and self.size > 1) else None
        # CTAs a fused kernel may occupy: the Policy object's own field, else the policy file's [runtime] key
        self.max_ctas = self.policy.max_ctas or (self.router.fused_max_ctas() if self.router is not None else 0)

    # ------------------------------------------------------------------ symmetric state
    def _ensure(self, half_bytes: int):
        if self._sig is None:
            flag_bytes = _lib.lib().cocclkFlagBytes()
            self._flag_bytes = flag_bytes
            self._sig = _Symm(self, flag_bytes + 256)
        if self._ws is None or self._ws_half < half_bytes:
            half = -(-max(half_bytes, 1 << 20) // (1 << 20)) * (1 << 20)
            old, self._ws, self._ws_half = self._ws, None, 0
            self._ws = _Symm.resized(self, old, 2 * half)
            self._ws_half = half

    def _leave_fused_path(self, why: Exception) -> None:
        import warnings
        warnings.warn(f"coccl_b200: group '{self.name}' falls back to native collectives on every rank: {why}")
        self.policy = NATIVE
        self.router = None

    def _fused(self, opc: int, inp: torch.Tensor, out: torch.Tensor, cfg) -> bool:
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
        a.codec = K.as_c(cfg, inp.dtype)
        a.slotBytes, a.regionBOffset = sb, region_b
        a.inp[self.rank], a.out[self.rank] = inp.data_ptr(), out.data_ptr()
        for p in range(n):
            a.ws[p] = self._ws.ptrs[p] + parity * self._ws_half
            a.flags[p] = self._sig.ptrs[p]
            a.status[p] = self._sig.ptrs[p] + self._flag_bytes
        if self._trace is not None:
            self._trace.zero_()
            a.trace[self.rank] = self._trace.data_ptr()
        with nvtx_range(f"coccl.fused.{K_NAMES.get(opc, opc)}.{a.codec.kind}"):
            rc = _lib.lib().cocclkFusedCollective(a, 1, self.max_ctas, _lib.cur_stream())
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

    def _route(self, op: str, inp: torch.Tensor, count: int, explicit: int = -1) -> Decision | None:
        """Ask the router. Returns the decision when the call runs as a fused compressed kernel, None when it runs
        natively (`self._last` keeps the decision either way, e.g. for the multimem variant of a native all-reduce).
        `count` is the count of the matching nccl* call."""
        self._last = None
        if self.router is None or not inp.is_cuda or inp.dtype not in NCCL_DTYPE:
            return None
        key = (op, inp.dtype, count, explicit)
        d = self._decisions.get(key)
        if d is None:   # the router is deterministic between two measurement updates: ask once per call shape
            d = self._decisions[key] = self.router.decide(self.role, op, inp.dtype, count, self.size, self.rank, explicit)
        self._last = d
        if not d.compressed:
            return None
        if not d.fusable or inp.dtype not in DTYPE_CODE or not (inp.is_contiguous() and inp.data_ptr() % 4 == 0):
            # a codec without a tile form (plugin-only: rANS, odd ZFP rates) is served by the staged pipeline of the
            # C API; this layer launches fused kernels only and leaves such calls native
            self.stats["unfused_codec_calls"] += 1
            return None
        return d

    def _native(self, nbytes):
        self.stats["native_calls"] += 1
        self.stats["native_bytes"] += nbytes

    def routing_summary(self) -> dict:
        """Effective policy hash, router counters and what was measured for the selector."""
        if self.router is None:
            return {"policy": "native"}
        return {"policy_hash": self.router.config_hash(), "training_mode": self.router.training_mode(),
                "router": self.router.stats(), "measured": list(self.router.tuning_log)}

    # ------------------------------------------------------------------ collectives
    def reduce_scatter(self, inp: torch.Tensor, out: torch.Tensor, role: str | None = None):
        """out = sum over ranks of inp[rank chunk]; inp has size*out.numel() elements."""
        if self.size == 1:
            out.copy_(inp.reshape(out.shape))
            return out
        nbytes = inp.numel() * inp.element_size()
        d = self._route("reduce_scatter", inp, out.numel())
        if d is None or not self._fused(K.OP_RS, inp, out, d.codec):
            self._native(nbytes)
            with nvtx_range("coccl.native.reduce_scatter"):
                dist.reduce_scatter_tensor(out, inp, group=self.group)
        return out

    def all_gather(self, inp: torch.Tensor, out: torch.Tensor, role: str | None = None, state=None):
        """Gather `inp` of every rank into `out`. When the policy puts a delta codec on this call (sdp4bit subAdd)
        the caller passes the state handle of the previous call (None the first time) and keeps the returned one;
        see all_gather_delta. Returns `out`, or (out, state) when `state` was given or a delta codec applies."""
        if self.size == 1:
            out.copy_(inp.reshape(out.shape))
            return out
        nbytes = out.numel() * out.element_size()
        d = self._route("all_gather", inp, inp.numel())
        if d is not None and d.delta:
            return out, self.all_gather_delta(inp, out, d.codec, state)
        if d is None or not self._fused(K.OP_AG, inp, out, d.codec):
            self._native(nbytes)
            with nvtx_range("coccl.native.all_gather"):
                dist.all_gather_into_tensor(out, inp, group=self.group)
        return out

    def uses_delta_all_gather(self, numel_per_rank: int, dtype: torch.dtype) -> bool:
        """Whether the policy routes an all-gather of this shape through a delta codec (the caller then keeps the
        previous values until the call has subtracted them)."""
        if self.router is None or self.size == 1:
            return False
        d = self.router.decide(self.role, "all_gather", dtype, numel_per_rank, self.size, self.rank)
        return bool(d.compressed and d.fusable and d.delta)

    # ------------------------------------------------------------------ NVSwitch (multimem) all-reduce
    def _ensure_nvls(self, nbytes: int) -> bool:
        """Symmetric buffer bound to a multicast object (torch symmetric memory does the allocation and the
        binding; the reduction kernel is csrc/kernels/nvls_kernels.cu). False when the fabric has no multicast."""
        if self._nvls is not None and self._nvls["bytes"] >= nbytes:
            return self._nvls["mc"] != 0
        if self._nvls is not None and self._nvls["mc"] == 0:
            return False
        size = max(nbytes, 64 << 20)
        if self._nvls is not None and isinstance(self._nvls.get("h"), _Symm):   # a larger region replaces the old one
            old = self._nvls["h"]
            self._nvls["t"] = self._nvls["h"] = None
            self._release_own_multicast(old)
        t, h, mc = self._own_multicast(size) if os.environ.get("COCCL_NVLS_BACKEND", "own") == "own" else (None, None, 0)
        if mc == 0:
            import torch.distributed._symmetric_memory as symm_mem
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
        self._nvls = {"t": t, "h": h, "mc": mc, "bytes": size, "flags": flags, "epoch": epoch, "used": 0}
        return mc != 0

    def _own_multicast(self, size: int):
        """(tensor over the local buffer, region, multicast address) from this library's own cuMem VMM region bound to an
        NVSwitch multicast object (csrc/symm/symm_vmm.cc), or (None, None, 0) on every rank when any rank cannot."""
        supported = _lib.declare("cocclSymmMulticastSupported", C.c_int, [])
        ok = torch.tensor([1 if supported() == 1 else 0], device=self.device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
        if int(ok.item()) == 0:
            return None, None, 0
        try:
            region = _Symm(self, size, backend=1)
        except SymmUnavailable:
            return None, None, 0
        create = _lib.declare("cocclSymmMulticastCreate", C.c_int, [C.c_void_p, C.c_int, C.c_void_p])
        join = _lib.declare("cocclSymmMulticastJoin", C.c_int, [C.c_void_p, C.c_void_p])
        bind = _lib.declare("cocclSymmMulticastBind", C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)])
        hbytes = int(_lib.declare("cocclSymmHandleBytes", C.c_int, [])())
        blob = C.create_string_buffer(hbytes)
        made = create(region.handle, self.size, blob) == 0 if self.rank == 0 else True
        box = [(made, bytes(blob.raw))]
        root = dist.get_global_rank(self.group, 0) if self.group is not None else 0
        dist.broadcast_object_list(box, src=root, group=self.group)

        def agreed(flag: bool) -> bool:   # also the barrier the protocol needs between its steps
            v = torch.tensor([1 if flag else 0], device=self.device)
            dist.all_reduce(v, op=dist.ReduceOp.MIN, group=self.group)
            return int(v.item()) == 1

        good = box[0][0]
        if good:
            good = join(region.handle, C.create_string_buffer(box[0][1], hbytes)) == 0
        good = agreed(good)            # every device has been added before anyone binds
        ptr = C.c_void_p()
        if good:
            good = bind(region.handle, C.byref(ptr)) == 0 and bool(ptr.value)
        good = agreed(good)
        if not good:
            self._release_own_multicast(region)
            return None, None, 0
        t = _lib.tensor_from_ptr(region.ptrs[self.rank], size, self.device, owner=region)
        return t, region, int(ptr.value)

    def _release_own_multicast(self, region) -> None:
        """Collective and ordered: unbind while every rank is alive, meet, unmap the peers, meet, free."""
        unbind = _lib.declare("cocclSymmMulticastUnbind", C.c_int, [C.c_void_p])
        torch.cuda.synchronize()
        if self.size > 1:
            dist.barrier(group=self.group)
        unbind(region.handle)
        if self.size > 1:
            dist.barrier(group=self.group)
        region.close_imports()
        if self.size > 1:
            dist.barrier(group=self.group)
        region.free()

    def symmetric_tensor(self, numel: int, dtype: torch.dtype) -> torch.Tensor | None:
        """A tensor inside this communicator's multicast-bound symmetric buffer (None when the fabric has no
        multicast). `all_reduce` on such a tensor runs the multimem kernel IN PLACE: no copy in, no copy out. Every
        rank must make the same sequence of requests (the offsets have to agree); the tensors live as long as the
        communicator and are never handed back."""
        nbytes = -(-numel * torch.empty(0, dtype=dtype).element_size() // 256) * 256
        used = self._nvls["used"] if self._nvls is not None else 0
        if used != 0 and used + nbytes > self._nvls["bytes"]:
            return None   # growing would move the tensors handed out before; callers fall back to ordinary tensors
        if not self._ensure_nvls(max(used + nbytes, 64 << 20)):
            return None
        st = self._nvls
        off = st["used"]
        st["used"] = off + nbytes
        return st["t"][off:off + numel * torch.empty(0, dtype=dtype).element_size()].view(dtype)

    def _nvls_offset(self, x: torch.Tensor):
        """Byte offset of x inside the symmetric buffer, or None if it lives elsewhere."""
        st = self._nvls
        if st is None or st["t"] is None:
            return None
        base = st["t"].data_ptr()
        off = x.data_ptr() - base
        return off if 0 <= off and off + x.numel() * x.element_size() <= st["bytes"] else None

    def all_reduce_nvls(self, x: torch.Tensor) -> bool:
        """In-place sum over ranks through the switch. Returns False (x untouched) when multicast is unavailable or
        the size does not split into 16-byte vectors per rank."""
        nbytes = x.numel() * x.element_size()
        if x.dtype not in DTYPE_CODE or nbytes % (16 * self.size) != 0 or not x.is_contiguous():
            return False
        inplace = self._nvls_offset(x)
        if inplace is not None and inplace % 16 == 0 and self._nvls["mc"] != 0:
            st, mc = self._nvls, self._nvls["mc"] + inplace
            buf = None
        else:
            # staging area = what is left of the buffer behind the tensors handed out by symmetric_tensor
            used = self._nvls["used"] if self._nvls is not None else 0
            if used != 0 and used + nbytes > self._nvls["bytes"]:
                return False   # growing would move the tensors that symmetric_tensor handed out
            if not self._ensure_nvls(used + nbytes):
                return False
            st = self._nvls
            buf = st["t"][st["used"]:st["used"] + nbytes].view(x.dtype)
            mc = st["mc"] + st["used"]
            buf.copy_(x.view(-1))
            self.stats["nvls_staged_copies"] = self.stats.get("nvls_staged_copies", 0) + 2
        st["epoch"] += 1
        fl = (C.c_void_p * self.size)(*[st["flags"].ptrs[p] for p in range(self.size)])
        status = st["flags"].ptrs[self.rank] + _lib.lib().cocclkNvlsFlagBytes()
        with nvtx_range("coccl.nvls.all_reduce"):
            rc = _lib.lib().cocclkNvlsAllReduce(mc, x.numel(), DTYPE_CODE[x.dtype], self.size, self.rank, fl, status,
                                                st["epoch"] & 0xFFFFFFFF, int(self.policy.timeout_ms * 1e6),
                                                self.max_ctas, _lib.cur_stream())
        _lib.check(rc, "cocclkNvlsAllReduce")
        if buf is not None:
            x.view(-1).copy_(buf)
        self.stats["nvls_calls"] = self.stats.get("nvls_calls", 0) + 1
        return True

    def all_reduce(self, x: torch.Tensor, role: str | None = None):
        if self.size == 1:
            return x
        nbytes = x.numel() * x.element_size()
        if self.router is not None and self.router.autotune and self.policy.measure and x.is_cuda and x.dtype in DTYPE_CODE:
            self._measure_all_reduce(x.dtype)
        d = self._route("all_reduce", x, x.numel())
        if d is not None:
            op = K.OP_AR1 if d.algorithm == ALGO_AR_ONESHOT else K.OP_AR2
            if self._fused(op, x, x, d.codec):
                return x
        last = self._last
        if last is not None and last.native_variant == 1 and self.policy.nvls and self.all_reduce_nvls(x):
            return x
        self._native(nbytes)
        with nvtx_range("coccl.native.all_reduce"):
            dist.all_reduce(x, group=self.group)
        return x

    def all_to_all(self, inp: torch.Tensor, out: torch.Tensor, role: str | None = None):
        if self.size == 1:
            out.copy_(inp)
            return out
        nbytes = inp.numel() * inp.element_size()
        d = self._route("all_to_all", inp, inp.numel() // self.size) if inp.numel() % self.size == 0 else None
        if d is None or not self._fused(K.OP_A2A, inp, out, d.codec):
            self._native(nbytes)
            with nvtx_range("coccl.native.all_to_all"):
                dist.all_to_all_single(out, inp, group=self.group)
        return out

    # ------------------------------------------------------------------ measurements for the selector
    def _time_calls(self, fn, iters: int = 5, warmup: int = 2) -> float:
        """Seconds per call of fn(): CUDA events on the current stream, maximum over the ranks of the group."""
        for _ in range(warmup):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / iters / 1e3], device=self.device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        return float(t.item())

    def _measure_all_reduce(self, dtype: torch.dtype) -> None:
        """Once per (datatype, group size) and routing session: time the fused one-shot and two-shot all-reduce on this
        group for a ladder of sizes, and, for calls that stay uncompressed, NCCL against the multimem kernel; hand the
        results to the selector (cocclRouterSetMeasured*), which from then on picks per call by nearest size. The
        reference fits cost models to point-to-point and codec timings instead
        (src/coccl-extend/core/tuning/coccl_autotune_profiler.cc:62-618); here the candidates themselves are timed.
        Collective: every rank reaches the first all-reduce of a datatype at the same call."""
        key = ("ar", dtype, self.size, self.role)
        r = self.router
        if key in r.measured:
            return
        r.measured.add(key)
        es = torch.empty(0, dtype=dtype).element_size()
        unit = self.size * 2048
        probe = r.decide(self.role, "all_reduce", dtype, unit * 4096, self.size, self.rank, ALGO_AR_TWOSHOT)
        sizes = [1 << 16, 1 << 18, 1 << 20, 1 << 22, 1 << 24, 1 << 26]
        if probe.compressed and probe.fusable:
            for nbytes in reversed(sizes):     # largest first: the workspace grows once
                numel = max(unit, nbytes // es // unit * unit)
                x = torch.zeros(numel, dtype=dtype, device=self.device)
                lg = (numel * es).bit_length() - 1
                row = {"what": "all_reduce", "dtype": str(dtype), "ranks": self.size, "bytes": numel * es}
                for algo, opc in ((ALGO_AR_ONESHOT, K.OP_AR1), (ALGO_AR_TWOSHOT, K.OP_AR2)):
                    if algo == ALGO_AR_ONESHOT and nbytes > (8 << 20):
                        continue   # every rank receives everything: N x the traffic, never competitive up here
                    t = self._time_calls(lambda: self._fused(opc, x, x, probe.codec))
                    r.set_measured("all_reduce", dtype, self.size, lg, algo, t)
                    row["oneshot_us" if algo == ALGO_AR_ONESHOT else "twoshot_us"] = t * 1e6
                r.tuning_log.append(row)
                del x
        if self.policy.nvls and self._ensure_nvls(8 << 20):
            for nbytes in (1 << 16, 1 << 18, 1 << 20, 1 << 22, 1 << 23):
                numel = max(unit, nbytes // es // unit * unit)
                x = torch.zeros(numel, dtype=dtype, device=self.device)
                lg = (numel * es).bit_length() - 1
                t_nccl = self._time_calls(lambda: dist.all_reduce(x, group=self.group))
                t_nvls = self._time_calls(lambda: self.all_reduce_nvls(x))
                r.set_measured_native(dtype, self.size, lg, 0, t_nccl)
                r.set_measured_native(dtype, self.size, lg, 1, t_nvls)
                r.tuning_log.append({"what": "all_reduce_uncompressed", "dtype": str(dtype), "ranks": self.size,
                                     "bytes": numel * es, "nccl_us": t_nccl * 1e6, "multimem_us": t_nvls * 1e6})
        self._decisions.clear()
        if os.environ.get("COCCL_DEBUG", "").upper() in ("INFO", "TRACE") and self.rank == 0:
            for row in r.tuning_log:
                print("[coccl tuning]", row, flush=True)

    # ------------------------------------------------------------------ tensor-parallel fusions
    def _ensure_tp(self, half_bytes: int):
        if self._tp_sig is None:
            self._tp_flag_bytes = _lib.lib().cocclkFlagBytes()
            self._tp_sig = _Symm(self, self._tp_flag_bytes + 256)
            self._tp_err = torch.zeros(1, dtype=torch.int32, device=self.device)
        if self._tp_ws is None or self._tp_half < half_bytes:
            half = -(-max(half_bytes, 1 << 20) // (1 << 20)) * (1 << 20)
            old, self._tp_ws, self._tp_half = self._tp_ws, None, 0
            self._tp_ws = _Symm.resized(self, old, 2 * half)
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
                gathered: torch.Tensor | None = None, payload: str | None = None):
        """concat_over_ranks(x_local) @ w.T (+ bias, GELU) in ONE kernel: the shards travel over peer memory
        while the tensor cores already work on the local shard. x_local [m, K] bf16; w [N, K], or [K, N] with
        b_mn=True (then the product is gather(x) @ w). save_preact: also return the pre-activation (GELU only).
        gathered: optional [M, K] tensor that receives the gathered input (for a later weight gradient).
        payload: "bf16", "fp8" (block-scaled E4M3 on the wire, dequantised on arrival) or None = what the policy's
        all-gather slot of this communicator's role says (MX-FP8 codec -> "fp8"); COCCL_TP_AG_PAYLOAD overrides."""
        from ..ops import tp_fused as T
        m, K = x_local.shape
        fp8 = self._ag_payload_fp8(m, K, payload)
        if fp8 and payload is None and not os.environ.get("COCCL_TP_AG_PAYLOAD") and \
                not self._ag_payload_pays(m, K, w.shape[1] if b_mn else w.shape[0]):
            fp8 = False
        N = w.shape[1] if b_mn else w.shape[0]
        M = m * self.size
        assert x_local.is_contiguous() and w.is_contiguous() and x_local.dtype == torch.bfloat16
        if out is None:
            out = torch.empty(M, N, dtype=torch.bfloat16, device=x_local.device)
        self._ensure_tp(T.ag_ws_bytes(M, K, T.PAYLOAD_FP8 if fp8 else T.PAYLOAD_BF16))
        a = self._tp_args(M, N, K)
        a.agPayload = T.PAYLOAD_FP8 if fp8 else T.PAYLOAD_BF16
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
            _lib.check(_lib.lib().cocclkAgGemm(a, 1, self.max_ctas, _lib.cur_stream()), "cocclkAgGemm")
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

    def _ag_payload_fp8(self, m: int, K: int, payload: str | None) -> bool:
        """Whether the shards of an all-gather fusion travel as block-scaled FP8 (needs whole 32-column blocks)."""
        forced = os.environ.get("COCCL_TP_AG_PAYLOAD", "") or payload
        if K % 32 != 0:
            return False
        if forced in ("bf16", "fp8"):
            return forced == "fp8"
        key = ("ag_payload", m, K)
        if key not in self._decisions:
            fp8 = False
            if self.router is not None:
                d = self.router.decide(self.role, "all_gather", torch.bfloat16, m * K, self.size, self.rank)
                fp8 = bool(d.compressed and d.fusable and d.codec.kind == 1)   # 1 = MX-FP8
            self._decisions[key] = fp8
        return self._decisions[key]

    def _ag_payload_pays(self, m: int, K: int, n_out: int) -> bool:
        """Inside the fusion the shards travel behind the tensor cores' work on the local shard, so halving the bytes
        helps only when the wire would otherwise be the longer of the two: bf16 bytes over the measured 770 GB/s per
        direction against the GEMM at the measured sustained 1.4 PFLOP/s (at 4 ranks and the MLP shapes the FP8
        payload was measured 1.46x SLOWER than bf16: the dequantisation on arrival is serial work the bf16 path does
        not have)."""
        wire_s = (self.size - 1) * m * K * 2 / 770e9
        gemm_s = 2.0 * m * self.size * n_out * K / 1.4e15
        return wire_s > gemm_s

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
            _lib.check(_lib.lib().cocclkGemmRs(a, 1, self.max_ctas, _lib.cur_stream()), "cocclkGemmRs")
        if bias is not None and _lib.lib().cocclkTpLastVariant() != 2:
            out += bias   # the single-CTA kernel's reducer has no bias operand
        self.stats["compressed_calls"] += 1
        self.stats["compressed_raw_bytes"] += M * N * 2
        return out

    def tp_fusable(self, rows_total: int, n_out_rs: int | None = None, width: int | None = None) -> bool:
        """Whether the one-kernel TP fusions serve a problem with `rows_total` gathered rows (and, for gemm_rs,
        `n_out_rs` output columns). The fusions quantise the reduce-scattered partial sums to block-scaled FP8, so
        they apply only where the router, asked about the two collectives the fusion replaces, answers "compressed" for
        both and names the MX-FP8 codec for the reduce-scatter (`width` = columns of the gathered operand). Otherwise the
        caller takes the unfused path, whose collectives are routed one by one."""
        if not (self.cuda and self.router is not None and 1 < self.size <= _lib.MAX_RANKS):
            return False
        key = ("tp_fusable", rows_total, n_out_rs, width)
        if key not in self._decisions:
            self._decisions[key] = self._tp_fusable(rows_total, n_out_rs, width)
        return self._decisions[key]

    def _tp_fusable(self, rows_total: int, n_out_rs: int | None, width: int | None) -> bool:
        per_rank = rows_total // self.size
        ag = self.router.decide(self.role, "all_gather", torch.bfloat16, per_rank * (width or n_out_rs or 0), self.size, self.rank)
        rs = self.router.decide(self.role, "reduce_scatter", torch.bfloat16, per_rank * (n_out_rs or width or 0), self.size, self.rank)
        if not (ag.compressed and ag.fusable and rs.compressed and rs.fusable and rs.codec.kind == 1):   # 1 = MX-FP8
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
        if not x.is_cuda:
            return self._moe_dispatch_host(x, expert_ids, n_experts, capacity, row_scale, pos, counts)
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
        _lib.check(_lib.lib().cocclkMoeDispatch(a, 1, self.max_ctas, _lib.cur_stream()), "cocclkMoeDispatch")
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
        if not y.is_cuda:
            return self._moe_combine_host(y, gates, handle, dot_with)
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
        _lib.check(_lib.lib().cocclkMoeCombine(a, 1, self.max_ctas, _lib.cur_stream()), "cocclkMoeCombine")
        return out if dot_with is None else (out, dots)

    # CPU tensors (the gloo tests, a launcher run without GPUs): the same exchange as plain PyTorch over
    # all_to_all_single, rows in the tensor's own datatype (no FP8 on the way), same row order and handle contents.
    def _moe_dispatch_host(self, x, expert_ids, n_experts, capacity, row_scale, pos, counts):
        from ..ops import moe as M
        n, le = self.size, n_experts // self.size
        tokens, topk = expert_ids.shape
        flat = expert_ids.reshape(-1).long()
        per_rank = counts.long().view(n, le)
        send_rows = per_rank.sum(1)
        slot = (torch.cumsum(send_rows, 0) - send_rows)[flat // le] + pos.reshape(-1).long()   # row of entry (t, j) in the send buffer
        rows = x.repeat_interleave(topk, dim=0)
        if row_scale is not None:
            rows = (rows.float() * row_scale.reshape(-1, 1)).to(x.dtype)
        send = torch.empty_like(rows)
        send[slot] = rows
        got = torch.empty_like(per_rank)                       # got[s, e]: rows source s sends to my local expert e
        dist.all_to_all_single(got, per_rank.contiguous(), group=self.group)
        recv_rows = got.sum(1)
        recv = x.new_empty(int(recv_rows.sum()), x.shape[1])
        dist.all_to_all_single(recv, send, output_split_sizes=recv_rows.tolist(), input_split_sizes=send_rows.tolist(),
                               group=self.group)
        # arrival order is source-major; the experts want their rows together: local expert, then source
        src_off = torch.cumsum(recv_rows, 0) - recv_rows
        in_src = torch.cumsum(got, 1) - got
        perm = torch.cat([torch.arange(int(got[s_, e]), dtype=torch.long) + int(src_off[s_] + in_src[s_, e])
                          for e in range(le) for s_ in range(n)]) if recv.shape[0] else torch.zeros(0, dtype=torch.long)
        roff = torch.zeros(le + 1, dtype=torch.int32)
        roff[1:] = torch.cumsum(got.sum(0), 0).to(torch.int32)
        h = M.Handle(expert_ids, pos, got.to(torch.int32), roff, capacity, n_experts)
        h.counts = counts
        h.host = (perm, send_rows.tolist(), recv_rows.tolist(), slot)
        self._native(rows.numel() * rows.element_size())
        return recv[perm], h

    def _moe_combine_host(self, y, gates, handle, dot_with):
        perm, send_rows, recv_rows, slot = handle.host
        tokens, topk = gates.shape
        back = y.new_empty(len(perm), y.shape[1])
        back[perm] = y[:len(perm)]
        ret = y.new_empty(tokens * topk, y.shape[1])
        dist.all_to_all_single(ret, back, output_split_sizes=send_rows, input_split_sizes=recv_rows, group=self.group)
        rows = ret[slot].view(tokens, topk, -1).float()
        out = (gates.float().unsqueeze(-1) * rows).sum(1).to(y.dtype)
        if dot_with is None:
            return out
        return out, (rows * dot_with.float().unsqueeze(1)).sum(-1)

    def moe_status(self) -> int:
        return 0 if self._moe is None else self._moe.status()

    def all_gather_delta(self, inp: torch.Tensor, out: torch.Tensor, cfg=None, state=None):
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
        if cfg is None:
            from ..ops.codec import CodecConfig
            cfg = CodecConfig("sdp4bit", 8, 2048, False, False)
        usable = self.cuda and inp.is_cuda and inp.dtype in DTYPE_CODE and inp.is_contiguous() and out.is_contiguous()
        seeded = (state is not None and state.get("out") is out and state.get("numel") == out.numel()
                  and state.get("version") == out._version)
        if not usable or not seeded or not self._fused(K.OP_AGD, inp, out, cfg):
            self._native(out.numel() * out.element_size())
            dist.all_gather_into_tensor(out, inp, group=self.group)
        if not usable or self.router is None:
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
        if self._nvls is not None and isinstance(self._nvls.get("h"), _Symm):
            region = self._nvls["h"]
            self._nvls["t"] = None
            self._nvls["h"] = None
            self._nvls["mc"] = 0
            self._release_own_multicast(region)
        self._ws = self._sig = self._tp_ws = self._tp_sig = self._moe = None
