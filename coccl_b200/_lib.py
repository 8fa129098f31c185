"""ctypes binding of libcoccl.so (the native runtime + sm_100a kernels).

The library is loaded from coccl_b200/lib; if it is missing it is built in
place. There is no Python fallback for a kernel: on a machine with a GPU a
missing or stale library is an error, never a silent slow path.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_ROOT = Path(__file__).resolve().parent
_SO = _ROOT / "lib" / "libcoccl.so"
# COCCL_CHECKED_KERNELS=1: load the bounds-checked twin (codec accesses range-checked, violations recorded in a
# device word instead of touching memory; see bounds_word())
if os.environ.get("COCCL_CHECKED_KERNELS", "") not in ("", "0"):
    _SO = _SO.with_name("libcoccl_checked.so")
_lib = None

c_void_p, c_int, c_long, c_float, c_uint, c_ulonglong = C.c_void_p, C.c_int, C.c_long, C.c_float, C.c_uint, C.c_ulonglong

MAX_RANKS = 8
MAX_SLICES = 4096


class Codec(C.Structure):
    """Mirror of cocclkCodec (csrc/kernels/kernels_api.h)."""
    _fields_ = [("kind", c_int), ("bits", c_int), ("group", c_int), ("asym", c_int), ("hadamard", c_int),
                ("stochastic", c_int), ("paramBytes", c_int), ("seed", C.c_uint32), ("aux", c_int),
                ("f0", c_float), ("f1", c_float), ("f2", c_float)]


class CollArgs(C.Structure):
    """Mirror of cocclkCollArgs."""
    _fields_ = [("op", c_int), ("nRanks", c_int), ("rankBase", c_int), ("dtype", c_int), ("count", c_long),
                ("sliceTiles", c_int), ("epoch", c_uint), ("timeoutNs", c_ulonglong), ("codec", Codec),
                ("slotBytes", c_long), ("regionBOffset", c_long),
                ("inp", c_void_p * MAX_RANKS), ("out", c_void_p * MAX_RANKS), ("ws", c_void_p * MAX_RANKS),
                ("flags", c_void_p * MAX_RANKS), ("status", c_void_p * MAX_RANKS), ("trace", c_void_p * MAX_RANKS)]


class TpArgs(C.Structure):
    """Mirror of cocclkTpArgs (csrc/kernels/tp_api.h)."""
    _fields_ = [("nRanks", c_int), ("rankBase", c_int), ("M", c_int), ("N", c_int), ("K", c_int), ("epi", c_int),
                ("bMN", c_int), ("epoch", c_uint), ("timeoutNs", c_ulonglong),
                ("a", c_void_p * MAX_RANKS), ("b", c_void_p * MAX_RANKS), ("c", c_void_p * MAX_RANKS),
                ("bias", c_void_p * MAX_RANKS), ("z", c_void_p * MAX_RANKS), ("ws", c_void_p * MAX_RANKS),
                ("flags", c_void_p * MAX_RANKS), ("status", c_void_p * MAX_RANKS), ("err", c_void_p * MAX_RANKS),
                ("gathered", c_void_p * MAX_RANKS), ("agPayload", c_int)]


class ExchangeArgs(C.Structure):
    """Mirror of cocclkExchangeArgs (csrc/kernels/kernels_api.h)."""
    _fields_ = [("nRanks", c_int), ("rankBase", c_int), ("gather", c_int), ("frames", c_int), ("pieces", c_int),
                ("frameStride", c_long), ("pieceBytes", c_long)] + \
               [(n, c_void_p * MAX_RANKS) for n in ("send", "recv", "sendMeta", "recvMeta", "staging", "flags", "status")] + \
               [("epoch", c_uint), ("timeoutNs", c_ulonglong)]


class MoeArgs(C.Structure):
    """Mirror of cocclkMoeArgs (csrc/kernels/moe_api.h)."""
    _fields_ = [("nRanks", c_int), ("rankBase", c_int), ("tokens", c_int), ("hidden", c_int), ("topk", c_int),
                ("experts", c_int), ("capacity", c_int), ("epoch", c_uint), ("timeoutNs", c_ulonglong)] + \
               [(n, c_void_p * MAX_RANKS) for n in ("x", "expertIds", "gates", "pos", "sendCounts", "recv", "recvOffsets",
                                                   "recvCounts", "y", "out", "rowScale", "dotWith", "dotOut", "ws", "flags",
                                                   "status")]


_PROTOS = {
    # kernels_api.h
    "cocclkEncodedChunkBytes": (c_long, [C.POINTER(Codec), c_long]),
    "cocclkTileCodecSupported": (c_int, [C.POINTER(Codec)]),
    "cocclkEncode": (c_int, [c_void_p, c_void_p, c_long, c_long, c_long, c_long, c_int, C.POINTER(Codec), c_void_p]),
    "cocclkDecodeReduce": (c_int, [c_void_p, c_void_p, c_long, c_long, c_long, c_long, c_long, c_int,
                                   C.POINTER(Codec), c_void_p]),
    "cocclkDecodeReduceEncode": (c_int, [c_void_p, c_void_p, c_long, c_long, c_long, c_long, c_long,
                                         C.POINTER(Codec), c_void_p]),
    "cocclkFlagBytes": (c_long, []),
    "cocclkTileElems": (c_int, []),
    "cocclkSlotBytes": (c_long, [C.POINTER(Codec), c_long]),
    "cocclkFusedCollective": (c_int, [C.POINTER(CollArgs), c_int, c_int, c_void_p]),
    "cocclkNvlsFlagBytes": (c_long, []),
    "cocclkNvlsAllReduce": (c_int, [c_void_p, c_long, c_int, c_int, c_int, C.POINTER(c_void_p), c_void_p, c_uint, c_ulonglong,
                                    c_int, c_void_p]),
    # gemm_api.h
    "cocclkGemmBf16": (c_int, [c_void_p, c_long, c_int, c_void_p, c_long, c_int, c_void_p, c_long, c_int, c_int, c_int,
                               c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "cocclkGemmSetVariant": (None, [c_int]),
    "cocclkGemmGetVariant": (c_int, []),
    # tp_api.h
    "cocclkAgGemmWorkspaceBytes": (c_long, [c_int, c_int]),
    "cocclkGemmRsWorkspaceBytes": (c_long, [c_int, c_int, c_int]),
    "cocclkAgGemm": (c_int, [C.POINTER(TpArgs), c_int, c_int, c_void_p]),
    "cocclkGemmRs": (c_int, [C.POINTER(TpArgs), c_int, c_int, c_void_p]),
    "cocclkTpLastVariant": (c_int, []),
    # moe_api.h
    "cocclkMoeWorkspaceBytes": (c_long, [c_int, c_int, c_int, c_int]),
    "cocclkMoeLayout": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "cocclkMoeDispatch": (c_int, [C.POINTER(MoeArgs), c_int, c_int, c_void_p]),
    "cocclkMoeCombine": (c_int, [C.POINTER(MoeArgs), c_int, c_int, c_void_p]),
    # train_api.h
    "cocclkLayerNormFwd": (c_int, [c_void_p] * 8 + [c_int, c_int, c_float, c_void_p]),
    "cocclkLayerNormBwdGrid": (c_int, [c_int]),
    "cocclkLayerNormBwd": (c_int, [c_void_p] * 9 + [c_int, c_void_p, c_int, c_int, c_void_p]),
    "cocclkColSumBlocks": (c_int, [c_int]),
    "cocclkColSum": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p]),
    "cocclkGeluFwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_int, c_void_p]),
    "cocclkGeluBwd": (c_int, [c_void_p, c_void_p, c_void_p, c_long, c_void_p]),
    "cocclkCrossEntropy": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_long, c_float, c_void_p]),
    "cocclkCrossEntropyStats": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_long, c_long, c_void_p]),
    "cocclkCrossEntropyFinish": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_long, c_long,
                                         c_float, c_void_p]),
    "cocclkAdam": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_long, c_float, c_float, c_float,
                           c_float, c_float, c_int, c_void_p, c_void_p]),
    "cocclkSumSqBlocks": (c_int, [c_long]),
    "cocclkSumSq": (c_int, [c_void_p, c_int, c_long, c_void_p, c_int, c_void_p, c_void_p]),
    "cocclkClipCoef": (c_int, [c_void_p, c_float, c_float, c_void_p, c_void_p, c_void_p]),
    "cocclkAccumBf16": (c_int, [c_void_p, c_void_p, c_long, c_int, c_void_p]),
}


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not _SO.exists():
            from . import _build
            _build.build()
        _lib = C.CDLL(str(_SO), mode=C.RTLD_GLOBAL)
        for name, (res, args) in _PROTOS.items():
            try:
                fn = getattr(_lib, name)
            except AttributeError as e:  # stale library
                raise RuntimeError(f"{_SO} lacks symbol {name}; rebuild with `python -m coccl_b200._build`") from e
            fn.restype = res
            fn.argtypes = args
    return _lib


def declare(name: str, restype, argtypes):
    """Attach a prototype for a symbol that is not in the static table (host runtime APIs)."""
    fn = getattr(lib(), name)
    fn.restype = restype
    fn.argtypes = argtypes
    return fn


def check(rc: int, what: str):
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}" + (" (unsupported configuration)" if rc == -1 else ""))


def ptr(t) -> int | None:
    """Device pointer of a tensor (None passes NULL)."""
    return None if t is None else t.data_ptr()


def cur_stream() -> int:
    import torch
    return torch.cuda.current_stream().cuda_stream


class _RawCudaMemory:
    """Exposes a device address range through __cuda_array_interface__ so that torch can view it."""

    def __init__(self, ptr: int, nbytes: int, owner=None):
        self.owner = owner   # kept alive for as long as the tensor lives
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (int(ptr), False), "version": 3,
                                         "strides": None}


def tensor_from_ptr(ptr: int, nbytes: int, device, owner=None):
    """uint8 tensor over device memory that this library allocated itself (symmetric buffers). The memory must stay
    valid while the tensor or any view of it is in use; `owner` is an object the tensor keeps alive."""
    import torch
    return torch.as_tensor(_RawCudaMemory(ptr, nbytes, owner), device=device)


def bounds_word(reset: bool = False) -> tuple[bool, list[int]]:
    """(whether the loaded library is the bounds-checked build, its error word: [0] = 0 or 0x80000000 | site, then the
    element index and the offending / allowed byte ends). Synchronises the device."""
    checked = bool(declare("cocclkBoundsChecked", C.c_int, [])())
    w = (C.c_uint * 8)()
    check(declare("cocclkBoundsWord", C.c_int, [C.POINTER(C.c_uint), C.c_int])(w, int(reset)), "cocclkBoundsWord")
    return checked, [int(v) for v in w]
