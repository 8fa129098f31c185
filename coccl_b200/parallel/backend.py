"""torch.distributed backend "coccl".

    import coccl_b200.parallel.backend            # registers the backend
    os.environ["COCCL_ENABLE"] = "1"; os.environ["COCCL_CONFIG_FILE"] = ".../normal-sdp4bit.toml"
    dist.init_process_group("coccl", ...)
    dist.all_reduce(t)                            # routed: compressed above the threshold, NCCL below

all_reduce / reduce_scatter_tensor / all_gather_into_tensor / all_to_all_single go through the library's
router; everything else (broadcast, barrier, send/recv, object collectives) is served by an inner
ProcessGroupNCCL over the same store. The native part lives in coccl_b200/_pg.so
(csrc/torch/process_group.cpp), built by `python -m coccl_b200._build --torch`.
"""
from __future__ import annotations

import importlib.util
from datetime import timedelta
from pathlib import Path

import torch.distributed as dist

_mod = None


def _native():
    global _mod
    if _mod is None:
        so = Path(__file__).resolve().parent.parent / "_pg.so"
        if not so.exists():
            from .. import _build
            _build.build()
            _build.build_torch_backend()
        from .. import _lib
        _lib.lib()  # libcoccl.so must be in the process before _pg.so resolves against it
        spec = importlib.util.spec_from_file_location("_pg", so)
        _mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(_mod)
    return _mod


def _create(store, rank, size, timeout=timedelta(minutes=10)):
    from torch.distributed import ProcessGroupNCCL
    opts = ProcessGroupNCCL.Options()
    opts._timeout = timeout
    inner = ProcessGroupNCCL(dist.PrefixStore("coccl_inner", store), rank, size, opts)
    return _native().ProcessGroupCoccl(inner, dist.PrefixStore("coccl", store), rank, size)


def register():
    if "COCCL" not in dist.Backend.backend_list and "coccl" not in dist.Backend.backend_list:
        dist.Backend.register_backend("coccl", _create, devices=["cuda"])


register()
