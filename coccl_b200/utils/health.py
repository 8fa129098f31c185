"""Host-side failure detection between steps.

The reference inherits NCCL's device-side abort flag and async error query (src/device/prims_simple.h:97-132,
src/init.cc:2166,2286) and has no elastic recovery. Here the device side is the bounded waits of the kernels
(status words read by `Communicator.status()`), and the host side is this heartbeat: every rank publishes
(step, wall time) in the rendezvous store after each step and consults its peers' entries BEFORE launching the
next step's kernels, so a rank that left, crashed or stalled is noticed on the host while no kernel or
collective of the survivors is in flight.
"""
from __future__ import annotations

import time
from dataclasses import dataclass

import torch.distributed as dist


class PeerLost(RuntimeError):
    def __init__(self, rank: int, reason: str):
        super().__init__(f"rank {rank}: {reason}")
        self.rank, self.reason = rank, reason


@dataclass
class PeerState:
    step: int
    wall: float
    leaving: bool


class Heartbeat:
    """store: a torch.distributed Store shared by all ranks (e.g. the TCPStore used for the rendezvous)."""

    def __init__(self, store, rank: int, world: int, prefix: str = "coccl/hb", stale_after_s: float = 30.0):
        self.store, self.rank, self.world, self.prefix, self.stale = store, rank, world, prefix, stale_after_s
        self.beat(-1)

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self, step: int, leaving: bool = False) -> None:
        self.store.set(self._key(self.rank), f"{step},{time.time():.3f},{int(leaving)}")

    def leave(self, step: int) -> None:
        """Announce an orderly departure (between steps, nothing in flight)."""
        self.beat(step, leaving=True)

    def peer(self, r: int) -> PeerState | None:
        try:
            if hasattr(self.store, "check") and not self.store.check([self._key(r)]):
                return None
            raw = self.store.get(self._key(r)).decode()
        except Exception:
            return None
        step, wall, leaving = raw.split(",")
        return PeerState(int(step), float(wall), leaving == "1")

    def check_peers(self, expect_step: int | None = None, wait_s: float = 0.0) -> None:
        """Raise PeerLost if a peer announced that it leaves, never registered, or has not finished
        `expect_step` within wait_s seconds and its last beat is older than `stale_after_s`."""
        deadline = time.time() + wait_s
        for r in range(self.world):
            if r == self.rank:
                continue
            while True:
                st = self.peer(r)
                if st is not None and st.leaving:
                    raise PeerLost(r, f"left after step {st.step}")
                if st is not None and (expect_step is None or st.step >= expect_step):
                    break
                now = time.time()
                if now >= deadline:
                    if st is None:
                        raise PeerLost(r, "never registered")
                    if now - st.wall > self.stale:
                        raise PeerLost(r, f"no heartbeat for {now - st.wall:.1f} s (last step {st.step})")
                    break
                time.sleep(0.01)


def default_store():
    """The store behind the default process group (None before init_process_group)."""
    if not dist.is_initialized():
        return None
    try:
        return dist.distributed_c10d._get_default_store()
    except Exception:
        return None
