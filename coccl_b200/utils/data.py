"""Token data for the trainer: a flat token file (or a synthetic stream) cut into training sequences, and a loader that
prepares every step's batch in pinned host memory on a background thread.

The reference ships no data path of its own: its launcher hands `--data-path` / `--dataset` to an external Megatron
trainer (examples/training_scripts/train_qwen_coccl.sh:96-131). The trainer of this package takes one pinned host
tensor [sequences, seq_len + 1] per step (train.py), so the loader's job is to have that tensor ready before the step
starts: the file is memory-mapped, a step's sequences are gathered by a worker thread into one of a small ring of
pinned buffers, and `next()` only hands over the buffer.

Which tokens a step sees is a pure function of (seed, step, data-parallel rank): a run that resumes at step k reads
exactly what an uninterrupted run would have read at step k, with no loader state in the checkpoint.
"""
from __future__ import annotations

import queue
import threading

import numpy as np
import torch


class TokenSource:
    """A stream of token ids addressed by position. `tokens(start, n)` returns n consecutive ids as int64."""

    length: int
    vocab: int | None = None

    def tokens(self, start: int, n: int) -> np.ndarray:
        raise NotImplementedError


class TokenFile(TokenSource):
    """A flat binary file of token ids (little-endian uint16 or uint32, no header), or a `.npy` array of any integer
    type. The file is memory-mapped; nothing is read until a batch needs it."""

    def __init__(self, path: str, dtype: str = "auto"):
        if path.endswith(".npy"):
            self.data = np.load(path, mmap_mode="r")
            if self.data.ndim != 1 or not np.issubdtype(self.data.dtype, np.integer):
                raise ValueError(f"{path}: expected a one-dimensional integer array, got {self.data.dtype}{self.data.shape}")
        else:
            if dtype == "auto":
                dtype = "uint32" if path.endswith((".u32", ".uint32")) else "uint16"
            if dtype not in ("uint16", "uint32"):
                raise ValueError(f"token dtype must be uint16 or uint32, got {dtype}")
            self.data = np.memmap(path, dtype=np.dtype(dtype).newbyteorder("<"), mode="r")
        self.length = int(self.data.shape[0])
        if self.length < 2:
            raise ValueError(f"{path}: fewer than two tokens")

    def tokens(self, start: int, n: int) -> np.ndarray:
        return np.asarray(self.data[start:start + n]).astype(np.int64, copy=False)


class SyntheticTokens(TokenSource):
    """Uniform-random token ids, reproducible by position: position p always holds the same id for a given seed."""

    def __init__(self, vocab: int, seed: int = 0, length: int = 1 << 40):
        self.vocab, self.seed, self.length = vocab, seed, length

    def tokens(self, start: int, n: int) -> np.ndarray:
        # a counter-based generator: block b of 4096 ids comes from Philox keyed by (seed, b)
        out = np.empty(n, dtype=np.int64)
        done, pos = 0, start
        while done < n:
            block, off = divmod(pos, 4096)
            ids = np.random.Generator(np.random.Philox(key=self.seed, counter=[block, 0, 0, 0])).integers(
                0, self.vocab, 4096, dtype=np.int64)
            take = min(4096 - off, n - done)
            out[done:done + take] = ids[off:off + take]
            done += take
            pos += take
        return out


def sequence_starts(length: int, seq_len: int, seed: int, step: int, global_batch: int) -> np.ndarray:
    """Start positions of the `global_batch` sequences of one step. The stream is cut into (length - 1) // seq_len
    windows of seq_len + 1 ids (inputs and their shifted targets); every epoch visits each window once in an order drawn from (seed, epoch), and a step takes
    the next `global_batch` windows of that order (wrapping into the next epoch's order at the end)."""
    windows = (length - 1) // seq_len   # neighbouring windows share one token: the target of the last position
    if windows < 1:
        raise ValueError(f"the token stream ({length} ids) is shorter than one sequence of {seq_len} + 1")
    first = step * global_batch
    out = np.empty(global_batch, dtype=np.int64)
    filled = 0
    while filled < global_batch:
        epoch, offset = divmod(first + filled, windows)
        order = _epoch_order(windows, seed, epoch)
        take = min(windows - offset, global_batch - filled)
        out[filled:filled + take] = order[offset:offset + take]
        filled += take
    return out * seq_len


_ORDER_CACHE: dict = {}
_ORDER_LOCK = threading.Lock()


def _epoch_order(windows: int, seed: int, epoch: int):
    """The visiting order of one epoch (an index array, or a stride walk for very long streams). Kept for the last few
    (stream, seed, epoch) triples; loaders of several ranks in one process share it from their worker threads."""
    key = (windows, seed, epoch)
    with _ORDER_LOCK:
        order = _ORDER_CACHE.get(key)
    if order is not None:
        return order
    rng = np.random.default_rng([seed, epoch])
    if windows > (1 << 26):
        # a permutation of a very long stream would not fit comfortably: a stride walk that is a bijection instead
        stride = int(rng.integers(windows // 3, windows)) | 1
        while np.gcd(stride, windows) != 1:
            stride += 2
        order = _StrideOrder(windows, stride, int(rng.integers(0, windows)))
    else:
        order = rng.permutation(windows)
    with _ORDER_LOCK:
        if len(_ORDER_CACHE) > 3:
            _ORDER_CACHE.clear()
        _ORDER_CACHE[key] = order
    return order


class _StrideOrder:
    def __init__(self, n, stride, start):
        self.n, self.stride, self.start = n, stride, start

    def __getitem__(self, s: slice) -> np.ndarray:
        idx = np.arange(s.start, s.stop, dtype=np.int64)
        return (self.start + idx * self.stride) % self.n


class BatchLoader:
    """Batches of one data-parallel rank: `next()` returns a pinned int64 tensor [sequences, seq_len + 1] for the next
    step. A worker thread fills a ring of `depth` pinned buffers ahead of the consumer.

    A handed-out buffer goes back to the worker `depth - 1` calls later. A consumer that copies the batch to a GPU
    asynchronously calls `copied()` right after issuing the copy: the loader records an event there and waits for it
    before the buffer is overwritten, so the host may run ahead of the device by `depth - 2` steps and no further."""

    def __init__(self, source: TokenSource, *, seq_len: int, global_batch: int, dp_rank: int = 0, dp_size: int = 1,
                 seed: int = 0, start_step: int = 0, depth: int = 3, pin: bool | None = None, vocab: int | None = None):
        if global_batch % dp_size:
            raise ValueError("the global batch must divide evenly over the data-parallel ranks")
        if depth < 2:
            raise ValueError("the loader needs at least two buffers")
        self.source, self.seq_len, self.global_batch = source, seq_len, global_batch
        self.dp_rank, self.dp_size, self.seed = dp_rank, dp_size, seed
        self.per_rank = global_batch // dp_size
        self.vocab, self.depth = vocab, depth
        pin = torch.cuda.is_available() if pin is None else pin
        self.buffers = [torch.empty((self.per_rank, seq_len + 1), dtype=torch.int64, pin_memory=pin) for _ in range(depth)]
        self.step = start_step
        self._free: queue.Queue = queue.Queue()
        self._ready: queue.Queue = queue.Queue()
        for i in range(depth):
            self._free.put(i)
        self._handed: list = []   # [buffer index, event or None], oldest first
        self._error: BaseException | None = None
        self._thread = threading.Thread(target=self._work, args=(start_step,), name="coccl-batch-loader", daemon=True)
        self._thread.start()

    def fill(self, step: int, out: torch.Tensor) -> None:
        """Write the batch of `step` for this rank into `out` (what the worker does; usable without the thread)."""
        starts = sequence_starts(self.source.length, self.seq_len, self.seed, step, self.global_batch)
        mine = starts[self.dp_rank * self.per_rank:(self.dp_rank + 1) * self.per_rank]
        dst = out.numpy()
        for i, s in enumerate(mine):
            ids = self.source.tokens(int(s), self.seq_len + 1)
            if self.vocab is not None and ids.size and int(ids.max()) >= self.vocab:
                raise ValueError(f"token id {int(ids.max())} near position {int(s)} is outside the model's vocabulary ({self.vocab})")
            dst[i, :] = ids

    def _work(self, step: int):
        try:
            while True:
                i = self._free.get()
                if i is None:
                    return
                self.fill(step, self.buffers[i])
                self._ready.put((step, i))
                step += 1
        except BaseException as e:   # surfaced by next()
            self._error = e
            self._ready.put((None, None))

    def next(self) -> torch.Tensor:
        # keep at most depth - 1 buffers out of the worker's hands, this call's included
        while len(self._handed) >= self.depth - 1:
            i, event = self._handed.pop(0)
            if event is not None:
                event.synchronize()
            self._free.put(i)
        step, i = self._ready.get()
        if step is None:
            raise RuntimeError("the batch loader's worker failed") from self._error
        assert step == self.step
        self._handed.append([i, None])
        self.step += 1
        return self.buffers[i]

    def copied(self) -> None:
        """The consumer has issued its (asynchronous) copy of the batch returned last on the current CUDA stream."""
        if self._handed and torch.cuda.is_available():
            event = torch.cuda.Event()
            event.record()
            self._handed[-1][1] = event

    def close(self):
        self._free.put(None)
        self._thread.join(timeout=5)
