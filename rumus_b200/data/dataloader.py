"""DataLoader: batching, shuffling, ``drop_last``, worker threads with bounded prefetch and
pinned host staging (rumus/src/data/dataloader.rs:16-274).

As in the reference, an epoch iterator feeds batch index lists to worker threads through a
bounded queue and collects finished batches from another; tearing the iterator down early cannot
dead-lock (workers poll a stop flag; queues are drained).  Shuffling uses the reference's
Fisher-Yates over a 64-bit LCG seeded with ``0xDEADBEEFCAFE1234`` (dataloader.rs:254-274).
Batches can be returned in pinned memory so the H2D copy is asynchronous.
"""
from __future__ import annotations

import queue
import threading
from typing import Iterator, List, Optional

import torch

from .dataset import DataItem, Dataset

_MASK = (1 << 64) - 1


class _Lcg:
    def __init__(self, seed=0xDEADBEEFCAFE1234):
        self.s = seed

    def next(self) -> int:
        self.s = (self.s * 6364136223846793005 + 1442695040888963407) & _MASK
        return self.s


_shuffle_rng = _Lcg()


def fisher_yates_shuffle(indices: List[int], rng: Optional[_Lcg] = None) -> None:
    rng = rng or _shuffle_rng
    for i in range(len(indices) - 1, 0, -1):
        j = rng.next() % (i + 1)
        indices[i], indices[j] = indices[j], indices[i]


def collate(items: List[DataItem], pin: bool = False) -> DataItem:
    """Stack inputs and targets along a new leading dimension (dataloader.rs:237-245)."""
    x = torch.stack([it.input for it in items])
    y = torch.stack([it.target for it in items])
    if pin and torch.cuda.is_available():
        x, y = x.pin_memory(), y.pin_memory()
    return DataItem(x, y)


class DataLoader:
    def __init__(self, dataset: Dataset, batch_size: int, shuffle: bool = False, drop_last: bool = False,
                 num_workers: int = 0, prefetch_factor: int = 2, pin_memory: bool = False):
        assert batch_size > 0 and prefetch_factor > 0
        self.dataset, self.batch_size, self.shuffle = dataset, batch_size, shuffle
        self.drop_last, self.num_workers, self.prefetch_factor = drop_last, num_workers, prefetch_factor
        self.pin_memory = pin_memory

    def __len__(self) -> int:
        n = len(self.dataset)
        return n // self.batch_size if self.drop_last else (n + self.batch_size - 1) // self.batch_size

    def _batches(self) -> List[List[int]]:
        idx = list(range(len(self.dataset)))
        if self.shuffle:
            fisher_yates_shuffle(idx)
        out = [idx[i:i + self.batch_size] for i in range(0, len(idx), self.batch_size)]
        if self.drop_last and out and len(out[-1]) < self.batch_size:
            out.pop()
        return out

    def iter(self) -> Iterator[DataItem]:
        return iter(self)

    def __iter__(self) -> Iterator[DataItem]:
        batches = self._batches()
        if self.num_workers == 0:
            for b in batches:
                yield collate([self.dataset.get(i) for i in b], self.pin_memory)
            return
        yield from _ThreadedIter(self, batches)


class _ThreadedIter:
    def __init__(self, loader: DataLoader, batches: List[List[int]]):
        self.loader, self.batches = loader, batches
        cap = loader.prefetch_factor * loader.num_workers
        self.todo: "queue.Queue" = queue.Queue()
        self.done: "queue.Queue" = queue.Queue(maxsize=cap)
        self.stop = threading.Event()
        for i, b in enumerate(batches):
            self.todo.put((i, b))
        self.threads = [threading.Thread(target=self._work, daemon=True) for _ in range(loader.num_workers)]
        for t in self.threads:
            t.start()

    def _work(self):
        while not self.stop.is_set():
            try:
                i, b = self.todo.get_nowait()
            except queue.Empty:
                return
            try:
                item = collate([self.loader.dataset.get(j) for j in b], self.loader.pin_memory)
            except Exception as e:  # noqa: BLE001 - surfaced to the consumer
                item = e
            while not self.stop.is_set():
                try:
                    self.done.put((i, item), timeout=0.05)
                    break
                except queue.Full:
                    continue

    def __iter__(self):
        pending, nxt = {}, 0
        try:
            while nxt < len(self.batches):
                while nxt not in pending:
                    i, item = self.done.get()
                    pending[i] = item
                item = pending.pop(nxt)
                nxt += 1
                if isinstance(item, Exception):
                    raise item
                yield item            # batches come out in order even though workers race
        finally:
            self.stop.set()
            while True:
                try:
                    self.done.get_nowait()
                except queue.Empty:
                    break
            for t in self.threads:
                t.join(timeout=1.0)
