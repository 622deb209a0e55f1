"""Storage access for files larger than RAM (``Loader(os_cache=False)``).

Role of the reference's ``ProcessCacheManager`` (``ffcv/memory_managers/process_cache/``): it knows
the epoch's batches in advance, loads the 8 MiB pages a batch needs into a ring of page slots a few
batches ahead of the pipeline and recycles a slot when the last batch that needs it is done
(``schedule.py:24-131``, ``page_reader.py``).  Here the file stays memory-mapped -- the native
staging threads read sample bytes from the mapping as with the OS cache -- and the schedule drives
the kernel's read-ahead instead of a private page ring: a helper thread asks for the byte ranges of
the next batches (``posix_fadvise(WILLNEED)``, which queues the reads without blocking) and hands
the ranges of finished batches back (``DONTNEED``), so resident memory stays bounded by the
window and no batch waits on a cold page.
"""
import os
import threading
from queue import Queue

import numpy as np

from .os_cache import MemoryContext, MemoryManager

PAGE = 4096


def merge_ranges(starts, sizes, gap=64 * 1024):
    """Byte ranges [start, start + size) rounded out to 4 KiB pages, sorted, with ranges closer than
    ``gap`` bytes merged (a batch in quasi-random order sits in a few long runs)."""
    lo = (np.asarray(starts, dtype=np.int64) // PAGE) * PAGE
    hi = ((np.asarray(starts, dtype=np.int64) + np.asarray(sizes, dtype=np.int64) + PAGE - 1) // PAGE) * PAGE
    order = np.argsort(lo, kind='stable')
    out = []
    for a, b in zip(lo[order].tolist(), hi[order].tolist()):
        if out and a <= out[-1][1] + gap:
            out[-1][1] = max(out[-1][1], b)
        else:
            out.append([a, b])
    return [(a, b - a) for a, b in out]


class ReadAheadContext(MemoryContext):
    def __init__(self, manager, batches):
        super().__init__(manager)
        self.batches = batches
        self.requested = 0          # batches whose ranges have been asked for
        self.queue = Queue()
        self.thread = None

    def ranges_of(self, b_ix):
        m = self.manager
        ptrs = m.sample_ptrs[np.asarray(self.batches[b_ix])]
        return merge_ranges(ptrs.ravel(), m.sizes_of(ptrs.ravel()))

    def __enter__(self):
        self.manager.open()
        self.thread = threading.Thread(target=self._work, daemon=True)
        self.thread.start()
        self._request_up_to(self.manager.window)
        return self

    def _request_up_to(self, limit):
        limit = min(limit, len(self.batches))
        while self.requested < limit:
            self.queue.put(('want', self.requested))
            self.requested += 1

    def start_batch(self, batch: int):
        # batch `batch` starts: everything up to `window` batches ahead should be on its way, and
        # the batch that left the pipeline's slot ring can go
        self._request_up_to(batch + 1 + self.manager.window)
        done = batch - self.manager.keep
        if done >= 0:
            self.queue.put(('drop', done))

    def _work(self):
        fd, advise = self.manager.fd, self.manager.advise
        while True:
            item = self.queue.get()
            if item is None:
                return
            kind, b_ix = item
            flag = os.POSIX_FADV_WILLNEED if kind == 'want' else os.POSIX_FADV_DONTNEED
            for start, length in self.ranges_of(b_ix):
                advise(fd, start, length, flag)

    def __exit__(self, *exc):
        if self.thread is not None:
            self.queue.put(None)
            self.thread.join()
            self.thread = None
        return False


class ReadAheadManager(MemoryManager):
    """Memory-mapped file plus schedule-driven read-ahead.  ``window``: batches requested ahead of
    the one being staged; ``keep``: batches behind it whose pages are still held (the loader's slot
    ring may still be copying from them)."""

    def __init__(self, reader, sample_ptrs, window=8, keep=6, advise=None):
        super().__init__(reader)
        self.sample_ptrs = np.asarray(sample_ptrs)   # [num_samples, k] file offsets of each sample's payloads
        self.window, self.keep = int(window), int(keep)
        self.mmap = None
        self.fd = None
        self.pinned = False
        self.pin = False
        self.advise = advise if advise is not None else os.posix_fadvise

    def open(self):
        if self.mmap is None:
            self.fd = os.open(self.reader.file_name, os.O_RDONLY)
            # the access pattern is scheduled explicitly: no sequential read-ahead heuristics
            self.advise(self.fd, 0, 0, os.POSIX_FADV_RANDOM)
            self.mmap = np.memmap(self.reader.file_name, 'uint8', mode='r')
        return self.mmap

    def file_base(self):
        return self.open().ctypes.data

    def schedule_epoch(self, batches):
        return ReadAheadContext(self, batches)

    def compile_reader(self):
        def read(address, mem_state):
            size = mem_state[2][np.searchsorted(mem_state[1], address)]
            return mem_state[0][address:address + size]
        return read

    def close(self):
        if self.fd is not None:
            os.close(self.fd)
            self.fd = None
        self.mmap = None
