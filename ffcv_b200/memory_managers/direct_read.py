"""Storage access for files larger than RAM (``Loader(os_cache=False)``).

Role of the reference's ``ProcessCacheManager`` (``ffcv/memory_managers/process_cache/``): it knows
the epoch's batches in advance, has reader threads load the 8 MiB pages a batch needs into a ring
of page slots a few batches ahead of the pipeline (``schedule.py:24-131``, ``page_reader.py:9-40``)
and the decoders copy the samples out of those slots.  Here the ring is the loader's own slot ring
of pinned staging buffers and the schedule is the loader's batch order: for batch ``b`` the native
staging threads ``pread`` every sample (for a raw image: the rows its crop touches) straight into
slot ``b mod slots`` while the GPU works on the batches before it, so a byte crosses host memory
once -- from the device that holds the file into the buffer the DMA engine reads -- and, with
``O_DIRECT``, never enters the page cache.  The file is not mapped; resident memory is the slot ring.
"""
import os
from collections import namedtuple

import numpy as np

from .os_cache import MemoryContext, MemoryManager

FileDescriptors = namedtuple('FileDescriptors', ['fd', 'fd_direct'])


class DirectReadContext(MemoryContext):
    @property
    def state(self):
        m = self.manager
        return (m.open(), m.ptrs, m.sizes)


class DirectReadManager(MemoryManager):
    """``direct_io``: try ``O_DIRECT`` (refused by some file systems, e.g. tmpfs before Linux 6.6:
    then reads are buffered and the pages they bring in are dropped again right after)."""

    direct = True
    pinned = False
    pin = False

    def __init__(self, reader, direct_io=True):
        super().__init__(reader)
        self.direct_io = bool(direct_io)
        self.fds = None
        self.context = DirectReadContext(self)

    def open(self):
        if self.fds is None:
            fd = os.open(self.reader.file_name, os.O_RDONLY)
            fd_direct = -1
            if self.direct_io and hasattr(os, 'O_DIRECT'):
                try:
                    fd_direct = os.open(self.reader.file_name, os.O_RDONLY | os.O_DIRECT)
                except OSError:
                    fd_direct = -1
            # the access pattern is the batch schedule: no sequential read-ahead heuristics
            os.posix_fadvise(fd, 0, 0, os.POSIX_FADV_RANDOM)
            self.fds = FileDescriptors(fd, fd_direct)
        return self.fds

    def file_base(self):
        return self.open()

    def schedule_epoch(self, batches):
        return self.context

    def compile_reader(self):
        def read(address, mem_state):
            fds, ptrs, sizes = mem_state
            size = int(sizes[np.searchsorted(ptrs, address)])
            return np.frombuffer(os.pread(fds.fd, size, int(address)), dtype=np.uint8)
        return read

    def close(self):
        if self.fds is not None:
            for fd in self.fds:
                if fd >= 0:
                    os.close(fd)
            self.fds = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
