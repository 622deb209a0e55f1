"""Storage access for the loader (reference: ``ffcv/memory_managers/base.py:32-80`` and
``os_cache.py``): the whole ``.beton`` file is memory-mapped and the operating system's page
cache keeps it in RAM.  The native staging threads read sample bytes straight from the mapping,
so beyond the reference's ``read(address, state)`` this manager exposes the mapping's base
address and a vectorised size lookup."""
from collections import defaultdict

import numpy as np


class MemoryContext:
    def __init__(self, manager):
        self.manager = manager

    @property
    def state(self):
        m = self.manager
        return (m.mmap, m.ptrs, m.sizes)

    def __enter__(self):
        self.manager.open()
        return self

    def start_batch(self, batch: int):
        pass

    def __exit__(self, *exc):
        return False


class MemoryManager:
    def __init__(self, reader):
        self.reader = reader
        table = reader.alloc_table
        order = np.argsort(table['ptr'])
        self.ptrs = np.ascontiguousarray(table['ptr'][order])
        self.sizes = np.ascontiguousarray(table['size'][order])
        shift = int(np.log2(reader.page_size))
        pages = table['ptr'] >> np.uint64(shift)
        self.page_to_samples = defaultdict(set)
        self.sample_to_pages = defaultdict(set)
        for sid, pid in zip(table['sample_id'].tolist(), pages.tolist()):
            self.page_to_samples[pid].add(sid)
            self.sample_to_pages[sid].add(pid)

    def sizes_of(self, data_ptrs):
        """Payload size of every address in ``data_ptrs`` (the allocation-table entry with that
        pointer, as ``read`` looks it up per sample in the reference)."""
        return np.ascontiguousarray(self.sizes[np.searchsorted(self.ptrs, data_ptrs)])


class OSCacheManager(MemoryManager):
    """``pin=False``: the file is memory-mapped (page cache) and the native staging threads copy
    each batch's bytes into pinned buffers.  ``pin=True``: the whole file is read once into
    page-locked host memory; the native library notices that its source is pinned and lets the GPU
    gather every batch's payloads over PCIe itself, so no CPU core touches sample bytes."""

    def __init__(self, reader, pin=False):
        super().__init__(reader)
        self.mmap = None
        self.pin = bool(pin)
        self.pinned = False
        self._keepalive = None
        self.context = MemoryContext(self)

    def open(self):
        if self.mmap is None:
            if self.pin:
                try:
                    self.mmap = self._read_pinned()
                    self.pinned = True
                except Exception as exc:  # not enough lockable memory, no CUDA: keep the staged path
                    print(f'ffcv_b200: could not pin {self.reader.file_name} ({exc}); using the page cache')
                    self.pin = False
            if self.mmap is None:
                self.mmap = np.memmap(self.reader.file_name, 'uint8', mode='r')
        return self.mmap

    def _read_pinned(self):
        import os
        import torch as ch
        size = os.path.getsize(self.reader.file_name)
        buf = ch.empty(size, dtype=ch.uint8, pin_memory=True)
        view = buf.numpy()
        with open(self.reader.file_name, 'rb', buffering=0) as fp:
            done = 0
            mv = memoryview(view)
            while done < size:
                got = fp.readinto(mv[done:done + (64 << 20)])
                if not got:
                    raise IOError('short read')
                done += got
        self._keepalive = buf
        return view

    def file_base(self):
        return self.open().ctypes.data

    def schedule_epoch(self, batches):
        return self.context

    def compile_reader(self):
        def read(address, mem_state):
            size = mem_state[2][np.searchsorted(mem_state[1], address)]
            return mem_state[0][int(address):int(address) + int(size)]
        return read
