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
    def __init__(self, reader):
        super().__init__(reader)
        self.mmap = None
        self.context = MemoryContext(self)

    def open(self):
        if self.mmap is None:
            self.mmap = np.memmap(self.reader.file_name, 'uint8', mode='r')
        return self.mmap

    def file_base(self):
        return self.open().ctypes.data

    def schedule_epoch(self, batches):
        return self.context

    def compile_reader(self):
        def read(address, mem_state):
            size = mem_state[2][np.searchsorted(mem_state[1], address)]
            return mem_state[0][int(address):int(address) + int(size)]
        return read
