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
    gather every batch's payloads over PCIe itself, so no CPU core touches sample bytes.
    ``pin='auto'``: a file on a memory file system is page-locked where it lies (one copy for
    the node, nothing extra is allocated); any other file gets a private page-locked copy only
    if the copies of all ranks of this host (``LOCAL_WORLD_SIZE``) together fit half of the
    memory that is available now -- page-locked memory cannot be swapped, and eight ranks
    copying a 40 GB file would lock 320 GB -- and is staged from the page cache otherwise."""

    def __init__(self, reader, pin=False):
        super().__init__(reader)
        self.mmap = None
        self.auto = pin == 'auto'
        self.pin = bool(pin)
        self.pinned = False
        self._keepalive = None
        self.context = MemoryContext(self)

    def open(self):
        if self.mmap is None:
            if self.pin:
                try:
                    self.mmap = self._register_shared()
                    if self.mmap is None and (not self.auto or self._private_copy_fits()):
                        self.mmap = self._read_pinned()
                    self.pinned = self.mmap is not None
                    self.pin = self.pinned
                except Exception as exc:  # not enough lockable memory, no CUDA: keep the staged path
                    print(f'ffcv_b200: could not pin {self.reader.file_name} ({exc}); using the page cache')
                    self.pin = False
            if self.mmap is None:
                self.mmap = np.memmap(self.reader.file_name, 'uint8', mode='r')
        return self.mmap

    def _private_copy_fits(self):
        import os
        ranks = max(1, int(os.environ.get('LOCAL_WORLD_SIZE', '1')))
        size = os.path.getsize(self.reader.file_name)
        if size > float(os.environ.get('FFCV_B200_PIN_LIMIT_GB', '64')) * (1 << 30):
            return False
        need = size * ranks
        try:
            with open('/proc/meminfo') as fp:
                avail = next(int(ln.split()[1]) * 1024 for ln in fp if ln.startswith('MemAvailable:'))
        except (OSError, StopIteration, ValueError):
            return False
        return need <= avail // 2

    def _register_shared(self):
        """Page-locks the file's own pages in place: a shared, writable mapping of a file on a
        memory file system (``/dev/shm``) can be registered with the CUDA driver, which makes the
        page cache itself the pinned copy -- nothing is read at start-up and every process of the
        node shares the one copy.  The driver only accepts a writable mapping, so the dataset file
        is opened read-write (a file this user cannot write is not registered); this code never
        stores through the mapping and hands out a read-only array.  (Read-only mappings and files on disk are refused by the
        driver; then the caller falls back to a private pinned copy.)  Nothing is ever written
        through the mapping.  Returns None when the file cannot be registered."""
        import mmap
        import os
        from .. import libffcv as L
        try:
            fd = os.open(self.reader.file_name, os.O_RDWR)
        except OSError:
            return None
        try:
            mm = mmap.mmap(fd, 0, flags=mmap.MAP_SHARED, prot=mmap.PROT_READ | mmap.PROT_WRITE)
        except (OSError, ValueError):
            os.close(fd)
            return None
        os.close(fd)
        view = np.frombuffer(mm, dtype=np.uint8)
        if not L.host_register(view.ctypes.data, view.size):
            del view
            mm.close()
            return None
        self._registered = (view.ctypes.data, mm)
        view.flags.writeable = False
        return view

    def close(self):
        """Releases the page lock taken by `_register_shared` (the mapping itself lives as long as
        arrays that view it)."""
        reg = getattr(self, '_registered', None)
        if reg is not None:
            from .. import libffcv as L
            L.host_unregister(reg[0])
            self._registered = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

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
