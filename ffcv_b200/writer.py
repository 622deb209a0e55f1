"""Writer of ``.beton`` files (reference: ``ffcv/writer.py``, ``ffcv/memory_allocator.py``).

Offline tool, outside the accelerated path; it exists so that datasets can be produced without
the reference installed.  Same file format: header, field descriptors, metadata table, data pages
(a sample's payload never straddles a page), allocation table.  Samples are encoded by a pool of
worker processes in chunks; pages are laid out by the parent in sample order, so the file is
deterministic for a given dataset.
"""
import multiprocessing as mp
from typing import Mapping

import numpy as np

from .fields.base import Field
from .types import (ALLOC_TABLE_TYPE, CURRENT_VERSION, FieldDescType, HeaderType, get_metadata_type)

MIN_PAGE_SIZE = 1 << 21
MAX_PAGE_SIZE = 1 << 32


def _type_id(field):
    from .types import type_id_table
    for tid, cls in type_id_table().items():
        if cls is not None and type(field) is cls:
            return tid
    for tid, cls in type_id_table().items():
        if cls is not None and isinstance(field, cls):
            return tid
    return 255


def _encode_chunk(args):
    dataset, fields, lo, hi = args
    mtype = get_metadata_type(list(fields.values()))
    meta = np.zeros(hi - lo, dtype=mtype)
    blobs = []
    for k, ix in enumerate(range(lo, hi)):
        sample = dataset[ix]
        if len(sample) != len(fields):
            raise ValueError(f"sample {ix} has {len(sample)} values for {len(fields)} fields")
        for f_ix, (field, value) in enumerate(zip(fields.values(), sample)):
            def malloc(size, _k=k, _f=f_ix):
                storage = np.zeros(int(size), dtype='<u1')
                blobs.append((_k, _f, storage))
                return 0, storage
            field.encode(meta[k:k + 1][f'f{f_ix}'], value, malloc)
    return lo, meta, blobs


class DatasetWriter:
    """Writes an indexed dataset (``__len__`` / ``__getitem__`` returning one value per field).

    Parameters
    ----------
    fname : str
        Output file.
    fields : Mapping[str, Field]
        Name and type of every field, in sample order.
    page_size : int
        Page size in bytes (power of two, default 8 MiB as the reference).
    num_workers : int
        Worker processes (< 1: one per core).
    """

    def __init__(self, fname: str, fields: Mapping[str, Field], page_size: int = 4 * MIN_PAGE_SIZE,
                 num_workers: int = -1, indices=None):
        if page_size & (page_size - 1) or not (MIN_PAGE_SIZE <= page_size <= MAX_PAGE_SIZE):
            raise ValueError(f'page_size has to be a power of two in [{MIN_PAGE_SIZE}, {MAX_PAGE_SIZE}]')
        self.fname = fname
        self.fields = dict(fields)
        self.page_size = page_size
        self.num_workers = num_workers if num_workers >= 1 else mp.cpu_count()
        self.indices = indices
        for name in self.fields:
            if len(name.encode('ascii')) > 16:
                raise ValueError(f"Field name '{name}' longer than 16 bytes")

    def from_indexed_dataset(self, dataset, indices=None, chunksize=64, shuffle_indices=False):
        if indices is None:
            indices = self.indices
        n_total = len(dataset)
        if indices is not None:
            dataset = _Subset(dataset, list(indices))
        n = len(dataset)
        del n_total
        fields = self.fields
        mtype = get_metadata_type(list(fields.values()))
        header_bytes = HeaderType.itemsize + FieldDescType.itemsize * len(fields) + mtype.itemsize * n
        data_start = (header_bytes + self.page_size - 1) // self.page_size * self.page_size
        metadata = np.zeros(n, dtype=mtype)
        allocs = []
        chunks = [(dataset, fields, lo, min(lo + chunksize, n)) for lo in range(0, n, chunksize)]
        with open(self.fname, 'wb') as fp:
            fp.write(np.zeros(data_start, dtype='<u1').tobytes())
            page = np.zeros(self.page_size, dtype='<u1')
            page_ix, page_off = 0, 0

            def flush():
                nonlocal page_ix, page_off
                if page_off:
                    fp.seek(data_start + page_ix * self.page_size)
                    fp.write(page.tobytes())
                    page[:] = 0
                    page_ix += 1
                    page_off = 0

            def consume(result):
                nonlocal page_off
                lo, meta, blobs = result
                metadata[lo:lo + len(meta)] = meta
                for k, f_ix, storage in blobs:
                    size = storage.size
                    if size > self.page_size:
                        raise ValueError(f"Tried allocating {size} but page size is {self.page_size}")
                    if size > self.page_size - page_off:
                        flush()
                    ptr = data_start + page_ix * self.page_size + page_off
                    page[page_off:page_off + size] = storage
                    page_off += size
                    column = metadata[f'f{f_ix}']
                    if column.dtype.names:  # image fields keep the pointer beside mode and size
                        column['data_ptr'][lo + k] = ptr
                    else:                   # array fields: the pointer is the whole entry
                        column[lo + k] = ptr
                    allocs.append((lo + k, ptr, size))

            if self.num_workers > 1 and len(chunks) > 1:
                with mp.get_context('fork').Pool(self.num_workers) as pool:
                    for result in pool.imap(_encode_chunk, chunks):
                        consume(result)
            else:
                for c in chunks:
                    consume(_encode_chunk(c))
            flush()
            alloc_ptr = data_start + page_ix * self.page_size
            table = np.array(allocs, dtype=ALLOC_TABLE_TYPE) if allocs else np.zeros(0, dtype=ALLOC_TABLE_TYPE)
            fp.seek(alloc_ptr)
            fp.write(table.tobytes())
            header = np.zeros(1, dtype=HeaderType)[0]
            header['version'] = CURRENT_VERSION
            header['num_fields'] = len(fields)
            header['page_size'] = self.page_size
            header['num_samples'] = n
            header['alloc_table_ptr'] = alloc_ptr
            descs = np.zeros(len(fields), dtype=FieldDescType)
            for i, (name, field) in enumerate(fields.items()):
                descs[i]['type_id'] = _type_id(field)
                raw = name.encode('ascii')
                descs[i]['name'][:len(raw)] = np.frombuffer(raw, dtype='<u1')
                descs[i]['arguments'][:] = np.frombuffer(np.asarray(field.to_binary()).tobytes(), dtype='<u1')
            fp.seek(0)
            fp.write(header.tobytes())
            fp.write(descs.tobytes())
            fp.write(metadata.tobytes())


class _Subset:
    def __init__(self, dataset, indices):
        self.dataset, self.indices = dataset, indices

    def __len__(self):
        return len(self.indices)

    def __getitem__(self, i):
        return self.dataset[self.indices[i]]
