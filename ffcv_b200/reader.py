"""Parser of the ``.beton`` header, field descriptors, metadata and allocation table
(reference: ``ffcv/reader.py:7-70``)."""
import numpy as np

from .types import (ALLOC_TABLE_TYPE, CURRENT_VERSION, FieldDescType, HeaderType, get_metadata_type,
                    type_id_table)


def _cstring(raw):
    return raw.tobytes().decode('ascii').split('\x00')[0]


class Reader:
    def __init__(self, fname, custom_handlers=None):
        self._fname = fname
        custom_handlers = custom_handlers or {}
        header = np.fromfile(fname, dtype=HeaderType, count=1)[0]
        if header['version'] != CURRENT_VERSION:
            raise AssertionError(f"file format mismatch: code={CURRENT_VERSION},file={header['version']}")
        self.header = header
        self.num_samples = int(header['num_samples'])
        self.page_size = int(header['page_size'])
        self.num_fields = int(header['num_fields'])

        descs = np.fromfile(fname, dtype=FieldDescType, count=self.num_fields, offset=HeaderType.itemsize)
        self.field_descriptors = descs
        self.field_names = [_cstring(d['name']) for d in descs]
        table = type_id_table()
        self.handlers = {}
        for name, d in zip(self.field_names, descs):
            if name in custom_handlers:
                self.handlers[name] = custom_handlers[name].from_binary(d['arguments'])
                continue
            cls = table.get(int(d['type_id']))
            if cls is None:
                raise ValueError(f"Must specify a custom_field entry for custom field {name}")
            self.handlers[name] = cls.from_binary(d['arguments'])
        self.metadata_type = get_metadata_type(list(self.handlers.values()))

        offset = HeaderType.itemsize + descs.nbytes
        self.metadata = np.fromfile(fname, dtype=self.metadata_type, count=self.num_samples, offset=offset)
        self.metadata.setflags(write=False)
        self.alloc_table = np.fromfile(fname, dtype=ALLOC_TABLE_TYPE, offset=int(header['alloc_table_ptr']))
        self.alloc_table.setflags(write=False)

    @property
    def file_name(self):
        return self._fname
