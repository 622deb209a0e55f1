"""On-disk layout of a ``.beton`` file, version 2 (reference: ``ffcv/types.py:22-77``).

All integers little-endian.  Header (24 B), ``num_fields`` field descriptors (1041 B each),
the per-sample metadata table, page-aligned data pages, then the allocation table to EOF.
"""
import numpy as np

CURRENT_VERSION = 2

HeaderType = np.dtype([('version', '<u2'), ('num_fields', '<u2'), ('page_size', '<u4'),
                       ('num_samples', '<u8'), ('alloc_table_ptr', '<u8')], align=True)

ALLOC_TABLE_TYPE = np.dtype([('sample_id', '<u8'), ('ptr', '<u8'), ('size', '<u8')])

FieldDescType = np.dtype([('type_id', '<u1'), ('name', ('<u1', 16)), ('arguments', ('<u1', (1024,)))],
                         align=True)

ARG_TYPE = np.dtype([('', '<u1', 1024)])


def type_id_table():
    from .fields import FloatField, IntField, NDArrayField, RGBImageField, TorchTensorField
    return {0: FloatField, 1: IntField, 2: RGBImageField, 4: NDArrayField, 6: TorchTensorField, 255: None}


def get_metadata_type(handlers):
    return np.dtype([('', h.metadata_type) for h in handlers], align=True)
