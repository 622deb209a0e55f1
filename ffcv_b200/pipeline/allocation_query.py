"""Buffer requests of operations (reference: ``ffcv/pipeline/allocation_query.py:8-42``):
numpy-typed requests become one pinned host array ``[slots, batch, *shape]``, torch-typed requests
one tensor ``[batch, *shape]`` per slot on the requested device."""
from dataclasses import dataclass
from typing import Optional, Sequence, Tuple, Union

import numpy as np
import torch as ch


@dataclass(frozen=True)
class AllocationQuery:
    shape: Tuple[int, ...]
    dtype: Union[np.dtype, ch.dtype]
    device: Optional[ch.device] = None


Allocation = Union[AllocationQuery, Sequence[AllocationQuery]]


def allocate_query(query: AllocationQuery, batch_size: int, slots: int):
    shape = [int(x) for x in query.shape]
    if isinstance(query.dtype, ch.dtype):
        out = []
        for _ in range(slots):
            t = ch.empty(batch_size, *shape, dtype=query.dtype, device=query.device)
            if t.device.type == 'cpu' and ch.cuda.is_available():
                t = t.pin_memory()
            out.append(t)
        return out
    ch_dtype = ch.from_numpy(np.empty(0, dtype=query.dtype)).dtype
    t = ch.empty(slots, batch_size, *shape, dtype=ch_dtype)
    if ch.cuda.is_available():
        t = t.pin_memory()
    return t.numpy()
