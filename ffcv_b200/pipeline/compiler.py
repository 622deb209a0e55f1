"""numba front-end (reference: ``ffcv/pipeline/compiler.py:9-42``).  Pixels never pass through
numba here; it compiles the per-batch random-parameter samplers so that they draw from numba's
``np.random`` stream exactly as the reference's augmentations do."""
from os import sched_getaffinity

import torch as ch
from numba import njit, set_num_threads


class Compiler:
    is_enabled = True
    num_threads = 1

    @classmethod
    def set_enabled(cls, b):
        cls.is_enabled = b

    @classmethod
    def set_num_threads(cls, n):
        if n < 1:
            n = len(sched_getaffinity(0))
        cls.num_threads = n
        try:
            set_num_threads(n)
        except ValueError:
            pass
        ch.set_num_threads(n)

    @classmethod
    def compile(cls, code, signature=None):
        if cls.is_enabled:
            return njit(signature, fastmath=True, nogil=True, error_model='numpy')(code)
        return code

    @classmethod
    def get_iterator(cls):
        return range
