"""Pipeline graph: turns the user's ``pipelines`` mapping into per-batch executables.

Role of ``ffcv/pipeline/graph.py`` in the reference (requirement collection, memory allocation,
staging of the operations), without its numba code generation: stage 0 of the reference (the
jitted CPU loops) does not exist here.  For an image field the longest fusable prefix of the
pipeline becomes one native GPU call (:mod:`ffcv_b200.pipeline.fusion`); every other operation
runs through the closure its ``generate_code`` returns, with the reference's call signatures.
"""
import threading
from typing import Dict

import numpy as np
import torch as ch

from .. import libffcv as L
from ..fields.basics import FloatDecoder, IntDecoder
from ..fields.ndarray import NDArrayDecoder
from ..fields.rgb_image import SimpleRGBImageDecoder
from .allocation_query import AllocationQuery, allocate_query
from .fusion import FusedImageExecutor, FusedImagePlan
from .pipeline_spec import PipelineSpec
from .state import State

INITIAL_STATE = State(jit_mode=True, device=ch.device('cpu'), dtype=np.dtype('u1'), shape=None)

_shared = {}
_shared_lock = threading.Lock()


def shared_context(device) -> L.Context:
    """Process-wide native context of a device, for operations used outside a fused plan."""
    device = ch.device(device)
    index = device.index if device.index is not None else ch.cuda.current_device()
    with _shared_lock:
        if index not in _shared:
            _shared[index] = L.Context(index, n_slots=1, n_threads=0)
        return _shared[index]


def standalone_decoder(op):
    """Closure with the reference's decoder signature
    ``decode(batch_indices, destination, metadata, storage_state)`` that decodes synchronously on
    the GPU into ``destination`` (a uint8 CUDA tensor)."""
    state = {}

    def decode(batch_indices, destination, metadata, storage_state):
        mmap, ptrs, sizes = storage_state
        if 'exe' not in state:
            plan = FusedImagePlan()
            op.fuse(plan)
            plan.device = destination.device
            sample_sizes = sizes[np.searchsorted(ptrs, metadata['data_ptr'])]
            state['exe'] = FusedImageExecutor(plan, shared_context(destination.device), metadata, sample_sizes,
                                              (lambda: mmap) if isinstance(mmap, tuple) else (lambda: mmap.ctypes.data),
                                              np.random.randint(0, 2 ** 31 - 1))
            state['calls'] = 0
        state['calls'] += 1
        stream = ch.cuda.current_stream(destination.device)
        out = state['exe'](np.asarray(batch_indices), 0, stream.cuda_stream, destination, 0, state['calls'])
        stream.synchronize()
        return out
    return decode


class _Pipeline:
    def __init__(self, name, source, f_ix, ops):
        self.name, self.source, self.f_ix, self.ops = name, source, f_ix, ops
        self.allocs = []
        self.executor = None  # FusedImageExecutor for the fused prefix
        self.n_fused = 0
        self.codes = []
        self.final_state = None
        self.rider_host = None  # index of the image pipeline whose staged bytes carry this field


class Graph:
    def __init__(self, pipeline_specs: Dict[str, PipelineSpec], handlers, fieldname_to_fix, metadata,
                 memory_manager, context_factory, seed):
        self.handlers = handlers
        self.metadata = metadata
        self.memory_manager = memory_manager
        self.memory_read = memory_manager.compile_reader()
        self.context_factory = context_factory
        self.seed = seed
        self.pipelines = []
        for output_name, spec in pipeline_specs.items():
            if not isinstance(spec.source, str):
                raise NotImplementedError("pipelines whose source is another operation are not supported")
            if spec.source not in handlers:
                raise ValueError(f"Field {output_name} has no source")
            field = handlers[spec.source]
            spec.accept_decoder(field.get_decoder_class(), output_name)
            assert spec.decoder is not None
            self.pipelines.append(_Pipeline(output_name, spec.source, fieldname_to_fix[spec.source],
                                            [spec.decoder] + list(spec.transforms)))
        self.collect_requirements()

    def collect_requirements(self):
        """Walks every pipeline root to leaf: ``accept_field``, ``accept_globals``,
        ``declare_state_and_memory`` (cf. ffcv/pipeline/graph.py:295-354), then fuses."""
        for pi, p in enumerate(self.pipelines):
            field = self.handlers[p.source]
            column = self.metadata[f'f{p.f_ix}']
            state = INITIAL_STATE
            p.allocs = []
            for op in p.ops:
                op.accept_field(field)
                op.accept_globals(column, self.memory_read)
                state, alloc = op.declare_state_and_memory(state)
                p.allocs.append(alloc)
            p.final_state = state
            p.n_fused = 0
            p.executor = None
            if isinstance(p.ops[0], SimpleRGBImageDecoder):
                plan = FusedImagePlan()
                k = 0
                while k < len(p.ops) and p.ops[k].fuse(plan):
                    plan.fused_ops.append(p.ops[k])
                    k += 1
                if k == 0:
                    raise RuntimeError("image decoder refused to open a GPU plan")
                p.n_fused = k
                mm = self.memory_manager
                p.executor = FusedImageExecutor(plan, self.context_factory(plan.device, pi), column,
                                                mm.sizes_of(column['data_ptr']), mm.file_base, self.seed)
        self.attach_riders()
        for p in self.pipelines:
            p.codes = [op.generate_code() for op in p.ops[p.n_fused:]]
        return self.pipelines

    def attach_riders(self):
        """A scalar or fixed-shape array field whose pipeline opens with ``decoder -> ToTensor ->
        ToDevice(gpu)`` does not get a host buffer and a copy of its own
        (ffcv/fields/basics.py:28-34, ffcv/fields/ndarray.py:37-43, ffcv/transforms/ops.py:50-57):
        its values ride in the staged bytes of an image pipeline decoded on that GPU and arrive
        with the same host->device transfer.  The rest of its pipeline runs unchanged on the
        device tensor."""
        from ..transforms.ops import ToDevice, ToTensor
        hosts = {}
        for pi, p in enumerate(self.pipelines):
            if p.executor is not None:
                hosts.setdefault(p.executor.device, []).append(pi)
        for p in self.pipelines:
            p.rider_host = None
        if not hosts:
            return
        load = {pi: 0 for pis in hosts.values() for pi in pis}
        for p in self.pipelines:
            p.rider_host = None
            if p.executor is not None or len(p.ops) < 3:
                continue
            dec, to_tensor, to_device = p.ops[:3]
            if type(dec) not in (IntDecoder, FloatDecoder, NDArrayDecoder) or type(to_tensor) is not ToTensor \
                    or type(to_device) is not ToDevice or to_device.device.type != 'cuda':
                continue
            dev = to_device.device
            if dev.index is None:
                dev = ch.device('cuda', ch.cuda.current_device())
            cands = [pi for pi in hosts.get(dev, []) if load[pi] < L.MAX_RIDERS]
            if not cands:
                continue
            p.rider_host = cands[0]
            load[cands[0]] += 1
            p.n_fused = 3

    def allocate_memory(self, batch_size, slots):
        buffers = {}
        for pi, p in enumerate(self.pipelines):
            if p.executor is not None:
                buffers[(pi, 'fused')] = p.executor.allocate(batch_size, slots)
            if p.rider_host is not None:
                buffers[(pi, 'rider')] = allocate_query(p.allocs[2], batch_size, slots)
            for k in range(p.n_fused, len(p.ops)):
                alloc = p.allocs[k]
                if isinstance(alloc, AllocationQuery):
                    buffers[(pi, k)] = allocate_query(alloc, batch_size, slots)
                elif isinstance(alloc, (tuple, list)):
                    buffers[(pi, k)] = tuple(allocate_query(q, batch_size, slots) for q in alloc)
                else:
                    buffers[(pi, k)] = None
        return buffers

    @staticmethod
    def _select(buffer, slot, count):
        if buffer is None:
            return None
        if isinstance(buffer, tuple):
            return tuple(Graph._select(b, slot, count) for b in buffer)
        return buffer[slot][:count]

    def run_batch(self, batch_indices, slot, stream_ptr, buffers, storage_state, epoch, batch_ix, lookahead=None):
        """One batch through every pipeline; returns the outputs in declaration order."""
        n = len(batch_indices)
        results = []
        for pi, p in enumerate(self.pipelines):
            if p.rider_host is not None:  # queued before the image pipeline stages its batch
                dst = buffers[(pi, 'rider')][slot][:n]
                values = np.ascontiguousarray(self.metadata[f'f{p.f_ix}'][batch_indices])
                if isinstance(p.ops[0], NDArrayDecoder):
                    rider = (None, values.astype(np.uint64), int(p.ops[0].field.element_size), dst.data_ptr())
                else:
                    rider = (values, None, values.dtype.itemsize, dst.data_ptr())
                self.pipelines[p.rider_host].executor.riders.append(rider)
        for pi, p in enumerate(self.pipelines):
            if p.rider_host is not None:
                value = buffers[(pi, 'rider')][slot][:n]
                first = p.n_fused
            elif p.executor is not None:
                value = p.executor(batch_indices, slot, stream_ptr, buffers[(pi, 'fused')][slot], epoch, batch_ix,
                                   lookahead=lookahead)
                first = p.n_fused
            else:
                code = p.codes[0]
                value = code(batch_indices, self._select(buffers[(pi, 0)], slot, n),
                             self.metadata[f'f{p.f_ix}'], storage_state)
                first = 1
            for k in range(first, len(p.ops)):
                begin = getattr(p.ops[k], 'begin_batch', None)
                if begin is not None:  # operations that draw random numbers of their own
                    begin(self.seed, epoch, batch_ix, pi * 64 + k)
                code = p.codes[k - p.n_fused]
                mem = self._select(buffers[(pi, k)], slot, n)
                if getattr(code, 'with_indices', False):
                    value = code(value, mem, batch_indices)
                else:
                    value = code(value, mem)
            results.append(value)
        return tuple(results)
