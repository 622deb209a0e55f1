"""The loader (reference: ``ffcv/loader/loader.py:52-277``): same constructor arguments and
iteration protocol; batches are decoded and augmented on the GPU of the calling process."""
import enum
from os import environ, sched_getaffinity
from typing import Any, Callable, Mapping, Sequence, Type, Union

import numpy as np
import torch as ch

from .. import libffcv as L
from ..fields.base import Field
from ..memory_managers import DirectReadManager, MemoryManager, OSCacheManager
from ..pipeline.compiler import Compiler
from ..pipeline.graph import Graph
from ..pipeline.operation import Operation
from ..pipeline.pipeline_spec import PipelineSpec
from ..reader import Reader
from ..traversal_order import QuasiRandom, Random, Sequential, TraversalOrder
from .epoch_iterator import EpochIterator


@enum.unique
class OrderOption(enum.Enum):
    SEQUENTIAL = enum.auto()
    RANDOM = enum.auto()
    QUASI_RANDOM = enum.auto()


ORDER_MAP = {
    OrderOption.RANDOM: Random,
    OrderOption.SEQUENTIAL: Sequential,
    OrderOption.QUASI_RANDOM: QuasiRandom,
}

DEFAULT_PROCESS_CACHE = int(environ.get('FFCV_DEFAULT_CACHE_PROCESS', "0"))
DEFAULT_OS_CACHE = not DEFAULT_PROCESS_CACHE


class Loader:
    """Drop-in for ``ffcv.loader.Loader``.

    Parameters
    ----------
    fname: str
        Path of the dataset (``.beton``).
    batch_size : int
        Batch size.
    num_workers : int
        Host threads that stage sample bytes into pinned memory (the reference's numba worker
        count); < 1 means every core this process may run on.
    os_cache : bool
        The file is memory-mapped and served from the operating system's page cache.  ``False``
        (the reference's process cache, for datasets larger than RAM): the file is neither mapped
        nor pinned; the staging threads read the samples of each batch (``pread``, with
        ``O_DIRECT`` where the file system allows) straight into the pinned staging buffer of the
        batch's slot, ``batches_ahead`` batches ahead of the consumer, so the bytes cross host
        memory once and resident memory is bounded by the slot ring.
    order : OrderOption or TraversalOrder subclass
        SEQUENTIAL, RANDOM, QUASI_RANDOM, or a custom order.
    distributed : bool
        Shard the samples over the ranks of the initialised ``torch.distributed`` process group,
        one process per GPU, as ``DistributedSampler`` does.  No collective is used.
    seed : int
        Seed of the sample order; here it also seeds the augmentations' random draws.
    indices : Sequence[int]
        Subset of the dataset.
    pipelines : Mapping[str, Sequence[Operation | torch.nn.Module]]
        Decoder and transforms of each field; ``None`` disables a field.
    custom_fields : Mapping[str, Field]
        Types of fields that use a custom type.
    drop_last : bool
        Drop the last, incomplete batch.
    batches_ahead : int
        Batches prepared in advance.
    recompile : bool
        Rebuild the pipeline executables every epoch.
    pin_file : bool
        (not in the reference) Keep the whole file in page-locked host memory and let the GPU
        fetch each batch's bytes itself over PCIe instead of staging them with CPU threads: the
        bytes cross host memory once instead of three times.  A file on a memory file system
        (``/dev/shm``) is page-locked where it lies, so all processes of a node share the one
        copy and nothing is read at start-up; any other file costs one pinned copy per process.
        Default (``None``): a file on a memory file system is page-locked where it lies, whatever
        its size (nothing is copied); any other file is copied into pinned memory only if it is at
        most ``FFCV_B200_PIN_LIMIT_GB`` (default 64) GiB and the copies of all ranks of the host
        (``LOCAL_WORLD_SIZE``) fit half of the memory available now; else the staged path is used.
        Measured on config 2: 1 GPU + 16 threads
        255-270 k img/s staged, 250-270 k gathered, 300-330 k split (below); 8 GPUs + 32 cores
        326 k staged, 1.15 M gathered.  ``FFCV_B200_PIN_FILE`` = 0 / 1 overrides.
    decode_index_gb : float
        (not in the reference; off by default) GiB of GPU memory for a decode index: the first
        decode of every JPEG sample records the decoder's state at the start of each of its
        subsequences (about 7 % of the stream's size); from the second epoch on the sample is
        decoded in one pass from those states instead of being re-synchronised by guess and
        repair.  Same pixels; entropy decode 2-3x faster.  Samples that do not fit the pool any
        more stay unindexed.
    cpu_stage_share : float
        (not in the reference) With a pinned file, the share of every batch's bytes that up to
        four staging threads copy and the copy engine moves while the GPU gathers the rest.
        Default (``None``): balanced from batch to batch by the native context when this process
        is the only rank on the host (``LOCAL_WORLD_SIZE`` <= 1) and has at least 8 staging
        threads, else 0 -- with several GPUs per host the CPU copies compete with every GPU's
        gather for host memory bandwidth (1 GPU + 16 cores: 305 k img/s balanced, 280 k gathered;
        2 GPUs + 24 cores: 570 k vs 563 k; 8 GPUs + 32 cores: 0.89 M vs 1.15 M).
    """

    def __init__(self, fname: str, batch_size: int, num_workers: int = -1,
                 os_cache: bool = DEFAULT_OS_CACHE,
                 order: Union[OrderOption, Type[TraversalOrder]] = OrderOption.SEQUENTIAL,
                 distributed: bool = False, seed: int = None, indices: Sequence[int] = None,
                 pipelines: Mapping[str, Sequence[Union[Operation, ch.nn.Module]]] = {},
                 custom_fields: Mapping[str, Type[Field]] = {}, drop_last: bool = True,
                 batches_ahead: int = 3, recompile: bool = False, order_kwargs: dict = dict(),
                 pin_file: bool = None, cpu_stage_share: float = None, decode_index_gb: float = 0):
        if distributed and order == OrderOption.RANDOM and (seed is None):
            print('Warning: no ordering seed was specified with distributed=True. '
                  'Setting seed to 0 to match PyTorch distributed sampler.')
            seed = 0
        elif seed is None:
            seed = int(np.random.randint(0, np.iinfo('int32').max))

        self._args = {
            'fname': fname, 'batch_size': batch_size, 'num_workers': num_workers, 'os_cache': os_cache,
            'order': order, 'distributed': distributed, 'seed': seed, 'indices': indices,
            'pipelines': pipelines, 'drop_last': drop_last, 'batches_ahead': batches_ahead,
            'recompile': recompile, 'pin_file': pin_file, 'cpu_stage_share': cpu_stage_share,
            'decode_index_gb': decode_index_gb,
        }
        self.fname = fname
        self.batch_size = batch_size
        self.decode_index_gb = float(decode_index_gb)
        if batches_ahead < 1:
            # the slot ring's reuse argument needs a bounded queue: Queue(0) would be unbounded
            raise ValueError("batches_ahead must be at least 1")
        self.batches_ahead = batches_ahead
        self.seed = seed
        self.reader = Reader(fname, custom_fields)
        self.num_workers = num_workers if num_workers >= 1 else len(sched_getaffinity(0))
        self.drop_last = drop_last
        self.distributed = distributed
        self.recompile = recompile
        self.device = ch.device('cuda', ch.cuda.current_device()) if ch.cuda.is_available() else ch.device('cpu')
        Compiler.set_num_threads(self.num_workers)

        if indices is None:
            self.indices = np.arange(self.reader.num_samples, dtype='uint64')
        else:
            self.indices = np.array(indices)

        if pin_file is None and environ.get('FFCV_B200_PIN_FILE') in ('0', '1'):
            pin_file = environ['FFCV_B200_PIN_FILE'] == '1'
        threads = num_workers if num_workers >= 1 else \
            len(sched_getaffinity(0)) // max(1, int(environ.get('LOCAL_WORLD_SIZE', '1')))
        if not os_cache:
            pin_file = False  # the file is taken to be larger than RAM
        if pin_file is None:
            # 'auto': page-lock the file where it lies if it is on a memory file system (no copy,
            # whatever its size); a private pinned copy only below the limit and if it fits
            pin_file = 'auto' if ch.cuda.is_available() else False
        self.pin_file = bool(pin_file)
        if cpu_stage_share is None and 'FFCV_B200_STAGE_SPLIT' in environ:
            cpu_stage_share = int(environ['FFCV_B200_STAGE_SPLIT']) / 1000
        if cpu_stage_share is not None and not 0 <= cpu_stage_share <= 1:
            raise ValueError("cpu_stage_share must lie in [0, 1]")
        if cpu_stage_share is None:
            # -1: balanced by the native context.  Only for a GPU that has the host to itself: with
            # two GPUs per host the split measured level with the pure gather, with eight it lost.
            alone = int(environ.get('LOCAL_WORLD_SIZE', '1')) <= 1
            self.stage_split = -1 if (threads >= 8 and alone) else 0
        else:
            self.stage_split = int(round(cpu_stage_share * 1000))
        if os_cache:
            self.memory_manager: MemoryManager = OSCacheManager(self.reader, pin=pin_file)
            if self.pin_file:  # settled now: the size of the staging pool depends on it
                self.memory_manager.open()
                self.pin_file = self.memory_manager.pinned
        else:
            # no mapping, no page cache: the staging threads read every batch straight into the
            # slot ring's pinned buffers (the reference's process cache role)
            self.memory_manager = DirectReadManager(self.reader)

        if order in ORDER_MAP:
            self.traversal_order: TraversalOrder = ORDER_MAP[order](self)
        elif isinstance(order, type) and issubclass(order, TraversalOrder):
            self.traversal_order = order(self, **order_kwargs)
        else:
            raise ValueError(f"Order {order} is not a supported order type or a subclass of TraversalOrder")

        self.next_epoch = 0
        self.pipeline_specs = {}
        self.field_name_to_f_ix = {}
        custom_specs = {}
        for output_name, spec in pipelines.items():
            if isinstance(spec, PipelineSpec):
                pass
            elif isinstance(spec, Sequence):
                spec = PipelineSpec(output_name, decoder=None, transforms=list(spec))
            elif spec is None:
                continue
            else:
                raise ValueError(f"The pipeline for {output_name} has to be "
                                 "either a PipelineSpec or a sequence of operations")
            custom_specs[output_name] = spec
        for f_ix, field_name in enumerate(self.reader.handlers.keys()):
            self.field_name_to_f_ix[field_name] = f_ix
            if field_name in custom_specs:
                self.pipeline_specs[field_name] = custom_specs[field_name]
            elif field_name not in pipelines:
                self.pipeline_specs[field_name] = PipelineSpec(field_name)
        for field_name, spec in custom_specs.items():
            if field_name not in self.pipeline_specs:
                self.pipeline_specs[field_name] = spec

        self._contexts = {}
        self._streams = None
        self._buffers = None
        self._slot_done = None
        self._live_iterator = None
        self.graph = None
        self.generate_code()
        self.first_traversal_order = self.next_traversal_order()

    # ---- resources shared by the epochs
    def _context_for(self, device, pipeline=0):
        """One native context per (device, image pipeline) of this loader; its slots are the
        loader's ring.  Two image fields never share a context: a context's slot holds the staged
        bytes and descriptors of exactly one batch of one field."""
        if not ch.cuda.is_available():
            raise RuntimeError("ffcv_b200 decodes images on the GPU and has no CPU fallback: "
                               "no CUDA device is visible")
        index = device.index if device is not None and device.index is not None else ch.cuda.current_device()
        index = (index, int(pipeline))
        if index not in self._contexts:
            # With the file pinned the GPU fetches most bytes itself: a few staging threads carry
            # the CPU's share, more of them only slow the gather down (measured).
            threads = min(self.num_workers, 4) if self.pin_file else self.num_workers
            self._contexts[index] = L.Context(index[0], n_slots=self.batches_ahead + 2, n_threads=threads)
            # the payload copy of a batch overlaps the drawing of the next batch's parameters
            self._contexts[index].set_async_staging(True)
            # this context only ever sees this loader's file: parsed headers are kept per sample
            self._contexts[index].set_header_cache(True)
            if self.pin_file:
                self._contexts[index].set_staging_split(self.stage_split)
            if self.decode_index_gb > 0:
                self._contexts[index].set_decode_index(int(self.decode_index_gb * (1 << 30)))
        return self._contexts[index]

    def slot_streams(self):
        if self._streams is None:
            self._streams = [ch.cuda.Stream(self.device) for _ in range(self.batches_ahead + 2)]
        return self._streams

    def slot_buffers(self):
        if self._buffers is None:
            self._buffers = self.graph.allocate_memory(self.batch_size, self.batches_ahead + 2)
        return self._buffers

    def slot_done_events(self):
        if self._slot_done is None:
            self._slot_done = [None] * (self.batches_ahead + 2)
        return self._slot_done

    def next_traversal_order(self):
        return self.traversal_order.sample_order(self.next_epoch)

    def __iter__(self):
        Compiler.set_num_threads(self.num_workers)
        order = self.next_traversal_order()
        selected_order = order[:len(self) * self.batch_size]
        epoch = self.next_epoch
        self.next_epoch += 1
        if self._live_iterator is not None:
            self._live_iterator.retire()
        if self.graph is None or self.recompile:
            self.generate_code()
        self._live_iterator = EpochIterator(self, selected_order, epoch)
        return self._live_iterator

    def filter(self, field_name: str, condition: Callable[[Any], bool]) -> 'Loader':
        new_args = {**self._args}
        pipelines = {name: None for name in self.reader.handlers.keys()}
        try:
            pipelines[field_name] = new_args['pipelines'][field_name]
        except KeyError:
            del pipelines[field_name]
        new_args['pipelines'] = pipelines
        new_args['order'] = OrderOption.SEQUENTIAL
        new_args['drop_last'] = False
        sub_loader = Loader(**new_args)
        selected = []
        for i, (batch,) in enumerate(sub_loader):
            for j, sample in enumerate(batch):
                if condition(sample):
                    selected.append(i * self.batch_size + j)
        final_args = {**self._args}
        final_args['indices'] = np.array(selected)
        return Loader(**final_args)

    def __len__(self):
        n = len(self.first_traversal_order)
        if self.drop_last:
            return n // self.batch_size
        return int(np.ceil(n / self.batch_size))

    def generate_code(self):
        specs = {k: PipelineSpec(v.source, v.decoder, list(v.transforms)) for k, v in self.pipeline_specs.items()}
        self.graph = Graph(specs, self.reader.handlers, self.field_name_to_f_ix, self.reader.metadata,
                           self.memory_manager, self._context_for, self.seed)
        self._buffers = None
        self.code = self.graph
