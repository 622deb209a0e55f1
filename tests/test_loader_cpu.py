"""Loader behaviour that needs no GPU: pipelines over the label field only (the image field is
disabled with `None`, as the reference allows), so everything runs on the host.  Mirrors the
reference's plumbing tests (tests/test_partial_batches.py, test_partial_pipeline.py,
test_loader_filter.py, test_basic_pipeline.py)."""
from dataclasses import replace

import numpy as np
import pytest
import torch as ch


@pytest.fixture(scope='module')
def beton(tmp_path_factory):
    from ffcv_b200.synthetic import write_dataset
    d = tmp_path_factory.mktemp('loadercpu')
    return write_dataset(0, str(d / 'c0.beton'), 203, num_workers=1)


def _labels(path):
    from ffcv_b200.reader import Reader
    return Reader(path).metadata['f1'].copy()


def _loader(path, **kw):
    from ffcv_b200 import Loader
    from ffcv_b200.fields.decoders import IntDecoder
    from ffcv_b200.transforms import ToTensor
    kw.setdefault('pipelines', {'image': None, 'label': [IntDecoder(), ToTensor()]})
    kw.setdefault('num_workers', 2)
    return Loader(path, **kw)


def test_sequential_batches_and_partial_last_batch(beton):
    truth = _labels(beton)
    loader = _loader(beton, batch_size=32, drop_last=False)
    assert len(loader) == 7
    got = [b[0].clone() for b in loader]  # batches are views of the slot ring: copy before it wraps
    assert [g.shape for g in got] == [(32, 1)] * 6 + [(11, 1)]
    assert np.array_equal(ch.cat(got).numpy().ravel(), truth)
    loader = _loader(beton, batch_size=32, drop_last=True)
    assert len(loader) == 6 and sum(b[0].shape[0] for b in loader) == 192


def test_default_pipeline_and_disabled_field(beton):
    from ffcv_b200 import Loader
    # `label` gets the default pipeline (decoder + ToTensor); the image field is switched off
    loader = Loader(beton, batch_size=50, num_workers=1, pipelines={'image': None})
    batch = next(iter(loader))
    assert len(batch) == 1 and isinstance(batch[0], ch.Tensor) and batch[0].dtype == ch.int64


def test_random_order_changes_per_epoch_and_is_seeded(beton):
    from ffcv_b200 import OrderOption
    truth = _labels(beton)
    a = _loader(beton, batch_size=64, order=OrderOption.RANDOM, seed=5, drop_last=False)
    b = _loader(beton, batch_size=64, order=OrderOption.RANDOM, seed=5, drop_last=False)
    e0 = ch.cat([x[0].clone() for x in a]).numpy().ravel()
    e1 = ch.cat([x[0].clone() for x in a]).numpy().ravel()
    f0 = ch.cat([x[0].clone() for x in b]).numpy().ravel()
    assert np.array_equal(e0, f0) and not np.array_equal(e0, e1)
    assert np.array_equal(np.sort(e0), np.sort(truth))
    order = np.random.default_rng(5).permutation(np.arange(203))
    assert np.array_equal(e0, truth[order])


def test_indices_subset_and_quasi_random(beton):
    from ffcv_b200 import OrderOption
    truth = _labels(beton)
    idx = np.arange(3, 203, 5)
    loader = _loader(beton, batch_size=16, indices=idx, drop_last=False)
    assert np.array_equal(ch.cat([b[0].clone() for b in loader]).numpy().ravel(), truth[idx])
    loader = _loader(beton, batch_size=16, indices=idx, order=OrderOption.QUASI_RANDOM, seed=1, drop_last=False)
    got = ch.cat([b[0].clone() for b in loader]).numpy().ravel()
    assert len(got) == len(idx) and np.array_equal(np.sort(got), np.sort(truth[idx]))


def test_filter_builds_a_subset_loader(beton):
    truth = _labels(beton)
    loader = _loader(beton, batch_size=40, drop_last=False)
    even = loader.filter('label', lambda x: int(x) % 2 == 0)
    got = ch.cat([b[0].clone() for b in even]).numpy().ravel()
    assert np.array_equal(got, truth[truth % 2 == 0])


def test_custom_operation_with_memory_and_indices(beton):
    """A user operation obeying the reference contract: allocation query, `(input, memory, indices)`
    call signature through `with_indices`."""
    from ffcv_b200.fields.decoders import IntDecoder
    from ffcv_b200.pipeline import AllocationQuery, Operation
    from ffcv_b200.transforms import ToTensor

    class AddIndex(Operation):
        def generate_code(self):
            def add(inp, dst, indices):
                dst[:len(indices), 0] = inp[:, 0] * 2 + np.asarray(indices)
                return dst[:len(indices)]
            add.with_indices = True
            return add

        def declare_state_and_memory(self, previous_state):
            return previous_state, AllocationQuery((1,), np.dtype('int64'))

    truth = _labels(beton)
    loader = _loader(beton, batch_size=25, drop_last=False,
                     pipelines={'image': None, 'label': [IntDecoder(), AddIndex(), ToTensor()]})
    got = ch.cat([b[0].clone() for b in loader]).numpy().ravel()
    assert np.array_equal(got, truth * 2 + np.arange(203))


def test_worker_exception_reaches_the_consumer(beton):
    """The reference leaves the consumer blocked forever when the worker thread dies
    (epoch_iterator.py:76-112,155); here the exception is re-raised in `__next__`."""
    from ffcv_b200.fields.decoders import IntDecoder
    from ffcv_b200.pipeline import Operation

    class Boom(Operation):
        def generate_code(self):
            def boom(inp, dst):
                if inp[0, 0] >= 0 and boom.calls >= 2:
                    raise RuntimeError('transform failed on purpose')
                boom.calls += 1
                return inp
            boom.calls = 0
            return boom

        def declare_state_and_memory(self, previous_state):
            return replace(previous_state, jit_mode=False), None

    loader = _loader(beton, batch_size=20, pipelines={'image': None, 'label': [IntDecoder(), Boom()]})
    it = iter(loader)
    next(it)
    next(it)
    with pytest.raises(RuntimeError, match='on purpose'):
        next(it)
    # the loader is usable again afterwards
    loader2 = _loader(beton, batch_size=20)
    assert sum(1 for _ in loader2) == 10


def test_abandoned_epoch_is_retired(beton):
    loader = _loader(beton, batch_size=10)
    it = iter(loader)
    next(it)
    first = loader._live_iterator
    second = iter(loader)
    assert not first.is_alive() and second is loader._live_iterator
    assert sum(1 for _ in second) == 20


def test_invalid_arguments(beton):
    from ffcv_b200 import Loader
    with pytest.raises(ValueError):
        Loader(beton, batch_size=8, order='shuffled', pipelines={'image': None})
    with pytest.raises(ValueError):
        Loader(beton, batch_size=8, pipelines={'image': None, 'label': 5})
    with pytest.raises(ValueError):
        Loader(beton, batch_size=8, pipelines={'image': None}, cpu_stage_share=1.5)


def test_direct_read_manager_reads_without_a_mapping(beton):
    """os_cache=False: the file is not mapped; `memory_read` serves payloads with pread, the
    label path is unchanged, and the native staging call gets the file descriptors."""
    from ffcv_b200.memory_managers import DirectReadManager, FileDescriptors, OSCacheManager
    from ffcv_b200.reader import Reader
    truth = _labels(beton)
    loader = _loader(beton, batch_size=32, drop_last=False, os_cache=False)
    mm = loader.memory_manager
    assert isinstance(mm, DirectReadManager) and not loader.pin_file and mm.direct
    got = ch.cat([b[0].clone() for b in loader]).numpy().ravel()
    assert np.array_equal(got, truth)
    fds = mm.file_base()
    assert isinstance(fds, FileDescriptors) and fds.fd >= 0
    # payload bytes read through the descriptor equal those of the mapping
    r = Reader(beton)
    mapped = OSCacheManager(r)
    read_fd, read_map = mm.compile_reader(), mapped.compile_reader()
    state_fd, state_map = mm.schedule_epoch([]).state, mapped.schedule_epoch([]).__enter__().state
    for ptr in r.metadata['f0']['data_ptr'][[0, 7, 202]]:
        assert np.array_equal(read_fd(ptr, state_fd), np.asarray(read_map(ptr, state_map)))
    mm.close()
    assert mm.fds is None


def test_ndarray_field_round_trip(tmp_path):
    """NDArrayField / TorchTensorField: same field arguments and stored bytes as the reference
    (ffcv/fields/ndarray.py), read back through the default pipeline on the host."""
    from ffcv_b200 import Loader
    from ffcv_b200.fields import FloatField, IntField, NDArrayField, TorchTensorField
    from ffcv_b200.reader import Reader
    from ffcv_b200.writer import DatasetWriter

    rng = np.random.default_rng(4)
    vec = rng.standard_normal((37, 3, 5)).astype(np.float32)
    ten = rng.integers(-1000, 1000, (37, 4)).astype(np.int16)

    class DS:
        def __len__(self):
            return 37

        def __getitem__(self, i):
            return vec[i], i * 3, float(i) / 7, ch.from_numpy(ten[i])

    path = str(tmp_path / 'nd.beton')
    DatasetWriter(path, {'vec': NDArrayField(np.dtype('float32'), (3, 5)), 'label': IntField(),
                         'weight': FloatField(), 'ten': TorchTensorField(ch.int16, (4,))},
                  num_workers=1).from_indexed_dataset(DS())
    r = Reader(path)
    assert type(r.handlers['vec']).__name__ == 'NDArrayField' and r.handlers['vec'].shape == (3, 5)
    assert r.handlers['vec'].dtype == np.float32 and r.handlers['ten'].dtype == np.int16
    assert [int(d['type_id']) for d in r.field_descriptors] == [4, 1, 0, 6]
    loader = Loader(path, batch_size=16, num_workers=1, drop_last=False)
    got = [[x.clone() for x in b] for b in loader]
    assert np.array_equal(ch.cat([g[0] for g in got]).numpy(), vec)
    assert np.array_equal(ch.cat([g[1] for g in got]).numpy().ravel(), np.arange(37) * 3)
    assert np.allclose(ch.cat([g[2] for g in got]).numpy().ravel(), np.arange(37) / 7)
    assert np.array_equal(ch.cat([g[3] for g in got]).numpy(), ten)
    with pytest.raises(ValueError):
        Loader(path, batch_size=16, batches_ahead=0)
