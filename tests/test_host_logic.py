"""CPU-only checks of the host side: the C-ABI library loads and exports what include/*.h
declares, the .beton writer/reader round-trip, traversal orders, samplers, the fusion pass, and
the loud failure when no GPU is present (there is no CPU fallback)."""
import os
import re

import numpy as np
import pytest
import torch as ch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from ffcv_b200 import libffcv
    header = open(os.path.join(ROOT, 'include', 'ffcv_b200.h')).read()
    header = re.sub(r'/\*.*?\*/', '', header, flags=re.S)
    names = set(re.findall(r'\b(ffcvb_\w+|imdecode|resize|my_memcpy|my_fread)\s*\(', header))
    assert {'ffcvb_create', 'ffcvb_stage_batch', 'ffcvb_submit_batch', 'ffcvb_transform_device', 'imdecode',
            'resize', 'my_memcpy', 'my_fread'} <= names
    for n in names:
        assert hasattr(libffcv.lib, n), f'{n} declared in include/ffcv_b200.h but not exported'


def test_plan_struct_layout_matches_header():
    from ffcv_b200 import libffcv as L
    import ctypes
    assert ctypes.sizeof(L.Op) == 12
    assert ctypes.sizeof(L.Plan) == 5 * 4 + 8 * 12 + 4 + 8  # 4 bytes of padding before the pointer
    plan = L.make_plan(224, 224, 1, L.OUT_F16_NHWC, [(L.OP_FLIP, 0, (0, 0, 0)), (L.OP_CUTOUT, 64, (1, 2, 3))], 0x1000)
    assert plan.n_ops == 2 and plan.ops[1].arg == 64 and list(plan.ops[1].fill)[:3] == [1, 2, 3]
    with pytest.raises(ValueError):
        L.make_plan(8, 8, 0, 0, [(L.OP_FLIP, 0, (0, 0, 0))] * 9)


@pytest.mark.skipif(ch.cuda.is_available(), reason='checks the no-GPU failure mode')
def test_no_gpu_fails_loudly(tmp_path):
    from ffcv_b200 import libffcv as L
    with pytest.raises(L.FFCVBError):
        L.Context(0, 1, 1)
    # the reference-signature call reports failure like tjDecompress2 does
    buf = np.zeros(64, np.uint8)
    assert L.imdecode(buf, np.zeros((8, 8, 3), np.uint8), 8, 8, 8, 8) == -1
    # and a loader with an image pipeline refuses to start
    from ffcv_b200 import Loader
    from ffcv_b200.synthetic import write_dataset
    path = write_dataset(0, str(tmp_path / 'c0.beton'), 64, num_workers=1)
    with pytest.raises(RuntimeError, match='no CPU fallback'):
        Loader(path, batch_size=16)


@pytest.fixture(scope='module')
def small_beton(tmp_path_factory):
    from ffcv_b200.synthetic import write_dataset
    d = tmp_path_factory.mktemp('host')
    return write_dataset(2, str(d / 'c2.beton'), 40, num_workers=2, page_size=1 << 21)


def test_beton_layout_and_payloads(small_beton):
    from ffcv_b200.memory_managers import OSCacheManager
    from ffcv_b200.reader import Reader
    from ffcv_b200.fields.rgb_image import resizer
    from ffcv_b200.synthetic import SyntheticImageDataset
    from parity import O
    r = Reader(small_beton)
    raw = open(small_beton, 'rb').read(24)
    assert int.from_bytes(raw[0:2], 'little') == 2 and int.from_bytes(raw[2:4], 'little') == 2
    assert int.from_bytes(raw[4:8], 'little') == 1 << 21 and int.from_bytes(raw[8:16], 'little') == 40
    assert r.metadata.dtype.itemsize == 24 and r.metadata.dtype.fields['f1'][1] == 16
    assert r.field_names == ['image', 'label']
    md = r.metadata['f0']
    assert set(np.unique(md['mode'])) == {0, 1}
    mm = OSCacheManager(r)
    sizes = mm.sizes_of(md['data_ptr'])
    read = mm.compile_reader()
    state = mm.schedule_epoch([]).__enter__().state
    ds = SyntheticImageDataset(2, 40)
    page = r.page_size
    for i in range(40):
        img, label = ds[i]
        img = resizer(img, 500)  # the writer bounds the longer side (rgb_image.py:37-45)
        assert r.metadata['f1'][i] == label
        payload = read(md['data_ptr'][i], state)
        assert len(payload) == sizes[i]
        assert int(md['data_ptr'][i]) // page == (int(md['data_ptr'][i]) + int(sizes[i]) - 1) // page
        assert (md['height'][i], md['width'][i]) == img.shape[:2] and max(img.shape[:2]) <= 500
        if md['mode'][i] == 1:
            assert np.array_equal(np.asarray(payload).reshape(img.shape), img)
        else:
            dec = O.jpeg_decode(np.asarray(payload))
            assert dec.shape == img.shape and np.abs(dec.astype(int) - img).mean() < 8


def test_write_time_resize_and_modes(tmp_path):
    from ffcv_b200.fields import IntField, RGBImageField
    from ffcv_b200.reader import Reader
    from ffcv_b200.writer import DatasetWriter

    class DS:
        def __len__(self):
            return 6

        def __getitem__(self, i):
            return np.full((300 + 10 * i, 600, 3), i * 9, np.uint8), i

    path = str(tmp_path / 'r.beton')
    DatasetWriter(path, {'image': RGBImageField(write_mode='jpg', max_resolution=256), 'label': IntField()},
                  num_workers=1).from_indexed_dataset(DS())
    md = Reader(path).metadata['f0']
    assert (md['width'] == 256).all() and (md['mode'] == 0).all()
    assert list(md['height']) == [int(256 / 600 * (300 + 10 * i)) for i in range(6)]
    with pytest.raises(ValueError):
        RGBImageField().encode(np.zeros(1, RGBImageField().metadata_type), np.zeros((4, 4, 3), np.float32), None)


def test_traversal_orders(small_beton):
    from types import SimpleNamespace
    from ffcv_b200.memory_managers import OSCacheManager
    from ffcv_b200.reader import Reader
    from ffcv_b200.traversal_order import QuasiRandom, Random, Sequential
    r = Reader(small_beton)
    fake = SimpleNamespace(indices=np.arange(40), seed=7, distributed=False, batch_size=4,
                           memory_manager=OSCacheManager(r))
    assert list(Sequential(fake).sample_order(0)) == list(range(40))
    a, b = Random(fake).sample_order(0), Random(fake).sample_order(1)
    assert sorted(a) == list(range(40)) and list(a) != list(b)
    assert list(a) == list(np.random.default_rng(7).permutation(np.arange(40)))
    q0, q0b, q1 = (QuasiRandom(fake).sample_order(e) for e in (0, 0, 1))
    assert sorted(q0) == list(range(40)) and list(q0) == list(q0b) and list(q0) != list(q1)
    sub = SimpleNamespace(indices=np.arange(0, 40, 3), seed=7, distributed=False, batch_size=4,
                          memory_manager=OSCacheManager(r))
    assert sorted(QuasiRandom(sub).sample_order(0)) == list(range(0, 40, 3))


def test_sampler_ranges_and_reproducibility():
    from ffcv_b200.pipeline import sampling as S
    n = 500
    h = np.full(n, 333, np.uint16)
    w = np.full(n, 500, np.uint16)
    a, b = np.zeros((n, 4), np.int32), np.zeros((n, 4), np.int32)
    S.sample_random_crops(11, h, w, np.array([0.08, 1.0]), np.array([0.75, 4 / 3]), a)
    S.sample_random_crops(11, h, w, np.array([0.08, 1.0]), np.array([0.75, 4 / 3]), b)
    assert np.array_equal(a, b)
    assert (a[:, 0] >= 0).all() and (a[:, 1] >= 0).all() and (a[:, 2] > 0).all() and (a[:, 3] > 0).all()
    assert (a[:, 0] + a[:, 2] <= 333).all() and (a[:, 1] + a[:, 3] <= 500).all()
    area = a[:, 2] * a[:, 3] / (333 * 500)
    assert 0.07 < area.min() and area.max() <= 1.0
    f = np.zeros((n, 2), np.int32)
    S.sample_flips(3, n, 0.5, f)
    assert 0.35 < f[:, 0].mean() < 0.65
    S.sample_flips(3, n, 1.0, f)
    assert f[:, 0].all()
    t = np.zeros((n, 2), np.int32)
    S.sample_translations(5, n, 2, t)
    assert t.min() == 0 and t.max() == 4
    c = np.zeros((n, 2), np.int32)
    S.sample_cutouts(5, n, 32, 32, 4, c)
    assert c.min() >= 0 and c.max() == 28
    seeds = {S.batch_seed(0, e, b, o) for e in range(4) for b in range(50) for o in range(4)}
    assert len(seeds) == 800


def test_fusion_pass_folds_the_reference_pipelines():
    from ffcv_b200 import libffcv as L
    from ffcv_b200.fields.decoders import RandomResizedCropRGBImageDecoder, SimpleRGBImageDecoder
    from ffcv_b200.pipeline.fusion import FusedImagePlan
    from ffcv_b200.transforms import (Convert, Cutout, ModuleWrapper, NormalizeImage, RandomHorizontalFlip,
                                      RandomTranslate, ToDevice, ToTensor, ToTorchImage)

    def fuse(ops):
        plan, k = FusedImagePlan(), 0
        while k < len(ops) and ops[k].fuse(plan):
            k += 1
        return plan, k

    mean, std = np.array([1., 2., 3.]), np.array([4., 5., 6.])
    dec = SimpleRGBImageDecoder()
    dec.metadata = np.zeros(3, dtype=[('width', '<u2'), ('height', '<u2')])
    dec.metadata['width'], dec.metadata['height'] = 32, 32
    ops = [dec, RandomHorizontalFlip(), RandomTranslate(2, (1, 2, 3)), Cutout(4, (4, 5, 6)), ToTensor(),
           ToDevice(ch.device('cuda:0')), ToTorchImage(), Convert(ch.float16), NormalizeImage(mean, std, np.float16)]
    plan, k = fuse(ops)
    assert k == len(ops) and [o[0] for o in plan.ops] == [L.OP_FLIP, L.OP_TRANSLATE, L.OP_CUTOUT]
    assert plan.out_kind == L.OUT_F16_NHWC and plan.torch_image and not plan.resize
    assert np.array_equal(plan.table, ops[-1].lookup_table)  # Convert's identity table was replaced
    plan, k = fuse([RandomResizedCropRGBImageDecoder((224, 224)), RandomHorizontalFlip(),
                    NormalizeImage(mean, std, np.float32), ToTorchImage(channels_last=False)])
    assert k == 4 and plan.out_kind == L.OUT_F32_NCHW and plan.buffer_shape == (3, 224, 224) and plan.resize
    # a spatial op after the table, or anything after a torch module, stays outside the plan
    plan, k = fuse([RandomResizedCropRGBImageDecoder((64, 64)), NormalizeImage(mean, std, np.float16), Cutout(8)])
    assert k == 2
    plan, k = fuse([RandomResizedCropRGBImageDecoder((64, 64)), ModuleWrapper(ch.nn.Identity()), Cutout(8)])
    assert k == 1 and plan.out_kind == L.OUT_U8_NHWC
    from ffcv_b200.transforms import RandomResizedCrop
    plan, k = fuse([dec, RandomResizedCrop((0.08, 1), (0.75, 4 / 3), 24), RandomHorizontalFlip()])
    assert k == 3 and plan.resize and plan.out_h == 24 and plan.crop_sampler is not None
    plan, k = fuse([dec, RandomHorizontalFlip(), RandomResizedCrop((0.08, 1), (0.75, 4 / 3), 24)])
    assert k == 2  # a crop after another augmentation is not the decoder's crop
    plan, k = fuse([RandomResizedCropRGBImageDecoder((64, 64)), Convert(ch.float32)])
    assert k == 2 and plan.table[200, 1] == 200.0


def test_state_contract():
    from ffcv_b200.pipeline import AllocationQuery, State
    with pytest.raises(AssertionError):
        State(jit_mode=True, device=ch.device('cuda:0'), shape=(1,), dtype=np.dtype('u1'))
    with pytest.raises(AssertionError):
        State(jit_mode=True, device=ch.device('cpu'), shape=(1,), dtype=ch.float16)
    q = AllocationQuery((2, 3), np.dtype('u1'))
    from ffcv_b200.pipeline.allocation_query import allocate_query
    buf = allocate_query(q, 4, 3)
    assert buf.shape == (3, 4, 2, 3) and buf.dtype == np.uint8
