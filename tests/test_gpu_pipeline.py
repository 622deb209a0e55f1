"""Parity of the whole loader path on the GPU against the CPU oracle, configuration by
configuration (reduced sample counts, full image sizes).  Bars: JPEG pixels bit-exact; resized
uint8 within 1 LSB (the oracle restates cv2 bit for bit, so 0 is asserted); flip / translate /
cutout bit-exact; normalised fp16 within 1 ULP (asserted: identical bit patterns, the table is
shared arithmetic)."""
import os

import numpy as np
import pytest
import torch as ch

from parity import (CIFAR_MEAN, CIFAR_STD, IMAGENET_MEAN, IMAGENET_STD, compare_epoch, image_executor)

pytestmark = pytest.mark.gpu


@pytest.fixture(scope='module')
def datasets(tmp_path_factory):
    from ffcv_b200.synthetic import write_dataset_isolated as write_dataset  # forks: not from this process
    d = tmp_path_factory.mktemp('betons')
    out = {}
    for cfg, n in [(0, 1536), (1, 192), (2, 128), (4, 6)]:
        out[cfg] = write_dataset(cfg, str(d / f'c{cfg}.beton'), n, num_workers=8)
    return out


def _loader(path, batch_size, pipelines, **kw):
    from ffcv_b200 import Loader, OrderOption
    kw.setdefault('order', OrderOption.SEQUENTIAL)
    kw.setdefault('seed', 0)
    kw.setdefault('num_workers', 8)
    return Loader(path, batch_size=batch_size, pipelines=pipelines, **kw)


def test_config0_cifar_raw_augment(datasets):
    from ffcv_b200 import OrderOption
    from ffcv_b200.fields.decoders import IntDecoder, SimpleRGBImageDecoder
    from ffcv_b200.transforms import (Convert, Cutout, NormalizeImage, RandomHorizontalFlip,
                                      RandomTranslate, Squeeze, ToDevice, ToTensor, ToTorchImage)
    dev = ch.device('cuda:0')
    fill = (125, 123, 114)
    pipes = {
        'image': [SimpleRGBImageDecoder(), RandomHorizontalFlip(0.5), RandomTranslate(padding=2, fill=fill),
                  Cutout(4, fill), ToTensor(), ToDevice(dev), ToTorchImage(), Convert(ch.float16),
                  NormalizeImage(CIFAR_MEAN, CIFAR_STD, np.float16)],
        'label': [IntDecoder(), ToTensor(), ToDevice(dev), Squeeze()],
    }
    loader = _loader(datasets[0], 512, pipes, order=OrderOption.RANDOM)
    exe = image_executor(loader)
    assert len(exe.plan.ops) == 3 and exe.plan.table is not None and exe.plan.torch_image
    n = compare_epoch(loader)
    assert n == 3 * 512 * 32 * 32 * 3
    # labels ride along unchanged
    loader2 = _loader(datasets[0], 512, pipes, order=OrderOption.SEQUENTIAL)
    labels = ch.cat([b[1] for b in loader2]).cpu().numpy()
    assert (labels == loader2.reader.metadata['f1'][:len(labels)]).all()
    # both halves of the augmentation space are exercised
    exe2 = image_executor(loader2)
    assert 0 < exe2.last_params[:, 4].mean() < 1


def test_config1_lowres_jpeg_rrc160(datasets):
    from ffcv_b200.fields.decoders import RandomResizedCropRGBImageDecoder
    from ffcv_b200.transforms import NormalizeImage, RandomHorizontalFlip, ToDevice, ToTensor, ToTorchImage
    dev = ch.device('cuda:0')
    pipes = {'image': [RandomResizedCropRGBImageDecoder((160, 160), scale=(0.08, 1), ratio=(3 / 4, 4 / 3)),
                       RandomHorizontalFlip(), ToTensor(), ToDevice(dev), ToTorchImage(),
                       NormalizeImage(IMAGENET_MEAN, IMAGENET_STD, np.float16)],
             'label': None}
    loader = _loader(datasets[1], 64, pipes)
    batch = next(iter(loader))
    assert batch[0].shape == (64, 3, 160, 160) and batch[0].dtype == ch.float16
    assert batch[0].is_contiguous(memory_format=ch.channels_last)
    compare_epoch(loader)


@pytest.mark.parametrize('pin_file,share', [(False, None), (True, 0.0), (True, 0.4), (True, 1.0)],
                         ids=['staged', 'pinned_gather', 'pinned_split', 'pinned_all_cpu'])
def test_config2_fullres_mix_rrc224(datasets, pin_file, share):
    """The ways the bytes can reach the GPU: staged by CPU threads from the memory-mapped file
    (crop box of raw samples only), gathered by the GPU from a pinned copy of the file, or split
    between the two."""
    from ffcv_b200 import OrderOption
    from ffcv_b200.fields.decoders import RandomResizedCropRGBImageDecoder
    from ffcv_b200.transforms import NormalizeImage, RandomHorizontalFlip, ToTorchImage
    pipes = {'image': [RandomResizedCropRGBImageDecoder((224, 224)), RandomHorizontalFlip(),
                       NormalizeImage(IMAGENET_MEAN, IMAGENET_STD, np.float16), ToTorchImage()],
             'label': None}
    loader = _loader(datasets[2], 32, pipes, order=OrderOption.QUASI_RANDOM, pin_file=pin_file,
                     cpu_stage_share=share)
    assert loader.memory_manager.open() is not None and loader.memory_manager.pinned == pin_file
    modes = loader.reader.metadata['f0']['mode']
    assert 0 < modes.mean() < 1  # both raw and jpg samples present
    compare_epoch(loader)


@pytest.mark.parametrize('cfg,interval,res', [(2, 4, 224), (1, 1, 160), (2, 25, 224), (4, 8, 384)])
def test_streams_with_restart_markers(tmp_path, cfg, interval, res):
    """Datasets written with the restart-interval option: every interval is decoded by its own
    thread (no speculation); the pixels must be those of the oracle, crop-limited decode included."""
    from ffcv_b200 import OrderOption
    from ffcv_b200.fields.decoders import RandomResizedCropRGBImageDecoder, SimpleRGBImageDecoder
    from ffcv_b200.synthetic import write_dataset_isolated as write_dataset
    from ffcv_b200.transforms import NormalizeImage, RandomHorizontalFlip, ToTorchImage
    n = 6 if cfg == 4 else 64
    path = write_dataset(cfg, str(tmp_path / f'c{cfg}_rst{interval}.beton'), n, num_workers=4, restart_interval=interval)
    pipes = {'image': [RandomResizedCropRGBImageDecoder((res, res)), RandomHorizontalFlip(),
                       NormalizeImage(IMAGENET_MEAN, IMAGENET_STD, np.float16), ToTorchImage()],
             'label': None}
    loader = _loader(path, min(n, 32), pipes, order=OrderOption.QUASI_RANDOM)
    exe = image_executor(loader)
    compare_epoch(loader)
    assert exe.ctx.launches(0) >= 4


def test_config3_center_crop_validation(datasets):
    from ffcv_b200.fields.decoders import CenterCropRGBImageDecoder
    from ffcv_b200.transforms import NormalizeImage, ToDevice, ToTensor, ToTorchImage
    dev = ch.device('cuda:0')
    pipes = {'image': [CenterCropRGBImageDecoder((256, 256), ratio=224 / 256), ToTensor(), ToDevice(dev),
                       ToTorchImage(), NormalizeImage(IMAGENET_MEAN, IMAGENET_STD, np.float16)],
             'label': None}
    loader = _loader(datasets[1], 64, pipes)
    compare_epoch(loader)
    # deterministic end to end: a second epoch gives the same tensors
    a = [b[0].clone() for b in loader]
    b = [x[0].clone() for x in loader]
    assert all(ch.equal(x, y) for x, y in zip(a, b))


def test_config4_highres_444_cutout(datasets):
    from ffcv_b200.fields.decoders import RandomResizedCropRGBImageDecoder
    from ffcv_b200.transforms import Cutout, NormalizeImage, RandomHorizontalFlip, ToTorchImage
    pipes = {'image': [RandomResizedCropRGBImageDecoder((384, 384), scale=(0.25, 1)), RandomHorizontalFlip(),
                       Cutout(64), NormalizeImage(IMAGENET_MEAN, IMAGENET_STD, np.float16),
                       ToTorchImage(channels_last=False)],
             'label': None}
    loader = _loader(datasets[4], 3, pipes)
    batch = next(iter(loader))
    assert batch[0].shape == (3, 3, 384, 384) and batch[0].is_contiguous()
    compare_epoch(loader)


def test_uint8_output_and_unfused_tail(datasets):
    """A pipeline that stops at uint8, and one whose tail cannot be fused (a torch module sits
    between the decoder and the augmentations): the tail runs op by op on the GPU and must give
    the same pixels as the oracle applied stage by stage."""
    from ffcv_b200.fields.decoders import SimpleRGBImageDecoder
    from ffcv_b200.transforms import Cutout, NormalizeImage, RandomHorizontalFlip, ToTorchImage
    pipes = {'image': [SimpleRGBImageDecoder(), RandomHorizontalFlip(1.0)], 'label': None}
    loader = _loader(datasets[0], 256, pipes)
    compare_epoch(loader, max_batches=2)
    batch = next(iter(loader))
    assert batch[0].dtype == ch.uint8 and batch[0].shape == (256, 32, 32, 3)

    ident = ch.nn.Identity()
    pipes = {'image': [SimpleRGBImageDecoder(), ident, RandomHorizontalFlip(1.0), Cutout(8, (9, 8, 7)),
                       NormalizeImage(CIFAR_MEAN, CIFAR_STD, np.float32), ToTorchImage()],
             'label': None}
    loader = _loader(datasets[0], 256, pipes)
    exe = image_executor(loader)
    assert len(exe.plan.ops) == 0 and exe.plan.table is None  # nothing after the module was fused
    got = next(iter(loader))[0]
    assert got.shape == (256, 3, 32, 32) and got.dtype == ch.float32
    raw = next(iter(_loader(datasets[0], 256, {'image': [SimpleRGBImageDecoder()], 'label': None})))[0]
    flipped = raw.flip(2).cpu().numpy()
    table = ((np.arange(256)[:, None] - CIFAR_MEAN[None]) / CIFAR_STD[None]).astype(np.float32)
    g = got.permute(0, 2, 3, 1).cpu().numpy()
    fillv = table[[9, 8, 7], [0, 1, 2]]
    is_fill = (g == fillv[None, None, None, :]).all(-1)
    assert (is_fill.sum((1, 2)) >= 64).all()  # an 8x8 square per image
    expect = table[flipped, np.arange(3)[None, None, None, :]]
    assert (np.where(is_fill[..., None], expect, g) == expect).all()


def test_random_resized_crop_transform(datasets):
    """The post-decode RandomResizedCrop: folded into the decoder's launch, and on its own."""
    from ffcv_b200.fields.decoders import SimpleRGBImageDecoder
    from ffcv_b200.transforms import NormalizeImage, RandomHorizontalFlip, RandomResizedCrop, ToTorchImage
    pipes = {'image': [SimpleRGBImageDecoder(), RandomResizedCrop((0.3, 1.0), (0.75, 4 / 3), 24), RandomHorizontalFlip(),
                       NormalizeImage(CIFAR_MEAN, CIFAR_STD, np.float16), ToTorchImage()], 'label': None}
    loader = _loader(datasets[0], 256, pipes)
    exe = image_executor(loader)
    assert exe.plan.resize and exe.plan.out_h == 24 and len(exe.plan.ops) == 1
    assert next(iter(loader))[0].shape == (256, 3, 24, 24)
    compare_epoch(loader, max_batches=3)
    # standalone (behind a torch module): same kernel on the decoded batch
    from parity import O
    pipes = {'image': [SimpleRGBImageDecoder(), ch.nn.Identity(), RandomResizedCrop((0.3, 1.0), (0.75, 4 / 3), 20)],
             'label': None}
    loader = _loader(datasets[0], 64, pipes)
    rrc = loader.graph.pipelines[0].ops[2]
    boxes = []
    orig = rrc.sample_crops
    rrc.sample_crops = lambda seed, h, w, out: (orig(seed, h, w, out), boxes.append(out.copy()))[0]
    got = next(iter(loader))[0].cpu().numpy()
    raw = next(iter(_loader(datasets[0], 64, {'image': [SimpleRGBImageDecoder()], 'label': None})))[0].cpu().numpy()
    assert got.shape == (64, 20, 20, 3)
    for i in range(64):
        r, c, h, w = (int(v) for v in boxes[0][i])
        assert np.array_equal(got[i], O.resize_area(raw[i], r, r + h, c, c + w, 20, 20))


def test_simple_decoder_rejects_variable_sizes(datasets):
    from ffcv_b200.fields.decoders import SimpleRGBImageDecoder
    with pytest.raises(TypeError):
        _loader(datasets[1], 16, {'image': [SimpleRGBImageDecoder()], 'label': None})


def test_partial_last_batch_and_drop_last(datasets):
    from ffcv_b200.fields.decoders import SimpleRGBImageDecoder
    pipes = {'image': [SimpleRGBImageDecoder()], 'label': None}
    loader = _loader(datasets[0], 1000, pipes, drop_last=False)
    sizes = [b[0].shape[0] for b in loader]
    assert sizes == [1000, 536]
    loader = _loader(datasets[0], 1000, pipes, drop_last=True)
    assert [b[0].shape[0] for b in loader] == [1000]


def test_corrupt_jpeg_is_reported_not_fatal(datasets, tmp_path):
    """A truncated stream must not hang or fault the GPU: the sample is flagged."""
    import shutil
    from ffcv_b200.fields.decoders import CenterCropRGBImageDecoder
    from ffcv_b200.reader import Reader
    path = str(tmp_path / 'broken.beton')
    shutil.copy(datasets[1], path)
    r = Reader(path)
    md = r.metadata['f0']
    row = int(np.where(r.alloc_table['ptr'] == md['data_ptr'][3])[0][0])
    with open(path, 'r+b') as fp:
        # halve the recorded size of sample 3 (its entropy data runs out), destroy sample 5's header
        entry = r.alloc_table[row:row + 1].copy()
        entry['size'] = int(entry['size'][0]) // 2
        fp.seek(int(r.header['alloc_table_ptr']) + row * r.alloc_table.dtype.itemsize)
        fp.write(entry.tobytes())
        fp.seek(int(md['data_ptr'][5]))
        fp.write(b'\x00\x00\x00\x00')
    pipes = {'image': [CenterCropRGBImageDecoder((64, 64), ratio=1.0)], 'label': None}
    loader = _loader(path, 16, pipes)
    it = iter(loader)
    batch = next(it)
    ch.cuda.synchronize()
    exe = image_executor(loader)
    status = exe.ctx.status(0, ch.cuda.current_stream().cuda_stream, 16)
    assert status[5] != 0 and status[3] != 0
    assert (np.delete(status, [3, 5]) == 0).all()
    assert batch[0].shape == (16, 64, 64, 3)


def test_file_on_memory_file_system_is_pinned_in_place(tmp_path):
    """A .beton on /dev/shm is page-locked where it lies (one copy for every process of the node);
    on disk the loader falls back to a private pinned copy.  Same pixels either way."""
    import shutil
    import uuid
    from ffcv_b200 import OrderOption
    from ffcv_b200.fields.decoders import RandomResizedCropRGBImageDecoder
    from ffcv_b200.synthetic import write_dataset_isolated
    from ffcv_b200.transforms import NormalizeImage, RandomHorizontalFlip, ToTorchImage
    if not (os.path.isdir('/dev/shm') and os.access('/dev/shm', os.W_OK)):
        pytest.skip('no writable /dev/shm')
    disk = write_dataset_isolated(2, str(tmp_path / 'c2.beton'), 48, num_workers=2)
    shm = f'/dev/shm/ffcv_b200_test_{uuid.uuid4().hex}.beton'
    shutil.copy(disk, shm)
    try:
        for path in (shm, disk):
            pipes = {'image': [RandomResizedCropRGBImageDecoder((96, 96)), RandomHorizontalFlip(),
                               NormalizeImage(IMAGENET_MEAN, IMAGENET_STD, np.float16), ToTorchImage()], 'label': None}
            loader = _loader(path, 16, pipes, order=OrderOption.QUASI_RANDOM, pin_file=True)
            mm = loader.memory_manager
            mm.open()
            assert mm.pinned
            # (the in-place lock is used where the driver grants it -- memory file systems -- else
            # the private pinned copy; which one a temporary directory gets depends on the machine)
            compare_epoch(loader)
            if loader._live_iterator is not None:
                loader._live_iterator.retire()
            del loader
    finally:
        os.remove(shm)


# ---- full-size batches, fixed-size JPEG datasets, several fields per sample ---------------------

@pytest.mark.parametrize('cfg,batch,res', [(2, 512, 224), (1, 1024, 160)])
def test_full_size_batches(tmp_path, cfg, batch, res):
    """One batch of the configuration's real size (512 x config 2, 1024 x config 1): the CTA sizes,
    subsequence lengths and grid shapes the benchmark runs with, checked against the oracle."""
    from ffcv_b200 import OrderOption
    from ffcv_b200.fields.decoders import RandomResizedCropRGBImageDecoder
    from ffcv_b200.synthetic import write_dataset_isolated as write_dataset
    from ffcv_b200.transforms import NormalizeImage, RandomHorizontalFlip, ToTorchImage
    path = write_dataset(cfg, str(tmp_path / f'c{cfg}_{batch}.beton'), batch, num_workers=8)
    pipes = {'image': [RandomResizedCropRGBImageDecoder((res, res)), RandomHorizontalFlip(),
                       NormalizeImage(IMAGENET_MEAN, IMAGENET_STD, np.float16), ToTorchImage()],
             'label': None}
    loader = _loader(path, batch, pipes, order=OrderOption.QUASI_RANDOM)
    assert compare_epoch(loader) == batch * res * res * 3
    status = image_executor(loader).ctx.status(0, ch.cuda.current_stream().cuda_stream, batch)
    assert (status == 0).all()


class _ManyFields:
    """(image, label, vector, weight, second image) samples with seeded content."""

    def __init__(self, n, h, w):
        self.n, self.h, self.w = n, h, w

    def __len__(self):
        return self.n

    def __getitem__(self, k):
        from ffcv_b200.synthetic import synth_content
        rng = np.random.default_rng([77, k])
        np.random.seed(k)
        return (synth_content(rng, self.h, self.w), int(rng.integers(0, 1000)),
                rng.standard_normal((5, 3)).astype(np.float32), float(rng.uniform()),
                synth_content(rng, self.h // 2, self.w // 2))


def _write_many_fields(path, n, h, w):
    """In a fresh interpreter: the writer forks, which a process that runs CUDA must not do."""
    import subprocess
    import sys
    code = ('import sys; sys.path[:0] = [%r, %r]; import numpy as np\n'
            'from test_gpu_pipeline import _ManyFields\n'
            'from ffcv_b200.fields import RGBImageField, IntField, NDArrayField, FloatField\n'
            'from ffcv_b200.writer import DatasetWriter\n'
            'DatasetWriter(%r, {"image": RGBImageField(write_mode="jpg"), "label": IntField(), '
            '"vec": NDArrayField(np.dtype("float32"), (5, 3)), "weight": FloatField(), '
            '"mask": RGBImageField(write_mode="proportion")}, num_workers=4).from_indexed_dataset(_ManyFields(%d, %d, %d))\n'
            % (os.path.dirname(os.path.dirname(os.path.abspath(__file__))), os.path.dirname(os.path.abspath(__file__)),
               path, n, h, w))
    subprocess.run([sys.executable, '-c', code], check=True, env=dict(os.environ, CUDA_VISIBLE_DEVICES=''))
    return path


def test_fixed_size_jpeg_labels_arrays_and_two_image_fields(tmp_path):
    """A fixed-size all-JPEG field through SimpleRGBImageDecoder; labels, a float field and an
    array field that ride in the image batch's staged bytes (one host->device transfer per batch);
    and a second image field, which must get a context of its own."""
    from ffcv_b200.fields.decoders import (FloatDecoder, IntDecoder, NDArrayDecoder, RandomResizedCropRGBImageDecoder,
                                           SimpleRGBImageDecoder)
    from ffcv_b200.reader import Reader
    from ffcv_b200.transforms import NormalizeImage, RandomHorizontalFlip, Squeeze, ToDevice, ToTensor, ToTorchImage
    n, h, w = 96, 72, 104
    path = _write_many_fields(str(tmp_path / 'many.beton'), n, h, w)
    dev = ch.device('cuda:0')
    pipes = {
        'image': [SimpleRGBImageDecoder(), RandomHorizontalFlip(), ToTensor(), ToDevice(dev), ToTorchImage(),
                  NormalizeImage(IMAGENET_MEAN, IMAGENET_STD, np.float16)],
        'label': [IntDecoder(), ToTensor(), ToDevice(dev), Squeeze()],
        'vec': [NDArrayDecoder(), ToTensor(), ToDevice(dev)],
        'weight': [FloatDecoder(), ToTensor(), ToDevice(dev)],
        'mask': [RandomResizedCropRGBImageDecoder((40, 40)), ToTensor(), ToDevice(dev), ToTorchImage()],
    }
    loader = _loader(path, 32, pipes)
    g = loader.graph
    by_name = {p.name: p for p in g.pipelines}
    assert all(by_name[k].rider_host is not None for k in ('label', 'vec', 'weight'))
    assert by_name['image'].executor.ctx is not by_name['mask'].executor.ctx
    r = Reader(path)
    mm = loader.memory_manager.open()
    truth_vec = np.stack([np.frombuffer(mm[int(p):int(p) + 60].tobytes(), np.float32).reshape(5, 3)
                          for p in r.metadata['f2']])
    labels, vecs, weights = [], [], []
    for batch in loader:
        assert all(t.device == dev for t in batch)
        labels.append(batch[1].clone())
        vecs.append(batch[2].clone())
        weights.append(batch[3].clone())
    assert labels[0].shape == (32,) and vecs[0].shape == (32, 5, 3) and weights[0].shape == (32, 1)
    assert np.array_equal(ch.cat(labels).cpu().numpy(), r.metadata['f1'])
    assert np.array_equal(ch.cat(vecs).cpu().numpy(), truth_vec)
    assert np.array_equal(ch.cat(weights).cpu().numpy().ravel(), r.metadata['f3'])
    # the riders add their bytes to the image batch's one transfer and nothing else is copied
    # (one batch per epoch, so that both loaders have staged the same samples when asked)
    full = _loader(path, n, pipes)
    bare = _loader(path, n, {'image': pipes['image'], 'label': None, 'vec': None, 'weight': None, 'mask': None})
    for ld in (full, bare):
        for _ in ld:
            pass
    extra = image_executor(full).h2d_bytes - image_executor(bare).h2d_bytes
    assert n * (8 + 60 + 8) <= extra <= n * (8 + 60 + 8) + 4 * 64
    # pixels of both image fields against the oracle (fresh loaders: every epoch redraws)
    assert compare_epoch(_loader(path, 32, pipes), field_pos=0, field='image') == n * h * w * 3
    assert compare_epoch(_loader(path, 32, pipes), field_pos=4, field='mask') == n * 40 * 40 * 3


def _resident_fraction(path):
    """Share of the file's pages that the page cache holds (mincore over a mapping)."""
    import ctypes
    import mmap
    size = os.path.getsize(path)
    with open(path, 'rb') as fp:
        mm = mmap.mmap(fp.fileno(), 0, prot=mmap.PROT_READ)
    pages = (size + mmap.PAGESIZE - 1) // mmap.PAGESIZE
    vec = (ctypes.c_ubyte * pages)()
    libc = ctypes.CDLL(None, use_errno=True)
    arr = np.frombuffer(mm, dtype=np.uint8)
    rc = libc.mincore(ctypes.c_void_p(arr.ctypes.data), ctypes.c_size_t(size), vec)
    frac = sum(v & 1 for v in vec) / pages if rc == 0 else None
    del arr
    mm.close()
    return frac


@pytest.mark.parametrize('direct_io', [True, False], ids=['o_direct', 'buffered'])
def test_larger_than_ram_path_reads_straight_into_pinned_buffers(tmp_path, direct_io):
    """Loader(os_cache=False): nothing is mapped, the staging threads pread every batch into the
    slot's pinned buffer (O_DIRECT where the file system takes it, else buffered reads whose pages
    are dropped again).  Same pixels and labels; the page cache does not fill up with the file."""
    from ffcv_b200 import OrderOption
    from ffcv_b200.fields.decoders import IntDecoder, RandomResizedCropRGBImageDecoder
    from ffcv_b200.memory_managers import DirectReadManager
    from ffcv_b200.synthetic import write_dataset_isolated as write_dataset
    from ffcv_b200.transforms import NormalizeImage, RandomHorizontalFlip, Squeeze, ToDevice, ToTensor, ToTorchImage
    path = write_dataset(2, str(tmp_path / 'c2_direct.beton'), 160, num_workers=8)
    dev = ch.device('cuda:0')
    pipes = {'image': [RandomResizedCropRGBImageDecoder((224, 224)), RandomHorizontalFlip(),
                       NormalizeImage(IMAGENET_MEAN, IMAGENET_STD, np.float16), ToTorchImage()],
             'label': [IntDecoder(), ToTensor(), ToDevice(dev), Squeeze()]}
    os.sync()  # freshly written pages are dirty, and dirty pages cannot be dropped
    fd = os.open(path, os.O_RDONLY)
    os.posix_fadvise(fd, 0, 0, os.POSIX_FADV_DONTNEED)
    os.close(fd)
    before = _resident_fraction(path)
    loader = _loader(path, 32, pipes, order=OrderOption.QUASI_RANDOM, os_cache=False)
    assert isinstance(loader.memory_manager, DirectReadManager)
    loader.memory_manager.direct_io = direct_io
    labels = []
    exe = image_executor(loader)
    exe.param_log = []
    for b in loader:
        labels.append(b[1].clone())
    order = np.concatenate([ix for (_, _, ix, _) in exe.param_log])
    exe.param_log = None
    assert np.array_equal(ch.cat(labels).cpu().numpy(), loader.reader.metadata['f1'][order])
    after = _resident_fraction(path)
    compare_epoch(loader)
    # On a file system that can drop clean pages (not tmpfs) an epoch leaves the cache as it found it.
    if before is not None and after is not None and before < 0.5:
        assert after < before + 0.15, (before, after)


@pytest.mark.parametrize('cfg,res,batch', [(4, 384, 3), (2, 96, 32), (1, 48, 64)])
def test_dct_domain_downscale_option(datasets, cfg, res, batch):
    """`dct_downscale=True`: JPEG samples whose crop box is at least twice the output size are
    decoded at 1/2, 1/4 or 1/8 scale and resized from the scaled image; raw samples and small crops
    are untouched.  Checked against the oracle, which applies the same rule with its own scaled
    decode (pinned on libjpeg-turbo's)."""
    from ffcv_b200 import OrderOption
    from ffcv_b200.fields.decoders import RandomResizedCropRGBImageDecoder
    from ffcv_b200.transforms import NormalizeImage, RandomHorizontalFlip, ToTorchImage
    pipes = {'image': [RandomResizedCropRGBImageDecoder((res, res), scale=(0.25, 1), dct_downscale=True),
                       RandomHorizontalFlip(), NormalizeImage(IMAGENET_MEAN, IMAGENET_STD, np.float16), ToTorchImage()],
             'label': None}
    loader = _loader(datasets[cfg], batch, pipes, order=OrderOption.QUASI_RANDOM)
    exe = image_executor(loader)
    assert exe.plan.dct_scale == -1
    compare_epoch(loader)
    # the rule did select reduced scales for part of the samples
    p = exe.last_params
    assert ((p[:, 2] >> 1) >= res).any() and ((p[:, 3] >> 1) >= res).any()
    # and the result is not the full-scale pipeline's (the option changes pixels: it is opt-in)
    plain = {'image': [RandomResizedCropRGBImageDecoder((res, res), scale=(0.25, 1)), RandomHorizontalFlip(),
                       NormalizeImage(IMAGENET_MEAN, IMAGENET_STD, np.float16), ToTorchImage()], 'label': None}
    a = next(iter(_loader(datasets[cfg], batch, pipes, order=OrderOption.QUASI_RANDOM)))[0]
    b = next(iter(_loader(datasets[cfg], batch, plain, order=OrderOption.QUASI_RANDOM)))[0]
    assert a.shape == b.shape and not ch.equal(a, b)
    assert (a.float() - b.float()).abs().mean() < 0.1  # same picture, different rounding path


@pytest.mark.parametrize('cfg,res,batch,epochs', [(2, 224, 32, 3), (1, 160, 64, 3), (4, 384, 3, 3)])
def test_decode_index_gives_the_same_pixels(datasets, cfg, res, batch, epochs):
    """`Loader(decode_index_gb=...)`: the first decode of a JPEG sample records the decoder states at
    the start of its subsequences, later epochs decode it in one pass from them.  Every epoch must
    still equal the oracle bit for bit (crops differ from epoch to epoch, so entries recorded for a
    small crop get extended by larger ones), and the index must actually be used."""
    from ffcv_b200 import OrderOption
    from ffcv_b200.fields.decoders import RandomResizedCropRGBImageDecoder
    from ffcv_b200.transforms import NormalizeImage, RandomHorizontalFlip, ToTorchImage
    pipes = {'image': [RandomResizedCropRGBImageDecoder((res, res)), RandomHorizontalFlip(),
                       NormalizeImage(IMAGENET_MEAN, IMAGENET_STD, np.float16), ToTorchImage()],
             'label': None}
    loader = _loader(datasets[cfg], batch, pipes, order=OrderOption.RANDOM, decode_index_gb=0.05, batches_ahead=1)
    ctx = image_executor(loader).ctx
    seen = []
    for _ in range(epochs):
        compare_epoch(loader)
        ch.cuda.synchronize()
        seen.append(ctx.decode_index_stats())
    n_jpeg = int((loader.reader.metadata['f0']['mode'] == 0).sum())
    assert seen[0]['recorded'] >= 1 and seen[-1]['entries'] >= min(n_jpeg, 1)
    assert seen[-1]['used'] > seen[0]['used'] and seen[-1]['used'] >= n_jpeg // 2, seen
    status = ctx.status(0, ch.cuda.current_stream().cuda_stream, 1)
    assert (status == 0).all()
