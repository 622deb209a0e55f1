"""Seeded synthetic images standing in for ImageNet / CIFAR records.

Image ``k`` of a configuration draws everything from ``np.random.default_rng([cfg_id, k])``:
short side uniform in ``[lo, hi]``, aspect ratio log-uniform in ``[r_lo, r_hi]``, orientation by a
fair coin, and per channel a smooth field ``128 + sum_m a_m sin(2 pi (cx_m x / W + cy_m y / H) +
phi_m)`` of 8 low-frequency sinusoids (``a ~ U(8, 32)``, ``cx, cy ~ U(-4, 4)`` cycles,
``phi ~ U(0, 2 pi)``) plus Gaussian noise ``sigma = 8``, rounded and clipped to uint8.
"""
import os

import numpy as np


def synth_shape(rng, short_lo, short_hi, ratio_lo, ratio_hi):
    short = int(rng.integers(short_lo, short_hi + 1))
    ratio = float(np.exp(rng.uniform(np.log(ratio_lo), np.log(ratio_hi))))
    long_side = int(round(short * max(ratio, 1.0 / ratio)))
    if rng.random() < 0.5:
        return short, long_side  # (h, w): landscape
    return long_side, short


def synth_content(rng, h, w, noise_sigma=8.0):
    ys = np.arange(h, dtype=np.float32)[:, None] / np.float32(h)
    xs = np.arange(w, dtype=np.float32)[None, :] / np.float32(w)
    img = np.empty((h, w, 3), dtype=np.float32)
    for c in range(3):
        acc = np.full((h, w), 128.0, dtype=np.float32)
        for _ in range(8):
            a = np.float32(rng.uniform(8, 32))
            cx, cy = rng.uniform(-4, 4, 2)
            ph = np.float32(rng.uniform(0, 2 * np.pi))
            acc += a * np.sin(np.float32(2 * np.pi) * (np.float32(cx) * xs + np.float32(cy) * ys) + ph)
        img[..., c] = acc
    if noise_sigma > 0:
        img += rng.standard_normal(img.shape, dtype=np.float32) * np.float32(noise_sigma)
    return np.clip(np.rint(img), 0, 255).astype(np.uint8)


def synth_image(cfg_id, k, short_lo, short_hi, ratio_lo=0.75, ratio_hi=4 / 3, noise_sigma=8.0):
    """Returns (image uint8 [h, w, 3], label rng) for sample ``k`` of configuration ``cfg_id``."""
    rng = np.random.default_rng([cfg_id, k])
    h, w = synth_shape(rng, short_lo, short_hi, ratio_lo, ratio_hi)
    return synth_content(rng, h, w, noise_sigma), rng


# ---------------------------------------------------------------------------------------------
# The five benchmark configurations as seeded synthetic datasets.

CONFIGS = {
    # id: image shape law, field arguments, label range
    0: dict(name='cifar_raw', fixed=(32, 32), field=dict(write_mode='raw'), labels=10, count=50_000),
    1: dict(name='imagenet_lowres_jpg', short=(200, 256), ratio=(3 / 4, 4 / 3),
            field=dict(write_mode='jpg', jpeg_quality=90, max_resolution=256), labels=1000, count=100_000),
    2: dict(name='imagenet_fullres_mix', short=(300, 500), ratio=(3 / 4, 4 / 3),
            field=dict(write_mode='proportion', compress_probability=0.5, jpeg_quality=90,
                       max_resolution=500), labels=1000, count=200_000),
    3: dict(name='imagenet_val_jpg', short=(200, 256), ratio=(3 / 4, 4 / 3),
            field=dict(write_mode='jpg', jpeg_quality=90, max_resolution=256), labels=1000, count=50_000),
    4: dict(name='highres_444', short=(1024, 1536), ratio=(3 / 4, 16 / 9),
            field=dict(write_mode='jpg', jpeg_quality=95), labels=1000, count=20_000, sampling=444),
}


class SyntheticImageDataset:
    """Indexed dataset of (image, label) for one configuration.  ``__getitem__`` also seeds numpy's
    global generator from the sample index, which makes the writer's 'proportion' coin
    (``np.random.rand() < compress_probability``) reproducible."""

    def __init__(self, cfg_id, count=None):
        self.cfg_id = cfg_id
        self.cfg = CONFIGS[cfg_id]
        self.count = self.cfg['count'] if count is None else int(count)

    def __len__(self):
        return self.count

    def __getitem__(self, k):
        cfg = self.cfg
        rng = np.random.default_rng([self.cfg_id, k])
        if 'fixed' in cfg:
            h, w = cfg['fixed']
            img = rng.integers(0, 256, (h, w, 3), dtype=np.uint8)
        else:
            h, w = synth_shape(rng, cfg['short'][0], cfg['short'][1], cfg['ratio'][0], cfg['ratio'][1])
            img = synth_content(rng, h, w)
        label = int(rng.integers(0, cfg['labels']))
        np.random.seed((self.cfg_id * 1_000_003 + k) % (2 ** 32))
        return img, label


def _field_444_class():
    from .fields import RGBImageField

    class RGBImageField444(RGBImageField):
        """Same metadata and payload kinds; JPEG written without chroma subsampling."""

        def encode_jpeg(self, image):
            import cv2
            flags = [int(cv2.IMWRITE_JPEG_QUALITY), self.jpeg_quality,
                     int(cv2.IMWRITE_JPEG_SAMPLING_FACTOR), int(cv2.IMWRITE_JPEG_SAMPLING_FACTOR_444)]
            if self.jpeg_restart_interval:
                flags += [int(cv2.IMWRITE_JPEG_RST_INTERVAL), self.jpeg_restart_interval]
            ok, res = cv2.imencode('.jpg', cv2.cvtColor(image, cv2.COLOR_RGB2BGR), flags)
            if not ok:
                raise ValueError("Impossible to encode image in jpeg")
            return res.reshape(-1)
    return RGBImageField444


RGBImageField444 = None


def make_field(cfg_id, restart_interval=0):
    from .fields import RGBImageField
    global RGBImageField444
    cfg = CONFIGS[cfg_id]
    if cfg.get('sampling') == 444:
        if RGBImageField444 is None:
            RGBImageField444 = _field_444_class()
            RGBImageField444.__qualname__ = 'RGBImageField444'  # picklable by module attribute
        return RGBImageField444(**cfg['field'], jpeg_restart_interval=restart_interval)
    return RGBImageField(**cfg['field'], jpeg_restart_interval=restart_interval)


def write_dataset(cfg_id, path, count=None, num_workers=-1, page_size=None, restart_interval=0):
    """Writes ``count`` samples (default: the configuration's full size) of a configuration;
    ``restart_interval`` > 0 writes the JPEG samples with a restart marker every that many MCUs."""
    from .fields import IntField
    from .writer import DatasetWriter
    kwargs = {} if page_size is None else {'page_size': page_size}
    if cfg_id == 4 and page_size is None:
        kwargs['page_size'] = 1 << 25  # 4:4:4 q95 images of ~2-4 MB: 32 MiB pages waste less
    writer = DatasetWriter(path, {'image': make_field(cfg_id, restart_interval), 'label': IntField()},
                           num_workers=num_workers, **kwargs)
    writer.from_indexed_dataset(SyntheticImageDataset(cfg_id, count), chunksize=16)
    return path


def write_dataset_isolated(cfg_id, path, count=None, num_workers=-1, page_size=None, restart_interval=0):
    """`write_dataset` in a fresh interpreter.  The writer forks its workers (as the reference's
    does); forking a process that already runs CUDA, NCCL or thread pools can deadlock the children,
    so programs that have initialised any of those write their datasets through this call."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = ('import sys; sys.path.insert(0, %r); from ffcv_b200.synthetic import write_dataset; '
            'write_dataset(%r, %r, %r, %r, %r, %r)' % (root, cfg_id, path, count, num_workers, page_size, restart_interval))
    env = dict(os.environ, CUDA_VISIBLE_DEVICES='')
    subprocess.run([sys.executable, '-c', code], check=True, env=env)
    return path


def replicate_samples(path, count):
    """Rewrites the tables of a freshly written file so that it presents ``count`` samples that
    cycle through the distinct samples already stored (sample k points at the payload of sample
    k mod distinct).  Lets a benchmark run epochs of a configuration's real length over a bounded
    set of distinct images; the payload pages are untouched."""
    from .reader import Reader
    from .types import ALLOC_TABLE_TYPE, FieldDescType, HeaderType
    r = Reader(path)
    distinct = r.num_samples
    if count <= distinct:
        return path
    reps = -(-count // distinct)
    metadata = np.tile(r.metadata, reps)[:count]
    first_payload = int(r.alloc_table['ptr'].min())
    header_bytes = HeaderType.itemsize + FieldDescType.itemsize * r.num_fields + metadata.nbytes
    if header_bytes > first_payload:
        raise ValueError('metadata of the replicated samples does not fit before the first data page')
    order = np.argsort(r.alloc_table['sample_id'], kind='stable')
    base = r.alloc_table[order]
    table = np.tile(base, reps)
    table['sample_id'] = np.repeat(np.arange(reps, dtype=np.uint64), len(base)) * np.uint64(distinct) + table['sample_id']
    table = table[table['sample_id'] < count]
    header = np.array(r.header)
    header['num_samples'] = count
    with open(path, 'r+b') as fp:
        fp.seek(0)
        fp.write(header.tobytes())
        fp.seek(HeaderType.itemsize + FieldDescType.itemsize * r.num_fields)
        fp.write(metadata.tobytes())
        fp.seek(int(r.header['alloc_table_ptr']))
        fp.write(table.astype(ALLOC_TABLE_TYPE).tobytes())
        fp.truncate()
    return path
