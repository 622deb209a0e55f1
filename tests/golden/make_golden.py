"""Generates tests/golden/*.npz.  Needs a checkout of the reference (libffcv/ffcv), cv2 and Pillow:

    python tests/golden/make_golden.py --reference <path of the ffcv checkout> [pixel]

jpeg_cases.npz    JPEG streams written by cv2.imencode (the call the reference's writer makes,
                  ffcv/fields/rgb_image.py:26-34) with their pixels as decoded by real libjpeg-turbo
                  binaries: `turbo_fast_fancy_*` = Pillow's bundled libjpeg-turbo driven through
                  the libjpeg API with dct_method = JDCT_IFAST and fancy upsampling on, i.e. the
                  configuration of the reference's TurboJPEG call (tests/libjpeg_direct.py);
                  `fast_replicate_*` = Pillow with decoder config (scale 1, draft 1) = fast integer
                  IDCT + replicated chroma; `accurate_fancy_*` = cv2.imdecode = accurate IDCT +
                  triangle ("fancy") upsampling.
jpeg_scaled_cases.npz the same streams decoded at 1/2, 1/4 and 1/8 scale by that library with the
                  fast integer IDCT selected (what TurboJPEG does with a scaling factor).
resize_cases.npz  inputs and outputs of cv2.resize(INTER_AREA), the call of libffcv.cpp:40-41.
crop_cases.npz    crop boxes from the reference's own get_random_crop / get_center_crop
                  (function source taken from ffcv/fields/rgb_image.py of the checkout at
                  generation time, run under numpy's legacy seeded stream).
normalize_cases.npz lookup tables built by the reference's NormalizeImage expression
                  (ffcv/transforms/normalize.py:42-43).
pixel_cases.npz   outputs of the reference's own RandomBrightness / RandomContrast /
                  RandomSaturation / ImageMixup / LabelMixup / Poison closures
                  (ffcv/transforms/color_jitter.py, mixup.py, poisoning.py), imported from
                  the checkout and compiled by the reference's Compiler with one thread (with
                  more, numba parallelises even the per-batch random draws and the result is not
                  reproducible), numba's random stream seeded before each call; the draws
                  themselves (made by the same calls in the same order) are stored beside them.
"""
import ast
import io
import os

import sys

import cv2
import numpy as np
from PIL import Image

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import libjpeg_direct  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
REF_ROOT = None  # set from --reference


def smooth(rng, h, w):
    y, x = np.mgrid[0:h, 0:w]
    img = np.zeros((h, w, 3))
    for c in range(3):
        v = 128.0
        for _ in range(8):
            a = rng.uniform(8, 32)
            cx, cy = rng.uniform(-4, 4, 2)
            ph = rng.uniform(0, 2 * np.pi)
            v = v + a * np.sin(2 * np.pi * (cx * x / w + cy * y / h) + ph)
        img[..., c] = v
    img += rng.normal(0, 8, img.shape)
    return np.clip(np.rint(img), 0, 255).astype(np.uint8)


def pil_draft(buf):
    im = Image.open(io.BytesIO(buf.tobytes()))
    im.decoderconfig = (1, 1)
    im.load()
    return np.array(im)


def jpeg_cases():
    rng = np.random.default_rng(2024)
    out = {}
    specs = [(48, 64, 90, 420, 0, 'smooth'), (37, 53, 90, 420, 0, 'smooth'), (17, 9, 75, 420, 0, 'noise'),
             (8, 8, 90, 420, 0, 'smooth'), (1, 1, 90, 420, 0, 'noise'), (3, 5, 90, 420, 0, 'noise'),
             (40, 56, 95, 444, 0, 'smooth'), (33, 31, 50, 444, 0, 'noise'), (30, 41, 90, 422, 0, 'smooth'),
             (64, 64, 100, 420, 0, 'binary'), (32, 32, 100, 444, 0, 'noise'), (50, 70, 90, 420, 3, 'smooth'),
             (45, 35, 90, 444, 5, 'noise'), (90, 120, 90, 420, 0, 'smooth')]
    for k, (h, w, q, samp, rst, kind) in enumerate(specs):
        if kind == 'noise':
            img = rng.integers(0, 256, (h, w, 3), dtype=np.uint8)
        elif kind == 'binary':
            img = (rng.integers(0, 2, (h, w, 3)) * 255).astype(np.uint8)
        else:
            img = smooth(rng, h, w)
        p = [cv2.IMWRITE_JPEG_QUALITY, q]
        if samp == 444:
            p += [cv2.IMWRITE_JPEG_SAMPLING_FACTOR, cv2.IMWRITE_JPEG_SAMPLING_FACTOR_444]
        if samp == 422:
            p += [cv2.IMWRITE_JPEG_SAMPLING_FACTOR, cv2.IMWRITE_JPEG_SAMPLING_FACTOR_422]
        if rst:
            p += [cv2.IMWRITE_JPEG_RST_INTERVAL, rst]
        ok, buf = cv2.imencode('.jpg', img[..., ::-1], p)
        buf = buf.reshape(-1)
        out[f'jpeg_{k}'] = buf
        out[f'fast_replicate_{k}'] = pil_draft(buf)
        out[f'accurate_fancy_{k}'] = np.ascontiguousarray(cv2.imdecode(buf, cv2.IMREAD_COLOR)[..., ::-1])
        out[f'turbo_fast_fancy_{k}'] = libjpeg_direct.decode(buf, libjpeg_direct.JDCT_IFAST, True)
    out['count'] = np.array(len(specs))
    np.savez_compressed(os.path.join(HERE, 'jpeg_cases.npz'), **out)


def jpeg_scaled_cases():
    """The streams of jpeg_cases.npz decoded at 1/2, 1/4 and 1/8 by Pillow's libjpeg-turbo through the
    libjpeg API (scale_num / scale_denom, fast integer IDCT selected, fancy upsampling on)."""
    z = np.load(os.path.join(HERE, 'jpeg_cases.npz'))
    out = {}
    kept = 0
    for k in range(int(z['count'])):
        buf = z[f'jpeg_{k}']
        for denom in (2, 4, 8):
            out[f'scaled_{k}_{denom}'] = libjpeg_direct.decode(buf, libjpeg_direct.JDCT_IFAST, True, denom)
        kept += 1
    out['count'] = np.array(kept)
    np.savez_compressed(os.path.join(HERE, 'jpeg_scaled_cases.npz'), **out)


def resize_cases():
    rng = np.random.default_rng(7)
    out = {}
    specs = [(40, 50, 0, 40, 0, 50, 40, 50), (64, 96, 0, 64, 0, 96, 32, 48), (66, 99, 3, 63, 4, 94, 20, 30),
             (96, 96, 0, 96, 0, 96, 32, 32), (96, 64, 0, 96, 0, 64, 32, 32), (70, 90, 5, 65, 7, 80, 24, 24),
             (50, 60, 2, 47, 3, 55, 32, 32), (20, 30, 0, 20, 0, 30, 56, 56), (30, 80, 0, 30, 0, 80, 56, 40),
             (80, 30, 1, 79, 2, 29, 40, 56), (9, 9, 4, 5, 4, 5, 16, 16), (100, 120, 10, 90, 10, 110, 7, 13),
             (45, 45, 0, 45, 0, 45, 45, 30), (128, 160, 0, 128, 0, 160, 64, 32)]
    for k, (H, W, r0, r1, c0, c1, dh, dw) in enumerate(specs):
        src = rng.integers(0, 256, (H, W, 3), dtype=np.uint8)
        out[f'src_{k}'] = src
        out[f'box_{k}'] = np.array([r0, r1, c0, c1, dh, dw])
        out[f'dst_{k}'] = cv2.resize(src[r0:r1, c0:c1], (dw, dh), interpolation=cv2.INTER_AREA)
    out['count'] = np.array(len(specs))
    np.savez_compressed(os.path.join(HERE, 'resize_cases.npz'), **out)


def reference_functions(names):
    REF = os.path.join(REF_ROOT, 'ffcv', 'fields', 'rgb_image.py')
    tree = ast.parse(open(REF).read())
    ns = {'np': np}
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in names:
            exec(compile(ast.Module([node], []), REF, 'exec'), ns)
    return [ns[n] for n in names]


def crop_cases():
    get_random_crop, get_center_crop = reference_functions(['get_random_crop', 'get_center_crop'])
    rng = np.random.default_rng(5)
    n = 64
    heights = rng.integers(20, 520, n).astype(np.uint16)
    widths = rng.integers(20, 520, n).astype(np.uint16)
    heights[:4] = [500, 20, 300, 33]
    widths[:4] = [20, 500, 300, 500]
    out = {'heights': heights, 'widths': widths}
    for name, seed, scale, ratio in [('default', 123, (0.08, 1.0), (0.75, 4 / 3)),
                                     ('quarter', 9, (0.25, 1.0), (0.75, 4 / 3))]:
        np.random.seed(seed)
        boxes = [get_random_crop(np.uint32(h), np.uint32(w), np.array(scale), np.array(ratio))
                 for h, w in zip(heights, widths)]
        out[f'random_{name}'] = np.array(boxes, dtype=np.int64)
        out[f'random_{name}_args'] = np.array([seed, *scale, *ratio])
    for r in (224 / 256, 1.0, 0.5):
        boxes = [get_center_crop(np.uint32(h), np.uint32(w), None, r) for h, w in zip(heights, widths)]
        out[f'center_{r:.4f}'] = np.array(boxes, dtype=np.int64)
    np.savez_compressed(os.path.join(HERE, 'crop_cases.npz'), **out)


def normalize_cases():
    out = {}
    for name, mean, std in [('imagenet', np.array([0.485, 0.456, 0.406]) * 255, np.array([0.229, 0.224, 0.225]) * 255),
                            ('cifar', np.array([125.3, 123.0, 113.9]), np.array([63.0, 62.1, 66.7]))]:
        for dt in (np.float16, np.float32):
            # the expression of ffcv/transforms/normalize.py:42-43
            table = (np.arange(256)[:, None] - mean[None, :]) / std[None, :]
            out[f'{name}_{np.dtype(dt).name}'] = table.astype(dt)
        out[f'{name}_mean'] = mean
        out[f'{name}_std'] = std
    np.savez_compressed(os.path.join(HERE, 'normalize_cases.npz'), **out)


def import_reference_transforms():
    """The reference's transform modules without its package __init__ (which loads the compiled
    extension that cannot be built here): a bare package object pointing at its source tree."""
    import importlib
    import types
    pkg = types.ModuleType('ffcv')
    pkg.__path__ = [os.path.join(REF_ROOT, 'ffcv')]
    sys.modules['ffcv'] = pkg
    stub = types.ModuleType('ffcv.libffcv')
    stub.ctypes_resize = stub.imdecode = stub.memcpy = stub.resize_crop = None
    sys.modules['ffcv.libffcv'] = stub
    importlib.import_module('ffcv.pipeline')
    mods = [importlib.import_module('ffcv.transforms.' + m) for m in ('color_jitter', 'mixup', 'poisoning')]
    from ffcv.pipeline.compiler import Compiler
    Compiler.set_enabled(True)
    Compiler.set_num_threads(1)
    return mods, Compiler


def pixel_cases():
    from numba import njit
    (cj, mx, po), Compiler = import_reference_transforms()

    @njit
    def seed_numba(s):
        np.random.seed(s)

    # the draw helpers are compiled by the reference's own Compiler (fastmath etc.), like the closures
    def jitter_draws(s, n, p, lo, hi):
        np.random.seed(s)
        apply = np.random.rand(n) < p
        mags = np.random.uniform(lo, hi, n)
        return apply, mags

    def beta_draws(s, alpha, n):
        np.random.seed(s)
        return np.random.beta(alpha, alpha, n)

    def beta_draw(s, alpha):
        np.random.seed(s)
        return np.random.beta(alpha, alpha)

    jitter_draws, beta_draws, beta_draw = (Compiler.compile(f) for f in (jitter_draws, beta_draws, beta_draw))

    rng = np.random.default_rng(77)
    n, h, w = 10, 24, 28
    images = np.stack([smooth(rng, h, w) for _ in range(n)])
    images[1] = rng.integers(0, 256, (h, w, 3), dtype=np.uint8)
    images[2] = 255
    images[3] = 0
    out = {'images': images}
    k = 0
    for cls, name in [(cj.RandomBrightness, 'brightness'), (cj.RandomContrast, 'contrast'),
                      (cj.RandomSaturation, 'saturation')]:
        for magnitude, p, seed in [(0.5, 0.7, 11), (1.5, 1.0, 12), (0.1, 0.5, 13)]:
            code = Compiler.compile(cls(magnitude, p).generate_code())
            seed_numba(seed)
            res = code(images.copy(), None)
            apply, mags = jitter_draws(seed, n, p, max(0, 1 - magnitude), 1 + magnitude)
            out[f'jitter_{k}_kind'] = np.array(name)
            out[f'jitter_{k}_args'] = np.array([magnitude, p, seed])
            out[f'jitter_{k}_apply'] = apply
            out[f'jitter_{k}_ratio'] = mags
            out[f'jitter_{k}_out'] = res
            k += 1
    out['jitter_count'] = np.array(k)
    k = 0
    for alpha, same, last_index in [(0.5, True, 41), (0.5, False, 42), (2.0, False, 43)]:
        indices = np.arange(last_index - n + 1, last_index + 1)
        code = Compiler.compile(mx.ImageMixup(alpha, same).generate_code())
        res = code(images.copy(), np.zeros_like(images), indices)
        labels = rng.integers(0, 1000, (n, 1)).astype(np.int64)
        lcode = Compiler.compile(mx.LabelMixup(alpha, same).generate_code())
        lres = lcode(labels.copy(), np.zeros((n, 3), np.float32), indices)
        lam = np.full(n, beta_draw(last_index, alpha)) if same else beta_draws(last_index, alpha, n)
        out[f'mixup_{k}_args'] = np.array([alpha, float(same), last_index])
        out[f'mixup_{k}_lam'] = lam
        out[f'mixup_{k}_out'] = res
        out[f'mixup_{k}_labels'] = labels
        out[f'mixup_{k}_labels_out'] = lres
        k += 1
    out['mixup_count'] = np.array(k)
    mask = rng.integers(0, 256, (h, w, 3)).astype(np.uint8)
    alpha = rng.uniform(0, 1, (h, w))
    alpha[:4] = 0
    alpha[-4:] = 1
    poisoned = np.array([2, 5, 103, 107])
    indices = np.arange(100, 100 + n)
    k = 0
    for clamp in [(0, 255), (30, 200)]:
        code = Compiler.compile(po.Poison(mask, alpha, poisoned, clamp).generate_code())
        res = code(images.copy(), np.zeros(images.shape, np.float32), indices)
        out[f'poison_{k}_clamp'] = np.array(clamp)
        out[f'poison_{k}_out'] = res
        k += 1
    out['poison_count'] = np.array(k)
    out['poison_mask'] = mask
    out['poison_alpha'] = alpha
    out['poison_indices'] = poisoned
    out['poison_batch_indices'] = indices
    np.savez_compressed(os.path.join(HERE, 'pixel_cases.npz'), **out)


if __name__ == '__main__':
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument('--reference', help='root of the libffcv/ffcv checkout (not needed for `scaled`)')
    ap.add_argument('what', nargs='?', default='all', choices=['all', 'pixel', 'scaled'])
    cli = ap.parse_args()
    if cli.what == 'scaled':
        jpeg_scaled_cases()
        raise SystemExit
    if not cli.reference:
        ap.error('--reference is required')
    REF_ROOT = os.path.abspath(cli.reference)
    if cli.what == 'pixel':
        pixel_cases()
        raise SystemExit
    jpeg_cases()
    jpeg_scaled_cases()
    resize_cases()
    crop_cases()
    normalize_cases()
    pixel_cases()
    for f in sorted(os.listdir(HERE)):
        print(f, os.path.getsize(os.path.join(HERE, f)))
