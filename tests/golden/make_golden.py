"""Generates tests/golden/*.npz.  Run in a container that has /root/reference, cv2 and Pillow:

    python tests/golden/make_golden.py

jpeg_cases.npz    JPEG streams written by cv2.imencode (the call the reference's writer makes,
                  ffcv/fields/rgb_image.py:26-34) with their pixels as decoded by real libjpeg-turbo
                  binaries: `turbo_fast_fancy_*` = Pillow's bundled libjpeg-turbo driven through
                  the libjpeg API with dct_method = JDCT_IFAST and fancy upsampling on, i.e. the
                  configuration of the reference's TurboJPEG call (tests/libjpeg_direct.py);
                  `fast_replicate_*` = Pillow with decoder config (scale 1, draft 1) = fast integer
                  IDCT + replicated chroma; `accurate_fancy_*` = cv2.imdecode = accurate IDCT +
                  triangle ("fancy") upsampling.
resize_cases.npz  inputs and outputs of cv2.resize(INTER_AREA), the call of libffcv.cpp:40-41.
crop_cases.npz    crop boxes from the reference's own get_random_crop / get_center_crop
                  (function source taken from /root/reference/ffcv/fields/rgb_image.py at
                  generation time, run under numpy's legacy seeded stream).
normalize_cases.npz lookup tables built by the reference's NormalizeImage expression
                  (ffcv/transforms/normalize.py:42-43).
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
REF = '/root/reference/ffcv/fields/rgb_image.py'


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


if __name__ == '__main__':
    jpeg_cases()
    resize_cases()
    crop_cases()
    normalize_cases()
    for f in sorted(os.listdir(HERE)):
        print(f, os.path.getsize(os.path.join(HERE, f)))
