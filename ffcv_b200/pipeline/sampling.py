"""Per-batch random parameters, drawn on the host and handed to the GPU as a table.

The reference draws inside numba ``prange`` bodies (``ffcv/fields/rgb_image.py:205``,
``transforms/flip.py:32``, ``translate.py:40-41``, ``cutout.py:39-42``), so its results depend on
thread scheduling.  Here each operation of each batch seeds numba's ``np.random`` stream once and
then draws serially, sample 0 first, with the same calls in the same order as the reference's
per-sample code.  The seed is a function of (loader seed, epoch, batch index, operation index),
so a run is reproducible and the oracle can be fed the very same table.
"""
import numpy as np
from numba import njit

_JIT = dict(fastmath=True, nogil=True, error_model='numpy', cache=True)


def batch_seed(base_seed, epoch, batch_ix, op_ix):
    """32-bit seed for one operation of one batch (SplitMix64-style mixing)."""
    x = (int(base_seed) * 0x9E3779B97F4A7C15 + int(epoch) * 0xBF58476D1CE4E5B9 +
         int(batch_ix) * 0x94D049BB133111EB + int(op_ix) * 0xD6E8FEB86659FD93) & 0xFFFFFFFFFFFFFFFF
    x ^= x >> 30
    x = (x * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
    x ^= x >> 27
    x = (x * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
    x ^= x >> 31
    return int(x & 0xFFFFFFFF)


@njit(**_JIT)
def _random_crop(height, width, scale, ratio):
    # torchvision-style RandomResizedCrop box, as ffcv/fields/rgb_image.py:48-72 draws it:
    # up to 10 attempts of (area fraction, log-uniform aspect), then a ratio-clamped centre crop.
    area = height * width
    log_ratio = np.log(ratio)
    for _ in range(10):
        target_area = area * np.random.uniform(scale[0], scale[1])
        aspect_ratio = np.exp(np.random.uniform(log_ratio[0], log_ratio[1]))
        w = int(round(np.sqrt(target_area * aspect_ratio)))
        h = int(round(np.sqrt(target_area / aspect_ratio)))
        if 0 < w <= width and 0 < h <= height:
            i = int(np.random.uniform(0, height - h + 1))
            j = int(np.random.uniform(0, width - w + 1))
            return i, j, h, w
    in_ratio = float(width) / float(height)
    if in_ratio < min(ratio):
        w = width
        h = int(round(w / min(ratio)))
    elif in_ratio > max(ratio):
        h = height
        w = int(round(h * max(ratio)))
    else:
        w = width
        h = height
    i = (height - h) // 2
    j = (width - w) // 2
    return i, j, h, w


@njit(**_JIT)
def sample_random_crops(seed, heights, widths, scale, ratio, out):
    np.random.seed(seed)
    for k in range(heights.shape[0]):
        i, j, h, w = _random_crop(np.uint32(heights[k]), np.uint32(widths[k]), scale, ratio)
        out[k, 0] = i
        out[k, 1] = j
        out[k, 2] = h
        out[k, 3] = w


@njit(**_JIT)
def sample_center_crops(heights, widths, ratio, out):
    # ffcv/fields/rgb_image.py:75-81
    for k in range(heights.shape[0]):
        height = np.uint32(heights[k])
        width = np.uint32(widths[k])
        s = min(height, width)
        c = int(ratio * s)
        out[k, 0] = (height - c) // 2
        out[k, 1] = (width - c) // 2
        out[k, 2] = c
        out[k, 3] = c


@njit(**_JIT)
def sample_flips(seed, n, flip_prob, out):
    # one vector draw per batch, ffcv/transforms/flip.py:32
    np.random.seed(seed)
    should_flip = np.random.rand(n) < flip_prob
    for k in range(n):
        out[k, 0] = 1 if should_flip[k] else 0
        out[k, 1] = 0


@njit(**_JIT)
def sample_translations(seed, n, pad, out):
    # y first, then x, ffcv/transforms/translate.py:40-41
    np.random.seed(seed)
    for k in range(n):
        out[k, 0] = np.random.randint(low=0, high=2 * pad + 1)
        out[k, 1] = np.random.randint(low=0, high=2 * pad + 1)


@njit(**_JIT)
def sample_cutouts(seed, n, height, width, crop_size, out):
    # ffcv/transforms/cutout.py:39-42
    np.random.seed(seed)
    for k in range(n):
        out[k, 0] = np.random.randint(height - crop_size + 1)
        out[k, 1] = np.random.randint(width - crop_size + 1)


@njit(**_JIT)
def sample_jitter(seed, n, p, low, high, apply, ratio):
    # the two vector draws of ffcv/transforms/color_jitter.py:44-45 (:86-87, :124-125), in that order
    np.random.seed(seed)
    chosen = np.random.rand(n) < p
    magnitudes = np.random.uniform(low, high, n)
    for k in range(n):
        apply[k] = 1 if chosen[k] else 0
        ratio[k] = magnitudes[k]


@njit(**_JIT)
def sample_mixup(seed, alpha, same_lambda, out):
    # ffcv/transforms/mixup.py:42-45 (:76-79): seeded with the last sample index of the batch, one
    # beta draw for the whole batch or one per sample
    np.random.seed(seed)
    n = out.shape[0]
    if same_lambda:
        lam = np.random.beta(alpha, alpha)
        for k in range(n):
            out[k] = lam
    else:
        lams = np.random.beta(alpha, alpha, n)
        for k in range(n):
            out[k] = lams[k]
