"""Seeded synthetic images standing in for ImageNet / CIFAR records.

Image ``k`` of a configuration draws everything from ``np.random.default_rng([cfg_id, k])``:
short side uniform in ``[lo, hi]``, aspect ratio log-uniform in ``[r_lo, r_hi]``, orientation by a
fair coin, and per channel a smooth field ``128 + sum_m a_m sin(2 pi (cx_m x / W + cy_m y / H) +
phi_m)`` of 8 low-frequency sinusoids (``a ~ U(8, 32)``, ``cx, cy ~ U(-4, 4)`` cycles,
``phi ~ U(0, 2 pi)``) plus Gaussian noise ``sigma = 8``, rounded and clipped to uint8.
"""
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
