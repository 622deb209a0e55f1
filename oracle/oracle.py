"""Python face of the CPU oracle (``liboracle.so`` built from the C files beside this one).

TEST INFRASTRUCTURE ONLY.  Importers: ``tests/``, ``__graft_entry__.smoke()`` and the CPU
baseline legs of ``bench.py``.  The product package never imports this module.
"""
import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, 'liboracle.so')

IDCT_FAST, IDCT_ACCURATE = 0, 1
UPSAMPLE_FANCY, UPSAMPLE_REPLICATE = 0, 1
OP_FLIP, OP_TRANSLATE, OP_CUTOUT = 1, 2, 3
OUT_U8_NHWC, OUT_F16_NHWC, OUT_F16_NCHW, OUT_F32_NHWC, OUT_F32_NCHW = range(5)


def build(force=False):
    srcs = [os.path.join(HERE, f) for f in ('jpeg_oracle.c', 'resize_oracle.c', 'pipeline_oracle.c', 'pixel_oracle.c')]
    stale = force or not os.path.exists(LIB_PATH) or any(
        os.path.getmtime(s) > os.path.getmtime(LIB_PATH) for s in srcs)
    if stale:
        subprocess.run(['make', '-C', HERE, '-B', 'liboracle.so'], check=True, capture_output=True)
    return LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(LIB_PATH)
        vp, ci, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
        L.oracle_jpeg_info.argtypes = [vp, sz, vp]
        L.oracle_jpeg_num_blocks.argtypes = [vp, sz]
        L.oracle_jpeg_num_blocks.restype = ctypes.c_int64
        L.oracle_jpeg_coefficients.argtypes = [vp, sz, vp]
        L.oracle_jpeg_decode.argtypes = [vp, sz, vp, ci, ci, ci, ci]
        L.oracle_jpeg_decode_scaled.argtypes = [vp, sz, vp, ci, ci, ci]
        L.oracle_jpeg_scalable.argtypes = [vp, sz]
        L.oracle_resize_area.argtypes = [vp, ci, ci, ci, ci, ci, vp, ci, ci]
        L.oracle_resize_area.restype = None
        L.oracle_augment.argtypes = [vp, ci, ci, vp, ci, vp]
        L.oracle_augment.restype = None
        L.oracle_normalize.argtypes = [vp, ci, ci, vp, ci, vp]
        L.oracle_normalize.restype = None
        L.oracle_run_batch.argtypes = [ci, vp, vp, vp, ci, ci, vp, ci, vp, ci, vp, ci, vp]
        for name in ('oracle_brightness', 'oracle_contrast', 'oracle_saturation'):
            getattr(L, name).argtypes = [vp, ci, ci, ci, vp, vp]
            getattr(L, name).restype = None
        L.oracle_mixup.argtypes = [vp, vp, ci, sz, vp]
        L.oracle_mixup.restype = None
        L.oracle_poison.argtypes = [vp, ci, sz, vp, vp, vp, ctypes.c_double, ctypes.c_double]
        L.oracle_poison.restype = None
        _lib = L
    return _lib


def jpeg_info(buf):
    buf = np.ascontiguousarray(buf, dtype=np.uint8)
    info = np.zeros(8, dtype=np.int64)
    rc = lib().oracle_jpeg_info(buf.ctypes.data, buf.size, info.ctypes.data)
    if rc:
        raise ValueError(f'oracle_jpeg_info: {rc}')
    keys = ('width', 'height', 'ncomp', 'hs', 'vs', 'restart_interval', 'scan_off', 'scan_len')
    return dict(zip(keys, (int(v) for v in info)))


def jpeg_decode(buf, idct=IDCT_FAST, upsample=UPSAMPLE_FANCY):
    """Decode to (h, w, 3) uint8 RGB.  The defaults are the reference's TurboJPEG configuration."""
    buf = np.ascontiguousarray(buf, dtype=np.uint8)
    info = jpeg_info(buf)
    out = np.empty((info['height'], info['width'], 3), dtype=np.uint8)
    rc = lib().oracle_jpeg_decode(buf.ctypes.data, buf.size, out.ctypes.data, info['height'],
                                  info['width'], idct, upsample)
    if rc:
        raise ValueError(f'oracle_jpeg_decode: {rc}')
    return out


def jpeg_decode_scaled(buf, denom):
    """Decode at 1 / denom (2, 4 or 8) to (ceil(h / denom), ceil(w / denom), 3) uint8 RGB, as
    libjpeg-turbo does with scale 1 / denom, the fast integer transform and fancy upsampling."""
    buf = np.ascontiguousarray(buf, dtype=np.uint8)
    info = jpeg_info(buf)
    h, w = -(-info['height'] // denom), -(-info['width'] // denom)
    out = np.empty((h, w, 3), dtype=np.uint8)
    rc = lib().oracle_jpeg_decode_scaled(buf.ctypes.data, buf.size, out.ctypes.data, h, w, int(denom))
    if rc:
        raise ValueError(f'oracle_jpeg_decode_scaled: {rc}')
    return out


def jpeg_scalable(buf):
    buf = np.ascontiguousarray(buf, dtype=np.uint8)
    return bool(lib().oracle_jpeg_scalable(buf.ctypes.data, buf.size))


def jpeg_coefficients(buf):
    buf = np.ascontiguousarray(buf, dtype=np.uint8)
    nb = lib().oracle_jpeg_num_blocks(buf.ctypes.data, buf.size)
    if nb < 0:
        raise ValueError('oracle_jpeg_num_blocks failed')
    coef = np.zeros((nb, 64), dtype=np.int16)
    rc = lib().oracle_jpeg_coefficients(buf.ctypes.data, buf.size, coef.ctypes.data)
    if rc:
        raise ValueError(f'oracle_jpeg_coefficients: {rc}')
    return coef


def resize_area(src, r0, r1, c0, c1, out_h, out_w):
    """cv2.resize(src[r0:r1, c0:c1], (out_w, out_h), interpolation=INTER_AREA) restated."""
    src = np.ascontiguousarray(src, dtype=np.uint8)
    assert src.ndim == 3 and src.shape[2] == 3
    dst = np.empty((out_h, out_w, 3), dtype=np.uint8)
    lib().oracle_resize_area(src.ctypes.data, src.shape[1], r0, r1, c0, c1, dst.ctypes.data, out_h, out_w)
    return dst


def pack_ops(ops):
    """ops: list of (type, p0, p1, p2, fill) -> int32 [nops, 8]."""
    arr = np.zeros((len(ops), 8), dtype=np.int32)
    for k, (typ, p0, p1, p2, fill) in enumerate(ops):
        arr[k, :4] = (typ, p0, p1, p2)
        arr[k, 4:7] = fill
    return arr


def augment(img, ops):
    """Applies flip / translate / cutout records (see pack_ops) to a copy of one image."""
    img = np.array(img, dtype=np.uint8, order='C', copy=True)
    h, w, _ = img.shape
    arr = pack_ops(ops)
    pad = max([o[1] for o in ops if o[0] == OP_TRANSLATE], default=0)
    scratch = np.zeros(((h + 2 * pad) * (w + 2 * pad) * 3 + 1,), dtype=np.uint8)
    lib().oracle_augment(img.ctypes.data, h, w, arr.ctypes.data, len(ops), scratch.ctypes.data)
    return img


def normalize_table(mean, std, dtype):
    """The lookup table of ffcv/transforms/normalize.py:42-43: float64 arithmetic, then a cast."""
    mean = np.asarray(mean, dtype=np.float64)
    std = np.asarray(std, dtype=np.float64)
    table = (np.arange(256)[:, None] - mean[None, :]) / std[None, :]
    return table.astype(dtype)


def run_batch(payloads, modes, heights, widths, crops, resize, out_h, out_w, ops_per_sample, lut,
              out_kind, nthreads=1, dct_scale=0):
    """Whole path for a batch.  payloads: list of uint8 arrays; crops: [n, 4] (i, j, h, w);
    ops_per_sample: list (per sample) of op records; lut: 256x3 table or None; dct_scale: 0 = JPEG
    samples decoded at full scale, 1..3 = at 1/2, 1/4, 1/8, -1 = per sample by its crop box."""
    n = len(payloads)
    payloads = [np.ascontiguousarray(p, dtype=np.uint8) for p in payloads]
    ptrs = (ctypes.c_void_p * n)(*[p.ctypes.data for p in payloads])
    sizes = np.array([p.size for p in payloads], dtype=np.uint64)
    desc = np.zeros((n, 8), dtype=np.int32)
    desc[:, 0] = modes
    desc[:, 1] = heights
    desc[:, 2] = widths
    desc[:, 3:7] = crops
    desc[:, 7] = int(bool(resize)) | ((255 if dct_scale < 0 else int(dct_scale)) << 8)
    nops = len(ops_per_sample[0]) if n else 0
    ops = np.zeros((n, max(nops, 1), 8), dtype=np.int32)
    for i in range(n):
        if nops:
            ops[i] = pack_ops(ops_per_sample[i])
    if out_kind == OUT_U8_NHWC:
        out = np.zeros((n, out_h, out_w, 3), dtype=np.uint8)
        lut_ptr = None
    else:
        f32 = out_kind in (OUT_F32_NHWC, OUT_F32_NCHW)
        planar = out_kind in (OUT_F16_NCHW, OUT_F32_NCHW)
        dt = np.float32 if f32 else np.float16
        lut = np.ascontiguousarray(lut, dtype=dt)
        assert lut.shape == (256, 3)
        lut_ptr = lut.ctypes.data
        out = np.zeros((n, 3, out_h, out_w) if planar else (n, out_h, out_w, 3), dtype=dt)
    status = np.zeros(n, dtype=np.int32)
    lib().oracle_run_batch(n, ptrs, sizes.ctypes.data, desc.ctypes.data, out_h, out_w, ops.ctypes.data,
                           nops, lut_ptr, out_kind, out.ctypes.data, nthreads, status.ctypes.data)
    return out, status


JITTER_BRIGHTNESS, JITTER_CONTRAST, JITTER_SATURATION = 0, 1, 2


def color_jitter(images, kind, apply, ratio):
    """Brightness / contrast / saturation of ffcv/transforms/color_jitter.py on a uint8
    [n, h, w, 3] batch; returns a new array.  apply: bool per image, ratio: float64 per image."""
    out = np.ascontiguousarray(images, dtype=np.uint8).copy()
    n, h, w, c = out.shape
    assert c == 3
    apply = np.ascontiguousarray(apply, dtype=np.uint8)
    ratio = np.ascontiguousarray(ratio, dtype=np.float64)
    assert apply.shape == (n,) and ratio.shape == (n,)
    fn = (lib().oracle_brightness, lib().oracle_contrast, lib().oracle_saturation)[kind]
    fn(out.ctypes.data, n, h, w, apply.ctypes.data, ratio.ctypes.data)
    return out


def mixup(images, lam):
    """ImageMixup of ffcv/transforms/mixup.py:41-50: image i blended with image i - 1."""
    src = np.ascontiguousarray(images, dtype=np.uint8)
    n = src.shape[0]
    lam = np.ascontiguousarray(np.broadcast_to(np.asarray(lam, dtype=np.float64), (n,)))
    out = np.empty_like(src)
    lib().oracle_mixup(src.ctypes.data, out.ctypes.data, n, src[0].size, lam.ctypes.data)
    return out


def poison(images, apply, mask, alpha, clamp=(0, 255)):
    """Poison of ffcv/transforms/poisoning.py:36-60.  mask: [h, w, 3], alpha: [h, w]."""
    out = np.ascontiguousarray(images, dtype=np.uint8).copy()
    n = out.shape[0]
    alpha3 = np.repeat(np.asarray(alpha)[:, :, None], 3, axis=2)
    m = np.ascontiguousarray(np.asarray(mask).astype('float') * alpha3, dtype=np.float64)
    oma = np.ascontiguousarray(1 - alpha3, dtype=np.float64)
    apply = np.ascontiguousarray(apply, dtype=np.uint8)
    lib().oracle_poison(out.ctypes.data, n, out[0].size, apply.ctypes.data, oma.ctypes.data, m.ctypes.data,
                        float(clamp[0]), float(clamp[1]))
    return out
