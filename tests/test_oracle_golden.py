"""Pins the CPU oracle (and the host-side samplers) on the committed golden vectors of
tests/golden/, produced by tests/golden/make_golden.py from real libjpeg-turbo / OpenCV binaries
and from the reference's own crop-sampling functions."""
import os

import numpy as np

from parity import O

G = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden')


def test_jpeg_decode_stages_against_libjpeg_turbo_vectors():
    z = np.load(os.path.join(G, 'jpeg_cases.npz'))
    n = int(z['count'])
    assert n >= 10
    for k in range(n):
        buf = z[f'jpeg_{k}']
        # the reference's configuration itself: fast integer IDCT + fancy upsampling
        assert np.array_equal(O.jpeg_decode(buf), z[f'turbo_fast_fancy_{k}']), k
        # entropy decode + dequantisation + fast integer IDCT + colour conversion
        a = O.jpeg_decode(buf, O.IDCT_FAST, O.UPSAMPLE_REPLICATE)
        assert np.array_equal(a, z[f'fast_replicate_{k}']), k
        # entropy decode + triangle upsampling + colour conversion
        b = O.jpeg_decode(buf, O.IDCT_ACCURATE, O.UPSAMPLE_FANCY)
        assert np.array_equal(b, z[f'accurate_fancy_{k}']), k


def test_resize_against_opencv_vectors():
    z = np.load(os.path.join(G, 'resize_cases.npz'))
    for k in range(int(z['count'])):
        r0, r1, c0, c1, dh, dw = (int(v) for v in z[f'box_{k}'])
        got = O.resize_area(z[f'src_{k}'], r0, r1, c0, c1, dh, dw)
        assert np.array_equal(got, z[f'dst_{k}']), k


def test_crop_samplers_against_reference_functions():
    from ffcv_b200.pipeline.sampling import sample_center_crops, sample_random_crops
    z = np.load(os.path.join(G, 'crop_cases.npz'))
    h, w = z['heights'], z['widths']
    for name in ('default', 'quarter'):
        args = z[f'random_{name}_args']
        out = np.zeros((len(h), 4), dtype=np.int32)
        sample_random_crops(int(args[0]), h, w, args[1:3].astype(np.float64), args[3:5].astype(np.float64), out)
        assert np.array_equal(out, z[f'random_{name}']), name
    for key in z.files:
        if key.startswith('center_'):
            out = np.zeros((len(h), 4), dtype=np.int32)
            sample_center_crops(h, w, float(key.split('_')[1]), out)
            assert np.array_equal(out, z[key]), key


def test_normalize_tables_against_reference_expression():
    from ffcv_b200.transforms import NormalizeImage
    z = np.load(os.path.join(G, 'normalize_cases.npz'))
    for name in ('imagenet', 'cifar'):
        for dt in (np.float16, np.float32):
            want = z[f'{name}_{np.dtype(dt).name}']
            op = NormalizeImage(z[f'{name}_mean'], z[f'{name}_std'], dt)
            assert op.lookup_table.dtype == want.dtype
            assert np.array_equal(op.lookup_table.view(np.uint16 if dt == np.float16 else np.uint32),
                                  want.view(np.uint16 if dt == np.float16 else np.uint32))
            assert np.array_equal(O.normalize_table(z[f'{name}_mean'], z[f'{name}_std'], dt), want)


def test_scaled_decode_against_libjpeg_turbo_vectors():
    """Decoding at 1/2, 1/4 and 1/8 (reduced-size inverse transforms; chroma of 4:2:0 streams at
    twice the luma's block size, hence no upsampling)."""
    z = np.load(os.path.join(G, 'jpeg_cases.npz'))
    s = np.load(os.path.join(G, 'jpeg_scaled_cases.npz'))
    checked = 0
    for k in range(int(z['count'])):
        buf = z[f'jpeg_{k}']
        if not O.jpeg_scalable(buf):
            continue  # 4:2:2: scaling is not offered for it
        for denom in (2, 4, 8):
            assert np.array_equal(O.jpeg_decode_scaled(buf, denom), s[f'scaled_{k}_{denom}']), (k, denom)
            checked += 1
    assert checked >= 30
