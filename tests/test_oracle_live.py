"""Pins the CPU oracle against the libjpeg-turbo and OpenCV binaries of this image on freshly
generated inputs (wider than the committed vectors): Pillow in draft configuration (fast integer
IDCT, replicated chroma), cv2.imdecode (accurate IDCT, fancy upsampling), cv2.resize INTER_AREA."""
import io

import cv2
import numpy as np
import pytest
from PIL import Image

from parity import O


def _pil_draft(buf):
    im = Image.open(io.BytesIO(buf.tobytes()))
    im.decoderconfig = (1, 1)
    im.load()
    return np.array(im)


def _encode(img, q, samp, rst=0, opt=0):
    p = [cv2.IMWRITE_JPEG_QUALITY, q]
    if samp == 444:
        p += [cv2.IMWRITE_JPEG_SAMPLING_FACTOR, cv2.IMWRITE_JPEG_SAMPLING_FACTOR_444]
    if samp == 422:
        p += [cv2.IMWRITE_JPEG_SAMPLING_FACTOR, cv2.IMWRITE_JPEG_SAMPLING_FACTOR_422]
    if rst:
        p += [cv2.IMWRITE_JPEG_RST_INTERVAL, rst]
    if opt:
        p += [cv2.IMWRITE_JPEG_OPTIMIZE, 1]
    ok, b = cv2.imencode('.jpg', img[..., ::-1], p)
    assert ok
    return b.reshape(-1)


def test_jpeg_random_streams():
    from ffcv_b200.synthetic import synth_content
    rng = np.random.default_rng(1)
    for t in range(48):
        h, w = int(rng.integers(1, 200)), int(rng.integers(1, 200))
        kind = t % 4
        if kind == 0:
            img = rng.integers(0, 256, (h, w, 3), dtype=np.uint8)
        elif kind == 1:
            img = (rng.integers(0, 2, (h, w, 3)) * 255).astype(np.uint8)
        elif kind == 2:
            img = np.zeros((h, w, 3), np.uint8)
            img[::2, ::2] = 255
        else:
            img = synth_content(rng, h, w, 40.0)
        q = int(rng.choice([100, 100, 97, 90, 30, 5]))
        buf = _encode(img, q, [420, 444, 422][t % 3], int(rng.integers(1, 9)) if t % 5 == 0 else 0, t % 7 == 0)
        assert np.array_equal(O.jpeg_decode(buf, O.IDCT_FAST, O.UPSAMPLE_REPLICATE), _pil_draft(buf)), t
        want = cv2.imdecode(buf, cv2.IMREAD_COLOR)[..., ::-1]
        assert np.array_equal(O.jpeg_decode(buf, O.IDCT_ACCURATE, O.UPSAMPLE_FANCY), want), t


def test_reference_configuration_against_libjpeg_turbo_directly():
    """Fast integer IDCT + fancy upsampling, the TurboJPEG configuration of libffcv.cpp:104-106,
    decoded by the libjpeg-turbo binary bundled with Pillow (see tests/libjpeg_direct.py)."""
    import libjpeg_direct as T
    from ffcv_b200.synthetic import synth_content
    if not T.available():
        pytest.skip('no bundled libjpeg-turbo to drive')
    rng = np.random.default_rng(9)
    cases = [(64, 64, 90, 420, 'smooth'), (385, 390, 90, 420, 'smooth'), (37, 53, 75, 420, 'noise'),
             (200, 250, 100, 420, 'noise'), (500, 333, 90, 420, 'smooth'), (17, 9, 90, 420, 'noise'),
             (300, 301, 95, 444, 'smooth'), (120, 90, 100, 444, 'binary'), (101, 100, 90, 422, 'smooth'),
             (8, 8, 50, 420, 'noise'), (256, 192, 30, 420, 'smooth'), (96, 160, 5, 420, 'noise')]
    for h, w, q, samp, kind in cases:
        if kind == 'noise':
            img = rng.integers(0, 256, (h, w, 3), dtype=np.uint8)
        elif kind == 'binary':
            img = (rng.integers(0, 2, (h, w, 3)) * 255).astype(np.uint8)
        else:
            img = synth_content(rng, h, w)
        buf = _encode(img, q, samp)
        assert np.array_equal(O.jpeg_decode(buf), T.decode(buf, T.JDCT_IFAST, True)), (h, w, q, samp)
        # the harness itself: library defaults reproduce cv2's decoder
        want = cv2.imdecode(buf, cv2.IMREAD_COLOR)[..., ::-1]
        assert np.array_equal(T.decode(buf, T.JDCT_ISLOW, True), want), (h, w, q, samp)


def test_jpeg_benchmark_shaped_images():
    from ffcv_b200.synthetic import synth_content
    rng = np.random.default_rng(2)
    for (h, w, q, samp) in [(385, 390, 90, 420), (256, 192, 90, 420), (500, 375, 90, 420), (700, 900, 95, 444)]:
        buf = _encode(synth_content(rng, h, w), q, samp)
        assert np.array_equal(O.jpeg_decode(buf, O.IDCT_FAST, O.UPSAMPLE_REPLICATE), _pil_draft(buf))
        want = cv2.imdecode(buf, cv2.IMREAD_COLOR)[..., ::-1]
        assert np.array_equal(O.jpeg_decode(buf, O.IDCT_ACCURATE, O.UPSAMPLE_FANCY), want)
        info = O.jpeg_info(buf)
        assert (info['height'], info['width']) == (h, w)


def test_grayscale_and_rejections():
    rng = np.random.default_rng(3)
    g = rng.integers(0, 256, (39, 50), dtype=np.uint8)
    ok, buf = cv2.imencode('.jpg', g, [cv2.IMWRITE_JPEG_QUALITY, 90])
    buf = buf.reshape(-1)
    out = O.jpeg_decode(buf, O.IDCT_FAST, O.UPSAMPLE_REPLICATE)
    assert np.array_equal(out[..., 0], _pil_draft(buf)) and np.array_equal(out[..., 0], out[..., 2])
    ok, prog = cv2.imencode('.jpg', g, [cv2.IMWRITE_JPEG_PROGRESSIVE, 1])
    with pytest.raises(ValueError):
        O.jpeg_decode(prog.reshape(-1))
    with pytest.raises(ValueError):
        O.jpeg_decode(rng.integers(0, 256, 300, dtype=np.uint8))


def test_resize_all_regimes():
    rng = np.random.default_rng(0)
    shapes = [(224, 224), (160, 160), (256, 256), (32, 32), (7, 13), (384, 384)]
    cases = []
    for t in range(150):
        H, W = int(rng.integers(8, 520)), int(rng.integers(8, 520))
        cases.append((H, W, int(rng.integers(1, H + 1)), int(rng.integers(1, W + 1))) + shapes[t % 6])
    for fy, fx in [(1, 1), (2, 2), (3, 3), (4, 4), (3, 2), (2, 3), (1, 2), (2, 1), (5, 1), (1, 3), (7, 7), (6, 11)]:
        cases.append((fy * 32 + 5, fx * 48 + 7, fy * 32, fx * 48, 32, 48))
    for t in range(12):
        dh, dw = [(224, 224), (384, 384), (160, 160)][t % 3]
        h, w = int(rng.integers(dh, dh * 4)), int(rng.integers(dw, dw * 4))
        cases.append((h + 3, w + 5, h, w, dh, dw))
    seen = set()
    for H, W, h, w, dh, dw in cases:
        src = rng.integers(0, 256, (H, W, 3), dtype=np.uint8)
        r0, c0 = int(rng.integers(0, H - h + 1)), int(rng.integers(0, W - w + 1))
        want = cv2.resize(src[r0:r0 + h, c0:c0 + w], (dw, dh), interpolation=cv2.INTER_AREA)
        got = O.resize_area(src, r0, r0 + h, c0, c0 + w, dh, dw)
        assert np.array_equal(got, want), (H, W, h, w, dh, dw)
        seen.add('same' if (h, w) == (dh, dw) else 'down' if (h >= dh and w >= dw) else 'up')
    assert seen == {'same', 'down', 'up'}


def test_augment_and_normalize_follow_numpy_semantics():
    """flip.py:31-39, translate.py:35-44, cutout.py:36-46, normalize.py:89-109 restated in numpy."""
    rng = np.random.default_rng(4)
    img = rng.integers(0, 256, (32, 40, 3), dtype=np.uint8)
    fill = (125, 123, 114)
    assert np.array_equal(O.augment(img, [(O.OP_FLIP, 1, 0, 0, (0, 0, 0))]), img[:, ::-1])
    assert np.array_equal(O.augment(img, [(O.OP_FLIP, 0, 0, 0, (0, 0, 0))]), img)
    for (ty, tx) in [(0, 0), (4, 4), (2, 2), (0, 3), (4, 1)]:
        pad = 2
        canvas = np.empty((32 + 2 * pad, 40 + 2 * pad, 3), np.uint8)
        canvas[:] = fill
        canvas[pad:pad + 32, pad:pad + 40] = img
        want = canvas[ty:ty + 32, tx:tx + 40]
        assert np.array_equal(O.augment(img, [(O.OP_TRANSLATE, pad, ty, tx, fill)]), want)
    want = img.copy()
    want[5:13, 30:38] = fill
    assert np.array_equal(O.augment(img, [(O.OP_CUTOUT, 8, 5, 30, fill)]), want)
    # chain in pipeline order: flip, translate, cutout
    step = img[:, ::-1]
    canvas = np.empty((36, 44, 3), np.uint8)
    canvas[:] = fill
    canvas[2:34, 2:42] = step
    step = canvas[1:33, 4:44].copy()
    step[0:4, 0:4] = (1, 2, 3)
    got = O.augment(img, [(O.OP_FLIP, 1, 0, 0, (0, 0, 0)), (O.OP_TRANSLATE, 2, 1, 4, fill), (O.OP_CUTOUT, 4, 0, 0, (1, 2, 3))])
    assert np.array_equal(got, step)
    table = O.normalize_table([125.3, 123.0, 113.9], [63.0, 62.1, 66.7], np.float16)
    out, st = O.run_batch([img.reshape(-1)], [1], [32], [40], np.array([[0, 0, 32, 40]]), 0, 32, 40, [[]], table,
                          O.OUT_F16_NCHW)
    want = table[img, np.arange(3)[None, None, :]].transpose(2, 0, 1)
    assert st[0] == 0 and np.array_equal(out[0].view(np.uint16), want.view(np.uint16))


def test_scaled_decode_against_libjpeg_turbo_directly():
    """Scales 1/2, 1/4, 1/8 with the fast integer IDCT selected, decoded by the libjpeg-turbo binary
    bundled with Pillow: random sizes and contents, 4:2:0 and 4:4:4, several qualities."""
    import libjpeg_direct
    if not libjpeg_direct.available():
        pytest.skip("Pillow's libjpeg-turbo binary is not present")
    from ffcv_b200.synthetic import synth_content
    rng = np.random.default_rng(5)
    for t in range(36):
        h, w = int(rng.integers(1, 260)), int(rng.integers(1, 260))
        img = rng.integers(0, 256, (h, w, 3), dtype=np.uint8) if t % 3 == 0 else synth_content(rng, h, w, 30.0)
        buf = _encode(img, int(rng.choice([100, 95, 90, 50, 10])), [420, 444][t % 2], 0, t % 5 == 0)
        for denom in (2, 4, 8):
            want = libjpeg_direct.decode(buf, libjpeg_direct.JDCT_IFAST, True, denom)
            assert np.array_equal(O.jpeg_decode_scaled(buf, denom), want), (t, denom)
