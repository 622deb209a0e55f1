"""Parity of the single-image C-ABI calls (`imdecode`, `resize`, same signatures as
libffcv/libffcv.cpp:33-112) on the GPU against the CPU oracle: decoded pixels bit-exact,
resized pixels within 1 LSB (0 asserted, the oracle restates cv2 exactly)."""
import cv2
import numpy as np
import pytest

from parity import O

pytestmark = pytest.mark.gpu


def _encode(img, q=90, samp=None, rst=0, opt=0, gray=False):
    p = [cv2.IMWRITE_JPEG_QUALITY, q]
    if samp == 444:
        p += [cv2.IMWRITE_JPEG_SAMPLING_FACTOR, cv2.IMWRITE_JPEG_SAMPLING_FACTOR_444]
    if samp == 422:
        p += [cv2.IMWRITE_JPEG_SAMPLING_FACTOR, cv2.IMWRITE_JPEG_SAMPLING_FACTOR_422]
    if rst:
        p += [cv2.IMWRITE_JPEG_RST_INTERVAL, rst]
    if opt:
        p += [cv2.IMWRITE_JPEG_OPTIMIZE, 1]
    ok, b = cv2.imencode('.jpg', img if gray else img[..., ::-1], p)
    assert ok
    return b.reshape(-1).copy()


CASES = [
    # h, w, quality, sampling, restart interval, optimised tables, content
    (64, 64, 90, None, 0, 0, 'smooth'), (200, 250, 90, None, 0, 0, 'smooth'), (37, 53, 90, None, 0, 0, 'smooth'),
    (385, 390, 90, None, 0, 0, 'smooth'), (17, 9, 75, None, 0, 0, 'smooth'), (8, 8, 90, None, 0, 0, 'smooth'),
    (1, 1, 90, None, 0, 0, 'smooth'), (3, 5, 90, None, 0, 0, 'noise'), (2, 2, 90, None, 0, 0, 'noise'),
    (300, 333, 95, 444, 0, 0, 'smooth'), (129, 255, 50, 444, 0, 0, 'smooth'), (100, 101, 90, 422, 0, 0, 'smooth'),
    (480, 500, 100, None, 0, 0, 'noise'), (256, 256, 100, 444, 0, 0, 'binary'), (90, 75, 5, None, 0, 0, 'noise'),
    (120, 130, 90, None, 3, 0, 'smooth'), (90, 70, 90, 444, 5, 1, 'noise'), (333, 222, 85, None, 0, 1, 'smooth'),
    (1100, 1300, 95, 444, 0, 0, 'smooth'), (1536, 1024, 95, 444, 0, 0, 'smooth'),
]


def _content(rng, h, w, kind):
    from ffcv_b200.synthetic import synth_content
    if kind == 'noise':
        return rng.integers(0, 256, (h, w, 3), dtype=np.uint8)
    if kind == 'binary':
        return (rng.integers(0, 2, (h, w, 3)) * 255).astype(np.uint8)
    return synth_content(rng, h, w)


@pytest.mark.parametrize('case', CASES, ids=lambda c: f'{c[0]}x{c[1]}q{c[2]}s{c[3]}r{c[4]}o{c[5]}{c[6]}')
def test_imdecode_bit_exact(case):
    from ffcv_b200.libffcv import imdecode
    h, w, q, samp, rst, opt, kind = case
    rng = np.random.default_rng(h * 10007 + w)
    buf = _encode(_content(rng, h, w, kind), q, samp, rst, opt)
    want = O.jpeg_decode(buf)
    got = np.zeros((h, w, 3), dtype=np.uint8)
    assert imdecode(buf, got, h, w, h, w, 0, 0, 1, 1, False, False) == 0
    assert np.array_equal(got, want)


def test_imdecode_grayscale_and_errors():
    from ffcv_b200.libffcv import imdecode
    rng = np.random.default_rng(3)
    g = rng.integers(0, 256, (40, 50), dtype=np.uint8)
    buf = _encode(g, gray=True)
    got = np.zeros((40, 50, 3), dtype=np.uint8)
    assert imdecode(buf, got, 40, 50, 40, 50) == 0
    assert np.array_equal(got, O.jpeg_decode(buf))
    # wrong dimensions, garbage and a progressive stream are rejected with -1, like tjDecompress2
    assert imdecode(buf, np.zeros((41, 50, 3), np.uint8), 41, 50, 41, 50) == -1
    junk = rng.integers(0, 256, 500, dtype=np.uint8)
    assert imdecode(junk, got, 40, 50, 40, 50) == -1
    ok, prog = cv2.imencode('.jpg', g, [cv2.IMWRITE_JPEG_PROGRESSIVE, 1])
    assert imdecode(prog.reshape(-1).copy(), got, 40, 50, 40, 50) == -1


def test_resize_crop_matches_inter_area():
    from ffcv_b200.libffcv import resize_crop
    rng = np.random.default_rng(11)
    shapes = [(224, 224), (160, 160), (256, 256), (32, 32), (7, 13), (384, 384)]
    cases = []
    for t in range(60):
        H, W = int(rng.integers(8, 520)), int(rng.integers(8, 520))
        h, w = int(rng.integers(1, H + 1)), int(rng.integers(1, W + 1))
        cases.append((H, W, h, w) + shapes[t % 6])
    for fy, fx in [(1, 1), (2, 2), (3, 3), (4, 4), (3, 2), (2, 3), (1, 2), (2, 1), (5, 1), (1, 3), (7, 7)]:
        cases.append((fy * 32 + 5, fx * 48 + 7, fy * 32, fx * 48, 32, 48))
    cases.append((1400, 1800, 1301, 1777, 384, 384))
    for H, W, h, w, dh, dw in cases:
        src = rng.integers(0, 256, (H, W, 3), dtype=np.uint8)
        r0, c0 = int(rng.integers(0, H - h + 1)), int(rng.integers(0, W - w + 1))
        want = O.resize_area(src, r0, r0 + h, c0, c0 + w, dh, dw)
        got = np.zeros((dh, dw, 3), dtype=np.uint8)
        resize_crop(src, r0, r0 + h, c0, c0 + w, got)
        diff = np.abs(got.astype(int) - want.astype(int))
        assert diff.max() == 0, (H, W, h, w, dh, dw, int(diff.max()), int((diff > 0).sum()))


def test_memcpy():
    from ffcv_b200.libffcv import memcpy
    rng = np.random.default_rng(0)
    a = rng.integers(0, 256, 4097, dtype=np.uint8)
    b = np.zeros_like(a)
    memcpy(a, b)
    assert np.array_equal(a, b)


# ---- the GPU against the third-party binaries themselves (no oracle in between) ----------------

@pytest.mark.parametrize('case', CASES,
                         ids=lambda c: f'{c[0]}x{c[1]}q{c[2]}s{c[3]}r{c[4]}o{c[5]}{c[6]}')
def test_imdecode_against_libjpeg_turbo(case):
    """`imdecode` on the GPU against libjpeg-turbo itself (Pillow's bundled binary, driven with
    dct_method = JDCT_IFAST and fancy upsampling, the configuration the reference's
    tjDecompress2(..., TJFLAG_FASTDCT) call selects, libffcv/libffcv.cpp:104-106): bit-exact."""
    import libjpeg_direct
    if not libjpeg_direct.available():
        pytest.skip("Pillow's libjpeg-turbo binary is not present")
    from ffcv_b200.libffcv import imdecode
    h, w, q, samp, rst, opt, kind = case
    rng = np.random.default_rng(h * 10007 + w)
    buf = _encode(_content(rng, h, w, kind), q, samp, rst, opt)
    want = libjpeg_direct.decode(buf, libjpeg_direct.JDCT_IFAST, True)
    got = np.zeros((h, w, 3), dtype=np.uint8)
    assert imdecode(buf, got, h, w, h, w, 0, 0, 1, 1, False, False) == 0
    assert np.array_equal(got, want)


def test_resize_crop_against_cv2_inter_area():
    """`resize` on the GPU against cv2.resize(..., INTER_AREA) itself, the call of
    libffcv/libffcv.cpp:40-41: bar 1 LSB, 0 asserted (all three regimes: integer factors,
    fractional shrink, enlargement)."""
    from ffcv_b200.libffcv import resize_crop
    rng = np.random.default_rng(12)
    shapes = [(224, 224), (160, 160), (256, 256), (32, 32), (7, 13), (384, 384)]
    cases = []
    for t in range(48):
        H, W = int(rng.integers(8, 520)), int(rng.integers(8, 520))
        h, w = int(rng.integers(1, H + 1)), int(rng.integers(1, W + 1))
        cases.append((H, W, h, w) + shapes[t % 6])
    for fy, fx in [(1, 1), (2, 2), (3, 3), (4, 4), (3, 2), (2, 3), (1, 2), (2, 1), (7, 7)]:
        cases.append((fy * 32 + 5, fx * 48 + 7, fy * 32, fx * 48, 32, 48))
    cases.append((1300, 1700, 1201, 1577, 384, 384))
    for H, W, h, w, dh, dw in cases:
        src = rng.integers(0, 256, (H, W, 3), dtype=np.uint8)
        r0, c0 = int(rng.integers(0, H - h + 1)), int(rng.integers(0, W - w + 1))
        want = cv2.resize(src[r0:r0 + h, c0:c0 + w], (dw, dh), interpolation=cv2.INTER_AREA)
        got = np.zeros((dh, dw, 3), dtype=np.uint8)
        resize_crop(src, r0, r0 + h, c0, c0 + w, got)
        diff = np.abs(got.astype(int) - want.astype(int))
        assert diff.max() == 0, (H, W, h, w, dh, dw, int(diff.max()), int((diff > 0).sum()))


def test_my_fread(tmp_path):
    """`my_fread(FILE *, offset, dst, size)` (libffcv/libffcv.cpp:48-51) through a C stream."""
    import ctypes
    from ffcv_b200.libffcv import lib
    libc = ctypes.CDLL(None)
    libc.fopen.restype = ctypes.c_void_p
    libc.fopen.argtypes = [ctypes.c_char_p, ctypes.c_char_p]
    libc.fclose.argtypes = [ctypes.c_void_p]
    data = np.random.default_rng(5).integers(0, 256, 10000, dtype=np.uint8)
    path = tmp_path / 'blob.bin'
    data.tofile(str(path))
    fp = libc.fopen(str(path).encode(), b'rb')
    assert fp
    lib.my_fread.argtypes = [ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64]
    lib.my_fread.restype = None
    out = np.zeros(777, dtype=np.uint8)
    lib.my_fread(fp, 1234, out.ctypes.data, out.size)
    libc.fclose(fp)
    assert np.array_equal(out, data[1234:1234 + 777])


@pytest.mark.parametrize('case', [c for c in CASES if c[3] != 422],
                         ids=lambda c: f'{c[0]}x{c[1]}q{c[2]}s{c[3]}r{c[4]}o{c[5]}{c[6]}')
def test_imdecode_scaled_bit_exact(case):
    """`imdecode(..., scale_num, scale_denom)` at 1/2, 1/4 and 1/8 (libffcv/libffcv.cpp:59,89-90,104:
    the output has TJSCALED(dim) = ceil(dim / denom) pixels a side) against the oracle and against
    libjpeg-turbo's own scaled decode with the fast integer IDCT selected: bit-exact."""
    import libjpeg_direct
    from ffcv_b200.libffcv import imdecode
    h, w, q, samp, rst, opt, kind = case
    rng = np.random.default_rng(h * 10007 + w)
    buf = _encode(_content(rng, h, w, kind), q, samp, rst, opt)
    for denom in (2, 4, 8):
        sh, sw = -(-h // denom), -(-w // denom)
        got = np.zeros((sh, sw, 3), dtype=np.uint8)
        assert imdecode(buf, got, h, w, h, w, 0, 0, 1, denom, False, False) == 0
        assert np.array_equal(got, O.jpeg_decode_scaled(buf, denom)), denom
        if libjpeg_direct.available():
            assert np.array_equal(got, libjpeg_direct.decode(buf, libjpeg_direct.JDCT_IFAST, True, denom)), denom


def test_imdecode_scaled_refuses_what_it_cannot_scale():
    from ffcv_b200.libffcv import imdecode
    rng = np.random.default_rng(9)
    img = _content(rng, 64, 80, 'smooth')
    got = np.zeros((32, 40, 3), dtype=np.uint8)
    assert imdecode(_encode(img, 90, 422), got, 64, 80, 64, 80, 0, 0, 1, 2) == -1   # 4:2:2
    assert imdecode(_encode(img, 90), got, 64, 80, 64, 80, 0, 0, 1, 3) == -1         # 1/3 is not offered
    assert imdecode(_encode(img, 90), got, 64, 80, 64, 80, 0, 0, 1, 2) == 0
