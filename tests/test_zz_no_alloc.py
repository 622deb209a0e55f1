"""The allocation-free decode entry point, `ffcvb_imdecode_static`.

It serves callers that may not allocate GPU memory while running (all device memory already
belongs to their own pool, or an allocation's device-wide synchronisation is unaffordable), so its
scratch is a fixed array inside the library.  Checked here through the C ABI against the regular
`imdecode` entry point and against the CPU oracle: identical pixels, on two calls in a row that
share the scratch (a large image first, then a small one, then the large one again), plus the
refusal of inputs beyond the fixed limits.  The buffers the *caller* passes are allocated by the test with torch."""
import cv2
import numpy as np
import pytest

from parity import O

pytestmark = pytest.mark.gpu


def _jpeg(rng, h, w, q, sampling=None, restart=0):
    from ffcv_b200.synthetic import synth_content
    p = [cv2.IMWRITE_JPEG_QUALITY, q]
    if sampling == 444:
        p += [cv2.IMWRITE_JPEG_SAMPLING_FACTOR, cv2.IMWRITE_JPEG_SAMPLING_FACTOR_444]
    if restart:
        p += [cv2.IMWRITE_JPEG_RST_INTERVAL, restart]
    ok, buf = cv2.imencode('.jpg', synth_content(rng, h, w)[..., ::-1], p)
    assert ok
    return buf.reshape(-1).copy()


def _decode_both(buf, h, w):
    import torch as ch
    from ffcv_b200 import libffcv as L
    want = np.zeros((h, w, 3), dtype=np.uint8)
    assert L.imdecode(buf, want, h, w, h, w) == 0
    dev = ch.device('cuda:0')
    src = ch.from_numpy(buf).to(dev)
    out = ch.full((h, w, 3), 77, dtype=ch.uint8, device=dev)
    stream = ch.cuda.current_stream(dev)
    rc = L.imdecode_static(buf, src.data_ptr(), h, w, out.data_ptr(), stream.cuda_stream)
    assert rc == 0
    stream.synchronize()
    return out.cpu().numpy(), want


def test_static_decode_matches_imdecode_on_consecutive_calls():
    rng = np.random.default_rng(42)
    big = _jpeg(rng, 500, 375, 90)
    small = _jpeg(rng, 61, 83, 95, sampling=444)
    marked = _jpeg(rng, 120, 200, 85, restart=4)
    for buf, (h, w) in [(big, (500, 375)), (small, (61, 83)), (big, (500, 375)), (marked, (120, 200)),
                        (small, (61, 83))]:
        got, want = _decode_both(buf, h, w)
        assert np.array_equal(got, want)
        assert np.array_equal(got, O.jpeg_decode(buf))  # and not merely equal to each other


def test_static_decode_refuses_what_does_not_fit():
    import torch as ch
    from ffcv_b200 import libffcv as L
    rng = np.random.default_rng(7)
    dev = ch.device('cuda:0')
    h, w = 700, 700  # 704 x 704 padded luma samples > 640 x 640
    buf = _jpeg(rng, h, w, 90)
    src = ch.from_numpy(buf).to(dev)
    out = ch.zeros((h, w, 3), dtype=ch.uint8, device=dev)
    assert L.imdecode_static(buf, src.data_ptr(), h, w, out.data_ptr()) == -6
    # a stream above the byte limit, and wrong dimensions
    huge = np.zeros(L.STATIC_MAX_STREAM_BYTES + 1, dtype=np.uint8)
    assert L.imdecode_static(huge, src.data_ptr(), 8, 8, out.data_ptr()) == -6
    ok = _jpeg(rng, 64, 64, 90)
    src2 = ch.from_numpy(ok).to(dev)
    assert L.imdecode_static(ok, src2.data_ptr(), 65, 64, out.data_ptr()) == -4
    ch.cuda.synchronize()
