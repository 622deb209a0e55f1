"""ctypes binding of ``libffcv_b200.so``.

Plays the role of ``ffcv/libffcv.py:1-56`` in the reference: it loads the native library and
exposes ``imdecode``, ``resize_crop`` and ``memcpy`` with the reference's Python signatures, plus
the batch calls (:class:`Context`) the loader uses.  There is no CPU implementation behind this
module: if the CUDA library is missing or cannot be loaded the import fails.
"""
import ctypes
import os
from ctypes import (CDLL, POINTER, Structure, c_bool, c_int, c_int32, c_int64, c_uint8, c_uint16,
                    c_uint32, c_uint64, c_void_p, c_char_p)

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, 'libffcv_b200.so')

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python ffcv_b200/_build.py` (needs nvcc). "
        "ffcv_b200 has no CPU fallback.")

lib = CDLL(LIB_PATH)

MODE_JPG, MODE_RAW = 0, 1
OUT_U8_NHWC, OUT_F16_NHWC, OUT_F16_NCHW, OUT_F32_NHWC, OUT_F32_NCHW = range(5)
OP_FLIP, OP_TRANSLATE, OP_CUTOUT = 1, 2, 3
MAX_OPS = 8


class Op(Structure):
    _fields_ = [('type', c_int32), ('arg', c_int32), ('fill', c_uint8 * 4)]


class Plan(Structure):
    _fields_ = [('out_h', c_int32), ('out_w', c_int32), ('resize', c_int32), ('out_kind', c_int32),
                ('n_ops', c_int32), ('ops', Op * MAX_OPS), ('dct_scale', c_int32), ('lut_dev', c_void_p)]


class Rider(Structure):
    _fields_ = [('host', c_void_p), ('ptrs', c_void_p), ('item_bytes', c_uint64), ('dst_dev', c_void_p)]


MAX_RIDERS = 8

lib.ffcvb_set_batch_riders.argtypes = [c_void_p, c_int, POINTER(Rider), c_int, c_int]
lib.ffcvb_set_batch_riders.restype = c_int
lib.ffcvb_create.argtypes = [c_int, c_int, c_int, POINTER(c_void_p)]
lib.ffcvb_create.restype = c_int
lib.ffcvb_destroy.argtypes = [c_void_p]
lib.ffcvb_destroy.restype = None
lib.ffcvb_last_error.argtypes = [c_void_p]
lib.ffcvb_last_error.restype = c_char_p
lib.ffcvb_stage_batch.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                  c_void_p, c_int, POINTER(Plan), c_void_p]
lib.ffcvb_stage_batch.restype = c_int
lib.ffcvb_stage_batch_fd.argtypes = [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_void_p, c_int, POINTER(Plan), c_void_p]
lib.ffcvb_stage_batch_fd.restype = c_int
lib.ffcvb_submit_batch.argtypes = [c_void_p, c_int, c_void_p, c_void_p]
lib.ffcvb_submit_batch.restype = c_int
lib.ffcvb_rerun_batch.argtypes = [c_void_p, c_int, c_void_p, c_void_p]
lib.ffcvb_rerun_batch.restype = c_int
lib.ffcvb_set_header_cache.argtypes = [c_void_p, c_int]
lib.ffcvb_set_header_cache.restype = c_int
lib.ffcvb_set_decode_index.argtypes = [c_void_p, c_uint64]
lib.ffcvb_set_decode_index.restype = c_int
lib.ffcvb_decode_index_stats.argtypes = [c_void_p, c_void_p]
lib.ffcvb_decode_index_stats.restype = c_int
lib.ffcvb_set_async_staging.argtypes = [c_void_p, c_int]
lib.ffcvb_set_async_staging.restype = c_int
lib.ffcvb_color_jitter.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p]
lib.ffcvb_color_jitter.restype = c_int
lib.ffcvb_mixup.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_void_p]
lib.ffcvb_mixup.restype = c_int
lib.ffcvb_poison.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p,
                             ctypes.c_double, ctypes.c_double]
lib.ffcvb_poison.restype = c_int
lib.ffcvb_set_staging_split.argtypes = [c_void_p, c_int]
lib.ffcvb_set_staging_split.restype = c_int
lib.ffcvb_host_register.argtypes = [c_void_p, c_uint64]
lib.ffcvb_host_register.restype = c_int
lib.ffcvb_host_unregister.argtypes = [c_void_p]
lib.ffcvb_host_unregister.restype = c_int
lib.ffcvb_staging_split.argtypes = [c_void_p]
lib.ffcvb_staging_split.restype = c_int
lib.ffcvb_set_profiling.argtypes = [c_void_p, c_int]
lib.ffcvb_set_profiling.restype = c_int
lib.ffcvb_batch_times.argtypes = [c_void_p, c_int, c_void_p]
lib.ffcvb_batch_times.restype = c_int
lib.ffcvb_staged_bytes.argtypes = [c_void_p, c_int]
lib.ffcvb_staged_bytes.restype = c_int64
lib.ffcvb_stage_times.argtypes = [c_void_p, c_int, c_void_p]
lib.ffcvb_stage_times.restype = c_int
lib.ffcvb_batch_info.argtypes = [c_void_p, c_int, c_void_p]
lib.ffcvb_batch_info.restype = c_int
lib.ffcvb_gather_time.argtypes = [c_void_p, c_int, c_void_p]
lib.ffcvb_gather_time.restype = c_int
lib.ffcvb_batch_launches.argtypes = [c_void_p, c_int]
lib.ffcvb_batch_launches.restype = c_int
lib.ffcvb_batch_status.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int]
lib.ffcvb_batch_status.restype = c_int
lib.ffcvb_transform_device.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                       POINTER(Plan), c_void_p, c_void_p]
lib.ffcvb_transform_device.restype = c_int

lib.ffcvb_imdecode_static.argtypes = [c_void_p, c_uint64, c_void_p, c_uint32, c_uint32, c_void_p, c_void_p]
lib.ffcvb_imdecode_static.restype = c_int
STATIC_MAX_STREAM_BYTES = 1 << 20
STATIC_MAX_PADDED_PIXELS = 640 * 640


def imdecode_static(jpeg_host: np.ndarray, jpeg_dev_ptr: int, height: int, width: int, rgb_dev_ptr: int,
                    stream: int = 0):
    """Decode one JPEG without any allocation by the library: ``jpeg_host`` is the stream in host
    memory, ``jpeg_dev_ptr`` the address of the same bytes on the GPU, ``rgb_dev_ptr`` the address of
    a ``height * width * 3`` byte output buffer on the GPU.  Asynchronous on ``stream``.  Returns the
    library's status code (0 on success, -6 when the image exceeds the fixed scratch)."""
    return lib.ffcvb_imdecode_static(jpeg_host.ctypes.data, jpeg_host.size, jpeg_dev_ptr, height, width,
                                     rgb_dev_ptr, stream or None)


def make_plan(out_h, out_w, resize, out_kind, ops=(), lut_dev=0, dct_scale=0):
    """ops: sequence of (type, arg, fill) with fill a 3-sequence of ints.  dct_scale: 0 full-scale
    decode, 1..3 every JPEG at 1/2, 1/4, 1/8, -1 per sample by its crop box (see ffcvb_plan)."""
    if len(ops) > MAX_OPS:
        raise ValueError(f'at most {MAX_OPS} fused augmentations')
    plan = Plan()
    plan.out_h, plan.out_w = int(out_h), int(out_w)
    plan.resize = int(bool(resize))
    plan.out_kind = int(out_kind)
    plan.n_ops = len(ops)
    for k, (typ, arg, fill) in enumerate(ops):
        plan.ops[k].type = int(typ)
        plan.ops[k].arg = int(arg)
        for c in range(3):
            plan.ops[k].fill[c] = int(fill[c]) & 255
    plan.dct_scale = int(dct_scale)
    plan.lut_dev = int(lut_dev) if lut_dev else None
    return plan


def _as(a, dtype):
    if isinstance(a, np.ndarray) and a.dtype == dtype and a.flags.c_contiguous:
        return a
    return np.ascontiguousarray(a, dtype=dtype)


class FFCVBError(RuntimeError):
    pass


def host_register(address, nbytes):
    """True when the range could be page-locked in place."""
    return lib.ffcvb_host_register(address, nbytes) == 0


def host_unregister(address):
    return lib.ffcvb_host_unregister(address) == 0


class Context:
    """A decode context on one GPU: staging threads, batch slots and device scratch."""

    def __init__(self, device=0, n_slots=1, n_threads=0):
        handle = c_void_p()
        rc = lib.ffcvb_create(int(device), int(n_slots), int(n_threads), ctypes.byref(handle))
        if rc != 0:
            raise FFCVBError(f'ffcvb_create failed with code {rc} (is a CUDA device visible?)')
        self._h = handle
        self.device = int(device)
        self.n_slots = int(n_slots)

    def _check(self, rc, what):
        if rc != 0:
            msg = lib.ffcvb_last_error(self._h)
            raise FFCVBError(f'{what} failed ({rc}): {msg.decode() if msg else ""}')

    def stage(self, slot, file_base, ptrs, sizes, modes, heights, widths, plan, params):
        """file_base: integer address (or uint8 array) the sample pointers are relative to, or a
        (fd, fd_direct) pair of descriptors of the file to read the samples from."""
        ptrs = _as(ptrs, np.uint64)
        sizes = _as(sizes, np.uint64)
        modes = _as(modes, np.uint8)
        heights = _as(heights, np.uint16)
        widths = _as(widths, np.uint16)
        params = _as(params, np.int32)
        n = len(ptrs)
        assert params.shape == (n, 4 + 2 * plan.n_ops), params.shape
        if isinstance(file_base, tuple):
            rc = lib.ffcvb_stage_batch_fd(self._h, slot, int(file_base[0]), int(file_base[1]), ptrs.ctypes.data,
                                          sizes.ctypes.data, modes.ctypes.data, heights.ctypes.data,
                                          widths.ctypes.data, n, ctypes.byref(plan), params.ctypes.data)
            self._check(rc, 'ffcvb_stage_batch_fd')
            return
        base = file_base.ctypes.data if isinstance(file_base, np.ndarray) else int(file_base)
        rc = lib.ffcvb_stage_batch(self._h, slot, base, ptrs.ctypes.data, sizes.ctypes.data,
                                   modes.ctypes.data, heights.ctypes.data, widths.ctypes.data, n,
                                   ctypes.byref(plan), params.ctypes.data)
        self._check(rc, 'ffcvb_stage_batch')

    def set_riders(self, slot, riders, n):
        """riders: sequence of (values, file_offsets, item_bytes, dst_ptr) -- exactly one of
        `values` (contiguous numpy array of n items) and `file_offsets` (uint64 array of n offsets
        from the file base given to stage) is not None.  Consumed by the next `stage` of the slot."""
        arr = (Rider * max(1, len(riders)))()
        keep = []
        for k, (values, offsets, item_bytes, dst_ptr) in enumerate(riders):
            if values is not None:
                values = np.ascontiguousarray(values)
                assert values.nbytes == n * item_bytes, (values.nbytes, n, item_bytes)
                arr[k].host, arr[k].ptrs = values.ctypes.data, None
                keep.append(values)
            else:
                offsets = _as(offsets, np.uint64)
                assert offsets.shape == (n,)
                arr[k].host, arr[k].ptrs = None, offsets.ctypes.data
                keep.append(offsets)
            arr[k].item_bytes = int(item_bytes)
            arr[k].dst_dev = int(dst_ptr)
        self._check(lib.ffcvb_set_batch_riders(self._h, slot, arr, len(riders), int(n)), 'ffcvb_set_batch_riders')

    def submit(self, slot, stream, out_ptr):
        self._check(lib.ffcvb_submit_batch(self._h, slot, stream or None, out_ptr), 'ffcvb_submit_batch')

    def rerun(self, slot, stream, out_ptr):
        self._check(lib.ffcvb_rerun_batch(self._h, slot, stream or None, out_ptr), 'ffcvb_rerun_batch')

    def set_staging_split(self, cpu_share_permille):
        self._check(lib.ffcvb_set_staging_split(self._h, int(cpu_share_permille)), 'ffcvb_set_staging_split')

    def color_jitter(self, stream_ptr, images_ptr, n, h, w, kind, apply, ratio):
        apply = np.ascontiguousarray(apply, dtype=np.uint8)
        ratio = np.ascontiguousarray(ratio, dtype=np.float64)
        assert apply.shape == (n,) and ratio.shape == (n,)
        self._check(lib.ffcvb_color_jitter(self._h, stream_ptr, images_ptr, n, h, w, kind, apply.ctypes.data,
                                           ratio.ctypes.data), 'ffcvb_color_jitter')

    def mixup(self, stream_ptr, src_ptr, dst_ptr, n, count, lam):
        lam = np.ascontiguousarray(lam, dtype=np.float64)
        assert lam.shape == (n,)
        self._check(lib.ffcvb_mixup(self._h, stream_ptr, src_ptr, dst_ptr, n, count, lam.ctypes.data), 'ffcvb_mixup')

    def poison(self, stream_ptr, images_ptr, n, count, apply, one_minus_alpha_ptr, mask_ptr, lo, hi):
        apply = np.ascontiguousarray(apply, dtype=np.uint8)
        assert apply.shape == (n,)
        self._check(lib.ffcvb_poison(self._h, stream_ptr, images_ptr, n, count, apply.ctypes.data,
                                     one_minus_alpha_ptr, mask_ptr, float(lo), float(hi)), 'ffcvb_poison')

    def staging_split(self):
        return int(lib.ffcvb_staging_split(self._h))

    def set_header_cache(self, enabled):
        """Remember parsed JPEG headers per sample offset (the context then serves one file)."""
        self._check(lib.ffcvb_set_header_cache(self._h, int(bool(enabled))), 'ffcvb_set_header_cache')

    def set_decode_index(self, nbytes):
        """Device memory for the decode index (0: off); see ffcvb_set_decode_index."""
        self._check(lib.ffcvb_set_decode_index(self._h, int(nbytes)), 'ffcvb_set_decode_index')

    def decode_index_stats(self):
        out = np.zeros(4, dtype=np.uint64)
        self._check(lib.ffcvb_decode_index_stats(self._h, out.ctypes.data), 'ffcvb_decode_index_stats')
        return dict(zip(('used', 'recorded', 'entries', 'bytes'), (int(v) for v in out)))

    def set_async_staging(self, enabled):
        self._check(lib.ffcvb_set_async_staging(self._h, int(bool(enabled))), 'ffcvb_set_async_staging')

    def set_profiling(self, enabled):
        self._check(lib.ffcvb_set_profiling(self._h, int(bool(enabled))), 'ffcvb_set_profiling')

    def batch_times(self, slot):
        """Milliseconds of (h2d copy, entropy decode, idct, colour, resize) of the slot's last run."""
        ms = np.zeros(5, dtype=np.float32)
        self._check(lib.ffcvb_batch_times(self._h, slot, ms.ctypes.data), 'ffcvb_batch_times')
        return ms

    def staged_bytes(self, slot):
        return int(lib.ffcvb_staged_bytes(self._h, slot))

    def stage_times(self, slot):
        """Host milliseconds of the slot's last staging: (header parse, layout, payload copy, total)."""
        ms = np.zeros(4, dtype=np.float64)
        self._check(lib.ffcvb_stage_times(self._h, slot, ms.ctypes.data), 'ffcvb_stage_times')
        return ms

    def batch_info(self, slot):
        info = np.zeros(8, dtype=np.int64)
        self._check(lib.ffcvb_batch_info(self._h, slot, info.ctypes.data), 'ffcvb_batch_info')
        keys = ('n', 'n_jpeg', 'blocks', 'scan_bytes', 'plane_bytes', 'rgb_bytes', 'raw_bytes', 'jpeg_bytes')
        return dict(zip(keys, (int(v) for v in info)))

    def gather_time(self, slot):
        """Milliseconds of the GPU's payload gather of the slot's last batch, or None."""
        ms = ctypes.c_float(-1.0)
        self._check(lib.ffcvb_gather_time(self._h, slot, ctypes.byref(ms)), 'ffcvb_gather_time')
        return float(ms.value) if ms.value >= 0 else None

    def launches(self, slot):
        return int(lib.ffcvb_batch_launches(self._h, slot))

    def status(self, slot, stream, n):
        st = np.zeros(n, dtype=np.int32)
        bad = lib.ffcvb_batch_status(self._h, slot, stream or None, st.ctypes.data, n)
        if bad < 0:
            self._check(bad, 'ffcvb_batch_status')
        return st

    def transform_device(self, stream, src_ptr, n, h, w, plan, params, out_ptr):
        params = np.ascontiguousarray(params, dtype=np.int32)
        assert params.shape == (n, 4 + 2 * plan.n_ops), params.shape
        rc = lib.ffcvb_transform_device(self._h, stream or None, src_ptr, n, h, w, ctypes.byref(plan),
                                        params.ctypes.data, out_ptr)
        self._check(rc, 'ffcvb_transform_device')

    def close(self):
        if getattr(self, '_h', None):
            lib.ffcvb_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# ---- the reference's single-image calls (ffcv/libffcv.py:22-55), same names and arguments -----

ctypes_resize = lib.resize
ctypes_resize.argtypes = 11 * [c_int64]
ctypes_resize.restype = None


def resize_crop(source, start_row, end_row, start_col, end_col, destination):
    ctypes_resize(0, source.ctypes.data, source.shape[0], source.shape[1], start_row, end_row,
                  start_col, end_col, destination.ctypes.data, destination.shape[0],
                  destination.shape[1])


ctypes_imdecode = lib.imdecode
ctypes_imdecode.argtypes = [c_void_p, c_uint64, c_uint32, c_uint32, c_void_p, c_uint32, c_uint32,
                            c_uint32, c_uint32, c_uint32, c_uint32, c_bool, c_bool]
ctypes_imdecode.restype = c_int


def imdecode(source: np.ndarray, dst: np.ndarray, source_height: int, source_width: int,
             crop_height=None, crop_width=None, offset_x=0, offset_y=0, scale_factor_num=1,
             scale_factor_denom=1, enable_crop=False, do_flip=False):
    if crop_height is None:
        crop_height = source_height
    if crop_width is None:
        crop_width = source_width
    return ctypes_imdecode(source.ctypes.data, source.size, source_height, source_width,
                           dst.ctypes.data, crop_height, crop_width, offset_x, offset_y,
                           scale_factor_num, scale_factor_denom, enable_crop, do_flip)


ctypes_memcopy = lib.my_memcpy
ctypes_memcopy.argtypes = [c_void_p, c_void_p, c_uint64]
ctypes_memcopy.restype = None


def memcpy(source: np.ndarray, dest: np.ndarray):
    return ctypes_memcopy(source.ctypes.data, dest.ctypes.data, source.size * source.itemsize)
