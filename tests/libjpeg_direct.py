"""Drives the libjpeg-turbo binary bundled with Pillow through its public libjpeg API (ctypes), so
that a test can select what no Python binding exposes: the fast integer IDCT (`dct_method =
JDCT_IFAST`) together with fancy chroma upsampling -- the configuration TurboJPEG uses for the
reference's call `tjDecompress2(..., TJFLAG_FASTDCT)` (libffcv/libffcv.cpp:104-106).

Only the stable public part of `struct jpeg_decompress_struct` is touched (x86-64 layout of
libjpeg API version 62: image_width at byte 48, image_height 52, num_components 56, dct_method 96,
do_fancy_upsampling 100).  The offsets are checked on every call: width/height must come out right
after jpeg_read_header and the two fields must hold their documented defaults (JDCT_ISLOW = 0,
TRUE = 1); with the defaults left alone the output must equal cv2.imdecode (tested).
The struct size is asked of the library itself: jpeg_CreateDecompress refuses a wrong size with a
message naming the right one (read in a child process, since the default error handler exits).
"""
import ctypes
import functools
import glob
import os
import re
import subprocess
import sys

import numpy as np

JDCT_ISLOW, JDCT_IFAST = 0, 1


def library_path():
    try:
        import PIL
    except ImportError:
        return None
    root = os.path.dirname(os.path.dirname(PIL.__file__))
    hits = sorted(glob.glob(os.path.join(root, 'pillow.libs', 'libjpeg*.so*')))
    return hits[0] if hits else None


@functools.lru_cache(maxsize=1)
def struct_size():
    path = library_path()
    if path is None:
        return None
    code = ("import ctypes;l=ctypes.CDLL(%r);c=ctypes.create_string_buffer(4096);e=ctypes.create_string_buffer(1024);"
            "l.jpeg_std_error.restype=ctypes.c_void_p;l.jpeg_std_error.argtypes=[ctypes.c_void_p];"
            "ctypes.cast(c,ctypes.POINTER(ctypes.c_void_p))[0]=l.jpeg_std_error(e);"
            "l.jpeg_CreateDecompress.argtypes=[ctypes.c_void_p,ctypes.c_int,ctypes.c_size_t];"
            "l.jpeg_CreateDecompress(c,62,1)") % path
    res = subprocess.run([sys.executable, '-c', code], capture_output=True, text=True)
    m = re.search(r'library thinks size is (\d+)', res.stderr + res.stdout)
    return int(m.group(1)) if m else None


@functools.lru_cache(maxsize=1)
def _lib():
    lib = ctypes.CDLL(library_path())
    vp = ctypes.c_void_p
    lib.jpeg_std_error.restype = vp
    lib.jpeg_std_error.argtypes = [vp]
    lib.jpeg_CreateDecompress.argtypes = [vp, ctypes.c_int, ctypes.c_size_t]
    lib.jpeg_mem_src.argtypes = [vp, vp, ctypes.c_ulong]
    lib.jpeg_read_header.argtypes = [vp, ctypes.c_int]
    lib.jpeg_read_header.restype = ctypes.c_int
    lib.jpeg_start_decompress.argtypes = [vp]
    lib.jpeg_read_scanlines.argtypes = [vp, vp, ctypes.c_uint]
    lib.jpeg_read_scanlines.restype = ctypes.c_uint
    lib.jpeg_finish_decompress.argtypes = [vp]
    lib.jpeg_destroy_decompress.argtypes = [vp]
    return lib


def available():
    return library_path() is not None and struct_size() is not None


def decode(buf, dct_method=JDCT_IFAST, fancy_upsampling=True, scale_denom=1):
    """RGB pixels of a 3-component JPEG stream as this libjpeg-turbo decodes them; with
    `scale_denom` > 1 at scale 1 / scale_denom (scale_num at byte 68, scale_denom at byte 72 of the
    struct, both 1 by default; output_width / output_height at bytes 136 / 140)."""
    lib = _lib()
    buf = np.ascontiguousarray(buf, dtype=np.uint8)
    cinfo = ctypes.create_string_buffer(4096)
    err = ctypes.create_string_buffer(1024)
    ctypes.cast(cinfo, ctypes.POINTER(ctypes.c_void_p))[0] = lib.jpeg_std_error(err)
    lib.jpeg_CreateDecompress(cinfo, 62, struct_size())
    lib.jpeg_mem_src(cinfo, buf.ctypes.data, buf.size)
    if lib.jpeg_read_header(cinfo, 1) != 1:
        raise ValueError('jpeg_read_header failed')
    ints = ctypes.cast(cinfo, ctypes.POINTER(ctypes.c_int))
    w, h, nc = ints[12], ints[13], ints[14]
    if not (0 < w < 65536 and 0 < h < 65536 and nc == 3 and ints[24] == JDCT_ISLOW and ints[25] == 1):
        raise RuntimeError('unexpected jpeg_decompress_struct layout')
    ints[24] = int(dct_method)
    ints[25] = 1 if fancy_upsampling else 0
    if scale_denom != 1:
        if ints[17] != 1 or ints[18] != 1:
            raise RuntimeError('unexpected jpeg_decompress_struct layout (scale)')
        ints[18] = int(scale_denom)
    lib.jpeg_start_decompress(cinfo)
    if scale_denom != 1:
        if ints[34] != -(-w // scale_denom) or ints[35] != -(-h // scale_denom):
            raise RuntimeError('unexpected jpeg_decompress_struct layout (output size)')
        w, h = ints[34], ints[35]
    out = np.zeros((h, w, 3), dtype=np.uint8)
    row = 0
    while row < h:
        ptr = (ctypes.c_void_p * 1)(out[row].ctypes.data)
        got = lib.jpeg_read_scanlines(cinfo, ptr, 1)
        if got == 0:
            raise ValueError('jpeg_read_scanlines made no progress')
        row += got
    lib.jpeg_finish_decompress(cinfo)
    lib.jpeg_destroy_decompress(cinfo)
    return out
