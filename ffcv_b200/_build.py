"""Builds libffcv_b200.so (CUDA kernels + C ABI) in-tree with nvcc for sm_100a."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, 'csrc')
LIB = os.path.join(HERE, 'libffcv_b200.so')
SOURCES = ['context.cu', 'entropy.cu', 'idct.cu', 'gather.cu', 'resize.cu', 'pixel_ops.cu', 'static_decode.cu', 'jpeg_header.cpp']
HEADERS = ['types.h', 'kernels.h', 'jpeg_header.h', os.path.join('..', '..', 'include', 'ffcv_b200.h')]


def _nvcc():
    for cand in (os.environ.get('NVCC'), '/usr/local/cuda/bin/nvcc', 'nvcc'):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    return 'nvcc'


def is_stale():
    if not os.path.exists(LIB):
        return True
    built = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS]
    return any(os.path.exists(d) and os.path.getmtime(d) > built for d in deps)


def build_native(force=False, verbose=False):
    """Compile the library if it is missing or older than its sources.  Returns the path."""
    if not force and not is_stale():
        return LIB
    cmd = [_nvcc(), '-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17',
           '-Xcompiler', '-fPIC,-O3,-pthread', '-shared', '-o', LIB]
    if verbose:
        cmd += ['-Xptxas', '-v']
    cmd += [os.path.join(CSRC, f) for f in SOURCES]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError('nvcc failed:\n' + res.stdout + res.stderr)
    if verbose:
        sys.stderr.write(res.stderr)
    return LIB


if __name__ == '__main__':
    print(build_native(force=True, verbose='-v' in sys.argv))
