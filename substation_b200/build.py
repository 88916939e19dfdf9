"""Builds the CUDA library in-tree with nvcc for sm_100a.

``python -m substation_b200.build`` (or :func:`build`) compiles
``csrc/*.cu`` into ``substation_b200/libsubstation_b200.so``.  The reference
instead generates a header per configuration and shells out to nvcc from
``Encoder._compile_module`` (pytorch_module/encoder.py:165-405); here sizes and
layouts are run-time arguments, so one build serves every configuration.
"""

import hashlib
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, 'csrc')
LIB_NAME = 'libsubstation_b200.so'
LIB_PATH = os.path.join(PKG_DIR, LIB_NAME)
#: one library per storage type (fp16 is the default one; the bf16 build is the same sources with -DSB_BF16)
LIB_PATHS = {'fp16': LIB_PATH, 'bf16': os.path.join(PKG_DIR, 'libsubstation_b200_bf16.so')}
DTYPE_FLAGS = {'fp16': [], 'bf16': ['-DSB_BF16']}
SOURCES = ('api.cu', 'fused_ops.cu', 'fused_lnbwd.cu', 'gemm.cu')
NVCC_FLAGS = ['-gencode', 'arch=compute_100a,code=sm_100a', '-O3', '-lineinfo', '-std=c++17',
              '-Xcompiler', '-fPIC', '-shared', '--threads', '0']


def _nvcc():
    for cand in (os.environ.get('NVCC'), shutil.which('nvcc'), '/usr/local/cuda/bin/nvcc'):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError('nvcc not found; set NVCC or put it on PATH')


def have_nvcc():
    try:
        _nvcc()
        return True
    except RuntimeError:
        return False


def stamp_matches(dtype='fp16'):
    """True when the library on disk was built from the current sources."""
    path = LIB_PATHS[dtype]
    stamp = path + '.md5'
    if not (os.path.exists(path) and os.path.exists(stamp)):
        return False
    with open(stamp) as f:
        return f.read().strip() == source_digest()


def source_digest():
    """md5 over the CUDA sources and the public header (same idea as the reference's
    per-configuration hash, pytorch_module/encoder.py:185-187)."""
    h = hashlib.md5()
    files = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC))]
    files.append(os.path.join(PKG_DIR, '..', 'include', 'substation_b200.h'))
    for f in files:
        if os.path.isfile(f):
            with open(f, 'rb') as fh:
                h.update(fh.read())
    return h.hexdigest()


def build(force=False, verbose=False, extra_flags=(), dtypes=('fp16', 'bf16')):
    """Compile the libraries whose sources changed since their last build (both storage types by default, the two
    nvcc runs side by side).  Returns the path of the fp16 library."""
    digest = source_digest()
    srcs = [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    running = []
    for dt in dtypes:
        path = LIB_PATHS[dt]
        if not force and stamp_matches(dt):
            continue
        cmd = [_nvcc(), *NVCC_FLAGS, *DTYPE_FLAGS[dt], *extra_flags, '-o', path, *srcs]
        if verbose:
            print(' '.join(cmd))
        running.append((dt, path, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for dt, path, proc in running:
        out, _ = proc.communicate()
        if proc.returncode != 0:
            raise RuntimeError(f'nvcc failed ({dt}):\n' + out)
        if verbose and out:
            print(out)
        with open(path + '.md5', 'w') as f:
            f.write(digest)
    return LIB_PATH


if __name__ == '__main__':
    print(build(force='--force' in sys.argv, verbose=True,
                extra_flags=('-Xptxas', '-v') if '--ptxas' in sys.argv else ()))
