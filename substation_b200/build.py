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


def stamp_matches():
    """True when the library on disk was built from the current sources."""
    stamp = LIB_PATH + '.md5'
    if not (os.path.exists(LIB_PATH) and os.path.exists(stamp)):
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


def build(force=False, verbose=False, extra_flags=()):
    """Compile the library if the sources changed since the last build."""
    stamp = LIB_PATH + '.md5'
    digest = source_digest()
    if not force and os.path.exists(LIB_PATH) and os.path.exists(stamp):
        with open(stamp) as f:
            if f.read().strip() == digest:
                return LIB_PATH
    srcs = [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    cmd = [_nvcc(), *NVCC_FLAGS, *extra_flags, '-o', LIB_PATH, *srcs]
    if verbose:
        print(' '.join(cmd))
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError('nvcc failed:\n' + res.stdout + res.stderr)
    if verbose and (res.stdout or res.stderr):
        print(res.stdout + res.stderr)
    with open(stamp, 'w') as f:
        f.write(digest)
    return LIB_PATH


if __name__ == '__main__':
    print(build(force='--force' in sys.argv, verbose=True,
                extra_flags=('-Xptxas', '-v') if '--ptxas' in sys.argv else ()))
