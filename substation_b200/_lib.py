"""ctypes binding of the C ABI declared in ``include/substation_b200.h``.

The reference loads its generated ``encoder.so`` the same way
(pytorch_module/encoder.py:395-405).  There is no fallback: if the library is
missing or fails to load, importing an operator raises.
"""

import ctypes
import os

from . import build as _build

SB_MAX_DIMS = 5
SB_OK = 0
SB_MASK_EXPLICIT, SB_MASK_PHILOX = 0, 1
SB_ACT_RELU, SB_ACT_GELU = 0, 1
SB_GEMM_AUTO, SB_GEMM_TCGEN05, SB_GEMM_SIMT = 0, 1, 2

c_void_p, c_int, c_float, c_char_p = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_char_p


class SbTensor(ctypes.Structure):
    _fields_ = [('ptr', c_void_p), ('ndim', ctypes.c_int32),
                ('size', ctypes.c_int64 * SB_MAX_DIMS), ('stride', ctypes.c_int64 * SB_MAX_DIMS)]


class SbDropout(ctypes.Structure):
    _fields_ = [('p', c_float), ('mode', ctypes.c_int32), ('seed', ctypes.c_uint64),
                ('offset', ctypes.c_uint64)]


class SbEpilogue(ctypes.Structure):
    _fields_ = [('kind', ctypes.c_int32), ('bias_dims', c_char_p), ('bias', ctypes.POINTER(SbTensor)),
                ('resid', ctypes.POINTER(SbTensor)), ('mask', ctypes.POINTER(SbTensor)),
                ('out2', ctypes.POINTER(SbTensor)), ('out3', ctypes.POINTER(SbTensor)),
                ('activation', ctypes.c_int32), ('dropout', ctypes.POINTER(SbDropout)),
                ('logical_dims', c_char_p), ('discard_c', ctypes.c_int32)]


class SbEncoderConfig(ctypes.Structure):
    _fields_ = [('batch', ctypes.c_int32), ('seq', ctypes.c_int32), ('heads', ctypes.c_int32),
                ('embed', ctypes.c_int32), ('activation', ctypes.c_int32),
                ('p_softmax', c_float), ('p_resid1', c_float), ('p_activation', c_float),
                ('p_resid2', c_float), ('n_tensors', ctypes.c_int32),
                ('names', ctypes.POINTER(c_char_p)), ('dims', ctypes.POINTER(c_char_p))]


class SubstationError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, status, message):
        super().__init__(f'substation_b200 status {status}: {message}')
        self.status = status
        self.message = message


_T = ctypes.POINTER(SbTensor)
_D = ctypes.POINTER(SbDropout)
_PP = ctypes.POINTER(c_void_p)

#: every exported symbol with (restype, argtypes); the CPU test suite checks the
#: library exports exactly these
SIGNATURES = {
    'sb_status_string': (c_char_p, [c_int]),
    'sb_last_error': (c_char_p, []),
    'sb_version': (c_char_p, []),
    'sb_workspace_bytes': (ctypes.c_size_t, []),
    'sb_attention_input_biases': (c_int, [c_void_p, _T, _T, _T]),
    'sb_softmax_dropout': (c_int, [c_void_p, _T, _T, _T, _T, c_float, _D]),
    'sb_bias_dropout_residual_layernorm': (c_int, [c_void_p] + [_T] * 11 + [_D]),
    'sb_bias_activation_dropout': (c_int, [c_void_p, _T, _T, _T, _T, _T, c_int, _D]),
    'sb_backward_scale_bias': (c_int, [c_void_p, c_void_p] + [_T] * 6),
    'sb_backward_layernorm_residual_dropout': (c_int, [c_void_p] + [_T] * 6),
    'sb_backward_dropout_activation_bias': (c_int, [c_void_p, c_void_p] + [_T] * 5 + [c_int]),
    'sb_extended_backward_scale_bias': (c_int, [c_void_p, c_void_p] + [_T] * 9),
    'sb_backward_attn_out_bias': (c_int, [c_void_p, c_void_p, _T, _T]),
    'sb_backward_scale_bias_layernorm': (c_int, [c_void_p, c_void_p] + [_T] * 11),
    'sb_extended_backward_scale_bias_layernorm': (c_int, [c_void_p, c_void_p] + [_T] * 15),
    'sb_backward_attn_out_bias_noalloc': (c_int, [c_void_p, _T, _T]),
    'sb_attention_scores_softmax': (c_int, [c_void_p, _T, _T, _T, _T, _T, _T, c_float, _D]),
    'sb_attention_scores_softmax_backward': (c_int, [c_void_p, _T, _T, _T, _T, _T, _T]),
    'sb_attention_score_contractions': (c_int, [c_void_p, _T, _T, _T, _T, _T, c_float]),
    'sb_backward_softmax': (c_int, [c_void_p, _T, _T, _T, _T]),
    'sb_backward_attention_input_biases': (c_int, [c_void_p, _T, _T]),
    'sb_backward_encoder_input': (c_int, [c_void_p, _T, _T, _T]),
    'sb_einsum': (c_int, [c_void_p, c_char_p, _T, c_char_p, _T, c_char_p, _T, c_float, c_int, c_void_p,
                        ctypes.c_size_t]),
    'sb_einsum_fused': (c_int, [c_void_p, c_char_p, _T, c_char_p, _T, c_char_p, _T, c_float, ctypes.POINTER(SbEpilogue)]),
    'sb_einsum_last_impl': (c_int, []),
    'sb_device_error': (c_int, [c_void_p, ctypes.POINTER(c_int)]),
    'sb_device_error_reset': (c_int, [c_void_p]),
    'sb_mma_peak_probe': (c_int, [c_void_p, c_int, c_int, ctypes.POINTER(ctypes.c_double)]),
    'sb_set_sm_budget': (c_int, [c_int]),
    'sb_encoder_create': (c_int, [ctypes.POINTER(SbEncoderConfig), ctypes.POINTER(c_void_p)]),
    'sb_encoder_destroy': (c_int, [c_void_p]),
    'sb_encoder_forward': (c_int, [c_void_p, c_void_p, c_void_p, _PP, _PP, c_void_p, c_int,
                                   ctypes.c_uint64, ctypes.c_uint64]),
    'sb_encoder_backward': (c_int, [c_void_p, c_void_p, c_void_p, _PP, _PP, _PP, _PP, c_void_p,
                                    c_void_p]),
    'sb_encoder_set_timing': (c_int, [c_void_p, c_int]),
    'sb_encoder_get_timing': (c_int, [c_void_p, c_int, ctypes.POINTER(c_char_p),
                                      ctypes.POINTER(c_float)]),
    'sb_encoder_set_graphs': (c_int, [c_void_p, c_int]),
    'sb_encoder_set_ffn_grads_event': (c_int, [c_void_p, c_void_p]),
    'sb_encoder_graph_stats': (c_int, [c_void_p, ctypes.POINTER(ctypes.c_longlong), ctypes.POINTER(ctypes.c_longlong)]),
    'sb_encoder_launch_count': (c_int, [c_void_p]),
    'sb_encoder_kernel_count': (c_int, [c_void_p]),
    'sb_encoder_set_fusion': (c_int, [c_void_p, c_int]),
    'sb_encoder_set_dead_stores': (c_int, [c_void_p, c_int]),
}

_libs = {}


def lib_path(dtype='fp16'):
    return _build.LIB_PATHS[dtype]


def dtype_key(dtype):
    """'fp16' / 'bf16' for a torch dtype (or one of those strings); anything else has no library."""
    if isinstance(dtype, str):
        key = dtype
    else:
        import torch
        key = {torch.float16: 'fp16', torch.bfloat16: 'bf16'}.get(dtype)
    if key not in _build.LIB_PATHS:
        raise NotImplementedError(
            f'substation_b200 stores activations and parameters in float16 or bfloat16 (fp32 accumulation); '
            f'{dtype} is not implemented')
    return key


def load(dtype='fp16'):
    """Load the library of one storage type, (re)building first whenever nvcc is at hand and the sources changed
    since the last build.  Without nvcc a library whose stamp does not match the sources is refused: results from
    a stale binary would describe code that no longer exists."""
    key = dtype_key(dtype)
    if key in _libs:
        return _libs[key]
    path = lib_path(key)
    if _build.have_nvcc():
        _build.build(dtypes=(key,))   # returns at once when the digest of the sources matches the stamp
    elif not os.path.exists(path):
        raise RuntimeError(f'{path} is missing and nvcc is not available to build it')
    elif not _build.stamp_matches(key):
        raise RuntimeError(f'{path} was built from other sources than the ones in csrc/ (stamp mismatch) '
                           'and nvcc is not available to rebuild it')
    lib = ctypes.CDLL(path)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)      # AttributeError if a declared symbol is missing
        fn.restype = restype
        fn.argtypes = argtypes
    if key.encode() not in lib.sb_version():
        raise RuntimeError(f'{path} reports {lib.sb_version()!r}, expected a {key} build')
    _libs[key] = lib
    return lib


_last_lib = [None]     # library of the most recent failing call (for the error text)


def check(status, lib=None):
    if status != SB_OK:
        raise SubstationError(status, (lib or load()).sb_last_error().decode())


def tensor_desc(t, order=None):
    """SbTensor for a torch tensor.  ``order``: permutation applied to (size, stride),
    i.e. ``t.permute(order)`` without creating a view."""
    d = SbTensor()
    d.ptr = t.data_ptr()
    dims = range(t.dim()) if order is None else order
    sizes = [t.size(i) for i in dims]
    strides = [t.stride(i) for i in dims]
    d.ndim = len(sizes)
    for i, (s, st) in enumerate(zip(sizes, strides)):
        d.size[i] = s
        d.stride[i] = st
    return d
