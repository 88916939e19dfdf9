"""Per-operator Python entry points over the C ABI (one per fused kernel, one
for contractions).  They take torch CUDA tensors *viewed in logical index
order* (any permuted view of the stored tensor is fine: strides carry the
layout) and run on the current torch stream.  This is the interface the
reference's kernel harness drives one generated launcher at a time
(pytorch_module/benchmark.py); it is also what the kernel-level parity tests call.
"""

import ctypes
import threading

import torch

from . import _lib
from ._lib import SubstationError  # noqa: F401
from ._lib import (SB_ACT_GELU, SB_ACT_RELU, SB_GEMM_AUTO, SB_GEMM_SIMT, SB_GEMM_TCGEN05,
                   SB_MASK_EXPLICIT, SB_MASK_PHILOX, SbDropout, tensor_desc)

_ACT = {'relu': SB_ACT_RELU, 'gelu': SB_ACT_GELU}
_MODE = {'explicit': SB_MASK_EXPLICIT, 'philox': SB_MASK_PHILOX}
_IMPL = {'auto': SB_GEMM_AUTO, 'tcgen05': SB_GEMM_TCGEN05, 'simt': SB_GEMM_SIMT}
_workspaces = {}


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def workspace(device=None):
    """Zero-initialised scratch for the token-reduction operators, one per
    (device, stream)."""
    dev = torch.device('cuda', torch.cuda.current_device()) if device is None else torch.device(device)
    key = (dev.index, torch.cuda.current_stream(dev).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None:
        ws = torch.zeros(_lib.load().sb_workspace_bytes(), dtype=torch.uint8, device=dev)
        _workspaces[key] = ws
    return ws


def _check_cuda(*tensors):
    for t in tensors:
        if not t.is_cuda:
            raise ValueError('substation_b200 operators need CUDA tensors (there is no CPU path)')


_tls = threading.local()


def _half(*tensors):
    """All floating-point operands of a call share one storage type, float16 or bfloat16; it selects the library
    build the call goes to (remembered per thread until the next call)."""
    dt = tensors[0].dtype
    if dt not in (torch.float16, torch.bfloat16):
        raise TypeError(f'expected float16 or bfloat16, got {dt}')
    for t in tensors:
        if t.dtype != dt:
            raise TypeError(f'operands mix {dt} and {t.dtype}')
    _tls.lib = _lib.load(dt)


def _cur():
    """Library of the current call (float16 build unless ``_half`` chose otherwise)."""
    lib = getattr(_tls, 'lib', None)
    return lib if lib is not None else _lib.load()


def check(status):
    _lib.check(status, _cur())


def _mask(t):
    if t.dtype != torch.uint8:
        raise TypeError(f'dropout masks are uint8, got {t.dtype}')


def _dropout(p, mode, seed, offset):
    d = SbDropout()
    d.p, d.mode, d.seed, d.offset = float(p), _MODE[mode], int(seed), int(offset)
    return d


def _d(t):
    return ctypes.byref(tensor_desc(t))


def _opt(t):
    """Descriptor of an output the caller may leave out (None -> NULL: the operator does not store it)."""
    return None if t is None else _d(t)


def _given(*tensors):
    return [t for t in tensors if t is not None]


def attention_input_biases(inp, bias, out):
    """out[n,p,h,b,j] = inp[n,p,h,b,j] + bias[n,p,h]."""
    _check_cuda(inp, bias, out); _half(inp, bias, out)
    check(_cur().sb_attention_input_biases(_stream(), _d(inp), _d(bias), _d(out)))


def softmax_dropout(beta, alpha, mask, drop, scale=1.0, p=0.0, mode='explicit', seed=0, offset=0):
    """alpha = softmax_k(scale*beta), drop = mask*alpha; all [H,B,J,K]."""
    _check_cuda(beta, alpha, mask, drop); _half(beta, alpha, drop); _mask(mask)
    d = _dropout(p, mode, seed, offset)
    check(_cur().sb_softmax_dropout(_stream(), _d(beta), _d(alpha), _d(mask), _d(drop),
                                         float(scale), ctypes.byref(d)))


def attention_scores_softmax(qq, kk, beta, alpha, mask, drop, scale, p=0.0, mode='explicit', seed=0, offset=0):
    """beta = scale*qq.kk, alpha = softmax(beta), drop = mask*alpha in one kernel; qq, kk are [P,H,B,J].
    ``beta=None``: the scores themselves are not stored."""
    _check_cuda(qq, kk, alpha); _half(qq, kk, alpha, drop, *_given(beta)); _mask(mask)
    d = _dropout(p, mode, seed, offset)
    check(_cur().sb_attention_scores_softmax(_stream(), _d(qq), _d(kk), _opt(beta), _d(alpha), _d(mask), _d(drop),
                                                  float(scale), ctypes.byref(d)))


def attention_scores_softmax_backward(dgamma, vv, alpha, mask, dattn_drop, dbeta):
    """dattn_drop = dgamma.vv and the softmax backward in one kernel; dgamma, vv are [P,H,B,J].
    ``dattn_drop=None``: that intermediate is not stored."""
    _check_cuda(dgamma, vv, alpha); _half(dgamma, vv, alpha, dbeta, *_given(dattn_drop)); _mask(mask)
    check(_cur().sb_attention_scores_softmax_backward(_stream(), _d(dgamma), _d(vv), _d(alpha), _d(mask),
                                                           _opt(dattn_drop), _d(dbeta)))


def attention_score_contractions(scores, x=None, out_rows=None, y=None, out_cols=None, alpha=1.0):
    """out_rows[p,h,b,j] = alpha * sum_k scores[h,b,j,k] x[p,h,b,k] and/or
    out_cols[p,h,b,k] = alpha * sum_j scores[h,b,j,k] y[p,h,b,j], reading scores once."""
    if (x is None) != (out_rows is None) or (y is None) != (out_cols is None):
        raise ValueError('an operand and its output are given together or not at all')
    given = [t for t in (x, out_rows, y, out_cols) if t is not None]
    _check_cuda(scores, *given); _half(scores, *given)
    opt = lambda t: _d(t) if t is not None else None
    check(_cur().sb_attention_score_contractions(_stream(), _d(scores), opt(x), opt(out_rows), opt(y),
                                                      opt(out_cols), float(alpha)))


def backward_softmax(alpha, mask, dattn_drop, dbeta):
    _check_cuda(alpha, mask, dattn_drop, dbeta); _half(alpha, dattn_drop, dbeta); _mask(mask)
    check(_cur().sb_backward_softmax(_stream(), _d(alpha), _d(mask), _d(dattn_drop), _d(dbeta)))


def bias_dropout_residual_layernorm(inp, bias, resid, gamma, beta, mask, lin, diff, istd, ln, out,
                                    p=0.0, mode='explicit', seed=0, offset=0):
    """``lin=None``: the biased input is not stored."""
    _check_cuda(inp, out); _half(inp, bias, resid, gamma, beta, diff, istd, ln, out, *_given(lin)); _mask(mask)
    d = _dropout(p, mode, seed, offset)
    check(_cur().sb_bias_dropout_residual_layernorm(
        _stream(), _d(inp), _d(bias), _d(resid), _d(gamma), _d(beta), _d(mask), _opt(lin), _d(diff),
        _d(istd), _d(ln), _d(out), ctypes.byref(d)))


def bias_activation_dropout(inp, bias, mask, lin1, drop2, activation='relu', p=0.0,
                            mode='explicit', seed=0, offset=0):
    _check_cuda(inp, drop2); _half(inp, bias, lin1, drop2); _mask(mask)
    d = _dropout(p, mode, seed, offset)
    check(_cur().sb_bias_activation_dropout(_stream(), _d(inp), _d(bias), _d(mask), _d(lin1),
                                                 _d(drop2), _ACT[activation], ctypes.byref(d)))


def backward_scale_bias(dy, ln, gamma, dln, dgamma, dbeta):
    _check_cuda(dy); _half(dy, ln, gamma, dln, dgamma, dbeta)
    ws = workspace(dy.device)
    check(_cur().sb_backward_scale_bias(_stream(), ctypes.c_void_p(ws.data_ptr()), _d(dy),
                                             _d(ln), _d(gamma), _d(dln), _d(dgamma), _d(dbeta)))


def backward_layernorm_residual_dropout(dln, istd, diff, mask, dresid, dlin):
    _check_cuda(dln); _half(dln, istd, diff, dresid, dlin); _mask(mask)
    check(_cur().sb_backward_layernorm_residual_dropout(
        _stream(), _d(dln), _d(istd), _d(diff), _d(mask), _d(dresid), _d(dlin)))


def backward_dropout_activation_bias(ddrop2, mask, lin1, dlin1, dbias, activation='relu'):
    _check_cuda(ddrop2); _half(ddrop2, lin1, dlin1, dbias); _mask(mask)
    ws = workspace(ddrop2.device)
    check(_cur().sb_backward_dropout_activation_bias(
        _stream(), ctypes.c_void_p(ws.data_ptr()), _d(ddrop2), _d(mask), _d(lin1), _d(dlin1),
        _d(dbias), _ACT[activation]))


def extended_backward_scale_bias(ln1, gamma1, dresid2, dlin1_linw1, dlin2, dln1, dgamma1, dbeta1,
                                 dlinb2):
    _check_cuda(ln1); _half(ln1, gamma1, dresid2, dlin1_linw1, dlin2, dln1, dgamma1, dbeta1, dlinb2)
    ws = workspace(ln1.device)
    check(_cur().sb_extended_backward_scale_bias(
        _stream(), ctypes.c_void_p(ws.data_ptr()), _d(ln1), _d(gamma1), _d(dresid2),
        _d(dlin1_linw1), _d(dlin2), _d(dln1), _d(dgamma1), _d(dbeta1), _d(dlinb2)))


def backward_scale_bias_layernorm(dy, ln, gamma, istd, diff, mask, dln, dresid, dlin, dgamma, dbeta):
    """backward_scale_bias + backward_layernorm_residual_dropout in one pass (``dln=None``: not stored)."""
    _check_cuda(dy); _half(dy, ln, gamma, istd, diff, dresid, dlin, dgamma, dbeta, *_given(dln)); _mask(mask)
    ws = workspace(dy.device)
    check(_cur().sb_backward_scale_bias_layernorm(
        _stream(), ctypes.c_void_p(ws.data_ptr()), _d(dy), _d(ln), _d(gamma), _d(istd), _d(diff), _d(mask),
        _opt(dln), _d(dresid), _d(dlin), _d(dgamma), _d(dbeta)))


def extended_backward_scale_bias_layernorm(ln1, gamma1, dresid2, dlin1_linw1, dlin2, istd, diff, mask, dln1,
                                           dresid1, datt, dgamma1, dbeta1, dlinb2, dbo):
    """extended_backward_scale_bias + backward_layernorm_residual_dropout + backward_attn_out_bias in one pass
    (``dln1=None``: not stored)."""
    _check_cuda(ln1); _mask(mask)
    _half(ln1, gamma1, dresid2, dlin1_linw1, dlin2, istd, diff, dresid1, datt, dgamma1, dbeta1, dlinb2, dbo, *_given(dln1))
    ws = workspace(ln1.device)
    check(_cur().sb_extended_backward_scale_bias_layernorm(
        _stream(), ctypes.c_void_p(ws.data_ptr()), _d(ln1), _d(gamma1), _d(dresid2), _d(dlin1_linw1), _d(dlin2),
        _d(istd), _d(diff), _d(mask), _opt(dln1), _d(dresid1), _d(datt), _d(dgamma1), _d(dbeta1), _d(dlinb2), _d(dbo)))


def backward_attn_out_bias(datt, dbo):
    _check_cuda(datt); _half(datt, dbo)
    ws = workspace(datt.device)
    check(_cur().sb_backward_attn_out_bias(_stream(), ctypes.c_void_p(ws.data_ptr()),
                                                _d(datt), _d(dbo)))


def backward_attention_input_biases(d, dbias):
    _check_cuda(d); _half(d, dbias)
    check(_cur().sb_backward_attention_input_biases(_stream(), _d(d), _d(dbias)))


def backward_encoder_input(dxatt, dresid1, dx):
    _check_cuda(dxatt); _half(dxatt, dresid1, dx)
    check(_cur().sb_backward_encoder_input(_stream(), _d(dxatt), _d(dresid1), _d(dx)))


def einsum(spec, a, b, c, alpha=1.0, impl='auto', workspace=None):
    """c = alpha * einsum(spec, a, b) with spec like 'phbk,phbj->hbjk'; the dims of
    each operand are named in the order of its own (size, stride) lists.  Returns
    'tcgen05' or 'simt' (the kernel that ran).  ``workspace``: optional uint8 CUDA
    tensor for split-K partial sums."""
    _check_cuda(a, b, c); _half(a, b, c)
    lhs, cd = spec.replace(' ', '').split('->')
    ad, bd = lhs.split(',')
    lib = _cur()
    ws_ptr = ctypes.c_void_p(workspace.data_ptr()) if workspace is not None else None
    ws_len = workspace.numel() * workspace.element_size() if workspace is not None else 0
    check(lib.sb_einsum(_stream(), ad.encode(), _d(a), bd.encode(), _d(b), cd.encode(), _d(c),
                        float(alpha), _IMPL[impl], ws_ptr, ws_len))
    return {SB_GEMM_TCGEN05: 'tcgen05', SB_GEMM_SIMT: 'simt'}.get(lib.sb_einsum_last_impl(), '?')


def einsum_fused(spec, a, b, c, alpha=1.0, *, kind, out2, bias=None, bias_dims=None, resid=None, mask=None, out3=None,
                 activation='relu', p=0.0, mode='explicit', seed=0, offset=0, logical_dims=None, discard_c=False):
    """einsum into c with the next elementwise operator folded into the contraction's epilogue:
    kind='bias' (out2 = c + bias), 'residual' (out2 = c + resid) or 'bias_act_dropout'
    (out2 = c + bias, out3 = mask * act(out2)).  Raises SubstationError with status 3 when the
    contraction does not run on the kernel that supports it."""
    _check_cuda(a, b, c, out2); _half(a, b, c, out2)
    lhs, cd = spec.replace(' ', '').split('->')
    ad, bd = lhs.split(',')
    ep = _lib.SbEpilogue()
    ep.kind = {'bias': 1, 'residual': 2, 'bias_act_dropout': 3}[kind]
    keep = [tensor_desc(out2)]
    ep.out2 = ctypes.pointer(keep[-1])
    if bias is not None:
        _half(bias)
        keep.append(tensor_desc(bias)); ep.bias = ctypes.pointer(keep[-1])
        ep.bias_dims = bias_dims.encode()
    if resid is not None:
        _half(resid)
        keep.append(tensor_desc(resid)); ep.resid = ctypes.pointer(keep[-1])
    if mask is not None:
        _mask(mask)
        keep.append(tensor_desc(mask)); ep.mask = ctypes.pointer(keep[-1])
    if out3 is not None:
        _half(out3)
        keep.append(tensor_desc(out3)); ep.out3 = ctypes.pointer(keep[-1])
    ep.activation = _ACT[activation]
    d = _dropout(p, mode, seed, offset)
    ep.dropout = ctypes.pointer(d)
    if logical_dims is not None:
        ep.logical_dims = logical_dims.encode()
    ep.discard_c = 1 if discard_c else 0      # c then only gives the geometry; it is not stored
    check(_cur().sb_einsum_fused(_stream(), ad.encode(), _d(a), bd.encode(), _d(b), cd.encode(), _d(c),
                                      float(alpha), ctypes.byref(ep)))


def _loaded():
    """Every library build this process has loaded (the float16 one is loaded if none is yet)."""
    return list(_lib._libs.values()) or [_lib.load()]


def device_error():
    """Code set on the current device when a bounded wait inside a kernel ran out (0 = none since the last
    ``device_error_reset``); every loaded build of the library is asked."""
    for lib in _loaded():
        code = ctypes.c_int(0)
        _lib.check(lib.sb_device_error(_stream(), ctypes.byref(code)), lib)
        if code.value:
            return code.value
    return 0


def device_error_reset():
    """Clear that code once the failed pass has been dealt with (while it is set, every tcgen05 kernel on the
    device gives up its waits at once)."""
    for lib in _loaded():
        _lib.check(lib.sb_device_error_reset(_stream()), lib)


def mma_peak_probe(k_blocks, bf16=False):
    """Enqueue one MMA-only launch (see ``sb_mma_peak_probe``) on the current stream; returns its FLOP count."""
    fl = ctypes.c_double(0.0)
    lib = _lib.load()
    _lib.check(lib.sb_mma_peak_probe(_stream(), int(k_blocks), 1 if bf16 else 0, ctypes.byref(fl)), lib)
    return fl.value


def set_sm_budget(n_sms):
    """Size every persistent grid of the library (contractions, attention, LayerNorm, reductions) for ``n_sms``
    SMs (0 = all), leaving the rest to a kernel that runs beside them, e.g. the NCCL allreduce of the
    data-parallel path.  Applies to both storage-type builds of the library."""
    for key in ('fp16', 'bf16'):
        lib = _lib.load(key)
        _lib.check(lib.sb_set_sm_budget(int(n_sms)), lib)
