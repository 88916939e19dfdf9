"""CPU checks of the C-ABI boundary: the library builds for sm_100a, loads, exports
every function the public header declares, and rejects bad requests with status
codes before touching a device (no compute calls here)."""

import ctypes
import os
import re

import pytest

from substation_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_builds_for_sm100a_and_loads():
    path = build.build()
    assert os.path.exists(path)
    lib = _lib.load()
    assert b'sm_100a' in lib.sb_version()
    assert lib.sb_workspace_bytes() >= 1 << 20


def test_every_declared_symbol_is_exported_and_bound():
    with open(os.path.join(ROOT, 'include', 'substation_b200.h')) as f:
        text = re.sub(r'/\*.*?\*/', '', f.read(), flags=re.S)
    declared = set(re.findall(r'\b(sb_[a-z0-9_]+)\s*\(', text))
    assert declared, 'no declarations found'
    for key in ('fp16', 'bf16'):                       # one build of the same sources per storage type
        lib = ctypes.CDLL(_lib.lib_path(key))
        for name in declared:
            assert hasattr(lib, name), f'{name} declared in the header but not exported by the {key} build'
        assert key.encode() in _lib.load(key).sb_version()
    assert declared == set(_lib.SIGNATURES), (declared ^ set(_lib.SIGNATURES))


def test_status_strings():
    lib = _lib.load()
    assert lib.sb_status_string(0) == b'ok'
    assert lib.sb_status_string(2) == b'invalid layout'
    assert lib.sb_status_string(99) == b'unknown status'


def _cfg(names, dims, **kw):
    cfg = _lib.SbEncoderConfig()
    cfg.batch, cfg.seq, cfg.heads, cfg.embed = kw.get('batch', 2), kw.get('seq', 8), kw.get('heads', 2), kw.get('embed', 16)
    cfg.activation = kw.get('activation', 0)
    cfg.p_softmax = cfg.p_resid1 = cfg.p_activation = cfg.p_resid2 = kw.get('p', 0.1)
    cfg.n_tensors = len(names)
    keep = ((ctypes.c_char_p * len(names))(*[n.encode() for n in names]),
            (ctypes.c_char_p * len(names))(*[d.encode() for d in dims]))
    cfg.names, cfg.dims = keep
    return cfg, keep


def _table():
    from substation_b200 import layouts as L
    t = L.validate(L.uniform_layouts())
    return list(t.keys()), list(t.values())


@pytest.mark.parametrize('mutate,status,fragment', [
    (lambda n, d: d.__setitem__(n.index('BETA'), 'HBJJ'), 2, 'not a permutation'),
    (lambda n, d: d.__setitem__(n.index('KKQQVV'), 'PQHBJ'), 2, 'Q outermost'),
    (lambda n, d: d.__setitem__(n.index('SB2'), 'IBJ'), 2, 'must be equal'),
    (lambda n, d: (n.pop(), d.pop()), 2, 'no layout given'),
    (lambda n, d: n.__setitem__(3, 'NOPE'), 2, 'unknown tensor'),
])
def test_encoder_create_rejects_bad_layouts_without_a_device(mutate, status, fragment):
    lib = _lib.load()
    names, dims = _table()
    mutate(names, dims)
    cfg, keep = _cfg(names, dims)
    handle = ctypes.c_void_p()
    st = lib.sb_encoder_create(ctypes.byref(cfg), ctypes.byref(handle))
    assert st == status, lib.sb_last_error()
    assert fragment in lib.sb_last_error().decode()
    assert not handle.value


def test_encoder_create_rejects_bad_sizes():
    lib = _lib.load()
    names, dims = _table()
    for kw, frag in ((dict(embed=15), 'multiple of the head count'), (dict(batch=0), 'positive'),
                     (dict(p=1.0), 'dropout'), (dict(activation=7), 'activation')):
        cfg, keep = _cfg(names, dims, **kw)
        handle = ctypes.c_void_p()
        assert lib.sb_encoder_create(ctypes.byref(cfg), ctypes.byref(handle)) == 1
        assert frag in lib.sb_last_error().decode()


def _tensor(sizes, strides, ptr=0x1000):
    t = _lib.SbTensor()
    t.ptr, t.ndim = ptr, len(sizes)
    for i, (s, st) in enumerate(zip(sizes, strides)):
        t.size[i], t.stride[i] = s, st
    return t


def test_einsum_planner_rejects_non_gemm_requests_before_any_launch():
    lib = _lib.load()
    a = _tensor([4, 6, 8], [48, 8, 1])
    b = _tensor([4, 6, 8], [48, 8, 1])
    c = _tensor([4, 4], [4, 1])
    call = lambda ad, bd, cd, aa=a, bb=b, cc=c: lib.sb_einsum(None, ad, ctypes.byref(aa), bd, ctypes.byref(bb), cd,
                                                             ctypes.byref(cc), 1.0, 0, None, 0)
    assert call(b'bmk', b'bnk', b'mnx') == 2            # rank mismatch
    assert b'rank' in lib.sb_last_error()
    assert call(b'bmm', b'bnk', b'mn') == 2             # repeated index
    c3 = _tensor([4, 6, 5], [30, 5, 1])
    assert call(b'bmk', b'bnk', b'bmn', cc=c3) == 1     # extent of n differs
    assert b'differs' in lib.sb_last_error()
    c3 = _tensor([4, 6, 6], [36, 6, 1])
    assert call(b'bmk', b'bnz', b'bmn', cc=c3) == 3     # index in one operand only
    # batch dims that do not collapse to one stride: (h,b) adjacent in A, interleaved in C
    a4 = _tensor([2, 3, 4, 8], [96, 32, 8, 1])
    b4 = _tensor([2, 3, 5, 8], [120, 40, 8, 1])
    c4 = _tensor([2, 4, 3, 5], [60, 15, 5, 1])          # h m b n
    st = lib.sb_einsum(None, b'hbmk', ctypes.byref(a4), b'hbnk', ctypes.byref(b4), b'hmbn', ctypes.byref(c4), 1.0, 0, None, 0)
    assert st == 3 and b'collapse' in lib.sb_last_error()


def test_operator_argument_validation_without_a_device():
    lib = _lib.load()
    d = _lib.SbDropout()
    d.p, d.mode = 0.1, 0
    x = _tensor([2, 3, 4, 8], [96, 32, 8, 1])
    bad = _tensor([2, 3, 4, 9], [108, 36, 9, 1])
    assert lib.sb_softmax_dropout(None, ctypes.byref(x), ctypes.byref(bad), ctypes.byref(x), ctypes.byref(x),
                                  1.0, ctypes.byref(d)) == 1
    assert b'extent mismatch' in lib.sb_last_error()
    d.p = 1.5
    assert lib.sb_softmax_dropout(None, ctypes.byref(x), ctypes.byref(x), ctypes.byref(x), ctypes.byref(x),
                                  1.0, ctypes.byref(d)) == 1
    assert b'probability' in lib.sb_last_error()
    x3 = _tensor([2, 3, 8], [24, 8, 1])
    v = _tensor([8], [2])
    vec = _tensor([8], [1])
    assert lib.sb_backward_scale_bias(None, None, ctypes.byref(x3), ctypes.byref(x3), ctypes.byref(v),
                                      ctypes.byref(x3), ctypes.byref(vec), ctypes.byref(vec)) == 3
    assert b'contiguous' in lib.sb_last_error()
    assert lib.sb_backward_scale_bias(None, None, ctypes.byref(x3), ctypes.byref(x3), ctypes.byref(vec),
                                      ctypes.byref(x3), ctypes.byref(vec), ctypes.byref(vec)) == 1
    assert b'workspace' in lib.sb_last_error()


def test_fused_epilogue_refuses_misaligned_side_inputs_before_any_launch():
    """The paired-CTA epilogue reads bias, residual and mask with 128-bit accesses; operands it could not read
    that way come back as SB_ERR_ALIGNMENT from the pointer values alone (no CUDA call has been made when the
    status returns: this runs without a device)."""
    lib = _lib.load()
    M, N, K = 512, 512, 256
    a = _tensor([M, K], [K, 1])
    b = _tensor([N, K], [K, 1])
    c = _tensor([M, N], [N, 1], ptr=0x100000)
    out2 = _tensor([M, N], [N, 1], ptr=0x200000)

    def call(ep):
        return lib.sb_einsum_fused(None, b'mk', ctypes.byref(a), b'nk', ctypes.byref(b), b'mn', ctypes.byref(c), 1.0,
                                   ctypes.byref(ep))
    # bias: a slice that starts one element into an aligned buffer
    bias = _tensor([N], [1], ptr=0x300000 + 2)
    ep = _lib.SbEpilogue()
    ep.kind, ep.bias_dims, ep.bias, ep.out2 = 1, b'n', ctypes.pointer(bias), ctypes.pointer(out2)
    assert call(ep) == 5, lib.sb_last_error()
    assert b'bias' in lib.sb_last_error()
    # residual with an odd base
    resid = _tensor([M, N], [N, 1], ptr=0x400000 + 8)
    ep = _lib.SbEpilogue()
    ep.kind, ep.resid, ep.out2 = 2, ctypes.pointer(resid), ctypes.pointer(out2)
    assert call(ep) == 5 and b'resid' in lib.sb_last_error()
    # mask: aligned base but a padded row pitch that is a multiple of 8 only
    Np = N + 8
    cp = _tensor([M, N], [Np, 1], ptr=0x100000)
    o2, o3 = _tensor([M, N], [Np, 1], ptr=0x200000), _tensor([M, N], [Np, 1], ptr=0x500000)
    mask = _tensor([M, N], [Np, 1], ptr=0x600000)
    bias = _tensor([N], [1], ptr=0x300000)
    d = _lib.SbDropout()
    d.p, d.mode = 0.1, 0
    ep = _lib.SbEpilogue()
    ep.kind, ep.bias_dims, ep.bias, ep.mask = 3, b'n', ctypes.pointer(bias), ctypes.pointer(mask)
    ep.out2, ep.out3, ep.activation, ep.dropout = ctypes.pointer(o2), ctypes.pointer(o3), 0, ctypes.pointer(d)
    st = lib.sb_einsum_fused(None, b'mk', ctypes.byref(a), b'nk', ctypes.byref(b), b'mn', ctypes.byref(cp), 1.0,
                             ctypes.byref(ep))
    assert st == 5 and b'mask' in lib.sb_last_error()
