"""The allocation-free bias-gradient entry point, called through the C ABI.

It exists for hosts that can pass inputs and outputs but neither a workspace nor
anything that allocates on the device (see the header).  The check: its result
must agree with what the ordinary entry point produces with a caller workspace
(rel-L2 <= 1e-2, the tolerance of the other parity tests; in practice both add the
same fp32 partial sums), on two calls in a row, because the second call finds the
first call's leftovers in the built-in array.  Oversized requests must be refused before anything is launched.
Collected last on purpose, so a failure here cannot hide another test's result.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_noalloc(datt, dbo):
    from substation_b200 import _lib
    lib = _lib.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    return lib.sb_backward_attn_out_bias_noalloc(stream, ctypes.byref(_lib.tensor_desc(datt)),
                                                 ctypes.byref(_lib.tensor_desc(dbo)))


@pytest.mark.parametrize('B,J,F,permute', [(8, 512, 1024, False), (3, 37, 200, False), (4, 64, 256, True),
                                               (2, 48, 16384, False)])   # the last: the largest feature extent accepted
def test_noalloc_matches_workspace_version_on_consecutive_calls(B, J, F, permute):
    from substation_b200 import _lib, ops
    g = torch.Generator(device='cuda:0').manual_seed(B * J + F)
    for call in range(2):
        datt = torch.randn(B, J, F, device='cuda:0', generator=g).half()
        if permute:                       # stored feature-outermost, viewed [B,J,F]
            datt = datt.permute(2, 0, 1).contiguous().permute(1, 2, 0)
        want = torch.full((F,), float('nan'), dtype=torch.float16, device='cuda:0')
        got = torch.full((F,), float('nan'), dtype=torch.float16, device='cuda:0')
        ops.backward_attn_out_bias(datt, want)
        st = _call_noalloc(datt, got)
        assert st == 0, _lib.load().sb_last_error()
        torch.cuda.synchronize()
        assert torch.isfinite(got).all()
        rel = ((got.float() - want.float()).norm() / want.float().norm().clamp_min(1e-6)).item()
        assert rel <= 1e-2, f'call {call}: rel-L2 {rel:.3e} against the workspace version'
        ref = datt.float().sum((0, 1))
        assert (got.float() - ref).norm() <= 1e-2 * ref.norm() + 1e-3


def test_noalloc_refuses_what_the_builtin_scratch_cannot_hold():
    from substation_b200 import _lib
    lib = _lib.load()
    F = 16384 + 8
    datt = torch.zeros(1, 2, F, dtype=torch.float16, device='cuda:0')
    dbo = torch.zeros(F, dtype=torch.float16, device='cuda:0')
    assert _call_noalloc(datt, dbo) == 3
    msg = lib.sb_last_error().decode()
    assert '16384' in msg and 'workspace' in msg
    # more tokens than the kernel's 32-bit token index can count: refused from the sizes alone (the tensor
    # descriptor below points at one element and is never dereferenced)
    one = torch.zeros(8, dtype=torch.float16, device='cuda:0')
    t = _lib.SbTensor()
    t.ptr, t.ndim = one.data_ptr(), 3
    for i, (sz, st) in enumerate(zip((65536, 65536, 8), (0, 0, 1))):
        t.size[i], t.stride[i] = sz, st
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.sb_backward_attn_out_bias_noalloc(stream, ctypes.byref(t), ctypes.byref(_lib.tensor_desc(one))) == 3
    assert 'tokens' in lib.sb_last_error().decode()
