"""Helpers for the GPU parity tests: place numpy data on the device in a given
memory layout and hand back the logical-order view the operators take."""

import numpy as np
import torch

from oracle import encoder_oracle as orc

DEV = 'cuda:0'


def h16(a):
    """Round to fp16 and return as float64 (what the kernels will see)."""
    return np.asarray(a).astype(np.float16).astype(np.float64)


def place(a, logical, layout, dtype=torch.float16, pad=0):
    """Device tensor stored as ``layout`` (optionally with ``pad`` extra elements on
    the innermost stored dim to make rows non-dense), viewed in ``logical`` order."""
    st = orc.to_layout(np.asarray(a), logical, layout)
    t = torch.from_numpy(np.ascontiguousarray(st))
    if pad:
        full = torch.zeros(*st.shape[:-1], st.shape[-1] + pad, dtype=t.dtype)
        full[..., :st.shape[-1]] = t
        t = full.to(DEV, dtype)[..., :st.shape[-1]]
    else:
        t = t.to(DEV, dtype)
    return t.permute([layout.index(c) for c in logical])


def empty(shape_logical, logical, layout, dtype=torch.float16, poison=True):
    """Uninitialised output in ``layout`` viewed logically; NaN/0xFF-filled so that
    elements a kernel fails to write are caught."""
    shape = [shape_logical[logical.index(c)] for c in layout]
    t = torch.empty(shape, dtype=dtype, device=DEV)
    if poison:
        t.fill_(float('nan') if dtype == torch.float16 else 255)
    return t.permute([layout.index(c) for c in logical])


def get(t):
    return t.detach().cpu().numpy().astype(np.float64)


def assert_close(got, want, tol=1e-2, what=''):
    got = get(got) if isinstance(got, torch.Tensor) else got
    assert np.isfinite(got).all(), f'{what}: non-finite output (unwritten elements?)'
    r = orc.rel_l2(got, want)
    assert r <= tol, f'{what}: rel-L2 {r:.3e} > {tol}'
    return r
