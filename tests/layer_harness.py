"""Shared driver for layer-level parity: build an ``Encoder`` for a layout
configuration, run forward+backward on seeded inputs through the public module
API, and compare every tensor the reference's own checks list
(pytorch_module/run_encoder.py:206-325 and the longer checklist of
pytorch_module/test_encoder.py:442-637) with the numpy oracle.

Tolerance: rel-L2 <= 1e-2 (fp16 storage / fp32 accumulation against float64),
masks bit-exact.
"""

import os

import numpy as np
import torch

from oracle import encoder_oracle as orc
from substation_b200 import Encoder, layouts as L

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden')


def get_layouts(which):
    """Package-held configurations by name; 'b8_l512' / 'b96_l128' are the reference's two shipped pickles,
    kept as JSON fixtures beside the golden vectors."""
    if isinstance(which, str) and which in ('b8_l512', 'b96_l128'):
        which = os.path.join(GOLDEN_DIR, f'layouts_{which}.json')
    return L.named_layouts(which)


def to_dev(a, logical, layout, device, dtype=torch.float16):
    return torch.from_numpy(orc.to_layout(np.asarray(a), logical, layout)).to(device=device, dtype=dtype)


def round_to(a, dtype):
    """Round float64 data to the storage type and return it as float64 (what the kernels will see)."""
    return torch.from_numpy(np.ascontiguousarray(a)).to(dtype).double().numpy()


def make_case(B, J, H, P, seed, p, random_affine=True, w_std=0.02, explicit_masks=True, dtype=torch.float16):
    """Seeded inputs in logical order, rounded to the storage type so that oracle and kernels see
    identical values.  X ~ N(0,1), weights ~ N(0, w_std), dY ~ N(0,1)."""
    rng = np.random.default_rng(seed)
    I, U = H * P, 4 * H * P
    params = orc.make_params(H, P, U, rng, w_std=w_std, random_affine=random_affine)
    params = {k: round_to(v, dtype) for k, v in params.items()}
    X = round_to(rng.normal(0, 1, (B, J, I)), dtype)
    DY = round_to(rng.normal(0, 1, (B, J, I)), dtype)
    masks = orc.make_masks(B, J, H, I, U, p, seed) if explicit_masks else None
    return X, DY, params, masks


def run_layer_case(B, J, H, P, layouts='uniform', p=0.1, activation='relu', mask_mode='explicit',
                   seed=0, device='cuda:0', tol=1e-2, random_affine=True, w_std=0.02,
                   case=None, return_report=False, dtype=torch.float16):
    """Returns the worst rel-L2 over all compared tensors (asserts each <= tol)."""
    lay = get_layouts(layouts)
    table = L.validate(lay)
    ps = (p, p, p, p) if np.isscalar(p) else tuple(p)
    if case is None:
        X, DY, params, masks = make_case(B, J, H, P, seed, ps, random_affine, w_std,
                                         explicit_masks=(mask_mode == 'explicit'), dtype=dtype)
    else:
        X, DY, params, masks = case
    I = H * P
    enc = Encoder('/tmp/substation_b200_unused', B, J, H, I, lay, dtype, *ps,
                  enable_debug=True, activation=activation, mask_mode=mask_mode, seed=seed)
    enc = enc.to(device)
    enc.train()
    with torch.no_grad():
        for (name, layout), prm in zip(lay['params'], enc.params):
            prm.copy_(to_dev(params[name], L.LOGICAL[name], layout, device, dtype))
    if mask_mode == 'explicit':
        enc.set_masks({n: to_dev(masks[n], L.LOGICAL[n], table[n], device, torch.uint8) for n in L.MASKS})
    Xd = to_dev(X, 'BJI', table['X'], device, dtype).requires_grad_(True)
    DYd = to_dev(DY, 'BJI', table['SB2'], device, dtype)
    first_offset = enc.philox_offset
    Y = enc(Xd)
    Y.backward(DYd)
    torch.cuda.synchronize(device)

    def dbg(name, layout_name=None):
        a = enc.debug[name]
        return orc.from_layout(a, table[layout_name or name], L.LOGICAL[layout_name or name]).astype(np.float64)

    if mask_mode == 'philox':
        # masks come from the kernels: check them bit-exactly against the CPU restatement of
        # the generator, then feed them to the oracle
        masks = {}
        for site, (n, prob) in enumerate(zip(L.MASKS, ps)):
            got = dbg(n).astype(np.uint8)
            want = orc.philox_mask(got.shape, prob, seed, first_offset + site)
            assert np.array_equal(got, want), f'{n}: Philox mask differs from the CPU restatement'
            masks[n] = got
    else:
        for n in L.MASKS:
            assert np.array_equal(dbg(n).astype(np.uint8), masks[n]), f'{n}: explicit mask was modified'

    f = orc.encoder_forward(X, params, masks, activation=activation)
    pattern = None
    if activation == 'relu':
        # relu' is discontinuous at 0: take the kernel's own activation pattern, after checking that it
        # departs from the float64 one only where LIN1 is within fp16 rounding of zero
        pattern = dbg('LIN1') > 0
        differs = pattern != (f['LIN1'] > 0)
        rms = max(1e-3, float(np.sqrt((f['LIN1'] ** 2).mean())))
        assert (np.abs(f['LIN1'][differs]) < 4e-3 * max(1.0, rms)).all(), 'ReLU pattern differs away from zero'
        assert differs.mean() < 5e-3
    g = orc.encoder_backward(X, DY, params, f, activation=activation, relu_pattern=pattern)
    report = {}

    def cmp(name, got, want):
        r = orc.rel_l2(got, want)
        report[name] = r
        assert np.isfinite(got).all(), f'{name}: non-finite values'
        assert r <= tol, f'{name}: rel-L2 {r:.3e} > {tol}'

    cmp('Y', orc.from_layout(Y.detach().float().cpu().numpy(), table['SB2'], 'BJI'), f['SB2'])
    for n in enc._fwd_names:
        if n in L.MASKS:
            continue
        if n in ('WKKWQQWVV', 'SB1_LINW1', 'DROP2_LINW2'):
            want = f[n]
        else:
            want = f[n]
        cmp(n, dbg(n), want)
    cmp('DX', orc.from_layout(Xd.grad.float().cpu().numpy(), table['X'], 'BJI'), g['DX'])
    for n in enc._bwd_names:
        got, want = dbg(n), g[n]
        cmp(n, got, want)
    for n in enc._param_names:
        got = orc.from_layout(enc.debug['D' + n], table[n], L.LOGICAL[n]).astype(np.float64)
        cmp('D' + n, got, g['D' + n])
        # the same gradient must reach autograd
        ag = getattr(enc, n).grad
        assert ag is not None and np.array_equal(ag.float().cpu().numpy(), enc.debug['D' + n].astype(np.float32)), n
    worst = max(report.values())
    return (worst, report) if return_report else worst
