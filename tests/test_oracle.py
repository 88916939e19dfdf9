"""The numpy oracle against (1) golden vectors produced by the reference's own
numpy path and (2) an independent torch-autograd restatement with all four
dropouts.  CPU only."""

import glob
import os

import numpy as np
import pytest
import torch

from oracle import encoder_oracle as orc

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), 'golden', 'encoder_*.npz')))


def _load(path):
    z = np.load(path)
    B, J, H, P, U = (int(v) for v in z['meta'])
    # inputs of the '*_fp16_*' cases are stored as float16 (exactly the values the reference computed on)
    z = {k: (z[k].astype(np.float64) if k.startswith('in_') and z[k].dtype == np.float16 else z[k]) for k in z.files}
    params = {k: z['in_' + k] for k in orc.PARAM_NAMES}
    masks = {k: z['in_' + k] for k in ('DROP1MASK', 'DROP2MASK', 'DROP3MASK')
             if 'in_' + k in z}
    return z, (B, J, H, P, U), params, masks


@pytest.mark.parametrize('path', GOLDEN, ids=[os.path.basename(p)[8:-4] for p in GOLDEN])
def test_oracle_matches_reference_numpy_path(path):
    """ln_mode='numpy' reproduces the reference (std + eps) to rounding error."""
    z, (B, J, H, P, U), params, masks = _load(path)
    act = str(z['activation'])
    f = orc.encoder_forward(z['in_X'], params, masks, activation=act, ln_mode='numpy')
    g = orc.encoder_backward(z['in_X'], z['in_DY'], params, f, activation=act, ln_mode='numpy')
    I = H * P

    def close(a, b, what):
        assert a.shape == b.shape, what
        np.testing.assert_allclose(a, b, rtol=1e-9, atol=1e-10, err_msg=what)

    close(f['SB2'], z['ref_y'], 'Y')
    # reference projections are [B,H,J,P] (attention.py:51-62); KKQQVV is [Q=K,Q,V][P,H,B,J]
    close(np.einsum('phbj->bhjp', f['KKQQVV'][0]), z['ref_proj_k'], 'KK')
    close(np.einsum('phbj->bhjp', f['KKQQVV'][1]), z['ref_proj_q'], 'QQ')
    close(np.einsum('phbj->bhjp', f['KKQQVV'][2]), z['ref_proj_v'], 'VV')
    close(np.einsum('hbjk->bhjk', f['ALPHA']), z['ref_scores'], 'ALPHA')
    close(np.einsum('phbj->bjhp', f['GAMMA']).reshape(B, J, I), z['ref_concat'], 'GAMMA')
    close(f['LN1'], z['ref_norm1_normed'], 'LN1')
    close(f['SB1'], z['ref_normed1'], 'SB1')
    close(1.0 / f['LN1STD'] - orc.LN_EPS, z['ref_norm1_std'][..., 0], 'LN1STD')
    close(f['LIN1'], z['ref_ff1_linear'], 'LIN1')
    close(f['DROP2'], z['ref_ff1'], 'DROP2')
    close(f['LN2'], z['ref_norm2_normed'], 'LN2')
    close(f['LN2DIFF'], z['ref_ff_resid'] - z['ref_ff_resid'].mean(-1, keepdims=True), 'LN2DIFF')

    # The reference's LayerNorm backward divides by std without the eps it
    # added in forward (transformer.py:106-118): agreement is to O(eps).
    def close_bwd(a, b, what):
        assert a.shape == b.shape, what
        np.testing.assert_allclose(a, b, rtol=2e-4, atol=2e-4, err_msg=what)

    close_bwd(g['DX'], z['ref_dx'], 'DX')
    close_bwd(np.einsum('phi->hpi', g['DWKQV'][0]), z['ref_dwk'], 'DWK')
    close_bwd(np.einsum('phi->hpi', g['DWKQV'][1]), z['ref_dwq'], 'DWQ')
    close_bwd(np.einsum('phi->hpi', g['DWKQV'][2]), z['ref_dwv'], 'DWV')
    dbqkv = np.stack([np.einsum('ph->hp', g['DBKQV'][q]) for q in (1, 0, 2)])
    close_bwd(dbqkv, z['ref_din_b'], 'DBKQV')
    close_bwd(np.einsum('iph->ihp', g['DWO']).reshape(I, I), z['ref_dwo'], 'DWO')
    close_bwd(g['DBO'], z['ref_dout_b'], 'DBO')
    close_bwd(g['DS1'], z['ref_dnorm1_scale'], 'DS1')
    close_bwd(g['DB1'], z['ref_dnorm1_bias'], 'DB1')
    close_bwd(g['DS2'], z['ref_dnorm2_scale'], 'DS2')
    close_bwd(g['DB2'], z['ref_dnorm2_bias'], 'DB2')
    close_bwd(g['DLINW1'].T, z['ref_dlinear1_w'], 'DLINW1')
    close_bwd(g['DLINB1'], z['ref_dlinear1_b'], 'DLINB1')
    close_bwd(g['DLINW2'].T, z['ref_dlinear2_w'], 'DLINW2')
    close_bwd(g['DLINB2'], z['ref_dlinear2_b'], 'DLINB2')


@pytest.mark.parametrize('path', GOLDEN, ids=[os.path.basename(p)[8:-4] for p in GOLDEN])
def test_cuda_layernorm_form_is_within_tolerance_of_reference(path):
    """rsqrt(var+eps) (CUDA path) vs 1/(std+eps) (numpy path): far inside 1e-2 rel-L2."""
    z, _, params, masks = _load(path)
    act = str(z['activation'])
    f = orc.encoder_forward(z['in_X'], params, masks, activation=act, ln_mode='cuda')
    g = orc.encoder_backward(z['in_X'], z['in_DY'], params, f, activation=act, ln_mode='cuda')
    assert orc.rel_l2(f['SB2'], z['ref_y']) < 1e-4
    assert orc.rel_l2(g['DX'], z['ref_dx']) < 1e-3
    assert orc.rel_l2(g['DLINW1'].T, z['ref_dlinear1_w']) < 1e-3


def _torch_layer(X, p, masks, activation):
    """Independent restatement with torch autograd (float64), four dropouts."""
    P = p['WKQV'].shape[1]
    kqv = torch.einsum('qphi,bji->qphbj', p['WKQV'], X) + p['BKQV'][:, :, :, None, None]
    beta = torch.einsum('phbk,phbj->hbjk', kqv[0], kqv[1]) / P ** 0.5
    alpha = torch.softmax(beta, dim=-1)
    gamma = torch.einsum('phbk,hbjk->phbj', kqv[2], alpha * masks['ATTN_DROP_MASK'])
    att = torch.einsum('iph,phbj->bji', p['WO'], gamma) + p['BO']
    I = X.shape[-1]
    sb1 = torch.nn.functional.layer_norm(att * masks['DROP1MASK'] + X, (I,), p['S1'], p['B1'], 1e-5)
    lin1 = sb1 @ p['LINW1'] + p['LINB1']
    a = torch.relu(lin1) if activation == 'relu' else torch.nn.functional.gelu(lin1, approximate='tanh')
    lin2 = (a * masks['DROP2MASK']) @ p['LINW2'] + p['LINB2']
    return torch.nn.functional.layer_norm(lin2 * masks['DROP3MASK'] + sb1, (I,), p['S2'], p['B2'], 1e-5)


@pytest.mark.parametrize('activation', ['relu', 'gelu'])
def test_oracle_matches_torch_autograd_with_four_dropouts(activation):
    B, J, H, P, U = 2, 7, 3, 4, 20
    I = H * P
    rng = np.random.default_rng(5)
    params = orc.make_params(H, P, U, rng, w_std=0.3, random_affine=True)
    masks = orc.make_masks(B, J, H, I, U, (0.2, 0.1, 0.3, 0.1), seed=3)
    X = rng.normal(0, 1, (B, J, I))
    DY = rng.normal(0, 1, (B, J, I))
    f = orc.encoder_forward(X, params, masks, activation=activation)
    g = orc.encoder_backward(X, DY, params, f, activation=activation)

    tp = {k: torch.tensor(v, dtype=torch.float64, requires_grad=True) for k, v in params.items()}
    tX = torch.tensor(X, requires_grad=True)
    tm = {k: torch.tensor(v, dtype=torch.float64) for k, v in masks.items()}
    Y = _torch_layer(tX, tp, tm, activation)
    Y.backward(torch.tensor(DY))
    np.testing.assert_allclose(f['SB2'], Y.detach().numpy(), rtol=1e-9, atol=1e-10)
    # gelu backward in the reference uses 6-digit constants (transformer.py:17-28)
    tol = 1e-9 if activation == 'relu' else 2e-5
    np.testing.assert_allclose(g['DX'], tX.grad.numpy(), rtol=tol, atol=tol)
    for k in orc.PARAM_NAMES:
        np.testing.assert_allclose(g['D' + k], tp[k].grad.numpy(), rtol=tol, atol=tol, err_msg=k)


def test_layout_round_trip():
    a = np.arange(2 * 3 * 4).reshape(2, 3, 4)
    b = orc.to_layout(a, 'BJI', 'IBJ')
    assert b.shape == (4, 2, 3)
    np.testing.assert_array_equal(orc.from_layout(b, 'IBJ', 'BJI'), a)


def test_philox_known_answer_and_statistics():
    # Known-answer vectors of Philox4x32-10 from the Random123 distribution's kat_vectors
    r = orc.philox4x32_10([0], [0], [0], [0], 0, 0)
    assert [int(x[0]) for x in r] == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    r = orc.philox4x32_10([0xffffffff], [0xffffffff], [0xffffffff], [0xffffffff], 0xffffffff, 0xffffffff)
    assert [int(x[0]) for x in r] == [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
    r = orc.philox4x32_10([0x243f6a88], [0x85a308d3], [0x13198a2e], [0x03707344], 0xa4093822, 0x299f31d0)
    assert [int(x[0]) for x in r] == [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]
    m = orc.philox_mask((64, 1000), 0.1, seed=7, offset=2)
    assert m.dtype == np.uint8 and set(np.unique(m)) == {0, 1}
    n = m.size
    keep = m.mean()
    assert abs(keep - 0.9) < 5 * np.sqrt(0.09 / n) + 1e-4
    assert not np.array_equal(m, orc.philox_mask((64, 1000), 0.1, seed=8, offset=2))
    assert not np.array_equal(m, orc.philox_mask((64, 1000), 0.1, seed=7, offset=3))
    np.testing.assert_array_equal(m, orc.philox_mask((64, 1000), 0.1, seed=7, offset=2))
