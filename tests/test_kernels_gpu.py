"""Kernel-level parity on the GPU: every fused operator, called through the C ABI,
against the numpy oracle on the same seeded inputs.  Mirrors the per-kernel
``compare_with_reference`` checks of pytorch_module/benchmark.py:375-1325
(tolerance there: allclose(1e-2, 1e-2); here rel-L2 <= 1e-2 and masks bit-exact).
Sizes are small enough for the oracle; each operator is run with contiguous
feature-innermost layouts (128-bit path), with permuted layouts (strided path)
and with ragged extents."""

import itertools

import numpy as np
import pytest
import torch

from oracle import encoder_oracle as orc
from tests.gpu_util import DEV, assert_close, empty, get, h16, place

pytestmark = pytest.mark.gpu

LAY3 = ['BJI', 'IBJ', 'JBI']


def _ops():
    from substation_b200 import ops
    return ops


@pytest.mark.parametrize('H,B,J,K,lay', [
    (2, 3, 16, 512, 'HBJK'), (2, 3, 10, 128, 'HBJK'), (1, 2, 5, 64, 'HBJK'), (2, 2, 7, 1024, 'HBJK'),
    (2, 2, 6, 37, 'HBJK'), (2, 3, 8, 40, 'KHBJ'), (2, 2, 8, 264, 'BJHK'), (1, 1, 3, 2048, 'HBJK'),
])
@pytest.mark.parametrize('scale', [1.0, 0.125])
def test_softmax_dropout_and_backward(H, B, J, K, lay, scale):
    ops = _ops()
    rng = np.random.default_rng(K + J)
    beta = h16(rng.normal(0, 2, (H, B, J, K)))
    mask = (rng.random((H, B, J, K)) >= 0.3).astype(np.uint8)
    d_beta = place(beta, 'HBJK', lay)
    d_mask = place(mask, 'HBJK', lay, torch.uint8)
    d_alpha, d_drop = empty((H, B, J, K), 'HBJK', lay), empty((H, B, J, K), 'HBJK', lay)
    ops.softmax_dropout(d_beta, d_alpha, d_mask, d_drop, scale=scale, p=0.3, mode='explicit')
    alpha, drop = orc.softmax_dropout(beta, mask, scale)
    assert_close(d_alpha, alpha, what='ALPHA')
    assert_close(d_drop, drop, what='ATTN_DROP')
    # exact structural property: DROP == mask * ALPHA element for element
    assert np.array_equal(get(d_drop), get(d_alpha) * mask)
    assert np.array_equal(get(d_mask), mask)

    g = h16(rng.normal(0, 1, (H, B, J, K)))
    alpha16 = h16(alpha)
    d_g, d_a = place(g, 'HBJK', lay), place(alpha16, 'HBJK', lay)
    d_out = empty((H, B, J, K), 'HBJK', lay)
    ops.backward_softmax(d_a, d_mask, d_g, d_out)
    assert_close(d_out, orc.softmax_dropout_backward(alpha16, mask, g), what='DBETA')


def test_softmax_philox_mask_matches_cpu_generator_and_is_layout_independent():
    ops = _ops()
    H, B, J, K = 2, 3, 8, 128
    beta = h16(np.random.default_rng(0).normal(0, 1, (H, B, J, K)))
    masks = []
    for lay in ('HBJK', 'KHBJ'):
        d_mask = empty((H, B, J, K), 'HBJK', lay, torch.uint8)
        d_alpha, d_drop = empty((H, B, J, K), 'HBJK', lay), empty((H, B, J, K), 'HBJK', lay)
        ops.softmax_dropout(place(beta, 'HBJK', lay), d_alpha, d_mask, d_drop, p=0.25, mode='philox',
                            seed=1234, offset=7)
        masks.append(get(d_mask).astype(np.uint8))
        assert np.array_equal(get(d_drop), get(d_alpha) * masks[-1])
    want = orc.philox_mask((H, B, J, K), 0.25, 1234, 7)
    assert np.array_equal(masks[0], want)
    assert np.array_equal(masks[1], want)


@pytest.mark.parametrize('B,J,F', [(2, 8, 1024), (3, 5, 256), (2, 4, 100), (1, 3, 2048), (2, 16, 64)])
@pytest.mark.parametrize('lays', ['same', 'mixed'])
def test_bdrln_and_blnrd(B, J, F, lays):
    ops = _ops()
    rng = np.random.default_rng(F + B)
    x = h16(rng.normal(0, 1, (B, J, F)))
    res = h16(rng.normal(0, 1, (B, J, F)))
    bias, gamma, beta = (h16(rng.normal(m, 0.1, F)) for m in (0, 1, 0))
    mask = (rng.random((B, J, F)) >= 0.1).astype(np.uint8)
    names = ['in', 'resid', 'mask', 'lin', 'diff', 'ln', 'out']
    lay = {n: 'BJI' for n in names} if lays == 'same' else dict(zip(names, itertools.cycle(LAY3[1:] + LAY3[:1])))
    sl = 'BJ' if lays == 'same' else 'JB'
    d = {
        'in': place(x, 'BJI', lay['in']), 'resid': place(res, 'BJI', lay['resid']),
        'mask': place(mask, 'BJI', lay['mask'], torch.uint8),
    }
    for n in ('lin', 'diff', 'ln', 'out'):
        d[n] = empty((B, J, F), 'BJI', lay[n])
    d_istd = empty((B, J), 'BJ', sl)
    tb, tg, tbt = (torch.tensor(v, dtype=torch.float16, device=DEV) for v in (bias, gamma, beta))
    ops.bias_dropout_residual_layernorm(d['in'], tb, d['resid'], tg, tbt, d['mask'], d['lin'], d['diff'],
                                        d_istd, d['ln'], d['out'], p=0.1, mode='explicit')
    lin, diff, istd, ln, out = orc.bias_dropout_residual_layernorm(x, bias, res, mask, gamma, beta)
    for n, want in (('lin', lin), ('diff', diff), ('ln', ln), ('out', out)):
        assert_close(d[n], want, what=n)
    assert_close(d_istd, istd, what='istd')

    # backward from the stored (fp16) diff / istd
    g = h16(rng.normal(0, 1, (B, J, F)))
    diff16, istd16 = h16(diff), h16(istd)
    d_res, d_lin = empty((B, J, F), 'BJI', lay['lin']), empty((B, J, F), 'BJI', lay['out'])
    ops.backward_layernorm_residual_dropout(place(g, 'BJI', lay['in']), place(istd16, 'BJ', sl),
                                            place(diff16, 'BJI', lay['diff']), d['mask'], d_res, d_lin)
    dres, dlin = orc.backward_layernorm_residual_dropout(g, diff16, istd16, mask)
    assert_close(d_res, dres, what='dresid')
    assert_close(d_lin, dlin, what='dlin')


def test_bdrln_in_place_and_philox():
    ops = _ops()
    B, J, F = 2, 8, 512
    rng = np.random.default_rng(3)
    x, res = h16(rng.normal(0, 1, (B, J, F))), h16(rng.normal(0, 1, (B, J, F)))
    bias = h16(rng.normal(0, 0.1, F))
    d_in = place(x, 'BJI', 'BJI')
    d_mask = empty((B, J, F), 'BJI', 'BJI', torch.uint8)
    outs = [empty((B, J, F), 'BJI', 'BJI') for _ in range(3)]
    d_istd = empty((B, J), 'BJ', 'BJ')
    one = torch.ones(F, dtype=torch.float16, device=DEV)
    zero = torch.zeros(F, dtype=torch.float16, device=DEV)
    ops.bias_dropout_residual_layernorm(d_in, torch.tensor(bias, dtype=torch.float16, device=DEV),
                                        place(res, 'BJI', 'BJI'), one, zero, d_mask, d_in, outs[0], d_istd,
                                        outs[1], outs[2], p=0.5, mode='philox', seed=5, offset=11)
    mask = get(d_mask).astype(np.uint8)
    assert np.array_equal(mask, orc.philox_mask((B, J, F), 0.5, 5, 11))
    lin, diff, istd, ln, out = orc.bias_dropout_residual_layernorm(x, bias, res, mask, np.ones(F), np.zeros(F))
    assert_close(d_in, lin, what='lin written over in')
    assert_close(outs[2], out, what='out')


@pytest.mark.parametrize('B,J,F,lay_in,lay_out', [
    (2, 8, 4096, 'BJI', 'BJI'), (2, 5, 1000, 'BJI', 'BJI'), (2, 8, 256, 'IBJ', 'BJI'), (3, 4, 72, 'JBI', 'IBJ')])
@pytest.mark.parametrize('activation', ['relu', 'gelu'])
def test_bad_and_bdrlb(B, J, F, lay_in, lay_out, activation):
    ops = _ops()
    rng = np.random.default_rng(F)
    x = h16(rng.normal(0, 1, (B, J, F)))
    bias = h16(rng.normal(0, 0.2, F))
    mask = (rng.random((B, J, F)) >= 0.2).astype(np.uint8)
    d_mask = place(mask, 'BJI', lay_out, torch.uint8)
    d_lin1, d_drop2 = empty((B, J, F), 'BJI', lay_out), empty((B, J, F), 'BJI', lay_in)
    tb = torch.tensor(bias, dtype=torch.float16, device=DEV)
    ops.bias_activation_dropout(place(x, 'BJI', lay_in), tb, d_mask, d_lin1, d_drop2, activation=activation,
                                p=0.2, mode='explicit')
    lin1, drop2 = orc.bias_activation_dropout(x, bias, mask, activation)
    assert_close(d_lin1, lin1, what='LIN1')
    assert_close(d_drop2, drop2, what='DROP2')

    g = h16(rng.normal(0, 1, (B, J, F)))
    lin16 = h16(lin1)
    d_dlin1 = empty((B, J, F), 'BJI', lay_in)
    d_db = torch.full((F,), float('nan'), dtype=torch.float16, device=DEV)
    ops.backward_dropout_activation_bias(place(g, 'BJI', lay_out), d_mask, place(lin16, 'BJI', lay_out), d_dlin1,
                                         d_db, activation=activation)
    dlin1, db = orc.backward_dropout_activation_bias(g, mask, lin16, activation)
    assert_close(d_dlin1, dlin1, what='DLIN1')
    assert_close(d_db, db, what='DLINB1')


@pytest.mark.parametrize('B,J,F,lay', [(4, 64, 1024, 'BJI'), (2, 9, 200, 'BJI'), (2, 16, 128, 'IBJ'),
                                       (3, 8, 520, 'JBI'), (16, 128, 64, 'BJI')])
def test_token_reductions_bsb_ebsb_baob(B, J, F, lay):
    ops = _ops()
    rng = np.random.default_rng(B * F)
    dy, ln = h16(rng.normal(0, 1, (B, J, F))), h16(rng.normal(0, 1, (B, J, F)))
    gamma = h16(rng.normal(1, 0.1, F))
    tg = torch.tensor(gamma, dtype=torch.float16, device=DEV)
    vec = lambda: torch.full((F,), float('nan'), dtype=torch.float16, device=DEV)
    d_dln, d_dg, d_db = empty((B, J, F), 'BJI', lay), vec(), vec()
    for _ in range(2):   # twice: the workspace counters must be left clean
        ops.backward_scale_bias(place(dy, 'BJI', lay), place(ln, 'BJI', 'BJI'), tg, d_dln, d_dg, d_db)
    dln, dg, db = orc.backward_scale_bias(dy, ln, gamma)
    assert_close(d_dln, dln, what='DLN')
    assert_close(d_dg, dg, what='dgamma')
    assert_close(d_db, db, what='dbeta')

    r2, lw, l2 = (h16(rng.normal(0, 1, (B, J, F))) for _ in range(3))
    d_dln1, d_dg1, d_db1, d_dl2 = empty((B, J, F), 'BJI', lay), vec(), vec(), vec()
    ops.extended_backward_scale_bias(place(ln, 'BJI', lay), tg, place(r2, 'BJI', 'BJI'), place(lw, 'BJI', lay),
                                     place(l2, 'BJI', 'BJI'), d_dln1, d_dg1, d_db1, d_dl2)
    dln1, dg1, db1, dl2 = orc.extended_backward_scale_bias(ln, gamma, r2, lw, l2)
    assert_close(d_dln1, dln1, what='DLN1')
    assert_close(d_dg1, dg1, what='dgamma1')
    assert_close(d_db1, db1, what='dbeta1')
    assert_close(d_dl2, dl2, what='dlinb2')

    d_dbo = vec()
    ops.backward_attn_out_bias(place(dy, 'BJI', lay), d_dbo)
    assert_close(d_dbo, orc.backward_attn_out_bias(dy), what='DBO')
    # determinism: a second run gives bit-identical sums
    again = vec()
    ops.backward_attn_out_bias(place(dy, 'BJI', lay), again)
    assert torch.equal(d_dbo, again)


@pytest.mark.parametrize('N,P,H,B,J,lin,lout', [
    (3, 8, 2, 2, 64, 'QPHBJ', 'QPHBJ'), (3, 4, 2, 3, 40, 'QPHBJ', 'QHBPJ'), (1, 4, 2, 2, 10, 'QPHBJ', 'QJBHP'),
    (3, 2, 2, 1, 1200, 'QPHBJ', 'QPHBJ')])
def test_aib_baib_bei(N, P, H, B, J, lin, lout):
    ops = _ops()
    rng = np.random.default_rng(J)
    x = h16(rng.normal(0, 1, (N, P, H, B, J)))
    bias = h16(rng.normal(0, 0.5, (N, P, H)))
    d_out = empty((N, P, H, B, J), 'QPHBJ', lout)
    ops.attention_input_biases(place(x, 'QPHBJ', lin), place(bias, 'QPH', 'QPH'), d_out)
    assert_close(d_out, orc.attention_input_biases(x, bias), what='KKQQVV')
    d_db = empty((N, P, H), 'QPH', 'QPH')
    ops.backward_attention_input_biases(place(x, 'QPHBJ', lout), d_db)
    assert_close(d_db, orc.backward_attention_input_biases(x), what='DBKQV')

    I = P * H * 4
    a, b = h16(rng.normal(0, 1, (B, J, I))), h16(rng.normal(0, 1, (B, J, I)))
    for la, lb, lo in (('BJI', 'BJI', 'BJI'), ('BJI', 'BJI', 'IBJ'), ('IBJ', 'JBI', 'BJI')):
        d_dx = empty((B, J, I), 'BJI', lo)
        ops.backward_encoder_input(place(a, 'BJI', la), place(b, 'BJI', lb), d_dx)
        assert_close(d_dx, a + b, tol=1e-3, what='DX')


def test_full_size_sweep_shapes_structural_properties():
    """Config-4 extents (H16 B96 J=K=128; [96,128,4096]): too large for the float64
    oracle in a test, so check size-independent properties and a torch fp32 restatement."""
    ops = _ops()
    H, B, J, K = 16, 96, 128, 128
    g = torch.Generator(device=DEV).manual_seed(0)
    beta = (torch.randn(H, B, J, K, device=DEV, generator=g) * 2).half()
    mask = (torch.rand(H, B, J, K, device=DEV, generator=g) >= 0.1).to(torch.uint8)
    alpha, drop = torch.empty_like(beta), torch.empty_like(beta)
    ops.softmax_dropout(beta, alpha, mask, drop, scale=0.125, p=0.1, mode='explicit')
    ref = torch.softmax(beta.float() * 0.125, dim=-1)
    assert (alpha.float() - ref).norm() / ref.norm() < 1e-3
    assert torch.equal(drop, alpha * mask)
    assert (alpha.float().sum(-1) - 1).abs().max() < 2e-2
    # Philox keep-rate at full size: binomial 5-sigma
    ops.softmax_dropout(beta, alpha, mask, drop, scale=0.125, p=0.1, mode='philox', seed=9, offset=0)
    n = mask.numel()
    keep = mask.float().mean().item()
    assert abs(keep - (1 - 6554 / 65536)) < 5 * (0.09 / n) ** 0.5
    # no correlation between neighbouring rows / columns
    m = mask.float() - keep
    assert abs((m[..., 1:] * m[..., :-1]).mean().item()) < 1e-3
    assert abs((m[:, :, 1:] * m[:, :, :-1]).mean().item()) < 1e-3

    Bt, Jt, U = 96, 128, 4096
    x = torch.randn(Bt, Jt, U, device=DEV, generator=g).half()
    bias = (torch.randn(U, device=DEV, generator=g) * 0.02).half()
    m2 = (torch.rand(Bt, Jt, U, device=DEV, generator=g) >= 0.1).to(torch.uint8)
    lin1, drop2 = torch.empty_like(x), torch.empty_like(x)
    ops.bias_activation_dropout(x, bias, m2, lin1, drop2, p=0.1, mode='explicit')
    ref = (x.float() + bias.float())
    assert (lin1.float() - ref).abs().max() < 4e-3
    assert torch.equal(drop2, torch.relu(lin1) * m2)
    dlin1, db = torch.empty_like(x), torch.empty(U, dtype=torch.float16, device=DEV)
    gy = torch.randn(Bt, Jt, U, device=DEV, generator=g).half()
    ops.backward_dropout_activation_bias(gy, m2, lin1, dlin1, db)
    refd = gy.float() * m2 * (lin1 > 0)
    assert torch.equal(dlin1, refd.half())
    refb = refd.sum((0, 1))
    assert (db.float() - refb).norm() / refb.norm() < 2e-3


@pytest.mark.parametrize('B,J,F,lay', [(4, 64, 1024, 'BJI'), (2, 9, 200, 'BJI'), (3, 8, 520, 'JBI'), (16, 128, 64, 'BJI'),
                                       (8, 512, 1024, 'BJI')])
def test_fused_layernorm_backward_operators(B, J, F, lay):
    """bsb+blnrd and ebsb+blnrd+baob in one pass each, against the oracle's separate operators."""
    ops = _ops()
    rng = np.random.default_rng(B * F + J)
    vec = lambda: torch.full((F,), float('nan'), dtype=torch.float16, device=DEV)
    dy, ln, diff = (h16(rng.normal(0, 1, (B, J, F))) for _ in range(3))
    istd = h16(rng.uniform(0.5, 2.0, (B, J)))
    gamma = h16(rng.normal(1, 0.1, F))
    mask = (rng.random((B, J, F)) >= 0.1).astype(np.uint8)
    tg = torch.tensor(gamma, dtype=torch.float16, device=DEV)
    d_mask = place(mask, 'BJI', lay, torch.uint8)
    d_dln, d_dres, d_dlin = (empty((B, J, F), 'BJI', lay) for _ in range(3))
    d_dg, d_db = vec(), vec()
    for _ in range(2):
        ops.backward_scale_bias_layernorm(place(dy, 'BJI', lay), place(ln, 'BJI', lay), tg, place(istd, 'BJ', 'BJ'),
                                          place(diff, 'BJI', lay), d_mask, d_dln, d_dres, d_dlin, d_dg, d_db)
    dln, dg, db = orc.backward_scale_bias(dy, ln, gamma)
    dres, dlin = orc.backward_layernorm_residual_dropout(dln, diff, istd, mask)
    for got, want, what in ((d_dln, dln, 'DLN'), (d_dres, dres, 'DRESID'), (d_dlin, dlin, 'DLIN'), (d_dg, dg, 'dgamma'),
                            (d_db, db, 'dbeta')):
        assert_close(got, want, what=what)

    r2, lw, l2 = (h16(rng.normal(0, 1, (B, J, F))) for _ in range(3))
    d_dln1, d_dres1, d_datt = (empty((B, J, F), 'BJI', lay) for _ in range(3))
    o = [vec() for _ in range(4)]
    ops.extended_backward_scale_bias_layernorm(place(ln, 'BJI', lay), tg, place(r2, 'BJI', lay), place(lw, 'BJI', lay),
                                               place(l2, 'BJI', lay), place(istd, 'BJ', 'BJ'), place(diff, 'BJI', lay),
                                               d_mask, d_dln1, d_dres1, d_datt, *o)
    dln1, dg1, db1, dl2 = orc.extended_backward_scale_bias(ln, gamma, r2, lw, l2)
    dres1, datt = orc.backward_layernorm_residual_dropout(dln1, diff, istd, mask)
    for got, want, what in ((d_dln1, dln1, 'DLN1'), (d_dres1, dres1, 'DRESID1'), (d_datt, datt, 'DATT'),
                            (o[0], dg1, 'dgamma1'), (o[1], db1, 'dbeta1'), (o[2], dl2, 'dlinb2'),
                            (o[3], orc.backward_attn_out_bias(datt), 'dbo')):
        assert_close(got, want, what=what)


def test_fused_layernorm_backward_declines_strided_views():
    ops = _ops()
    from substation_b200._lib import SubstationError
    B, J, F = 2, 8, 64
    x = torch.zeros(F, B, J, dtype=torch.float16, device=DEV).permute(1, 2, 0)     # feature-outermost
    m = torch.zeros(B, J, F, dtype=torch.uint8, device=DEV)
    v = torch.zeros(F, dtype=torch.float16, device=DEV)
    s2 = torch.zeros(B, J, dtype=torch.float16, device=DEV)
    with pytest.raises(SubstationError) as e:
        ops.backward_scale_bias_layernorm(x, x, v, s2, x, m, x, x, x, v, v)
    assert e.value.status == 3


@pytest.mark.parametrize('H,B,L,lay', [(2, 2, 512, 'PHBJ'), (2, 3, 128, 'PHBJ'), (1, 2, 64, 'PHBJ'), (2, 1, 384, 'HBPJ'),
                                       (3, 2, 256, 'HBJP')])
@pytest.mark.parametrize('mode', ['explicit', 'philox'])
def test_fused_attention_scores_forward_and_backward(H, B, L, lay, mode):
    """QKT+softmax+dropout and dX1gamma+softmax-backward, each in one kernel with the score tile in
    tensor memory, against the oracle's separate steps."""
    ops = _ops()
    P = 64
    rng = np.random.default_rng(L + H)
    qq, kk, vv, dg = (h16(rng.normal(0, 1, (P, H, B, L))) for _ in range(4))
    mask = (rng.random((H, B, L, L)) >= 0.2).astype(np.uint8)
    d_mask = place(mask, 'HBJK', 'HBJK', torch.uint8) if mode == 'explicit' else empty((H, B, L, L), 'HBJK', 'HBJK', torch.uint8)
    d_beta, d_alpha, d_drop = (empty((H, B, L, L), 'HBJK', 'HBJK') for _ in range(3))
    scale = 0.125
    ops.attention_scores_softmax(place(qq, 'PHBJ', lay), place(kk, 'PHBJ', lay), d_beta, d_alpha, d_mask, d_drop, scale,
                                 p=0.2, mode=mode, seed=77, offset=5)
    assert ops.device_error() == 0
    if mode == 'philox':
        mask = get(d_mask).astype(np.uint8)
        assert np.array_equal(mask, orc.philox_mask((H, B, L, L), 0.2, 77, 5))
    beta = scale * np.einsum('phbk,phbj->hbjk', kk, qq)
    alpha, drop = orc.softmax_dropout(beta, mask)
    assert_close(d_beta, beta, what='BETA')
    assert_close(d_alpha, alpha, what='ALPHA')
    assert_close(d_drop, drop, what='ATTN_DROP')
    assert np.array_equal(get(d_drop), get(d_alpha) * mask)

    alpha16 = h16(alpha)
    d_dad, d_dbeta = empty((H, B, L, L), 'HBJK', 'HBJK'), empty((H, B, L, L), 'HBJK', 'HBJK')
    ops.attention_scores_softmax_backward(place(dg, 'PHBJ', lay), place(vv, 'PHBJ', lay), place(alpha16, 'HBJK', 'HBJK'),
                                          place(mask, 'HBJK', 'HBJK', torch.uint8), d_dad, d_dbeta)
    assert ops.device_error() == 0
    dad = np.einsum('phbk,phbj->hbjk', vv, dg)
    assert_close(d_dad, dad, what='DATTN_DROP')
    assert_close(d_dbeta, orc.softmax_dropout_backward(alpha16, mask, h16(dad)), what='DBETA')


def test_fused_attention_scores_decline_what_they_do_not_cover():
    ops = _ops()
    from substation_b200._lib import SubstationError
    H, B, L, P = 1, 1, 96, 64                       # L not a multiple of 64
    q = torch.zeros(P, H, B, L, dtype=torch.float16, device=DEV)
    s = torch.zeros(H, B, L, L, dtype=torch.float16, device=DEV)
    m = torch.zeros(H, B, L, L, dtype=torch.uint8, device=DEV)
    with pytest.raises(SubstationError) as e:
        ops.attention_scores_softmax(q, q, s, s.clone(), m, s.clone(), 1.0)
    assert e.value.status == 3


@pytest.mark.parametrize('H,B,L,lay_in,lay_out', [(2, 2, 512, 'PHBJ', 'PHBJ'), (1, 3, 128, 'PHBJ', 'PHBJ'),
                                                  (2, 1, 256, 'HBPJ', 'PHBJ'), (3, 2, 384, 'HBJP', 'HBJP'),
                                                  (2, 2, 256, 'PHBJ', 'HBJP')])
@pytest.mark.parametrize('which', ['rows', 'cols', 'both'])
def test_attention_score_contractions(H, B, L, lay_in, lay_out, which):
    """gamma / dX2gamma / the dX1QKT+dX2QKT pair as one pass over the score tensor, against float64 einsums."""
    ops = _ops()
    P = 64
    rng = np.random.default_rng(L + H + len(which))
    sc = h16(rng.normal(0, 0.3, (H, B, L, L)))
    x, y = h16(rng.normal(0, 1, (P, H, B, L))), h16(rng.normal(0, 1, (P, H, B, L)))
    d_r, d_c = empty((P, H, B, L), 'PHBJ', lay_out), empty((P, H, B, L), 'PHBJ', lay_out)
    kw = {}
    if which in ('rows', 'both'):
        kw.update(x=place(x, 'PHBJ', lay_in), out_rows=d_r)
    if which in ('cols', 'both'):
        kw.update(y=place(y, 'PHBJ', lay_in), out_cols=d_c)
    ops.attention_score_contractions(place(sc, 'HBJK', 'HBJK'), alpha=0.125, **kw)
    assert ops.device_error() == 0
    if 'x' in kw:
        assert_close(d_r, 0.125 * np.einsum('hbjk,phbk->phbj', sc, x), what='rows')
    if 'y' in kw:
        assert_close(d_c, 0.125 * np.einsum('hbjk,phbj->phbk', sc, y), what='cols')


def test_attention_score_contractions_decline_what_they_do_not_cover():
    ops = _ops()
    from substation_b200._lib import SubstationError
    H, B, L, P = 1, 1, 192, 64                      # L not a multiple of 128
    sc = torch.zeros(H, B, L, L, dtype=torch.float16, device=DEV)
    x = torch.zeros(P, H, B, L, dtype=torch.float16, device=DEV)
    with pytest.raises(SubstationError) as e:
        ops.attention_score_contractions(sc, x=x, out_rows=x.clone())
    assert e.value.status == 3


def test_optional_outputs_can_be_left_out_without_changing_the_others():
    """BETA, DATTN_DROP, LIN and DLN are only intermediates of their fused operators: with None in their place the
    operator stores nothing for them and every other output keeps its bits."""
    ops = _ops()
    g = torch.Generator(device=DEV).manual_seed(31)
    rnd = lambda *shape: torch.randn(*shape, device=DEV, generator=g).half()
    nan = lambda *shape: torch.full(shape, float('nan'), dtype=torch.float16, device=DEV)
    # fused attention scores, forward and backward
    H, B, L, P = 2, 3, 256, 64
    qq, kk, vv, dg = (rnd(P, H, B, L) for _ in range(4))
    mask = (torch.rand(H, B, L, L, device=DEV, generator=g) >= 0.2).to(torch.uint8)
    outs = {}
    for keep in (True, False):
        beta, alpha, drop = (nan(H, B, L, L) for _ in range(3))
        ops.attention_scores_softmax(qq, kk, beta if keep else None, alpha, mask, drop, 0.125)
        dad, dbeta = nan(H, B, L, L), nan(H, B, L, L)
        ops.attention_scores_softmax_backward(dg, vv, alpha, mask, dad if keep else None, dbeta)
        outs[keep] = (alpha, drop, dbeta)
    assert ops.device_error() == 0
    for a, b in zip(outs[True], outs[False]):
        assert torch.isfinite(b).all() and torch.equal(a, b)
    # bias + dropout + residual + LayerNorm
    B, J, F = 4, 96, 1024
    x, resid, bias, gamma, beta_ = rnd(B, J, F), rnd(B, J, F), rnd(F), rnd(F), rnd(F)
    m3 = (torch.rand(B, J, F, device=DEV, generator=g) >= 0.1).to(torch.uint8)
    outs = {}
    for keep in (True, False):
        lin, diff, ln, out = (nan(B, J, F) for _ in range(4))
        istd = nan(B, J)
        ops.bias_dropout_residual_layernorm(x, bias, resid, gamma, beta_, m3, lin if keep else None, diff, istd, ln, out)
        outs[keep] = (diff, istd, ln, out)
    for a, b in zip(outs[True], outs[False]):
        assert torch.isfinite(b).all() and torch.equal(a, b)
    # fused LayerNorm backward, both forms
    dy, lnv, dfv, r2, lw, l2 = (rnd(B, J, F) for _ in range(6))
    istd = (torch.rand(B, J, device=DEV, generator=g) + 0.5).half()
    outs = {}
    for keep in (True, False):
        dln, dres, dlin = (nan(B, J, F) for _ in range(3))
        v = [nan(F) for _ in range(6)]
        ops.backward_scale_bias_layernorm(dy, lnv, gamma, istd, dfv, m3, dln if keep else None, dres, dlin, v[0], v[1])
        dln1, dres1, datt = (nan(B, J, F) for _ in range(3))
        ops.extended_backward_scale_bias_layernorm(lnv, gamma, r2, lw, l2, istd, dfv, m3, dln1 if keep else None, dres1,
                                                   datt, *v[2:])
        outs[keep] = (dres, dlin, dres1, datt, *v)
    for a, b in zip(outs[True], outs[False]):
        assert torch.isfinite(b).all() and torch.equal(a, b)
