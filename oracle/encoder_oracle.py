"""numpy restatement of the BERT encoder-layer forward+backward (CPU oracle).

TEST INFRASTRUCTURE ONLY: imported by tests, the smoke check and the CPU-baseline
timing leg; never by the shipped package.

Every function restates one operator of the reference, in float64, on tensors
held in *logical* index order (the order given in each docstring), with dropout
masks passed in explicitly as {0,1} arrays.  Citations are paths inside the
spcl/substation tree.

Conventions taken from the reference's CUDA path (the numpy path differs in
places; both are supported where it matters for pinning):
  * dropout keeps with value 1, no rescale: ``blocks.cuh:24-45``
  * stacked projections are ordered K, Q, V: ``encoder.cu:93-103``
  * LayerNorm uses rsqrt(var + 1e-5) and stores the reciprocal in ``LN*STD``
    (``block_bdrln.cuh:81-91``); the numpy path divides by (std + 1e-5)
    (``substation/transformer.py:100-103``).  ``ln_mode`` selects which.

Letters: B batch, J query position, K key position, H heads, P head size,
I embedding (= H*P), U feed-forward width, Q in {K,Q,V}.
"""

import numpy as np

LN_EPS = 1e-5

# ----------------------------------------------------------------------------
# Layout helpers
# ----------------------------------------------------------------------------

#: logical dim order of every tensor the layer touches (names as in the layout
#: pickles written by ``config_selection/optimize.py:443-493``)
LOGICAL = {
    'X': 'BJI', 'SB2': 'BJI',
    'WKQV': 'QPHI', 'BKQV': 'QPH', 'WO': 'IPH', 'BO': 'I',
    'S1': 'I', 'B1': 'I', 'S2': 'I', 'B2': 'I',
    'LINW1': 'IU', 'LINB1': 'U', 'LINW2': 'UI', 'LINB2': 'I',
    'KKQQVV': 'QPHBJ', 'WKKWQQWVV': 'QPHBJ',
    'BETA': 'HBJK', 'ALPHA': 'HBJK', 'ATTN_DROP_MASK': 'HBJK', 'ATTN_DROP': 'HBJK',
    'GAMMA': 'PHBJ', 'ATT': 'BJI', 'DROP1MASK': 'BJI', 'SB1': 'BJI',
    'SB1_LINW1': 'BJU', 'DROP2': 'BJU', 'LIN1': 'BJU', 'DROP2_LINW2': 'BJI',
    'LIN2': 'BJI', 'LN2': 'BJI', 'LN2STD': 'BJ', 'LN2DIFF': 'BJI',
    'DROP2MASK': 'BJU', 'DROP3MASK': 'BJI', 'LN1': 'BJI', 'LN1STD': 'BJ',
    'LN1DIFF': 'BJI',
    'DLN2': 'BJI', 'DRESID2': 'BJI', 'DLIN2': 'BJI', 'DDROP2': 'BJU',
    'DLIN1': 'BJU', 'DLIN1_LINW1': 'BJI', 'DLN1': 'BJI', 'DRESID1': 'BJI',
    'DATT': 'BJI', 'DXATT': 'BJI', 'DGAMMA': 'PHBJ', 'DATTN_DROP': 'HBJK',
    'DBETA': 'HBJK', 'DKKQQVV': 'QPHBJ',
    'DX': 'BJI', 'DSB2': 'BJI',
}
for _p in ('WKQV', 'BKQV', 'WO', 'BO', 'S1', 'B1', 'S2', 'B2',
           'LINW1', 'LINB1', 'LINW2', 'LINB2'):
    LOGICAL['D' + _p] = LOGICAL[_p]

PARAM_NAMES = ('WKQV', 'BKQV', 'WO', 'BO', 'S1', 'B1', 'LINB1', 'LINW1',
               'S2', 'B2', 'LINB2', 'LINW2')


def to_layout(a, logical, layout):
    """Permute ``a`` (dims in order ``logical``) into memory order ``layout``."""
    assert sorted(logical) == sorted(layout), (logical, layout)
    return np.ascontiguousarray(np.transpose(a, [logical.index(c) for c in layout]))


def from_layout(a, layout, logical):
    """Inverse of :func:`to_layout`: view ``a`` (stored as ``layout``) in logical order."""
    assert sorted(logical) == sorted(layout), (logical, layout)
    return np.transpose(a, [layout.index(c) for c in logical])


# ----------------------------------------------------------------------------
# Counter-based dropout masks (Philox4x32-10, public algorithm of Salmon et al.,
# "Parallel random numbers: as easy as 1, 2, 3", SC'11).  The reference draws
# its masks from cuRAND's Philox4_32_10 per thread (blocks.cuh:24-51); thread
# geometry is not part of any contract, so the new kernels key the generator by
# the element's logical linear index instead, which this function restates.
# ----------------------------------------------------------------------------

_PHILOX_M0 = np.uint64(0xD2511F53)
_PHILOX_M1 = np.uint64(0xCD9E8D57)
_PHILOX_W0 = 0x9E3779B9
_PHILOX_W1 = 0xBB67AE85
_M32 = np.uint64(0xFFFFFFFF)


def philox4x32_10(c0, c1, c2, c3, k0, k1):
    """Ten rounds of Philox-4x32 on uint64 arrays holding 32-bit words."""
    c0, c1, c2, c3 = (np.asarray(c, dtype=np.uint64) & _M32 for c in (c0, c1, c2, c3))
    k0 = int(k0) & 0xFFFFFFFF
    k1 = int(k1) & 0xFFFFFFFF
    for _ in range(10):
        p0 = _PHILOX_M0 * c0
        p1 = _PHILOX_M1 * c2
        hi0, lo0 = p0 >> np.uint64(32), p0 & _M32
        hi1, lo1 = p1 >> np.uint64(32), p1 & _M32
        c0, c1, c2, c3 = (hi1 ^ c1 ^ np.uint64(k0), lo1,
                          hi0 ^ c3 ^ np.uint64(k1), lo0)
        k0 = (k0 + _PHILOX_W0) & 0xFFFFFFFF
        k1 = (k1 + _PHILOX_W1) & 0xFFFFFFFF
    return c0, c1, c2, c3


def dropout_threshold(p):
    """16-bit drop threshold: an element is dropped when its 16 random bits are < thr."""
    return int(min(65535, max(0, round(float(p) * 65536.0))))


def philox_mask(shape, p, seed, offset):
    """{0,1} uint8 keep-mask for a tensor of logical ``shape``.

    Element with logical linear index e uses Philox counter (e>>3 lo, e>>3 hi,
    offset lo, offset hi), key (seed lo, seed hi); its 16 random bits are half
    (e&1) of output word ((e&7)>>1).  keep = bits >= round(p*65536): the same
    rule as ``mask = u < p ? 0 : 1`` (blocks.cuh:33-34) at 16-bit resolution.
    """
    n = int(np.prod(shape))
    e = np.arange(n, dtype=np.uint64)
    g = e >> np.uint64(3)
    ng = (n + 7) // 8
    gg = np.arange(ng, dtype=np.uint64)
    r = philox4x32_10(gg & _M32, gg >> np.uint64(32),
                      np.uint64(offset & 0xFFFFFFFF), np.uint64((offset >> 32) & 0xFFFFFFFF),
                      seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)
    words = np.stack(r, axis=1)                       # [ng, 4]
    t = (e & np.uint64(7)).astype(np.int64)
    w = words[g.astype(np.int64), t >> 1]
    bits = (w >> ((t & 1) * 16).astype(np.uint64)) & np.uint64(0xFFFF)
    thr = dropout_threshold(p)
    return (bits >= np.uint64(thr)).astype(np.uint8).reshape(shape)


# ----------------------------------------------------------------------------
# Fused operators (one function per reference launcher)
# ----------------------------------------------------------------------------

def relu(x):
    """substation/transformer.py:31-33"""
    return np.maximum(0, x)


def relu_backward(x, dy):
    """substation/transformer.py:36-38; the CUDA path tests LIN1 > 0 (block_bdrlb.cuh:72)."""
    return (x > 0) * dy


def gelu(x):
    """tanh form, substation/transformer.py:11-14"""
    return 0.5 * x * (1 + np.tanh(np.sqrt(2.0 / np.pi) * (x + 0.044715 * (x ** 3))))


def gelu_backward(x, dy):
    """substation/transformer.py:17-28 (same constants)."""
    x3 = x ** 3
    inner = 0.0356774 * x3 + 0.797885 * x
    sech2 = 1.0 / np.cosh(inner) ** 2
    return (0.5 * np.tanh(inner) + (0.0535161 * x3 + 0.398942 * x) * sech2 + 0.5) * dy


_ACT = {'relu': (relu, relu_backward), 'gelu': (gelu, gelu_backward)}


def attention_input_biases(wkkwqqwvv, bkqv):
    """KKQQVV[q,p,h,b,j] = WKKWQQWVV[q,p,h,b,j] + BKQV[q,p,h]  (block_aib.cuh:17-62)."""
    return wkkwqqwvv + bkqv[:, :, :, None, None]


def softmax_dropout(beta, mask, scale=1.0):
    """ALPHA = softmax_k(scale*BETA); ATTN_DROP = mask*ALPHA.

    block_softmax.cuh:12-124 (row max, exp, sum, normalise, mask) and
    substation/attention.py:14-17.  Inside the layer the 1/sqrt(P) factor is
    already in BETA (encoder.cu:116) and scale is 1.
    """
    x = scale * beta
    e = np.exp(x - x.max(axis=-1, keepdims=True))
    alpha = e / e.sum(axis=-1, keepdims=True)
    return alpha, alpha * mask


def softmax_dropout_backward(alpha, mask, dattn_drop):
    """DBETA = ALPHA*(da - sum_k da*ALPHA), da = mask*DATTN_DROP.

    block_bs.cuh:13-98; substation/attention.py:20-29.
    """
    da = mask * dattn_drop
    s = (da * alpha).sum(axis=-1, keepdims=True)
    return alpha * (da - s)


def bias_dropout_residual_layernorm(inp, bias, resid, mask, gamma, beta, ln_mode='cuda'):
    """LIN, DIFF, ISTD, LN, OUT of block_bdrln.cuh:17-103 / :195-272.

    LIN = IN + bias; r = mask*LIN + RESID; DIFF = r - mean_I(r);
    ISTD = rsqrt(var_I(r) + eps) [cuda] or 1/(std + eps) [numpy,
    substation/transformer.py:100-103]; LN = DIFF*ISTD; OUT = LN*gamma + beta.
    """
    lin = inp + bias
    r = mask * lin + resid
    mean = r.mean(axis=-1, keepdims=True)
    diff = r - mean
    var = (diff * diff).mean(axis=-1, keepdims=True)
    if ln_mode == 'cuda':
        istd = 1.0 / np.sqrt(var + LN_EPS)
    else:
        istd = 1.0 / (np.sqrt(var) + LN_EPS)
    ln = diff * istd
    out = ln * gamma + beta
    return lin, diff, istd[..., 0], ln, out


def bias_activation_dropout(inp, bias, mask, activation='relu'):
    """LIN1 = IN + bias; DROP2 = mask*act(LIN1)  (block_bad.cuh:28-81; ReLU at :74)."""
    lin1 = inp + bias
    return lin1, mask * _ACT[activation][0](lin1)


def backward_scale_bias(dy, ln, gamma):
    """DLN = DY*gamma; dgamma = sum_{b,j} DY*LN; dbeta = sum_{b,j} DY (block_bsb_ebsb.cuh:12-169)."""
    return dy * gamma, (dy * ln).sum(axis=(0, 1)), dy.sum(axis=(0, 1))


def backward_layernorm_residual_dropout(dln, diff, istd, mask, ln_mode='cuda'):
    """LayerNorm backward-data from stored DIFF and reciprocal std, then dropout.

    block_blnrd.cuh:14-69: with g=DLN, d=DIFF, s=ISTD, n=I
      D_LN_IN = g*s - (sum g)*s/n - d*(sum g*d)*s^3/n ;  D_DROP_IN = mask*D_LN_IN.
    The numpy path (substation/transformer.py:106-118) is the same formula with
    s = 1/std (no eps), selected by ln_mode='numpy' when istd was made that way.
    """
    n = dln.shape[-1]
    s = istd[..., None]
    sg = dln.sum(axis=-1, keepdims=True)
    sgd = (dln * diff).sum(axis=-1, keepdims=True)
    dres = dln * s - sg * s / n - diff * sgd * s ** 3 / n
    return dres, mask * dres


def backward_dropout_activation_bias(ddrop2, mask, lin1, activation='relu'):
    """DLIN1 = act'(LIN1)*(mask*DDROP2); dLINB1 = sum_{b,j} DLIN1 (block_bdrlb.cuh:13-96)."""
    dlin1 = _ACT[activation][1](lin1, ddrop2 * mask)
    return dlin1, dlin1.sum(axis=(0, 1))


def extended_backward_scale_bias(ln1, gamma1, dresid2, dlin1_linw1, dlin2):
    """block_bsb_ebsb.cuh:228-366.

    dLINB2 = sum DLIN2; g = DRESID2 + DLIN1_LINW1; DLN1 = g*gamma1;
    dgamma1 = sum g*LN1; dbeta1 = sum g.
    """
    g = dresid2 + dlin1_linw1
    return (g * gamma1, (g * ln1).sum(axis=(0, 1)), g.sum(axis=(0, 1)),
            dlin2.sum(axis=(0, 1)))


def backward_attn_out_bias(datt):
    """dBO[i] = sum_{b,j} DATT[b,j,i] (block_baob.cuh:10-73)."""
    return datt.sum(axis=(0, 1))


def backward_attention_input_biases(dkkqqvv):
    """dBKQV[q,p,h] = sum_{b,j} DKKQQVV[q,p,h,b,j] (block_baib.cuh:15-154)."""
    return dkkqqvv.sum(axis=(3, 4))


def backward_encoder_input(dxatt, dresid1):
    """DX = DXATT + DRESID1 (block_bei.cuh:12-50)."""
    return dxatt + dresid1


# ----------------------------------------------------------------------------
# Whole layer: operator sequence of encoder.cu:87-157 (forward) and :158-299
# (backward); contractions are the 18 einsums listed there, written with
# np.einsum on logical index order.
# ----------------------------------------------------------------------------

def encoder_forward(X, params, masks, activation='relu', ln_mode='cuda'):
    """Forward pass.  ``params``: dict of the 12 parameters in logical order.

    ``masks``: dict with ATTN_DROP_MASK [H,B,J,K], DROP1MASK [B,J,I],
    DROP2MASK [B,J,U], DROP3MASK [B,J,I] ({0,1}); a missing/None entry means
    "keep everything".  Returns a dict with every forward intermediate of
    ``layouts['forward_interm']`` plus 'SB2', all in logical order, float64.
    """
    f = {}
    X = np.asarray(X, dtype=np.float64)
    p = {k: np.asarray(v, dtype=np.float64) for k, v in params.items()}
    Q, P, H, I = p['WKQV'].shape
    B, J, _ = X.shape
    U = p['LINW1'].shape[1]
    scale = 1.0 / np.sqrt(P)

    def m(name, shape):
        v = masks.get(name) if masks else None
        return np.ones(shape) if v is None else np.asarray(v, dtype=np.float64)

    # F1 QKV-fused (encoder.cu:90) and aib (:105-113)
    f['WKKWQQWVV'] = np.einsum('qphi,bji->qphbj', p['WKQV'], X, optimize=True)
    f['KKQQVV'] = attention_input_biases(f['WKKWQQWVV'], p['BKQV'])
    KK, QQ, VV = f['KKQQVV'][0], f['KKQQVV'][1], f['KKQQVV'][2]
    # F2 QKT with alpha = 1/sqrt(P) (encoder.cu:116)
    f['BETA'] = scale * np.einsum('phbk,phbj->hbjk', KK, QQ, optimize=True)
    f['ATTN_DROP_MASK'] = m('ATTN_DROP_MASK', f['BETA'].shape)
    f['ALPHA'], f['ATTN_DROP'] = softmax_dropout(f['BETA'], f['ATTN_DROP_MASK'])
    # F3 gamma (encoder.cu:124), F4 out (:128)
    f['GAMMA'] = np.einsum('phbk,hbjk->phbj', VV, f['ATTN_DROP'], optimize=True)
    att = np.einsum('iph,phbj->bji', p['WO'], f['GAMMA'], optimize=True)
    # bdrln1 writes ATT + BO back into ATT (encoder.cu:134-135)
    f['DROP1MASK'] = m('DROP1MASK', (B, J, I))
    f['ATT'], f['LN1DIFF'], f['LN1STD'], f['LN1'], f['SB1'] = \
        bias_dropout_residual_layernorm(att, p['BO'], X, f['DROP1MASK'],
                                        p['S1'], p['B1'], ln_mode)
    # F5 lin1 (:139), bad (:143), F6 lin2 (:148), bdrln2 (:152)
    f['SB1_LINW1'] = np.einsum('bji,iu->bju', f['SB1'], p['LINW1'], optimize=True)
    f['DROP2MASK'] = m('DROP2MASK', (B, J, U))
    f['LIN1'], f['DROP2'] = bias_activation_dropout(
        f['SB1_LINW1'], p['LINB1'], f['DROP2MASK'], activation)
    f['DROP2_LINW2'] = np.einsum('bju,ui->bji', f['DROP2'], p['LINW2'], optimize=True)
    f['DROP3MASK'] = m('DROP3MASK', (B, J, I))
    f['LIN2'], f['LN2DIFF'], f['LN2STD'], f['LN2'], f['SB2'] = \
        bias_dropout_residual_layernorm(f['DROP2_LINW2'], p['LINB2'], f['SB1'],
                                        f['DROP3MASK'], p['S2'], p['B2'], ln_mode)
    return f


def encoder_backward(X, DY, params, f, activation='relu', ln_mode='cuda', relu_pattern=None):
    """Backward pass (encoder.cu:158-299).  ``f`` is the dict from encoder_forward.

    Returns a dict with the 14 backward intermediates, 'DX' and 'D'+param for
    the 12 parameters, logical order, float64.

    ``relu_pattern`` (bool [B,J,U], ReLU only): evaluate relu' on this pattern
    instead of ``LIN1 > 0``.  relu' is discontinuous at 0, so an fp16 LIN1 within
    rounding of zero can have the other sign than the float64 one and the whole
    gradient element (and everything summed from it) differs; tests pass the
    pattern of the implementation under test after checking that it departs from
    the oracle's only on such elements.
    """
    g = {}
    X = np.asarray(X, dtype=np.float64)
    DY = np.asarray(DY, dtype=np.float64)
    p = {k: np.asarray(v, dtype=np.float64) for k, v in params.items()}
    P = p['WKQV'].shape[1]
    scale = 1.0 / np.sqrt(P)
    KK, QQ, VV = f['KKQQVV'][0], f['KKQQVV'][1], f['KKQQVV'][2]

    g['DLN2'], g['DS2'], g['DB2'] = backward_scale_bias(DY, f['LN2'], p['S2'])
    g['DRESID2'], g['DLIN2'] = backward_layernorm_residual_dropout(
        g['DLN2'], f['LN2DIFF'], f['LN2STD'], f['DROP3MASK'], ln_mode)
    g['DDROP2'] = np.einsum('bji,ui->bju', g['DLIN2'], p['LINW2'], optimize=True)     # B1
    g['DLINW2'] = np.einsum('bju,bji->ui', f['DROP2'], g['DLIN2'], optimize=True)     # B2
    if relu_pattern is not None and activation == 'relu':
        g['DLIN1'] = relu_pattern * (g['DDROP2'] * f['DROP2MASK'])
        g['DLINB1'] = g['DLIN1'].sum(axis=(0, 1))
    else:
        g['DLIN1'], g['DLINB1'] = backward_dropout_activation_bias(
            g['DDROP2'], f['DROP2MASK'], f['LIN1'], activation)
    g['DLIN1_LINW1'] = np.einsum('bju,iu->bji', g['DLIN1'], p['LINW1'], optimize=True)  # B3
    g['DLINW1'] = np.einsum('bji,bju->iu', f['SB1'], g['DLIN1'], optimize=True)       # B4
    g['DLN1'], g['DS1'], g['DB1'], g['DLINB2'] = extended_backward_scale_bias(
        f['LN1'], p['S1'], g['DRESID2'], g['DLIN1_LINW1'], g['DLIN2'])
    g['DRESID1'], g['DATT'] = backward_layernorm_residual_dropout(
        g['DLN1'], f['LN1DIFF'], f['LN1STD'], f['DROP1MASK'], ln_mode)
    g['DBO'] = backward_attn_out_bias(g['DATT'])
    g['DWO'] = np.einsum('phbj,bji->iph', f['GAMMA'], g['DATT'], optimize=True)        # B5
    g['DGAMMA'] = np.einsum('iph,bji->phbj', p['WO'], g['DATT'], optimize=True)        # B6
    g['DATTN_DROP'] = np.einsum('phbk,phbj->hbjk', VV, g['DGAMMA'], optimize=True)     # B7
    dvv = np.einsum('phbj,hbjk->phbk', g['DGAMMA'], f['ATTN_DROP'], optimize=True)     # B8
    g['DBETA'] = softmax_dropout_backward(f['ALPHA'], f['ATTN_DROP_MASK'], g['DATTN_DROP'])
    dqq = scale * np.einsum('phbk,hbjk->phbj', KK, g['DBETA'], optimize=True)          # B9
    dkk = scale * np.einsum('phbj,hbjk->phbk', QQ, g['DBETA'], optimize=True)          # B10
    g['DKKQQVV'] = np.stack((dkk, dqq, dvv))
    g['DXATT'] = np.einsum('qphi,qphbj->bji', p['WKQV'], g['DKKQQVV'], optimize=True)  # B11
    g['DWKQV'] = np.einsum('bji,qphbj->qphi', X, g['DKKQQVV'], optimize=True)          # B12
    g['DBKQV'] = backward_attention_input_biases(g['DKKQQVV'])
    g['DX'] = backward_encoder_input(g['DXATT'], g['DRESID1'])
    return g


# ----------------------------------------------------------------------------
# Synthetic inputs shared by tests, fixtures and the benchmark
# ----------------------------------------------------------------------------

def make_params(H, P, U, rng, w_std=0.02, random_affine=False):
    """The 12 parameters in logical order.  Default: weights ~ N(0, w_std),
    biases 0, LayerNorm gamma 1 / beta 0.  ``random_affine`` draws the biases
    and LayerNorm parameters too so that every gradient path is exercised."""
    I = H * P
    p = {
        'WKQV': rng.normal(0, w_std, (3, P, H, I)),
        'WO': rng.normal(0, w_std, (I, P, H)),
        'LINW1': rng.normal(0, w_std, (I, U)),
        'LINW2': rng.normal(0, w_std, (U, I)),
    }
    if random_affine:
        p.update(BKQV=rng.normal(0, 0.1, (3, P, H)), BO=rng.normal(0, 0.1, I),
                 S1=rng.normal(1, 0.1, I), B1=rng.normal(0, 0.1, I),
                 S2=rng.normal(1, 0.1, I), B2=rng.normal(0, 0.1, I),
                 LINB1=rng.normal(0, 0.1, U), LINB2=rng.normal(0, 0.1, I))
    else:
        p.update(BKQV=np.zeros((3, P, H)), BO=np.zeros(I), S1=np.ones(I), B1=np.zeros(I),
                 S2=np.ones(I), B2=np.zeros(I), LINB1=np.zeros(U), LINB2=np.zeros(I))
    return p


def make_masks(B, J, H, I, U, ps, seed):
    """Four explicit Bernoulli keep-masks (uint8) from seeds seed+1..seed+4."""
    shapes = {'ATTN_DROP_MASK': (H, B, J, J), 'DROP1MASK': (B, J, I),
              'DROP2MASK': (B, J, U), 'DROP3MASK': (B, J, I)}
    out = {}
    for n, (name, shape) in enumerate(shapes.items()):
        r = np.random.default_rng(seed + 1 + n)
        out[name] = (r.random(shape) >= ps[n]).astype(np.uint8)
    return out


def rel_l2(a, b):
    """||a-b|| / ||b|| (0 when both are zero)."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    den = np.linalg.norm(b)
    num = np.linalg.norm(a - b)
    return 0.0 if num == 0 else num / max(den, 1e-30)
