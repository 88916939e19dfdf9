"""Generate golden vectors by running the reference's own numpy encoder path.

Run in a container where the spcl/substation tree is mounted:

    SUBSTATION_REF=/path/to/substation python tests/golden/make_golden.py

It imports ``substation.transformer`` from that tree (with a stub ``dace``
module, which the numpy functions never touch: substation/attention.py:9),
replaces only ``substation.transformer.dropout`` by a function that applies
caller-supplied {0,1} masks (the stock one draws unseeded masks,
substation/transformer.py:134-138), runs ``encoder`` and ``encoder_backward``
(substation/transformer.py:176-285) on seeded inputs and writes inputs and
outputs to ``tests/golden/encoder_<case>.npz``.  The committed .npz files are
what the tests read; this script is kept so they can be regenerated.
"""

import os
import sys
import types
from unittest import mock

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, '..', '..'))

from oracle.encoder_oracle import make_params, make_masks  # noqa: E402

CASES = {
    # name: (B, J, H, P, U, dropout p (0 = off), activation, random_affine, seed)
    'relu_p0': (2, 6, 2, 4, 32, 0.0, 'relu', False, 11),
    'relu_masks': (2, 6, 2, 4, 32, 0.1, 'relu', True, 12),
    'gelu_masks': (3, 5, 2, 4, 32, 0.25, 'gelu', True, 13),
    'relu_masks_mid': (2, 16, 4, 8, 128, 0.1, 'relu', True, 14),
    # inputs that fp16 holds exactly (weights ~ N(0, 0.1)) at 64 features: what the kernels are given is what the
    # reference computed on, so the fp16 path can be held to the layer tolerance of 1e-2 against these
    'relu_masks_fp16_e64': (2, 16, 1, 64, 256, 0.1, 'relu', True, 15, 'fp16'),
    'gelu_masks_fp16_e64': (2, 8, 1, 64, 256, 0.1, 'gelu', True, 16, 'fp16'),
}


def import_reference():
    ref = os.environ.get('SUBSTATION_REF') or sys.exit('set SUBSTATION_REF to a checkout of spcl/substation')
    sys.modules.setdefault('dace', mock.MagicMock())
    sys.path.insert(0, ref)
    import substation.transformer as tr  # noqa
    return tr


def run_case(tr, B, J, H, P, U, p, activation, random_affine, seed, inputs='float64'):
    rng = np.random.default_rng(seed)
    I = H * P
    fp16 = inputs == 'fp16'
    params = make_params(H, P, U, rng, w_std=0.1 if fp16 else 0.3, random_affine=random_affine)
    X = rng.normal(0, 1, (B, J, I))
    DY = rng.normal(0, 1, (B, J, I))
    if fp16:
        params = {k: v.astype(np.float16).astype(np.float64) for k, v in params.items()}
        X, DY = X.astype(np.float16).astype(np.float64), DY.astype(np.float16).astype(np.float64)
    masks = make_masks(B, J, H, I, U, (0.0, p, p, p), seed) if p > 0 else {}
    masks.pop('ATTN_DROP_MASK', None)     # the numpy path has no dropout on the probabilities

    queue = [masks.get('DROP1MASK'), masks.get('DROP2MASK'), masks.get('DROP3MASK')]

    def dropout(x, prob):
        if prob == 0:
            return x, None
        mk = queue.pop(0).astype(np.float64)
        return x * mk, mk

    tr.dropout = dropout

    # reference argument layout (pytorch_module/run_encoder.py:155-184)
    wk, wq, wv = (np.einsum('phi->hpi', params['WKQV'][q]) for q in range(3))
    bqkv = np.stack([np.einsum('ph->hp', params['BKQV'][q]) for q in (1, 0, 2)])
    wo = np.einsum('iph->ihp', params['WO']).reshape(I, I)
    w1, w2 = params['LINW1'].T.copy(), params['LINW2'].T.copy()
    scale = 1 / np.sqrt(P)
    common = (params['S1'], params['B1'], params['S2'], params['B2'],
              w1, params['LINB1'], w2, params['LINB2'], p, p, p)

    fwd = tr.encoder(X, wq, wk, wv, wo, bqkv, params['BO'], scale, *common,
                     activation=activation)
    (y, concat, pq, pk, pv, scores, m1, n1mean, n1std, n1normed, m2, m3,
     n2mean, n2std, n2normed, ff_resid, ff1, ff1_linear, normed1, attn_resid) = fwd
    bwd = tr.encoder_backward(X, DY, *fwd[1:], wq, wk, wv, wo, scale, *common,
                              activation=activation)
    (dx, dwq, dwk, dwv, dwo, din_b, dout_b, dn1s, dn1b, dn2s, dn2b,
     dw1, db1, dw2, db2) = bwd

    store = (lambda a: a.astype(np.float16)) if fp16 else (lambda a: a)     # exact either way
    out = {'in_X': store(X), 'in_DY': store(DY)}
    out.update({'in_' + k: store(v) for k, v in params.items()})
    out['inputs'] = np.array(inputs)
    out.update({'in_' + k: v for k, v in masks.items()})
    out['meta'] = np.array([B, J, H, P, U], dtype=np.int64)
    out['p'] = np.array(p)
    out['activation'] = np.array(activation)
    # reference outputs, still in the reference's own index orders
    out.update(
        ref_y=y, ref_concat=np.stack(concat), ref_proj_q=np.stack(pq),
        ref_proj_k=np.stack(pk), ref_proj_v=np.stack(pv),
        ref_scores=np.stack(scores), ref_norm1_std=n1std, ref_norm1_normed=n1normed,
        ref_norm2_std=n2std, ref_norm2_normed=n2normed, ref_ff_resid=ff_resid,
        ref_ff1=ff1, ref_ff1_linear=ff1_linear, ref_normed1=normed1,
        ref_attn_resid=attn_resid,
        ref_dx=dx, ref_dwq=dwq, ref_dwk=dwk, ref_dwv=dwv, ref_dwo=dwo,
        ref_din_b=din_b, ref_dout_b=dout_b, ref_dnorm1_scale=dn1s,
        ref_dnorm1_bias=dn1b, ref_dnorm2_scale=dn2s, ref_dnorm2_bias=dn2b,
        ref_dlinear1_w=dw1, ref_dlinear1_b=db1, ref_dlinear2_w=dw2, ref_dlinear2_b=db2)
    return out


def main():
    tr = import_reference()
    for name, cfg in CASES.items():
        out = run_case(tr, *cfg)
        path = os.path.join(HERE, f'encoder_{name}.npz')
        np.savez_compressed(path, **out)
        print(name, os.path.getsize(path), 'bytes')


if __name__ == '__main__':
    main()
