"""Time every operator of the layer under candidate layouts, on the GPU, through
the C ABI, and write the tables the layout optimizer reads.

    python -m substation_b200.layout_selection.sweep --out DIR [--batch 8 --seq 512]

Output formats are the reference's:
  * fused kernels: ``<kernel>-combined.csv`` with one line per configuration,
    ``NAME = layout ... time = t s`` (pytorch_module/benchmark.py:1440-1444,
    read back by config_selection/load_data.py:11-41);
  * contractions: ``<op>-result.csv`` with columns A,B,C,M,N,K,batch,Time,
    Implementation (subset of config_selection/parse_tc_results.py:15-18,38-62;
    the cuBLAS-specific columns trans_a/lda/... have no meaning here and are
    left out).
Search-space pruning (the reference prunes too, pytorch_module/benchmark.py:365-373):
contractions take the full product of their operands' candidate layouts; a fused
kernel is timed with all of its tensors in one common family of layouts and with
one tensor at a time deviating from it.
"""

import argparse
import itertools
import os

import torch

from .. import layouts as L
from .. import ops
from .spec import DOMAINS, OPS

H, DEV = 16, 'cuda'


def _alloc(name, layout, sizes, kind='h'):
    shape = L.shape_of(layout, sizes)
    if name in L.MASKS:
        t = (torch.rand(shape, device=DEV) >= 0.1).to(torch.uint8)
    else:
        t = (torch.randn(shape, device=DEV) * 0.5).half()
    logical = L.LOGICAL[name]
    return t.permute([layout.index(c) for c in logical])        # logical-order view


def _vec(n):
    return torch.ones(n, device=DEV).half()


def fused_call(name, T, sizes):
    """Closure running fused operator ``name`` on logical views ``T`` (dict by tensor name)."""
    I, U = sizes['I'], sizes['U']
    vi, vu = _vec(I), _vec(U)
    if name == 'aib':
        return lambda: ops.attention_input_biases(T['WKKWQQWVV'], T['BKQV'], T['KKQQVV'])
    if name == 'softmax':
        return lambda: ops.softmax_dropout(T['BETA'], T['ALPHA'], T['ATTN_DROP_MASK'], T['ATTN_DROP'], p=0.1)
    if name == 'bdrln1':
        return lambda: ops.bias_dropout_residual_layernorm(T['ATT'], vi, T['X'], vi, vi, T['DROP1MASK'], T['ATT'],
                                                           T['LN1DIFF'], T['LN1STD'], T['LN1'], T['SB1'], p=0.1)
    if name == 'bdrln2':
        return lambda: ops.bias_dropout_residual_layernorm(T['DROP2_LINW2'], vi, T['SB1'], vi, vi, T['DROP3MASK'],
                                                           T['LIN2'], T['LN2DIFF'], T['LN2STD'], T['LN2'], T['SB2'], p=0.1)
    if name == 'bad':
        return lambda: ops.bias_activation_dropout(T['SB1_LINW1'], vu, T['DROP2MASK'], T['LIN1'], T['DROP2'], p=0.1)
    if name == 'bsb':
        dg, db = _vec(I), _vec(I)
        return lambda: ops.backward_scale_bias(T['SB2'], T['LN2'], vi, T['DLN2'], dg, db)
    if name in ('blnrd1', 'blnrd2'):
        k = ('DLN2', 'LN2STD', 'LN2DIFF', 'DROP3MASK', 'DRESID2', 'DLIN2') if name == 'blnrd1' else \
            ('DLN1', 'LN1STD', 'LN1DIFF', 'DROP1MASK', 'DRESID1', 'DATT')
        return lambda: ops.backward_layernorm_residual_dropout(*(T[n] for n in k))
    if name == 'bdrlb':
        db = _vec(U)
        return lambda: ops.backward_dropout_activation_bias(T['DDROP2'], T['DROP2MASK'], T['LIN1'], T['DLIN1'], db)
    if name == 'ebsb':
        a, b, c = _vec(I), _vec(I), _vec(I)
        return lambda: ops.extended_backward_scale_bias(T['LN1'], vi, T['DRESID2'], T['DLIN1_LINW1'], T['DLIN2'],
                                                        T['DLN1'], a, b, c)
    if name == 'baob':
        d = _vec(I)
        return lambda: ops.backward_attn_out_bias(T['DATT'], d)
    if name == 'bs':
        return lambda: ops.backward_softmax(T['ALPHA'], T['ATTN_DROP_MASK'], T['DATTN_DROP'], T['DBETA'])
    if name == 'baib':
        return lambda: ops.backward_attention_input_biases(T['DKKQQVV'], T['BKQV'])
    if name == 'bei':
        return lambda: ops.backward_encoder_input(T['DXATT'], T['DRESID1'], T['X'])
    raise KeyError(name)


def time_graph(fn, reps=8, replays=3):
    """Median device time (s) of one call: `reps` calls captured in a CUDA graph (so host
    launch cost is out of the picture), replayed a few times."""
    fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        fn()
        with torch.cuda.graph(g, stream=s):
            for _ in range(reps):
                fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(replays):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) / reps / 1e3)
    return sorted(times)[len(times) // 2]


def fused_configs(op):
    """Common-family configurations plus single-tensor deviations."""
    names = op['tensors']
    doms = [DOMAINS[n] for n in names]
    width = max(len(d) for d in doms)
    seen = []
    for fam in range(width):
        base = tuple(d[min(fam, len(d) - 1)] for d in doms)
        if base not in seen:
            seen.append(base)
        if fam == 0:
            for i, d in enumerate(doms):
                for alt in d[1:]:
                    cfg = base[:i] + (alt,) + base[i + 1:]
                    if cfg not in seen:
                        seen.append(cfg)
    return seen


def sweep(out_dir, batch, seq, heads=H, embed=1024, only=None, verbose=True):
    os.makedirs(out_dir, exist_ok=True)
    sizes = L.sizes_map(batch, seq, heads, embed)
    for op in OPS:
        if only and op['name'] not in only:
            continue
        names = op['tensors']
        if op['kind'] == 'gemm':
            path = os.path.join(out_dir, f"{op['name']}-result.csv")
            rows = ['A,B,C,M,N,K,batch,Time,Implementation']
            for lay in itertools.product(*(DOMAINS[n] for n in names)):
                if names[0] == names[1] and lay[0] != lay[1]:
                    continue                      # the same tensor read twice
                dims = [v(l) for v, l in zip(op['views'], lay)]
                try:
                    t = [(torch.randn(L.shape_of(d, sizes), device=DEV) * 0.1).half() for d in dims]
                    spec = f'{dims[0].lower()},{dims[1].lower()}->{dims[2].lower()}'
                    impl = ops.einsum(spec, t[0], t[1], t[2])
                    sec = time_graph(lambda: ops.einsum(spec, t[0], t[1], t[2]))
                except ops.SubstationError:
                    continue                      # not a GEMM under these layouts (index groups do not collapse)
                ks = [c for c in dims[0] if c in dims[1] and c not in dims[2]]
                bs = [c for c in dims[0] if c in dims[1] and c in dims[2]]
                ms = [c for c in dims[0] if c not in dims[1]]
                ns = [c for c in dims[1] if c not in dims[0]]
                prod = lambda cs: int(torch.tensor([sizes[c] for c in cs]).prod()) if cs else 1
                rows.append(f'{lay[0]},{lay[1]},{lay[2]},{prod(ms)},{prod(ns)},{prod(ks)},{prod(bs)},{sec:.9f},{impl}')
                del t
            with open(path, 'w') as f:
                f.write('\n'.join(rows) + '\n')
        else:
            path = os.path.join(out_dir, f"{op['name']}-combined.csv")
            lines = []
            for lay in fused_configs(op):
                T = {}
                for n, l in zip(names, lay):
                    T[n] = _alloc(n, l, sizes)
                sec = time_graph(fused_call(op['name'], T, sizes))
                lines.append(' '.join(f'{n} = {l}' for n, l in zip(names, lay)) + f' time = {sec:.9f} s')
                del T
            with open(path, 'w') as f:
                f.write('\n'.join(lines) + '\n')
        torch.cuda.empty_cache()
        if verbose:
            print(op['name'], 'done', flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--out', required=True)
    ap.add_argument('--batch', type=int, default=8)
    ap.add_argument('--seq', type=int, default=512)
    ap.add_argument('--only', nargs='*')
    a = ap.parse_args()
    sweep(a.out, a.batch, a.seq, only=a.only)


if __name__ == '__main__':
    main()
