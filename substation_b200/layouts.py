"""The layout-configuration contract of the reference's ``Encoder``.

A configuration is the dict pickled by ``config_selection/optimize.py:443-493``:
``input``/``output`` = (name, dims), ``params`` (12), ``forward_interm`` (23),
``backward_interm`` (14) = lists of (name, dims), plus ``special_dims`` and
``algorithms`` (hints for the reference's kernels and cuBLAS; accepted and
ignored here, they have no meaning for these kernels).  ``dims`` is the memory
order of the tensor, outermost first, one letter per dim:
B batch, J/K sequence, H heads, P head size, I embedding, U = 4 I, Q = 3.
"""

import pickle

#: logical index order of every tensor (the order operators are defined in)
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
    'DROP2MASK': 'BJU', 'DROP3MASK': 'BJI', 'LN1': 'BJI', 'LN1STD': 'BJ', 'LN1DIFF': 'BJI',
    'DLN2': 'BJI', 'DRESID2': 'BJI', 'DLIN2': 'BJI', 'DDROP2': 'BJU', 'DLIN1': 'BJU',
    'DLIN1_LINW1': 'BJI', 'DLN1': 'BJI', 'DRESID1': 'BJI', 'DATT': 'BJI', 'DXATT': 'BJI',
    'DGAMMA': 'PHBJ', 'DATTN_DROP': 'HBJK', 'DBETA': 'HBJK', 'DKKQQVV': 'QPHBJ',
}

PARAMS = ('WKQV', 'BKQV', 'WO', 'BO', 'S1', 'B1', 'LINB1', 'LINW1', 'S2', 'B2', 'LINB2', 'LINW2')
FORWARD_INTERM = ('KKQQVV', 'WKKWQQWVV', 'BETA', 'ALPHA', 'ATTN_DROP_MASK', 'ATTN_DROP', 'GAMMA',
                  'ATT', 'DROP1MASK', 'SB1', 'SB1_LINW1', 'DROP2', 'LIN1', 'DROP2_LINW2', 'LIN2',
                  'LN2', 'LN2STD', 'LN2DIFF', 'DROP2MASK', 'DROP3MASK', 'LN1', 'LN1STD', 'LN1DIFF')
BACKWARD_INTERM = ('DLN2', 'DRESID2', 'DLIN2', 'DDROP2', 'DLIN1', 'DLIN1_LINW1', 'DLN1', 'DRESID1',
                   'DATT', 'DXATT', 'DGAMMA', 'DATTN_DROP', 'DBETA', 'DKKQQVV')
MASKS = ('ATTN_DROP_MASK', 'DROP1MASK', 'DROP2MASK', 'DROP3MASK')
STACKED = ('KKQQVV', 'DKKQQVV', 'WKKWQQWVV', 'BKQV', 'WKQV')


class LayoutError(ValueError):
    pass


def load_layouts(path):
    """Read a layout pickle as shipped with the reference
    (pytorch_module/layouts-bert-*.pickle; pytorch_module/run_encoder.py:110-111)."""
    with open(path, 'rb') as f:
        return pickle.load(f)


def validate(layouts):
    """Check a configuration dict; returns {name: dims} over all 51 tensors.

    Mirrors the checks the reference makes while generating its header
    (pytorch_module/encoder.py:318-327) and the same-layout constraints of the
    layout optimizer (config_selection/ops.py:265-289)."""
    for key in ('input', 'output', 'params', 'forward_interm', 'backward_interm'):
        if key not in layouts:
            raise LayoutError(f"layout configuration has no '{key}' entry")
    if layouts['input'][0] != 'X' or layouts['output'][0] != 'SB2':
        raise LayoutError("input tensor must be named 'X' and output 'SB2'")
    table = dict([tuple(layouts['input']), tuple(layouts['output'])])
    for key, names in (('params', PARAMS), ('forward_interm', FORWARD_INTERM),
                       ('backward_interm', BACKWARD_INTERM)):
        got = [n for n, _ in layouts[key]]
        if sorted(got) != sorted(names):
            missing = sorted(set(names) - set(got))
            extra = sorted(set(got) - set(names))
            raise LayoutError(f"'{key}' must list exactly {len(names)} tensors "
                              f"(missing {missing}, unexpected {extra})")
        table.update((n, d) for n, d in layouts[key])
    for name, dims in table.items():
        if sorted(dims) != sorted(LOGICAL[name]):
            raise LayoutError(f"layout '{dims}' of {name} is not a permutation of '{LOGICAL[name]}'")
    for name in STACKED:
        if table[name][0] != 'Q':
            raise LayoutError(f'stacked tensor {name} must have Q outermost (got {table[name]})')
    if table['X'] != table['SB2']:
        raise LayoutError('input and output layouts must be equal so that layers chain')
    return table


def sizes_map(batch_size, max_seq_len, num_heads, embedding_size):
    """Letter -> extent (pytorch_module/encoder.py:43-53)."""
    return {'Q': 3, 'B': batch_size, 'S': max_seq_len, 'H': num_heads,
            'P': embedding_size // num_heads, 'I': embedding_size, 'U': 4 * embedding_size,
            'J': max_seq_len, 'K': max_seq_len}


def shape_of(dims, sizes):
    return tuple(sizes[c] for c in dims)


def permutation(src, dst):
    """Axes such that a tensor stored as ``src`` permuted by them has dim order ``dst``."""
    return [src.index(c) for c in dst]


def uniform_layouts(feature_inner=True):
    """A configuration with every activation token-major and feature-innermost
    (the natural choice for 128-bit row access); weights as in the shipped pickles."""
    fwd = {n: LOGICAL[n] for n in FORWARD_INTERM}
    bwd = {n: LOGICAL[n] for n in BACKWARD_INTERM}
    return {
        'input': ('X', 'BJI'), 'output': ('SB2', 'BJI'),
        'params': [(n, LOGICAL[n]) for n in PARAMS],
        'forward_interm': [(n, fwd[n]) for n in FORWARD_INTERM],
        'backward_interm': [(n, bwd[n]) for n in BACKWARD_INTERM],
        'special_dims': {}, 'algorithms': {},
    }


def selected_layouts(tag='b8_l512'):
    """The configuration the layout search chose for these kernels on B200
    (``layout_selection/results_<tag>/layouts_b200_<tag>.json``; regenerate with
    ``python -m substation_b200.layout_selection.sweep`` then ``.optimize``)."""
    import json
    import os
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'layout_selection', f'results_{tag}',
                        f'layouts_b200_{tag}.json')
    with open(path) as f:
        d = json.load(f)
    for k in ('params', 'forward_interm', 'backward_interm'):
        d[k] = [tuple(x) for x in d[k]]
    d['input'], d['output'] = tuple(d['input']), tuple(d['output'])
    return d


def read_json(path):
    """A configuration stored as JSON (the pickle's dict with tuples written as lists)."""
    import json
    with open(path) as f:
        d = json.load(f)
    for k in ('params', 'forward_interm', 'backward_interm'):
        d[k] = [tuple(x) for x in d[k]]
    d['input'], d['output'] = tuple(d['input']), tuple(d['output'])
    return d


def named_layouts(which):
    """A configuration by name: a dict (returned as is), 'uniform', 'b200_<tag>' (what the layout search chose for
    these kernels, see ``selected_layouts``), or the path of a ``.json`` / ``.pickle`` file."""
    if isinstance(which, dict):
        return which
    if which == 'uniform':
        return uniform_layouts()
    if which.startswith('b200_'):
        return selected_layouts(which[5:])
    if which.endswith('.pickle') or which.endswith('.pkl'):
        return load_layouts(which)
    if which.endswith('.json'):
        return read_json(which)
    raise LayoutError(f"unknown layout configuration '{which}'")
