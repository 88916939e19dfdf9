"""Operators of the layer as the layout search sees them: which tensors each one
touches (names as in the layout configuration) and, for contractions, how its
einsum is spelled from the operands' layouts (pytorch_module/encoder.cu:87-299).
"""

from .. import layouts as L

#: candidate memory orders per tensor class
_ACT_I = ('BJI', 'JBI', 'IBJ')
_ACT_U = ('BJU', 'JBU', 'UBJ')
_SCORE = ('HBJK', 'BHJK')
_STACK = ('QPHBJ', 'QHPBJ', 'QHBPJ')
_HEADS = ('PHBJ', 'HPBJ', 'BJPH', 'BJHP')

DOMAINS = {}
for _n in ('X', 'SB2', 'ATT', 'DROP1MASK', 'SB1', 'DROP2_LINW2', 'LIN2', 'LN2', 'LN2DIFF', 'DROP3MASK', 'LN1',
           'LN1DIFF', 'DLN2', 'DRESID2', 'DLIN2', 'DLIN1_LINW1', 'DLN1', 'DRESID1', 'DATT', 'DXATT'):
    DOMAINS[_n] = _ACT_I
for _n in ('SB1_LINW1', 'DROP2', 'LIN1', 'DROP2MASK', 'DDROP2', 'DLIN1'):
    DOMAINS[_n] = _ACT_U
for _n in ('BETA', 'ALPHA', 'ATTN_DROP_MASK', 'ATTN_DROP', 'DATTN_DROP', 'DBETA'):
    DOMAINS[_n] = _SCORE
for _n in ('KKQQVV', 'WKKWQQWVV', 'DKKQQVV'):
    DOMAINS[_n] = _STACK
for _n in ('GAMMA', 'DGAMMA'):
    DOMAINS[_n] = _HEADS
DOMAINS.update({
    'LN1STD': ('BJ', 'JB'), 'LN2STD': ('BJ', 'JB'),
    'WKQV': ('QPHI', 'QHPI', 'QIPH'), 'BKQV': ('QPH', 'QHP'), 'WO': ('IPH', 'PHI', 'IHP', 'HPI'),
    'LINW1': ('IU', 'UI'), 'LINW2': ('UI', 'IU'),
    'BO': ('I',), 'S1': ('I',), 'B1': ('I',), 'S2': ('I',), 'B2': ('I',), 'LINB1': ('U',), 'LINB2': ('I',),
})

#: tensors that must share one layout (layers chain: config_selection/ops.py:265-289)
TIED = [('X', 'SB2')]

_r = lambda s: s.replace('J', 'K')


def _g(name, a, b, c, a_view=None, b_view=None, c_view=None):
    """Contraction: operand tensor names and optional view functions (slice of a stacked
    tensor with J relabelled K)."""
    return {'kind': 'gemm', 'name': name, 'tensors': (a, b, c),
            'views': (a_view or (lambda l: l), b_view or (lambda l: l), c_view or (lambda l: l))}


_sl = lambda l: l[1:]            # one projection of a stacked tensor
_slk = lambda l: _r(l[1:])       # ... read with the sequence index named K

OPS = [
    _g('QKV-fused', 'X', 'WKQV', 'WKKWQQWVV'),
    {'kind': 'fused', 'name': 'aib', 'tensors': ('WKKWQQWVV', 'BKQV', 'KKQQVV')},
    _g('QKT', 'KKQQVV', 'KKQQVV', 'BETA', _slk, _sl),
    {'kind': 'fused', 'name': 'softmax', 'tensors': ('BETA', 'ALPHA', 'ATTN_DROP_MASK', 'ATTN_DROP')},
    _g('gamma', 'KKQQVV', 'ATTN_DROP', 'GAMMA', _slk),
    _g('out', 'WO', 'GAMMA', 'ATT'),
    {'kind': 'fused', 'name': 'bdrln1', 'tensors': ('ATT', 'X', 'DROP1MASK', 'LN1DIFF', 'LN1STD', 'LN1', 'SB1')},
    _g('lin1', 'SB1', 'LINW1', 'SB1_LINW1'),
    {'kind': 'fused', 'name': 'bad', 'tensors': ('SB1_LINW1', 'DROP2MASK', 'LIN1', 'DROP2')},
    _g('lin2', 'DROP2', 'LINW2', 'DROP2_LINW2'),
    {'kind': 'fused', 'name': 'bdrln2',
     'tensors': ('DROP2_LINW2', 'SB1', 'DROP3MASK', 'LIN2', 'LN2DIFF', 'LN2STD', 'LN2', 'SB2')},
    {'kind': 'fused', 'name': 'bsb', 'tensors': ('SB2', 'LN2', 'DLN2')},
    {'kind': 'fused', 'name': 'blnrd1', 'tensors': ('DLN2', 'LN2STD', 'LN2DIFF', 'DROP3MASK', 'DRESID2', 'DLIN2')},
    _g('dXlin2', 'DLIN2', 'LINW2', 'DDROP2'),
    _g('dWlin2', 'DLIN2', 'DROP2', 'LINW2'),
    {'kind': 'fused', 'name': 'bdrlb', 'tensors': ('DDROP2', 'DROP2MASK', 'LIN1', 'DLIN1')},
    _g('dXlin1', 'DLIN1', 'LINW1', 'DLIN1_LINW1'),
    _g('dWlin1', 'DLIN1', 'SB1', 'LINW1'),
    {'kind': 'fused', 'name': 'ebsb', 'tensors': ('LN1', 'DRESID2', 'DLIN1_LINW1', 'DLIN2', 'DLN1')},
    {'kind': 'fused', 'name': 'blnrd2', 'tensors': ('DLN1', 'LN1STD', 'LN1DIFF', 'DROP1MASK', 'DRESID1', 'DATT')},
    {'kind': 'fused', 'name': 'baob', 'tensors': ('DATT',)},
    _g('dWout', 'GAMMA', 'DATT', 'WO'),
    _g('dXout', 'WO', 'DATT', 'DGAMMA'),
    _g('dX1gamma', 'KKQQVV', 'DGAMMA', 'DATTN_DROP', _slk),
    _g('dX2gamma', 'DGAMMA', 'ATTN_DROP', 'DKKQQVV', None, None, _slk),
    {'kind': 'fused', 'name': 'bs', 'tensors': ('ALPHA', 'ATTN_DROP_MASK', 'DATTN_DROP', 'DBETA')},
    _g('dX1QKT', 'KKQQVV', 'DBETA', 'DKKQQVV', _slk, None, _sl),
    _g('dX2QKT', 'KKQQVV', 'DBETA', 'DKKQQVV', _sl, None, _slk),
    _g('dXQKV-fused', 'WKQV', 'DKKQQVV', 'DXATT'),
    _g('dWQKV-fused', 'X', 'DKKQQVV', 'WKQV'),
    {'kind': 'fused', 'name': 'baib', 'tensors': ('DKKQQVV', 'BKQV')},
    {'kind': 'fused', 'name': 'bei', 'tensors': ('DXATT', 'DRESID1', 'X')},
]


def op_key(op, table):
    """The layouts an operator's cost depends on, as a hashable key."""
    return tuple(table[t] for t in op['tensors'])


def default_table():
    return L.validate(L.uniform_layouts())
