"""The layer as the layout search sees it: operator groups in execution order, the tensors each group's time
depends on (names as in the layout configuration) and every memory order a tensor may take.

A group is what the layer runs between two points where only contract tensors are live: a fused operator
(one launch) or, when that operator declines for the layouts at hand, the separate operators that replace it
(pytorch_module/encoder.cu:87-299 lists the separate sequence).  The search measures groups, so a layout that
makes a fused operator fall back is charged what the fall-back really costs.
"""

import itertools

from .. import layouts as L

#: tensors that must share one layout (layers chain: config_selection/ops.py:265-289)
TIED = [('X', 'SB2')]


def _perms(dims, fixed_first=False):
    if fixed_first:
        return tuple(dims[0] + ''.join(p) for p in itertools.permutations(dims[1:]))
    return tuple(''.join(p) for p in itertools.permutations(dims))


#: candidate memory orders per tensor: every permutation of its dims; stacked tensors keep Q outermost (they are
#: sliced by pointer offset, pytorch_module/encoder.py:318-327).  The logical order comes first.
DOMAINS = {}
for _n, _d in L.LOGICAL.items():
    _p = _perms(_d, fixed_first=_n in L.STACKED)
    DOMAINS[_n] = (_d,) + tuple(x for x in _p if x != _d)


def _grp(name, members, tensors, kind='fused'):
    return {'name': name, 'members': tuple(members), 'tensors': tuple(tensors), 'kind': kind}


#: execution order; 'members' = every operator name the layer may report for this group (fused or separate)
OPS = [
    _grp('QKV-fused+aib', ('QKV-fused+aib', 'QKV-fused', 'aib'), ('X', 'WKQV', 'BKQV', 'WKKWQQWVV', 'KKQQVV')),
    _grp('QKT+softmax', ('QKT+softmax', 'QKT', 'softmax'), ('KKQQVV', 'BETA', 'ALPHA', 'ATTN_DROP_MASK', 'ATTN_DROP')),
    _grp('gamma', ('gamma',), ('KKQQVV', 'ATTN_DROP', 'GAMMA'), 'gemm'),
    _grp('out', ('out',), ('WO', 'GAMMA', 'ATT'), 'gemm'),
    _grp('bdrln1', ('bdrln1',), ('ATT', 'X', 'DROP1MASK', 'LN1DIFF', 'LN1STD', 'LN1', 'SB1')),
    _grp('lin1+bad', ('lin1+bad', 'lin1', 'bad'), ('SB1', 'LINW1', 'SB1_LINW1', 'DROP2MASK', 'LIN1', 'DROP2')),
    _grp('lin2', ('lin2',), ('DROP2', 'LINW2', 'DROP2_LINW2'), 'gemm'),
    _grp('bdrln2', ('bdrln2',), ('DROP2_LINW2', 'SB1', 'DROP3MASK', 'LIN2', 'LN2DIFF', 'LN2STD', 'LN2', 'SB2')),
    _grp('bsb+blnrd1', ('bsb+blnrd1', 'bsb', 'blnrd1'), ('SB2', 'LN2', 'DLN2', 'LN2STD', 'LN2DIFF', 'DROP3MASK', 'DRESID2', 'DLIN2')),
    _grp('dXlin2', ('dXlin2',), ('DLIN2', 'LINW2', 'DDROP2'), 'gemm'),
    _grp('dWlin2', ('dWlin2',), ('DLIN2', 'DROP2', 'LINW2'), 'gemm'),
    _grp('bdrlb', ('bdrlb',), ('DDROP2', 'DROP2MASK', 'LIN1', 'DLIN1')),
    _grp('dXlin1', ('dXlin1',), ('DLIN1', 'LINW1', 'DLIN1_LINW1'), 'gemm'),
    _grp('dWlin1', ('dWlin1',), ('DLIN1', 'SB1', 'LINW1'), 'gemm'),
    _grp('ebsb+blnrd2+baob', ('ebsb+blnrd2+baob', 'ebsb', 'blnrd2', 'baob'),
         ('LN1', 'DRESID2', 'DLIN1_LINW1', 'DLIN2', 'DLN1', 'LN1STD', 'LN1DIFF', 'DROP1MASK', 'DRESID1', 'DATT')),
    _grp('dWout', ('dWout',), ('GAMMA', 'DATT', 'WO'), 'gemm'),
    _grp('dXout', ('dXout',), ('WO', 'DATT', 'DGAMMA'), 'gemm'),
    _grp('dX1gamma+bs', ('dX1gamma+bs', 'dX1gamma', 'bs'), ('KKQQVV', 'DGAMMA', 'ALPHA', 'ATTN_DROP_MASK', 'DATTN_DROP', 'DBETA')),
    _grp('dX2gamma', ('dX2gamma',), ('DGAMMA', 'ATTN_DROP', 'DKKQQVV'), 'gemm'),
    _grp('dX1QKT+dX2QKT', ('dX1QKT+dX2QKT', 'dX1QKT', 'dX2QKT'), ('KKQQVV', 'DBETA', 'DKKQQVV')),
    _grp('dXQKV-fused+bei', ('dXQKV-fused+bei', 'dXQKV-fused', 'bei'), ('WKQV', 'DKKQQVV', 'DXATT', 'DRESID1', 'X')),
    _grp('dWQKV-fused', ('dWQKV-fused',), ('X', 'DKKQQVV', 'WKQV'), 'gemm'),
    _grp('baib', ('baib',), ('DKKQQVV', 'BKQV')),
]

#: operator name -> group name
GROUP_OF = {m: op['name'] for op in OPS for m in op['members']}


def op_key(op, table):
    """The layouts a group's cost depends on, as a hashable key."""
    return tuple(table[t] for t in op['tensors'])


def default_table():
    return L.validate(L.uniform_layouts())


def tie_groups():
    """Tensors that move together, each group once, in a fixed order."""
    tied = {}
    for g in TIED:
        for n in g:
            tied[n] = g
    seen, out = set(), []
    for n in DOMAINS:
        if n in seen:
            continue
        g = tied.get(n, (n,))
        seen.update(g)
        out.append(g)
    return out
