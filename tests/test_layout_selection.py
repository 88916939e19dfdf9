"""CPU checks of the layout optimizer on synthetic tables: file formats of the
reference (config_selection/load_data.py:11-41, parse_tc_results.py:38-62) are read
back, the search prefers cheaper layouts, ties inputs to outputs, and emits a
configuration the Encoder accepts."""

import itertools
import os

from substation_b200 import layouts as L
from substation_b200.layout_selection import optimize as opt
from substation_b200.layout_selection.spec import DOMAINS, OPS
from substation_b200.layout_selection.sweep import fused_configs


def _write_tables(d, cost):
    for op in OPS:
        names = op['tensors']
        if op['kind'] == 'gemm':
            rows = ['A,B,C,M,N,K,batch,Time,Implementation']
            for lay in itertools.product(*(DOMAINS[n] for n in names)):
                if names[0] == names[1] and lay[0] != lay[1]:
                    continue
                rows.append(f'{lay[0]},{lay[1]},{lay[2]},1,1,1,1,{cost(op, lay):.9f},tcgen05')
            with open(os.path.join(d, f"{op['name']}-result.csv"), 'w') as f:
                f.write('\n'.join(rows) + '\n')
        else:
            with open(os.path.join(d, f"{op['name']}-combined.csv"), 'w') as f:
                for lay in fused_configs(op):
                    f.write(' '.join(f'{n} = {l}' for n, l in zip(names, lay)) + f' time = {cost(op, lay):.9f} s\n')


def test_optimizer_reads_tables_and_prefers_cheaper_layouts(tmp_path):
    # every operator costs 10 us, plus 5 us per [*,*,I]-type tensor not stored feature-innermost,
    # minus 3 us for lin2 when LINW2 is stored 'IU'
    def cost(op, lay):
        c = 10e-6 + 5e-6 * sum(1 for l in lay if len(l) == 3 and l[-1] not in 'IU')
        if op['name'] == 'lin2' and lay[1] == 'IU':
            c -= 3e-6
        return c
    _write_tables(str(tmp_path), cost)
    tables = opt.load_tables(str(tmp_path))
    assert len(tables['lin2']) == 3 * 2 * 3 and len(tables['softmax']) == 6
    start = L.validate(L.uniform_layouts())
    start['X'] = start['SB2'] = 'IBJ'                  # a deliberately bad start
    cfg, report = opt.optimize(str(tmp_path), start=start)
    table = L.validate(cfg)
    assert table['X'] == table['SB2'] and table['X'][-1] == 'I'
    assert table['LINW2'] == 'IU'
    assert report['chosen_cost_s'] < report['start_cost_s']
    assert set(cfg) == {'input', 'output', 'params', 'forward_interm', 'backward_interm', 'special_dims',
                        'algorithms'}
    assert [n for n, _ in cfg['params']] == list(L.PARAMS)


def test_missing_costs_are_never_chosen(tmp_path):
    def cost(op, lay):
        return 10e-6
    _write_tables(str(tmp_path), cost)
    # remove every aib row that does not keep the default stacked layouts
    path = os.path.join(str(tmp_path), 'aib-combined.csv')
    keep = [l for l in open(path) if 'KKQQVV = QPHBJ' in l]
    open(path, 'w').writelines(keep)
    cfg, _ = opt.optimize(str(tmp_path))
    assert dict(cfg['forward_interm'])['KKQQVV'] == 'QPHBJ'
