"""CPU checks of the layout search on synthetic measurements: the tables are written in the reference's file
formats (config_selection/load_data.py:11-41, parse_tc_results.py:38-62) and read back, a sweep appends and
resumes by key, the search prefers cheaper layouts, keeps tied tensors together, never picks what was not
measured, and emits a configuration the Encoder accepts."""

import os

from substation_b200 import layouts as L
from substation_b200.layout_selection import optimize as opt
from substation_b200.layout_selection import sweep as sw
from substation_b200.layout_selection.spec import DOMAINS, OPS, default_table, op_key


def _fake_measure(cost, calls=None):
    def measure(table):
        if calls is not None:
            calls.append(dict(table))
        return {op['name']: cost(op, op_key(op, table)) for op in OPS}
    return measure


def test_domains_cover_every_permutation_and_keep_stacked_tensors_sliceable():
    assert len(DOMAINS['BETA']) == 24 and len(DOMAINS['X']) == 6 and len(DOMAINS['LINW1']) == 2
    assert len(DOMAINS['KKQQVV']) == 24 and all(l[0] == 'Q' for l in DOMAINS['KKQQVV'])
    assert all(DOMAINS[n][0] == L.LOGICAL[n] for n in DOMAINS)
    touched = {t for op in OPS for t in op['tensors']}
    assert set(L.LOGICAL) - touched == {'B1', 'B2', 'BO', 'LINB1', 'LINB2', 'S1', 'S2'}    # one layout only


def test_sweep_appends_resumes_and_optimizer_prefers_cheaper_layouts(tmp_path):
    # every group costs 10 us, plus 5 us per [*,*,I]- or [*,*,U]-type tensor not stored feature-innermost,
    # minus 3 us for lin2 when LINW2 is stored 'IU'
    def cost(op, key):
        c = 10e-6 + 5e-6 * sum(1 for l in key if len(l) == 3 and l[-1] not in 'IU')
        if op['name'] == 'lin2' and key[1] == 'IU':
            c -= 3e-6
        return c
    out = str(tmp_path)
    start = default_table()
    start['X'] = start['SB2'] = 'IBJ'                  # a deliberately bad start
    calls = []
    n1 = sw.sweep(out, 2, 8, heads=2, embed=16, around=start, measure=_fake_measure(cost, calls), limit=100, verbose=False)
    assert n1 == 100
    n2 = sw.sweep(out, 2, 8, heads=2, embed=16, around=start, measure=_fake_measure(cost, calls), verbose=False)
    assert n1 + n2 == len(calls) == 394                # resumed where the first call stopped, nothing measured twice
    assert sw.sweep(out, 2, 8, heads=2, embed=16, around=start, measure=_fake_measure(cost, calls), verbose=False) == 0
    # file formats
    with open(os.path.join(out, 'lin2-result.csv')) as f:
        rows = f.read().splitlines()
    assert rows[0] == 'A,B,C,M,N,K,batch,Time,Implementation' and len(rows) == 1 + 1 + 5 + 1 + 5
    with open(os.path.join(out, 'bdrlb-combined.csv')) as f:
        assert all(' time = ' in line and line.rstrip().endswith(' s') for line in f)
    tables = opt.load_tables(out)
    assert len(tables['lin2']) == 12 and len(tables['baib']) == 1 + 23 + 1
    cfg, report = opt.optimize(out, start=start)
    table = L.validate(cfg)
    assert table['X'] == table['SB2'] and table['X'][-1] == 'I'
    assert table['LINW2'] == 'IU'
    assert report['chosen_cost_s'] < report['start_cost_s']
    assert set(cfg) == {'input', 'output', 'params', 'forward_interm', 'backward_interm', 'special_dims',
                        'algorithms'}
    assert [n for n, _ in cfg['params']] == list(L.PARAMS)
    # a second sweep around the result adds the neighbours of the new point to the same files
    assert sw.sweep(out, 2, 8, heads=2, embed=16, around=table, measure=_fake_measure(cost), verbose=False) > 0
    assert len(opt.load_tables(out)['lin2']) > 12


def test_missing_costs_are_never_chosen(tmp_path):
    # everything costs the same except that KKQQVV in another order would be much cheaper for aib's group;
    # that row is then removed from the table, and the search must not pick it
    def cost(op, key):
        return 1e-6 if op['name'] == 'baib' and key[0] != 'QPHBJ' else 10e-6
    out = str(tmp_path)
    sw.sweep(out, 2, 8, heads=2, embed=16, measure=_fake_measure(cost), verbose=False)
    cfg, _ = opt.optimize(out)
    assert dict(cfg['backward_interm'])['DKKQQVV'] != 'QPHBJ'
    path = os.path.join(out, 'baib-combined.csv')
    keep = [l for l in open(path) if 'DKKQQVV = QPHBJ' in l]
    open(path, 'w').writelines(keep)
    cfg, _ = opt.optimize(out)
    assert dict(cfg['backward_interm'])['DKKQQVV'] == 'QPHBJ'
