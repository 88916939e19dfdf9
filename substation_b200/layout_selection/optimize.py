"""Choose per-tensor layouts from the sweep tables and write a configuration in the
reference's pickle schema (config_selection/optimize.py:443-493).

    python -m substation_b200.layout_selection.optimize RESULTS_DIR --output_config out.pickle

The reference expands the operator DAG into a layered graph and runs a
single-source shortest path over (position, layouts of the variables cut there)
(config_selection/optimize.py:109-134, 233-266, 346-392), then binds leftovers
greedily (config_selection/ops.py:1440-1480).  Here the same objective, the sum
over the layer's operator groups of the measured time under the layouts of their tensors, is
minimised in two stages: (1) the chain of forward groups is solved exactly by
shortest path over layered states (position, layout of the tensor carried to the
next group); (2) every remaining tensor is bound by coordinate descent on the
full objective until no single change improves it.  Tensors tied together
(input = output so that layers chain) move as one.  Costs missing from the
tables are treated as infinite, so only measured configurations can be chosen; the
sweep measures every single-tensor change around a starting point, and sweeping
again around the result (``sweep --rounds``) extends the tables where the search goes.
"""

import argparse
import csv
import json
import os
import pickle
import re

from .. import layouts as L
from .spec import DOMAINS, OPS, op_key, tie_groups

INF = float('inf')


def load_tables(results_dir):
    """{op name: {tuple of layouts: seconds}} from <op>-result.csv / <kernel>-combined.csv."""
    tables = {}
    for op in OPS:
        t = {}
        if op['kind'] == 'gemm':
            path = os.path.join(results_dir, f"{op['name']}-result.csv")
            if os.path.exists(path):
                with open(path) as f:
                    for row in csv.DictReader(f):
                        key = (row['A'], row['B'], row['C'])
                        t[key] = min(t.get(key, INF), float(row['Time']))
        else:
            path = os.path.join(results_dir, f"{op['name']}-combined.csv")
            if os.path.exists(path):
                with open(path) as f:
                    for line in f:
                        pairs = dict(re.findall(r'(\w+) = (\S+)', line))
                        if 'time' not in pairs:
                            continue
                        key = tuple(pairs[n] for n in op['tensors'])
                        t[key] = min(t.get(key, INF), float(pairs['time']))
        tables[op['name']] = t
    return tables


def op_cost(op, table, tables):
    return tables[op['name']].get(op_key(op, table), INF)


def total_cost(table, tables):
    return sum(op_cost(op, table, tables) for op in OPS)


def forward_chain_shortest_path(table, tables):
    """Exact minimisation over the tensors handed from one forward group to the next (KKQQVV, ATTN_DROP, GAMMA,
    ATT, SB1, DROP2, DROP2_LINW2): layered graph, node = (position, layout of the carried tensor), edge = the
    producing group's time given that layout with all other tensors as in the best path so far."""
    chain = ['KKQQVV', 'ATTN_DROP', 'GAMMA', 'ATT', 'SB1', 'DROP2', 'DROP2_LINW2']
    fwd_ops = OPS[:8]            # QKV-fused+aib ... bdrln2
    best = {None: (0.0, dict(table))}
    for pos, name in enumerate(chain):
        nxt = {}
        for lay in DOMAINS[name]:
            cand = (INF, None)
            for _, (cost_so_far, tab) in best.items():
                t2 = dict(tab)
                t2[name] = lay
                c = cost_so_far + op_cost(fwd_ops[pos], t2, tables)      # the group producing this tensor
                if c < cand[0]:
                    cand = (c, t2)
            if cand[1] is not None:
                nxt[lay] = cand
        if not nxt or all(v[0] == INF for v in nxt.values()):
            return table
        best = nxt
    final = min(best.values(), key=lambda v: v[0] + op_cost(fwd_ops[7], v[1], tables))
    return final[1] if final[0] < INF else table


def coordinate_descent(table, tables, max_rounds=20, min_gain=0.005):
    """A change must win at least `min_gain` of the total (0.5 %, about 3 us of a 0.6 ms step): the tables are
    medians of a few in-layer measurements that repeat to about one percent per group, and a difference inside
    that noise must not move a tensor."""
    table = dict(table)
    cur = total_cost(table, tables)
    for _ in range(max_rounds):
        improved = False
        for group in tie_groups():
            dom = DOMAINS[group[0]]
            if len(dom) < 2:
                continue
            keep = table[group[0]]
            best_lay, best_cost = keep, cur
            for lay in dom:
                if lay == keep:
                    continue
                for n in group:
                    table[n] = lay
                c = total_cost(table, tables)
                if c < best_cost - min_gain * cur:
                    best_lay, best_cost = lay, c
            for n in group:
                table[n] = best_lay
            if best_lay != keep:
                cur, improved = best_cost, True
        if not improved:
            break
    return table, cur


def to_configuration(table):
    """Reference schema: input, output, params, forward_interm, backward_interm, special_dims, algorithms."""
    return {
        'input': ('X', table['X']), 'output': ('SB2', table['SB2']),
        'params': [(n, table[n]) for n in L.PARAMS],
        'forward_interm': [(n, table[n]) for n in L.FORWARD_INTERM],
        'backward_interm': [(n, table[n]) for n in L.BACKWARD_INTERM],
        'special_dims': {}, 'algorithms': {},
    }


def optimize(results_dir, start=None):
    tables = load_tables(results_dir)
    start = dict(start or L.validate(L.uniform_layouts()))
    base_cost = total_cost(start, tables)
    table = forward_chain_shortest_path(start, tables)
    if total_cost(table, tables) > base_cost:
        table = start
    table, cost = coordinate_descent(table, tables)
    L.validate(to_configuration(table))
    report = {'start_cost_s': base_cost, 'chosen_cost_s': cost,
              'changed': {n: (start[n], table[n]) for n in table if table[n] != start[n]},
              'per_op_s': {op['name']: op_cost(op, table, tables) for op in OPS}}
    return to_configuration(table), report


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('results_dir')
    ap.add_argument('--output_config', required=True)
    ap.add_argument('--report')
    a = ap.parse_args()
    cfg, report = optimize(a.results_dir)
    if a.output_config.endswith('.json'):
        with open(a.output_config, 'w') as f:
            json.dump(cfg, f, indent=1)
    else:
        with open(a.output_config, 'wb') as f:
            pickle.dump(cfg, f)
    if a.report:
        with open(a.report, 'w') as f:
            json.dump(report, f, indent=1)
    print(json.dumps(report['changed'], indent=1))
    print('sum of operator times: %.1f us -> %.1f us' % (1e6 * report['start_cost_s'], 1e6 * report['chosen_cost_s']))


if __name__ == '__main__':
    main()
