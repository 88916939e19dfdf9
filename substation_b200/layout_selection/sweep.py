"""Measure the layer's operator groups under candidate layouts, on the GPU, and keep the tables the layout
optimizer reads.

    python -m substation_b200.layout_selection.sweep --out DIR [--batch 8 --seq 512] [--around CONFIG.json]
                                                     [--rounds 3] [--tag b8_l512]

What is timed is what runs: for every candidate configuration an ``Encoder`` is built with those layouts and
one forward+backward step is run a few times with the library's per-operator CUDA events on, inside the real
operator sequence (inputs as the previous operator left them in the caches, fused operators where the layouts
allow them, their separate replacements where they decline).  A group's time is the sum over the operators the
layer reported for it.  The reference instead benchmarks every kernel and every cuBLAS call in isolation
(pytorch_module/benchmark.py:1328-1359, tc_profiling/einsum_perms.py:397-470); its table formats are kept:
  * groups that are one contraction: ``<group>-result.csv`` with columns A,B,C,M,N,K,batch,Time,Implementation
    (subset of config_selection/parse_tc_results.py:15-18,38-62; cuBLAS-only columns have no meaning here);
  * all other groups: ``<group>-combined.csv``, one line per configuration,
    ``NAME = layout ... time = t s`` (pytorch_module/benchmark.py:1440-1444, config_selection/load_data.py:11-41).
Candidates: the configuration given with ``--around`` (default: every tensor in its logical order) and every
configuration that differs from it in ONE tensor (or one group of tied tensors), over every permutation of that
tensor's dims.  Tables are appended to, never rewritten: a configuration whose groups are all present is skipped,
so an interrupted sweep resumes and a later sweep around another configuration adds to the same files
(the reference: ``--resume``, pytorch_module/benchmark.py:1388-1399).  With ``--rounds N`` the optimizer runs after
each sweep and the next sweep goes around what it chose, until nothing changes.
"""

import argparse
import json
import os
import statistics

from .. import layouts as L
from .spec import DOMAINS, OPS, default_table, op_key, tie_groups

H = 16


def table_path(out_dir, op):
    return os.path.join(out_dir, f"{op['name']}-{'result' if op['kind'] == 'gemm' else 'combined'}.csv")


def load_keys(out_dir):
    """{group name: set of layout keys already measured}."""
    from .optimize import load_tables
    return {name: set(t) for name, t in load_tables(out_dir).items()}


def _extents(dims, sizes):
    n = 1
    for c in dims:
        n *= sizes[c]
    return n


def append_rows(out_dir, table, times, sizes, have):
    """Append one line per group whose key is new; ``times``: {group name: seconds}."""
    os.makedirs(out_dir, exist_ok=True)
    for op in OPS:
        key = op_key(op, table)
        if key in have.setdefault(op['name'], set()) or op['name'] not in times:
            continue
        path = table_path(out_dir, op)
        new = not os.path.exists(path)
        with open(path, 'a') as f:
            if op['kind'] == 'gemm':
                if new:
                    f.write('A,B,C,M,N,K,batch,Time,Implementation\n')
                a, b, c = (L.LOGICAL[t] for t in op['tensors'])
                batch = [x for x in a if x in b and x in c]
                ks = [x for x in a if x in b and x not in c]
                ms = [x for x in a if x not in b]
                ns = [x for x in b if x not in a]
                f.write(f'{key[0]},{key[1]},{key[2]},{_extents(ms, sizes)},{_extents(ns, sizes)},{_extents(ks, sizes)},'
                        f'{_extents(batch, sizes)},{times[op["name"]]:.9f},layer\n')
            else:
                f.write(' '.join(f'{n} = {l}' for n, l in zip(op['tensors'], key)) + f' time = {times[op["name"]]:.9f} s\n')
        have[op['name']].add(key)


def candidates(base):
    """The base table and every single-tensor (tie-group) deviation from it."""
    yield dict(base)
    for group in tie_groups():
        for lay in DOMAINS[group[0]]:
            if lay == base[group[0]]:
                continue
            t = dict(base)
            for n in group:
                t[n] = lay
            yield t


def measure_layer(table, batch, seq, heads=H, embed=1024, reps=5, warmup=2, device='cuda'):
    """{group name: seconds} for one configuration: median over ``reps`` steps of the per-operator event times."""
    import torch
    from ..encoder import Encoder
    from .optimize import to_configuration
    from .spec import GROUP_OF
    cfg = to_configuration(table)
    dev = torch.device(device)
    enc = Encoder('', batch, seq, heads, embed, cfg, torch.float16, 0.1, 0.1, 0.1, 0.1, profiling=True,
                  mask_mode='explicit').to(dev)
    gen = torch.Generator(device=dev).manual_seed(0)
    with torch.no_grad():
        for prm in enc.params:
            prm.copy_((torch.randn(prm.shape, device=dev, generator=gen) * 0.02).half())
    shape_x = L.shape_of(table['X'], enc.sizes)
    X = torch.randn(shape_x, device=dev, generator=gen).half()
    DY = torch.randn(shape_x, device=dev, generator=gen).half()
    masks = {n: (torch.rand(L.shape_of(table[n], enc.sizes), device=dev, generator=gen) >= 0.1).to(torch.uint8)
             for n in L.MASKS}
    enc.set_masks(masks)
    weights = [p.detach() for p in enc.params]
    fwd = enc._alloc(enc._fwd_plan, dev)
    fwd.update(masks)
    bwd = enc._alloc(enc._bwd_plan, dev)
    grads = enc._alloc(enc._grad_plan, dev)
    Y, DX = torch.empty_like(X), torch.empty_like(X)
    per = {}
    for i in range(warmup + reps):
        enc.forward_raw(X, weights, fwd, Y)
        enc.backward_raw(DY, grads, bwd, weights, fwd, X, DX)
        torch.cuda.synchronize(dev)
        times = enc.op_times()
        if i >= warmup:
            step = {}
            for name, ms in times:
                g = GROUP_OF.get(name)
                if g is not None:
                    step[g] = step.get(g, 0.0) + ms * 1e-3
            for g, s in step.items():
                per.setdefault(g, []).append(s)
    enc._destroy()
    del enc, fwd, bwd, grads
    torch.cuda.empty_cache()
    return {g: statistics.median(v) for g, v in per.items()}


def sweep(out_dir, batch, seq, heads=H, embed=1024, around=None, measure=None, limit=None, verbose=True):
    """Measure every candidate around ``around`` whose groups are not all in the tables yet; returns how many
    configurations were run."""
    base = dict(around or default_table())
    sizes = L.sizes_map(batch, seq, heads, embed)
    have = load_keys(out_dir) if os.path.isdir(out_dir) else {}
    measure = measure or (lambda t: measure_layer(t, batch, seq, heads, embed))
    done = 0
    for table in candidates(base):
        if all(op_key(op, table) in have.get(op['name'], ()) for op in OPS):
            continue
        if limit is not None and done >= limit:
            break
        try:
            times = measure(table)
        except Exception as exc:        # a layout the layer refuses outright: nothing to record
            if verbose:
                print('skipped', {n: table[n] for n in table if table[n] != base[n]}, '-', exc, flush=True)
            continue
        append_rows(out_dir, table, times, sizes, have)
        done += 1
        if verbose and done % 25 == 0:
            print(done, 'configurations measured', flush=True)
    return done


def main():
    from . import optimize as opt
    ap = argparse.ArgumentParser()
    ap.add_argument('--out', required=True, help='directory of the tables (appended to)')
    ap.add_argument('--batch', type=int, default=8)
    ap.add_argument('--seq', type=int, default=512)
    ap.add_argument('--around', help='configuration (.json) to sweep around; default: all tensors in logical order')
    ap.add_argument('--rounds', type=int, default=1, help='sweep, optimize, sweep around the result, ...')
    ap.add_argument('--tag', help='write the chosen configuration and report into the package as results_<tag>/')
    ap.add_argument('--limit', type=int, help='at most this many configurations per sweep')
    a = ap.parse_args()
    table = L.validate(L.read_json(a.around)) if a.around else default_table()
    cfg = report = None
    for r in range(max(1, a.rounds)):
        n = sweep(a.out, a.batch, a.seq, around=table, limit=a.limit)
        cfg, report = opt.optimize(a.out, start=table)
        new = L.validate(cfg)
        print(f'round {r}: {n} configurations measured; sum of groups {1e6 * report["start_cost_s"]:.1f} us -> '
              f'{1e6 * report["chosen_cost_s"]:.1f} us; changed: {report["changed"]}', flush=True)
        if new == table:
            break
        table = new
    if a.tag:
        d = os.path.join(os.path.dirname(os.path.abspath(__file__)), f'results_{a.tag}')
        os.makedirs(d, exist_ok=True)
        with open(os.path.join(d, f'layouts_b200_{a.tag}.json'), 'w') as f:
            json.dump(cfg, f, indent=1)
        with open(os.path.join(d, 'report.json'), 'w') as f:
            json.dump(report, f, indent=1)


if __name__ == '__main__':
    main()
