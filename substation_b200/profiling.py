"""Turn Nsight Compute output into the short text summaries kept under ``profiles/``.

    # launch list: every kernel of a step with its device time (one pass, cheap on the full workload)
    ncu --metrics gpu__time_duration.sum --clock-control none -s <skip> -c <count> --csv --log-file launches.csv <cmd>
    python -m substation_b200.profiling launches launches.csv > profiles/<name>.md

    # full capture of one kernel (small case, one to three launches), exported as raw CSV
    ncu --set full --clock-control none -k regex:<kernel> -s 3 -c 3 -o prof <cmd>
    ncu -i prof.ncu-rep --page raw --csv > prof.csv
    python -m substation_b200.profiling kernel prof.csv
    python -m substation_b200.profiling traffic OPERATOR=prof.csv[:launch] ... > profiles/dram_traffic_<shape>.md

``traffic`` writes the table bench.py reads its ``roofline.traffic`` from (DRAM bytes read + written per launch).
The reference profiles with nvprof / cudaProfilerStart around whole kernels (pytorch_module/encoder.cu:32-53,
pycudaprof/); this is its counterpart for Nsight Compute reports.
"""

import csv
import sys

_SCALE = {'byte': 1.0, 'Kbyte': 1e3, 'Mbyte': 1e6, 'Gbyte': 1e9, 'ns': 1e-3, 'us': 1.0, 'ms': 1e3, 's': 1e6}

KERNEL_METRICS = (
    ('gpu__time_duration.sum', 'duration_us'),
    ('dram__bytes_read.sum', 'dram_read_bytes'),
    ('dram__bytes_write.sum', 'dram_write_bytes'),
    ('gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed', 'dram_pct'),
    ('sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active', 'tensor_pipe_pct'),
    ('sm__issue_active.avg.pct_of_peak_sustained_elapsed', 'issue_active_pct'),
    ('lts__t_sector_hit_rate.pct', 'l2_hit_pct'),
    ('launch__registers_per_thread', 'registers'),
    ('launch__grid_size', 'grid'),
    ('launch__shared_mem_per_block_dynamic', 'dyn_smem_bytes'),
)


def short_name(kernel):
    """'void unnamed>::lnbwd_ring_kernel<1>(...)' -> 'lnbwd_ring_kernel<1>'."""
    k = kernel.split('(')[0].replace('void ', '')
    return k.split('::')[-1].strip()


def read_launch_list(path):
    """[(kernel, microseconds)] from ``ncu --metrics gpu__time_duration.sum --csv`` (lines before the CSV header,
    which the profiler prints for its own messages, are skipped)."""
    with open(path) as f:
        lines = [l for l in f if l.startswith('"')]
    out = []
    for row in csv.DictReader(lines):
        if row.get('Metric Name') != 'gpu__time_duration.sum':
            continue
        scale = {'ns': 1e-3, 'us': 1.0, 'ms': 1e3}.get(row['Metric Unit'], 1.0)
        out.append((short_name(row['Kernel Name']), float(row['Metric Value'].replace(',', '')) * scale))
    return out


def summarise_launch_list(path):
    """Markdown table: per kernel its launches, total time and share of the captured launches."""
    rows = read_launch_list(path)
    total = sum(us for _, us in rows) or 1.0
    agg = {}
    for name, us in rows:
        n, t = agg.get(name, (0, 0.0))
        agg[name] = (n + 1, t + us)
    lines = ['| kernel | launches | total us | mean us | share |', '|---|---:|---:|---:|---:|']
    for name, (n, t) in sorted(agg.items(), key=lambda kv: -kv[1][1]):
        lines.append(f'| {name} | {n} | {t:.1f} | {t / n:.1f} | {100 * t / total:.1f}% |')
    lines.append(f'| all {len(rows)} launches | | {total:.1f} | | 100% |')
    return '\n'.join(lines)


def read_raw_csv(path):
    """[{metric: value in base units}] per captured launch from ``ncu --page raw --csv`` (row 0: metric names,
    row 1: units)."""
    with open(path) as f:
        rows = [r for r in csv.reader(f) if r]
    start = next(i for i, r in enumerate(rows) if 'Kernel Name' in r)
    hdr, units = rows[start], rows[start + 1]
    out = []
    for r in rows[start + 2:]:
        d = {'kernel': short_name(r[hdr.index('Kernel Name')])}
        for metric, key in KERNEL_METRICS:
            if metric in hdr:
                i = hdr.index(metric)
                try:
                    d[key] = float(r[i].replace(',', '')) * _SCALE.get(units[i], 1.0)
                except ValueError:
                    pass
        out.append(d)
    return out


def summarise_kernel(path):
    lines = ['| kernel | duration us | dram read MB | dram write MB | dram % | tensor pipe % | issue active % | L2 hit % | regs | grid |',
             '|---|---:|---:|---:|---:|---:|---:|---:|---:|---:|']
    for d in read_raw_csv(path):
        g = lambda k, f='{:.1f}': f.format(d[k]) if k in d else '-'
        lines.append(f"| {d['kernel']} | {g('duration_us')} | {d.get('dram_read_bytes', 0) / 1e6:.1f} | "
                     f"{d.get('dram_write_bytes', 0) / 1e6:.1f} | {g('dram_pct')} | {g('tensor_pipe_pct')} | "
                     f"{g('issue_active_pct')} | {g('l2_hit_pct')} | {g('registers', '{:.0f}')} | {g('grid', '{:.0f}')} |")
    return '\n'.join(lines)


def traffic_table(specs, stores='live'):
    """``specs``: ['OPERATOR=file.csv[:launch index]', ...] -> the '| operator | bytes | stores |' table."""
    lines = ['| operator | dram bytes per launch (read + write) | stores |', '|---|---:|---|']
    for spec in specs:
        op, src = spec.split('=', 1)
        path, _, idx = src.partition(':')
        launches = read_raw_csv(path)
        d = launches[int(idx) if idx else 0]
        lines.append(f"| {op} | {d.get('dram_read_bytes', 0) + d.get('dram_write_bytes', 0):.0f} | {stores} |")
    return '\n'.join(lines)


def main(argv):
    if len(argv) < 3 or argv[1] not in ('launches', 'kernel', 'traffic'):
        sys.exit(__doc__)
    if argv[1] == 'launches':
        print(summarise_launch_list(argv[2]))
    elif argv[1] == 'kernel':
        for p in argv[2:]:
            print(summarise_kernel(p))
    else:
        stores = 'live'
        specs = []
        for a in argv[2:]:
            if a.startswith('--stores='):
                stores = a.split('=', 1)[1]
            else:
                specs.append(a)
        print(traffic_table(specs, stores))


if __name__ == '__main__':
    main(sys.argv)
