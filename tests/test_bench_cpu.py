"""CPU checks of the measurement code: the reference arm's JSON line (the numpy port timed on the host, the way
pytorch_module/run_encoder.py:345-383 times one layer), the DRAM-traffic table the bench reads, the byte and FLOP
models, and the profiler-output summarisers."""

import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import bench  # noqa: E402
from substation_b200 import profiling  # noqa: E402


def test_reference_arm_prints_the_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, 'bench.py'), '--impl', 'reference', '--steps', '1',
                          '--warmup', '0', '--batch', '1', '--seq', '64'], capture_output=True, text=True, timeout=600,
                         cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line['impl'] == 'reference' and line['metric'] == bench.METRIC and line['unit'] == bench.UNIT
    assert line['higher_is_better'] is True and line['n_gpus'] == 1 and line['steps'] == 1 and line['warmup'] == 0
    assert line['value'] > 0 and line['ms_per_step'] > 0 and line['gpu_launches'] == 0
    assert line['cpu_baseline']['kind'] == 'port' and line['cpu_baseline']['cores'] >= 1
    assert line['cpu_baseline']['value'] == line['value'] == line['e2e']['value']
    assert line['e2e']['h2d_bytes_per_step'] == 0 and line['e2e']['d2h_bytes_per_step'] == 0
    assert 'workload' in line['config'] and 'model' not in line['config']


def test_reference_arm_is_silent_on_other_ranks():
    env = dict(os.environ, RANK='1')
    out = subprocess.run([sys.executable, os.path.join(ROOT, 'bench.py'), '--impl', 'reference', '--steps', '1',
                          '--warmup', '0', '--batch', '1', '--seq', '64', '--gpus', '2'], capture_output=True, text=True,
                         timeout=600, cwd=ROOT, env=env)
    assert out.returncode == 0 and out.stdout.strip() == ''


def test_dram_traffic_table_is_read_per_store_setting():
    live = bench.load_dram_traffic(8, 512, keep_all=False)
    kept = bench.load_dram_traffic(8, 512, keep_all=True)
    for name in ('QKT+softmax', 'dX1gamma+bs'):
        assert 5e7 < live[name] < kept[name] < 4e8        # skipping a score tensor's store shows in DRAM bytes
    assert bench.load_dram_traffic(96, 128, keep_all=False) == {}


def test_byte_and_flop_models():
    B, L = 8, 512
    T, S = B * L, bench.H * B * L * L
    assert bench.GEMM_FLOPS['lin1'](B, L) == 2 * T * bench.E * bench.U
    assert bench.FUSED_BYTES['bdrln1'](B, L) == 13 * T * bench.E and bench.FUSED_BYTES_SKIP['bdrln1'](B, L) == 11 * T * bench.E
    assert bench.FUSED_BYTES['QKT+softmax'](B, L) - bench.FUSED_BYTES_SKIP['QKT+softmax'](B, L) == 2 * S
    assert set(bench.GEMM_SHAPES) == {n.split('+')[0] for n in bench.GEMM_FLOPS if n.split('+')[0] in bench.GEMM_SHAPES}
    M, N, K = bench.GEMM_SHAPES['dWout'](T)
    assert (M, N, K) == (bench.E, bench.E, T)


def test_profiler_summaries(tmp_path):
    csv_path = tmp_path / 'launches.csv'
    csv_path.write_text(
        '==PROF== some message\n'
        '"ID","Process ID","Process Name","Host Name","Kernel Name","Context","Stream","Block Size","Grid Size",'
        '"Device","CC","Section Name","Metric Name","Metric Unit","Metric Value"\n'
        '"0","1","python","h","void sb::<unnamed>::bdrln_ring_kernel<4>(sb::BdrlnParams, int, int)","1","7","(544, 1, 1)",'
        '"(148, 1, 1)","0","10.0","Command line profiler metrics","gpu__time_duration.sum","us","14.0"\n'
        '"1","1","python","h","void sb::<unnamed>::bdrln_ring_kernel<4>(sb::BdrlnParams, int, int)","1","7","(544, 1, 1)",'
        '"(148, 1, 1)","0","10.0","Command line profiler metrics","gpu__time_duration.sum","ns","16000"\n'
        '"2","1","python","h","void pair::gemm_tc_pair_kernel<0, 8>(CUtensorMap_st)","1","7","(320, 1, 1)",'
        '"(148, 1, 1)","0","10.0","Command line profiler metrics","gpu__time_duration.sum","us","30.0"\n')
    rows = profiling.read_launch_list(str(csv_path))
    assert [n for n, _ in rows] == ['bdrln_ring_kernel<4>', 'bdrln_ring_kernel<4>', 'gemm_tc_pair_kernel<0, 8>']
    assert [round(us, 3) for _, us in rows] == [14.0, 16.0, 30.0]
    table = profiling.summarise_launch_list(str(csv_path))
    assert '| gemm_tc_pair_kernel<0, 8> | 1 | 30.0 | 30.0 | 50.0% |' in table
    assert '| bdrln_ring_kernel<4> | 2 | 30.0 | 15.0 | 50.0% |' in table

    raw = tmp_path / 'raw.csv'
    raw.write_text(
        '"ID","Kernel Name","gpu__time_duration.sum","dram__bytes_read.sum","dram__bytes_write.sum","launch__grid_size"\n'
        '"","","us","Mbyte","Mbyte",""\n'
        '"0","void attn::attn_scores_kernel<1>(CUtensorMap_st)","45.0","117.5","25.9","148"\n')
    rec = profiling.read_raw_csv(str(raw))[0]
    assert rec['kernel'] == 'attn_scores_kernel<1>' and rec['duration_us'] == 45.0
    assert rec['dram_read_bytes'] == pytest.approx(117.5e6) and rec['grid'] == 148
    assert '| dX1gamma+bs | 143400000 | live |' in profiling.traffic_table([f'dX1gamma+bs={raw}:0'])
