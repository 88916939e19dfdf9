"""Benchmark of the encoder-layer hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--layouts b200_b8_l512|uniform|b8_l512|b96_l128|<file.json>] [--batch B] [--seq L]
    python bench.py --kernels        every fused operator alone at the kernel-sweep shapes, one JSON line
    python bench.py --layers 24      the 24-layer stack, one JSON line

One "step" = one BERT-large encoder layer forward+backward (B=8, L=512, H=16,
E=1024, fp16 storage / fp32 accumulation, dropout p=0.1 with seeded explicit
masks) on each GPU; with N>1 every rank runs its own batch of 8 (weak scaling)
and the layer's 12 parameter gradients are sum-allreduced over NCCL, overlapped
with the next step.  Rank 0 prints ONE JSON line.

value        sequences/s over all ranks, inputs resident in HBM, CUDA-event timed
e2e          same through the public ``Encoder`` module with host buffers:
             pinned-host X and dY copied in, Y and dX copied out, every step;
             copy_only_ms_per_step = the same copies with no compute
sustained    the same step repeated for at least two seconds, with the SM clock
             sampled while it runs (ms x MHz is the clock-normalised figure)
roofline     the operator with the largest device time: algorithmic bytes (or
             FLOPs) / its mean duration, against MEASURED_PEAKS.json
operators    every operator of the step: device time, GB/s or TFLOP/s, and for the
             large contractions the time torch.matmul (cuBLAS) takes for the same
             shape on this GPU (measured outside the timed region, never on the
             product path)
fused_kernels  each fused operator alone at H=16, B=96, J=K=128 (kernel sweep)
cpu_baseline the numpy port of the reference path (oracle/) timed on the host
N>1 only     dp_check (summed gradients against the sum of the gathered per-rank
             gradients and against one GPU on the concatenated batch), strong
             (global batch 96 at L=128 split over the ranks), stack (24 layers)
--impl reference  the numpy port as its own arm (rank 0 only)
"""

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

H, E = 16, 1024
P, U = E // H, 4 * E
P_DROP = 0.1
METRIC = 'bert_large_encoder_layer_fwd_bwd_sequences_per_s'
UNIT = 'seq/s'
FALLBACK_PEAKS = {'hbm_gbs': 6650.0, 'bf16_tflops': 1590.0, 'bf16_tflops_sustained': 1400.0}
NOMINAL_HBM_GBS = 8000.0

# contraction name -> FLOPs as a function of (B, L): 2*batch*M*N*K of the 18 einsums
GEMM_FLOPS = {
    'QKV-fused': lambda B, L: 2 * 3 * E * E * B * L, 'out': lambda B, L: 2 * E * E * B * L,
    'lin1': lambda B, L: 2 * E * U * B * L, 'lin2': lambda B, L: 2 * E * U * B * L,
    'dXlin2': lambda B, L: 2 * E * U * B * L, 'dWlin2': lambda B, L: 2 * E * U * B * L,
    'dXlin1': lambda B, L: 2 * E * U * B * L, 'dWlin1': lambda B, L: 2 * E * U * B * L,
    'dWout': lambda B, L: 2 * E * E * B * L, 'dXout': lambda B, L: 2 * E * E * B * L,
    'dXQKV-fused': lambda B, L: 2 * 3 * E * E * B * L, 'dWQKV-fused': lambda B, L: 2 * 3 * E * E * B * L,
}
GEMM_FLOPS['QKV-fused+aib'] = GEMM_FLOPS['QKV-fused']
GEMM_FLOPS['lin1+bad'] = GEMM_FLOPS['lin1']
GEMM_FLOPS['dXQKV-fused+bei'] = GEMM_FLOPS['dXQKV-fused']
for _n in ('QKT', 'gamma', 'dX1gamma', 'dX2gamma', 'dX1QKT', 'dX2QKT'):
    GEMM_FLOPS[_n] = lambda B, L: 2 * H * B * L * L * P
# (M, N, K) of the twelve large contractions as functions of the token count T
GEMM_SHAPES = {
    'QKV-fused': lambda T: (T, 3 * E, E), 'out': lambda T: (T, E, E), 'lin1': lambda T: (T, U, E),
    'lin2': lambda T: (T, E, U), 'dXlin2': lambda T: (T, U, E), 'dWlin2': lambda T: (U, E, T),
    'dXlin1': lambda T: (T, E, U), 'dWlin1': lambda T: (E, U, T), 'dWout': lambda T: (E, E, T),
    'dXout': lambda T: (T, E, E), 'dXQKV-fused': lambda T: (T, E, 3 * E), 'dWQKV-fused': lambda T: (3 * E, E, T),
}
# attention contractions are HBM-bound: minimum operand bytes (two [P,L] operands + one [L,L], or v.v.)
ATTN_BYTES = {n: (lambda B, L: 2 * H * B * (2 * P * L + L * L))
              for n in ('QKT', 'gamma', 'dX1gamma', 'dX2gamma', 'dX1QKT', 'dX2QKT')}
# fused operators: algorithmic bytes, every input read once + every output written once,
# 2 B per fp16 element, 1 B per mask element (T = B*L tokens, S = H*B*L*L scores)
FUSED_BYTES = {
    'aib': lambda B, L: 12 * B * L * E, 'softmax': lambda B, L: 7 * H * B * L * L,
    'bdrln1': lambda B, L: 13 * B * L * E, 'bdrln2': lambda B, L: 13 * B * L * E,
    'bad': lambda B, L: 7 * B * L * U, 'bsb': lambda B, L: 6 * B * L * E,
    'blnrd1': lambda B, L: 9 * B * L * E, 'blnrd2': lambda B, L: 9 * B * L * E,
    'bdrlb': lambda B, L: 7 * B * L * U, 'ebsb': lambda B, L: 10 * B * L * E,
    'baob': lambda B, L: 2 * B * L * E, 'bs': lambda B, L: 7 * H * B * L * L,
    'baib': lambda B, L: 6 * B * L * E, 'bei': lambda B, L: 6 * B * L * E,
    # fused LayerNorm-backward passes: inputs once, outputs once
    'bsb+blnrd1': lambda B, L: 13 * B * L * E, 'ebsb+blnrd2+baob': lambda B, L: 17 * B * L * E,
    # fused attention scores: projections in, mask in, BETA/ALPHA/ATTN_DROP (resp. ALPHA in, DATTN_DROP/DBETA) out
    'dX1QKT+dX2QKT': lambda B, L: H * B * (2 * L * L + 8 * P * L),
    'QKT+softmax': lambda B, L: H * B * (4 * P * L + 7 * L * L), 'dX1gamma+bs': lambda B, L: H * B * (4 * P * L + 7 * L * L),
}
# the same operators when the intermediates nothing reads again are not stored (the default; --keep-all 1 stores them):
# LIN (2*T*E) in both bdrln calls, DLN (2*T*E) in both LayerNorm-backward passes, BETA / DATTN_DROP (2*S)
FUSED_BYTES_SKIP = dict(FUSED_BYTES)
FUSED_BYTES_SKIP.update({
    'bdrln1': lambda B, L: 11 * B * L * E, 'bdrln2': lambda B, L: 11 * B * L * E,
    'bsb+blnrd1': lambda B, L: 11 * B * L * E, 'ebsb+blnrd2+baob': lambda B, L: 15 * B * L * E,
    'QKT+softmax': lambda B, L: H * B * (4 * P * L + 5 * L * L), 'dX1gamma+bs': lambda B, L: H * B * (4 * P * L + 5 * L * L),
})


def load_peaks():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d, 'measured'
    return dict(FALLBACK_PEAKS), 'fallback'


def load_dram_traffic(B, S, keep_all):
    """DRAM bytes (read + write) per launch from the ncu captures summarised under profiles/: the table rows of
    profiles/dram_traffic_b8_l512.md, '| operator | bytes | stores |' (the file names the capture command that
    regenerates it).  Only known for the shapes and store setting that were captured."""
    if (B, S) != (8, 512):
        return {}
    path = os.path.join(ROOT, 'profiles', 'dram_traffic_b8_l512.md')
    out = {}
    try:
        with open(path) as f:
            for line in f:
                c = [x.strip() for x in line.strip().strip('|').split('|')]
                if len(c) >= 3 and c[2] in ('all', 'live'):
                    try:
                        nbytes = float(c[1])
                    except ValueError:
                        continue
                    if (c[2] == 'all') == bool(keep_all):
                        out[c[0]] = nbytes
    except OSError:
        pass
    return out


class ClockSampler:
    """nvidia-smi clock/throttle samples while the timed region runs."""
    Q = ('index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,'
         'clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
         'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')

    def __init__(self, gpu_index, interval_ms=100):
        self.proc, self.rows, self.idx, self.interval = None, [], gpu_index, interval_ms

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ['nvidia-smi', f'--query-gpu={self.Q}', '--format=csv,noheader,nounits', '-lms', str(self.interval),
                 '-i', str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self, skip_first=0):
        if self.proc is None:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['nvidia-smi unavailable']}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, smax, power, reasons = [], [], [], set()
        for line in out.strip().splitlines()[skip_first:]:
            c = [x.strip() for x in line.split(',')]
            if len(c) < 9:
                continue
            try:
                sm.append(float(c[1])); smax.append(float(c[2]))
            except ValueError:
                continue
            try:
                power.append(float(c[3]))
            except ValueError:
                pass
            for name, val in zip(('hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap'), c[5:9]):
                if val.lower().startswith('active'):
                    reasons.add(name)
        return {'sm_mhz': statistics.median(sm) if sm else None,
                'sm_max_mhz': max(smax) if smax else None, 'samples': len(sm),
                'power_w_max': max(power) if power else None, 'reasons': sorted(reasons)}


# ------------------------------------------------------------------------------------------
# CPU arm: numpy port of the reference path
# ------------------------------------------------------------------------------------------
def cpu_pass(batch, seq, seed=0):
    """One forward+backward of the numpy port on `batch` sequences; returns seconds."""
    import numpy as np
    from oracle import encoder_oracle as orc
    rng = np.random.default_rng(seed)
    params = orc.make_params(H, P, U, rng)
    X = rng.normal(0, 1, (batch, seq, E)).astype(np.float32)
    DY = rng.normal(0, 1, (batch, seq, E)).astype(np.float32)
    masks = orc.make_masks(batch, seq, H, E, U, (P_DROP,) * 4, seed)
    t0 = time.perf_counter()
    f = orc.encoder_forward(X, params, masks)
    orc.encoder_backward(X, DY, params, f)
    return time.perf_counter() - t0


def host_cores():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def run_reference_arm(args):
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return
    sample_b = 1
    for _ in range(args.warmup):
        cpu_pass(sample_b, args.seq)
    times = [cpu_pass(sample_b, args.seq, seed=i) for i in range(args.steps)]
    total = sum(times)
    value = sample_b * args.steps / total
    sample = (f'{sample_b} of the {args.batch} sequences (L={args.seq}) per step, numpy float64 port of '
              f'substation/transformer.py encoder+encoder_backward with four explicit dropout masks')
    line = {
        'impl': 'reference', 'metric': METRIC, 'value': value, 'unit': UNIT, 'n_gpus': args.gpus,
        'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': 1e3 * total / args.steps,
        'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'f64',
        'data': 'synthetic',
        'config': workload_config(args, 'numpy-port'),
        'cpu_baseline': {'value': value, 'unit': UNIT, 'cores': host_cores(), 'kind': 'port', 'sample': sample},
        'e2e': {'value': value, 'unit': UNIT, 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    }
    print(json.dumps(line))


def workload_config(args, layouts_name):
    return {'workload': f'BERT-large encoder layer fwd+bwd, B={args.batch} per GPU, L={args.seq}, H={H}, P={P}, '
                        f'E={E}, U={U}, ReLU, dropout p={P_DROP} (seeded explicit masks)',
            'batch_per_gpu': args.batch, 'seq_len': args.seq, 'layouts': layouts_name,
            'parallelism': f'dp{args.gpus}', 'comm_ctas': args.comm_ctas if args.gpus > 1 else 0,
            'intermediates': 'all stored' if args.keep_all else 'the nine tensors nothing reads again are not stored',
            'l2': 'per-step working set (~0.9 GB of intermediates) is larger than the 126 MB L2; no flush needed'}


def resolve_layouts(name):
    """--layouts value -> configuration dict.  'b8_l512' and 'b96_l128' are the reference's two shipped
    configurations, kept as JSON data files beside the golden vectors."""
    from substation_b200 import layouts as L
    if name in ('b8_l512', 'b96_l128'):
        name = os.path.join(ROOT, 'tests', 'golden', f'layouts_{name}.json')
    return L.named_layouts(name)


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
def dist_env(args):
    import torch
    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local_rank = int(os.environ.get('LOCAL_RANK', '0'))
    if world != args.gpus:
        raise SystemExit(f'--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run')
    if not torch.cuda.is_available():
        raise SystemExit('bench.py needs a CUDA device: the product path has no CPU fallback')
    torch.cuda.set_device(local_rank)
    return world, rank, local_rank, torch.device('cuda', local_rank)


def init_nccl(args, world, dev):
    """One process per GPU over NCCL.  Few NCCL CTAs are enough for a 25 MB bucket over NVLink; the persistent
    contraction kernels leave exactly those SMs free so that the allreduce runs beside them."""
    import torch
    import torch.distributed as dist
    if world == 1:
        return
    opts = None
    try:
        opts = dist.ProcessGroupNCCL.Options()
        opts.config.max_ctas = args.comm_ctas
        opts.config.min_ctas = min(4, args.comm_ctas)
    except Exception:
        opts = None
    dist.init_process_group('nccl', device_id=dev, pg_options=opts)
    from substation_b200 import ops as _ops
    _ops.set_sm_budget(torch.cuda.get_device_properties(dev).multi_processor_count - args.comm_ctas)


class LayerBench:
    """One encoder layer with preallocated buffers and seeded inputs: what a step runs on."""

    def __init__(self, B, S, lay, dev, rank, keep_all, weight_seed=1234, data_seed=100, heads=H, embed=E,
                 profiling=True, X=None, DY=None, masks=None):
        import torch
        from substation_b200 import Encoder, layouts as L
        self.B, self.S, self.dev = B, S, dev
        self.table = L.validate(lay)
        self.enc = Encoder('/tmp/substation_b200_unused', B, S, heads, embed, lay, torch.float16,
                           P_DROP, P_DROP, P_DROP, P_DROP, profiling=profiling, mask_mode='explicit',
                           keep_all_intermediates=bool(keep_all)).to(dev)
        enc = self.enc
        gen = torch.Generator(device=dev).manual_seed(weight_seed)        # same weights on every rank
        with torch.no_grad():
            for (name, layout), prm in zip(lay['params'], enc.params):
                if name in ('WKQV', 'WO', 'LINW1', 'LINW2'):
                    prm.copy_((torch.randn(prm.shape, device=dev, generator=gen) * 0.02).half())
                elif name in ('S1', 'S2'):
                    prm.fill_(1.0)
                else:
                    prm.zero_()
        gen = torch.Generator(device=dev).manual_seed(data_seed + rank)    # different data per rank
        shape_x = L.shape_of(self.table['X'], enc.sizes)
        self.X = torch.randn(shape_x, device=dev, generator=gen).half() if X is None else X
        self.DY = torch.randn(shape_x, device=dev, generator=gen).half() if DY is None else DY
        if masks is None:
            masks = {}
            for n in L.MASKS:
                shp = L.shape_of(self.table[n], enc.sizes)
                masks[n] = (torch.rand(shp, device=dev, generator=gen) >= P_DROP).to(torch.uint8)
        self.masks = masks
        enc.set_masks(masks)
        self.weights = [p.detach() for p in enc.params]
        self.fwd = enc._alloc(enc._fwd_plan, dev)
        self.fwd.update(masks)
        self.bwd = enc._alloc(enc._bwd_plan, dev)
        self.Y, self.DX = torch.empty_like(self.X), torch.empty_like(self.X)

    def run(self, grads):
        self.enc.forward_raw(self.X, self.weights, self.fwd, self.Y)
        self.enc.backward_raw(self.DY, grads, self.bwd, self.weights, self.fwd, self.X, self.DX)


def event_time_ms(fn, n, torch):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(n):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1)


def graph_time_ms(fn, n, torch):
    """The same n calls captured once into a CUDA graph and replayed: the device time of back-to-back launches,
    whatever the host needs to issue one (a Python call with a dozen tensor arguments costs 20-60 us, more than
    the shorter operators run).  None when the calls cannot be captured; the caller then times them eagerly."""
    try:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(n):
                fn(i)
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        del g
        return ms
    except Exception as exc:  # capture refused (an operator that synchronises or allocates): eager timing instead
        sys.stderr.write(f'kernel sweep: graph capture not possible ({type(exc).__name__}: {exc}); timing eagerly\n')
        torch.cuda.synchronize()
        return None


def cublas_anchors(T, dev, torch, reps=100, nset=4):
    """The twelve large contractions at the layer's shapes, alone: this library's kernel (with the epilogue the layer
    fuses into it) and torch.matmul (cuBLAS), both operands K-major, rotating operand sets so that every launch
    starts cold in L2, the `reps` launches replayed as one CUDA graph between two events (no host in the loop, no
    event between launches).  name -> (this kernel us, cuBLAS us).  A yardstick only: never on the product path."""
    from substation_b200 import ops
    g = torch.Generator(device=dev).manual_seed(3)
    rnd = lambda *s, std=1.0: (torch.randn(*s, device=dev, generator=g) * std).half()
    out = {}
    for name, shape in GEMM_SHAPES.items():
        M, N, K = shape(T)
        As = [rnd(1, M, K, std=K ** -0.5) for _ in range(nset)]
        Bs = [rnd(1, N, K) for _ in range(nset)]
        Cs = [torch.empty(1, M, N, device=dev, dtype=torch.float16) for _ in range(nset)]
        if name == 'QKV-fused':      # + bias, C itself not stored
            O2 = [torch.empty_like(c) for c in Cs]
            bias = rnd(N, std=0.02)
            ours = lambda i: ops.einsum_fused('bmk,bnk->bmn', As[i % nset], Bs[i % nset], Cs[i % nset], kind='bias',
                                              out2=O2[i % nset], bias=bias, bias_dims='n', discard_c=True)
        elif name == 'dXQKV-fused':  # + residual, C itself not stored
            O2 = [torch.empty_like(c) for c in Cs]
            R = [rnd(1, M, N) for _ in range(nset)]
            ours = lambda i: ops.einsum_fused('bmk,bnk->bmn', As[i % nset], Bs[i % nset], Cs[i % nset], kind='residual',
                                              out2=O2[i % nset], resid=R[i % nset], discard_c=True)
        elif name == 'lin1':         # + bias, activation, dropout: two outputs, C itself not stored
            O2 = [torch.empty_like(c) for c in Cs]
            O3 = [torch.empty_like(c) for c in Cs]
            bias = rnd(N, std=0.02)
            mask = [(torch.rand(1, M, N, device=dev, generator=g) >= P_DROP).to(torch.uint8) for _ in range(nset)]
            ours = lambda i: ops.einsum_fused('bmk,bnk->bmn', As[i % nset], Bs[i % nset], Cs[i % nset],
                                              kind='bias_act_dropout', out2=O2[i % nset], out3=O3[i % nset], bias=bias,
                                              bias_dims='n', mask=mask[i % nset], p=P_DROP, discard_c=True)
        else:
            ours = lambda i: ops.einsum('bmk,bnk->bmn', As[i % nset], Bs[i % nset], Cs[i % nset], impl='tcgen05')
        lib = lambda i: torch.matmul(As[i % nset][0], Bs[i % nset][0].t(), out=Cs[i % nset][0])
        res = []
        for f in (ours, lib):
            for i in range(nset + 2):
                f(i)
            torch.cuda.synchronize()
            ms = graph_time_ms(f, reps, torch)
            if ms is None:
                ms = event_time_ms(f, reps, torch)
            res.append(1e3 * ms / reps)
        out[name] = tuple(res)
        del As, Bs, Cs
    torch.cuda.empty_cache()
    return out


def tensor_peak_probe(torch):
    """fp16 tcgen05 rate with operands resident in shared memory (no loads, no epilogue): a short burst and a
    ~50 ms run (the power cap pulls the clock down within a few milliseconds of dense MMA work)."""
    from substation_b200 import ops
    res = {}
    for label, kb in (('burst', 4096), ('long', 200000)):
        ops.mma_peak_probe(64)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fl = ops.mma_peak_probe(kb)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        res[label] = {'tflops': round(fl / ms / 1e9, 1), 'ms': round(ms, 3)}
    if ops.device_error() != 0:
        res['error'] = 'a bounded wait ran out'
        ops.device_error_reset()
    return res


# ---- kernel sweep: every fused operator alone -------------------------------------------------------
def fused_kernel_sweep(dev, torch, warmup=20, reps=200, Hh=16, B=96, L=128, nset=2):
    """Each fused operator and its backward counterpart alone at H=16, B=96, J=K=128, E=1024, U=4096: scores
    ~ N(0,4) with scale 1/8 and dropout p=0.1, bdrln over [B,J,E] with bias ~ N(0,0.02) and residual ~ N(0,1),
    bad over [B,J,U], gradients ~ N(0,1), saved tensors from the matching forward.  20 + 200 launches over
    rotating buffer sets (a set is 50-350 MB, above the 126 MB L2), the 200 replayed as one CUDA graph between two
    CUDA events so that the host's issue rate does not enter, GB/s = algorithmic bytes / time.
    Mirrors the reference's per-kernel harness (pytorch_module/benchmark.py:375-393, :1475-1493)."""
    from substation_b200 import ops
    peaks, _ = load_peaks()
    hbm = float(peaks['hbm_gbs'])
    g = torch.Generator(device=dev).manual_seed(7)
    Pp = E // Hh
    rnd = lambda *s, std=1.0: (torch.randn(*s, device=dev, generator=g) * std).half()
    empty = lambda *s: torch.empty(*s, device=dev, dtype=torch.float16)
    keep = lambda *s: (torch.rand(*s, device=dev, generator=g) >= P_DROP).to(torch.uint8)
    results = {}

    def timed(name, nbytes, calls):
        for i in range(warmup):
            calls[i % len(calls)]()
        torch.cuda.synchronize()
        ms = graph_time_ms(lambda i: calls[i % len(calls)](), reps, torch)
        how = 'graph replay'
        if ms is None:
            ms, how = event_time_ms(lambda i: calls[i % len(calls)](), reps, torch), 'eager'
        us = 1e3 * ms / reps
        results[name] = {'us': round(us, 2), 'launch': how, 'gbs': round(nbytes / us / 1e3, 1),
                         'frac_of_measured_copy': round(nbytes / us / 1e3 / hbm, 3),
                         'frac_of_8tbs': round(nbytes / us / 1e3 / NOMINAL_HBM_GBS, 3)}

    S4, T3, TU = (Hh, B, L, L), (B, L, E), (B, L, U)
    ns, nt, nu = Hh * B * L * L, B * L * E, B * L * U
    # ---- softmax + dropout, and its backward (separate operators and the fused attention-score forms)
    sets = []
    for _ in range(nset):
        d = {'beta': rnd(*S4, std=2.0), 'alpha': empty(*S4), 'mask': keep(*S4), 'drop': empty(*S4),
             'dad': rnd(*S4), 'dbeta': empty(*S4), 'qq': rnd(Pp, Hh, B, L), 'kk': rnd(Pp, Hh, B, L),
             'vv': rnd(Pp, Hh, B, L), 'dg': rnd(Pp, Hh, B, L)}
        sets.append(d)
    timed('softmax', 7 * ns, [lambda d=d: ops.softmax_dropout(d['beta'], d['alpha'], d['mask'], d['drop'], 0.125, P_DROP)
                              for d in sets])
    timed('bs', 7 * ns, [lambda d=d: ops.backward_softmax(d['alpha'], d['mask'], d['dad'], d['dbeta']) for d in sets])
    timed('QKT+softmax', 5 * ns + 4 * nt, [lambda d=d: ops.attention_scores_softmax(
        d['qq'], d['kk'], None, d['alpha'], d['mask'], d['drop'], 0.125, P_DROP) for d in sets])
    timed('dX1gamma+bs', 5 * ns + 4 * nt, [lambda d=d: ops.attention_scores_softmax_backward(
        d['dg'], d['vv'], d['alpha'], d['mask'], None, d['dbeta']) for d in sets])
    del sets
    # ---- bias + dropout + residual + LayerNorm and the LayerNorm backward family over [B,J,E]
    vec = lambda std=1.0: rnd(E, std=std)
    sets = []
    for _ in range(nset + 1):
        d = {'in': rnd(*T3), 'resid': rnd(*T3), 'mask': keep(*T3), 'lin': empty(*T3), 'diff': empty(*T3),
             'istd': empty(B, L), 'ln': empty(*T3), 'out': empty(*T3), 'dy': rnd(*T3), 'dln': empty(*T3),
             'dres': empty(*T3), 'dlin': empty(*T3), 'r2': rnd(*T3), 'lw': rnd(*T3), 'l2': rnd(*T3),
             'bias': vec(0.02), 'gamma': vec(), 'beta': vec(), 'v': [empty(E) for _ in range(4)]}
        sets.append(d)
    timed('bdrln', 13 * nt, [lambda d=d: ops.bias_dropout_residual_layernorm(
        d['in'], d['bias'], d['resid'], d['gamma'], d['beta'], d['mask'], d['lin'], d['diff'], d['istd'], d['ln'], d['out'],
        P_DROP) for d in sets])
    timed('bsb', 6 * nt, [lambda d=d: ops.backward_scale_bias(d['dy'], d['ln'], d['gamma'], d['dln'], d['v'][0], d['v'][1])
                          for d in sets])
    timed('blnrd', 9 * nt, [lambda d=d: ops.backward_layernorm_residual_dropout(
        d['dln'], d['istd'], d['diff'], d['mask'], d['dres'], d['dlin']) for d in sets])
    timed('ebsb', 10 * nt, [lambda d=d: ops.extended_backward_scale_bias(
        d['ln'], d['gamma'], d['r2'], d['lw'], d['l2'], d['dln'], d['v'][0], d['v'][1], d['v'][2]) for d in sets])
    timed('baob', 2 * nt, [lambda d=d: ops.backward_attn_out_bias(d['dlin'], d['v'][3]) for d in sets])
    timed('bei', 6 * nt, [lambda d=d: ops.backward_encoder_input(d['r2'], d['lw'], d['dres']) for d in sets])
    timed('bsb+blnrd', 11 * nt, [lambda d=d: ops.backward_scale_bias_layernorm(
        d['dy'], d['ln'], d['gamma'], d['istd'], d['diff'], d['mask'], None, d['dres'], d['dlin'], d['v'][0], d['v'][1])
        for d in sets])
    timed('ebsb+blnrd+baob', 15 * nt, [lambda d=d: ops.extended_backward_scale_bias_layernorm(
        d['ln'], d['gamma'], d['r2'], d['lw'], d['l2'], d['istd'], d['diff'], d['mask'], None, d['dres'], d['dlin'], *d['v'])
        for d in sets])
    del sets
    # ---- attention input biases and their gradient over [3,P,H,B,J]
    sets = [{'in': rnd(3, Pp, Hh, B, L), 'out': empty(3, Pp, Hh, B, L), 'bias': rnd(3, Pp, Hh), 'db': empty(3, Pp, Hh)}
            for _ in range(nset + 1)]
    timed('aib', 12 * nt, [lambda d=d: ops.attention_input_biases(d['in'], d['bias'], d['out']) for d in sets])
    timed('baib', 6 * nt, [lambda d=d: ops.backward_attention_input_biases(d['in'], d['db']) for d in sets])
    del sets
    # ---- bias + activation + dropout and its backward over [B,J,U]
    sets = [{'in': rnd(*TU), 'bias': rnd(U, std=0.02), 'mask': keep(*TU), 'lin1': empty(*TU), 'drop2': empty(*TU),
             'dd': rnd(*TU), 'dlin1': empty(*TU), 'db': empty(U)} for _ in range(nset)]
    timed('bad', 7 * nu, [lambda d=d: ops.bias_activation_dropout(d['in'], d['bias'], d['mask'], d['lin1'], d['drop2'],
                                                                  'relu', P_DROP) for d in sets])
    timed('bdrlb', 7 * nu, [lambda d=d: ops.backward_dropout_activation_bias(d['dd'], d['mask'], d['lin1'], d['dlin1'],
                                                                             d['db'], 'relu') for d in sets])
    del sets
    torch.cuda.empty_cache()
    return {'shape': f'H={Hh}, B={B}, J=K={L}, E={E}, U={U}', 'launches_per_operator': f'{warmup} + {reps}',
            'peaks_gbs': {'measured_copy': hbm, 'nominal': NOMINAL_HBM_GBS}, 'operators': results}


def run_kernels(args):
    import torch
    _, rank, _, dev = dist_env(args)
    if rank != 0:
        return
    sampler = ClockSampler(dev.index)
    sampler.start()
    sweep = fused_kernel_sweep(dev, torch)
    clocks = sampler.stop()
    worst = min(sweep['operators'], key=lambda n: sweep['operators'][n]['frac_of_measured_copy'])
    print(json.dumps({'metric': 'fused_operator_hbm_gbs', 'unit': 'GB/s', 'value': sweep['operators'][worst]['gbs'],
                      'value_is': f'the slowest operator of the sweep ({worst})', 'higher_is_better': True,
                      'n_gpus': 1, 'dtype': 'f16', 'data': 'synthetic', 'clocks': clocks,
                      'config': {'workload': 'each fused operator alone, ' + sweep['shape']}, **sweep}))


def run_ours(args):
    import torch
    import torch.distributed as dist
    from substation_b200 import layouts as L
    from substation_b200.data_parallel import GradientBucketReducer, shard_batch

    world, rank, local_rank, dev = dist_env(args)
    init_nccl(args, world, dev)
    B, S = args.batch, args.seq
    lay = resolve_layouts(args.layouts)
    lb = LayerBench(B, S, lay, dev, rank, args.keep_all)
    enc = lb.enc
    fused_bytes = FUSED_BYTES if args.keep_all else FUSED_BYTES_SKIP
    # double-buffered gradient buckets: the allreduce of step i overlaps step i+1
    reducer = GradientBucketReducer(enc.arena_bytes('grads'), dev, buffers=2)
    grad_views = [enc.views('grads', reducer.arenas[b]) for b in range(len(reducer.arenas))]

    # The whole bucket is allreduced beside the next step.  With --early-allreduce 1 the gradients of the
    # feed-forward half, final in the middle of the backward pass, are allreduced beside the attention half of the
    # pass instead: measured slower in steady state (the allreduce then competes with the HBM-bound attention
    # kernels rather than with the next step's tensor-bound projections).
    # The LAST step of a timed region has no next step to hide behind: there the feed-forward half is started early
    # (--early-last 1, the default), which shortens the drain that ends the region.
    early = None
    if world > 1 and (args.early_allreduce or args.early_last):
        ffn_event = torch.cuda.Event()
        enc.set_ffn_grads_event(ffn_event)
        early = (enc.early_grad_offset(), ffn_event)

    def step(i, last=False):
        reducer.wait(i)                                   # this bucket's previous reduction has finished
        lb.run(grad_views[i % len(grad_views)])
        reducer.reduce_async(i, early=early if (args.early_allreduce or (last and args.early_last)) else None)

    drain = reducer.drain

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    lib = __import__('substation_b200._lib', fromlist=['load']).load()

    def set_timing(on):
        lib.sb_encoder_set_timing(enc._native(dev), 1 if on else 0)

    def timed_region(n_steps, sampler=None):
        """n_steps steps bracketed by barrier + synchronize; device time, max over ranks."""
        barrier()
        if sampler is not None and rank == 0:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n_steps):
            step(i, last=(i == n_steps - 1))
        drain()
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1))

    # ---- headline: K steps, device timed, per-operator events off -----------------------
    set_timing(False)
    for i in range(args.warmup):
        step(i)
    drain()
    sampler = ClockSampler(local_rank)
    total_ms = timed_region(args.steps, sampler)
    clocks = sampler.stop() if rank == 0 else None
    ms_per_step = total_ms / args.steps
    value = world * B * args.steps / (total_ms / 1e3)

    # ---- the same step for at least --sustain-s seconds: what the power cap leaves of the short-run figure ----
    sustained = None
    if args.sustain_s > 0:
        n_sus = max(args.steps, int(args.sustain_s * 1e3 / ms_per_step) + 1)
        sampler = ClockSampler(local_rank)
        sus_ms = timed_region(n_sus, sampler)
        sc = sampler.stop(skip_first=2) if rank == 0 else None      # the first samples precede the load
        sustained = {'steps': n_sus, 'seconds': round(sus_ms / 1e3, 3), 'ms_per_step': sus_ms / n_sus,
                     'value': world * B * n_sus / (sus_ms / 1e3), 'clocks': sc}
        if sc and sc.get('sm_mhz'):
            sustained['ms_x_mhz'] = round(sus_ms / n_sus * sc['sm_mhz'], 1)
    if clocks and clocks.get('sm_mhz'):
        clocks['ms_x_mhz'] = round(ms_per_step * clocks['sm_mhz'], 1)

    # ---- per-operator device times (CUDA events on the launching stream around every launch) ----
    launches_per_step = []
    set_timing(True)
    enc.op_times()
    per = {}
    reps = max(3, min(args.steps, 20))
    for i in range(reps):
        step(i)
        drain()
        times = enc.op_times()
        launches_per_step.append(enc.kernel_count())
        for name, ms in times:
            per.setdefault(name, []).append(ms)
    set_timing(False)
    torch.cuda.synchronize(dev)
    launches = max(launches_per_step) * args.steps    # kernels launched inside the timed region (the library's count)
    peaks, peak_kind = load_peaks()
    hbm = float(peaks['hbm_gbs'])
    tf_burst = float(peaks['bf16_tflops'])
    tf_sustained = float(peaks.get('bf16_tflops_sustained', tf_burst))

    # ---- yardsticks, outside every timed region (rank 0 of a single-GPU run) ----
    anchors, probe = {}, None
    if rank == 0 and world == 1 and not args.no_anchors:
        anchors = cublas_anchors(B * S, dev, torch)
        probe = tensor_peak_probe(torch)

    ops = {}
    ideal_us = 0.0
    for name, v in per.items():
        us = 1e3 * statistics.mean(v)
        rec = {'us': round(us, 2)}
        if name in GEMM_FLOPS:
            fl = GEMM_FLOPS[name](B, S)
            rec['tflops'] = round(fl / us / 1e6, 1)
            rec['frac_tensor'] = round(fl / us / 1e6 / tf_burst, 3)
            ideal = fl / (tf_burst * 1e6)
            if name in ATTN_BYTES:
                by = ATTN_BYTES[name](B, S)
                rec['gbs'] = round(by / us / 1e3, 1)
                rec['frac_hbm'] = round(by / us / 1e3 / hbm, 3)
                ideal = max(ideal, by / (hbm * 1e3))
            base = name.split('+')[0]
            if base in anchors:
                # alone, back to back under graph replay: this kernel with its fused epilogue, and cuBLAS on the plain
                # contraction of the same shape (`us` above carries the per-operator events' 5-10 us)
                rec['replay_us'] = round(anchors[base][0], 2)
                rec['frac_tensor_replay'] = round(fl / anchors[base][0] / 1e6 / tf_burst, 3)
                rec['cublas_us'] = round(anchors[base][1], 2)
        else:
            by = fused_bytes[name](B, S)
            rec['gbs'] = round(by / us / 1e3, 1)
            rec['frac_hbm'] = round(by / us / 1e3 / hbm, 3)
            ideal = by / (hbm * 1e3)
        ideal_us += ideal
        ops[name] = rec
    sum_us = sum(r['us'] for r in ops.values())
    T_tok = B * S
    ref_bytes = 142 * T_tok * E + 14 * H * B * S * S
    ref_flops = 72 * E * E * T_tok + 12 * B * S * S * E
    ref_list_us = ref_bytes / (hbm * 1e3) + ref_flops / (tf_sustained * 1e6)
    ref_list_burst_us = ref_bytes / (hbm * 1e3) + ref_flops / (tf_burst * 1e6)
    top = max(ops, key=lambda n: ops[n]['us'])
    if top in GEMM_FLOPS and top not in ATTN_BYTES:
        roof = {'kernel': f'gemm_tc_pair_kernel ({top})', 'bound': 'tensor', 'achieved': ops[top]['tflops'],
                'peak': tf_burst, 'unit': 'TFLOP/s', 'frac': round(ops[top]['tflops'] / tf_burst, 3)}
    else:
        roof = {'kernel': top, 'bound': 'hbm', 'achieved': ops[top]['gbs'], 'peak': hbm, 'unit': 'GB/s',
                'frac': round(ops[top]['gbs'] / hbm, 3)}
    roof['traffic'] = load_dram_traffic(B, S, args.keep_all).get(top)
    roof['traffic_unit'] = 'bytes per launch (ncu dram__bytes_read.sum + dram__bytes_write.sum; null: not captured for this setting)'
    roof['algorithmic_bytes'] = (fused_bytes.get(top) or ATTN_BYTES.get(top, lambda b, l: None))(B, S)
    roof['peak_source'] = f'{peak_kind} (MEASURED_PEAKS.json: torch copy / cuBLAS bf16 burst)'
    roof['share_of_step'] = round(ops[top]['us'] / sum_us, 3)

    # ---- end to end through the public module with host buffers -------------------------
    e2e = None
    if not args.no_e2e:
        X, DY = lb.X, lb.DY
        hX, hDY = X.cpu().pin_memory(), DY.cpu().pin_memory()
        hY, hDX = torch.empty_like(hX).pin_memory(), torch.empty_like(hX).pin_memory()

        # Three streams: host->device copies of step i+1 and device->host copies of step i-1 run
        # beside the compute of step i (PCIe is full duplex); every step still copies its own X and
        # dY in and its own Y and dX out, all inside the timed region.
        cur = torch.cuda.current_stream(dev)
        s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        xd = [torch.empty_like(X) for _ in range(2)]
        dyd = [torch.empty_like(X) for _ in range(2)]
        yd = [torch.empty_like(X) for _ in range(2)]
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_free = [torch.cuda.Event() for _ in range(2)]       # compute no longer reads input buffer b
        ev_out = [torch.cuda.Event() for _ in range(2)]
        keep = [None, None]
        works = [None, None]
        for prm in enc.params:
            prm.requires_grad_(True)
        # The module keeps two sets of buffers for its autograd path and uses them in turn (set_buffer_pool): the
        # pointers of a pass repeat every other step, so passes replay as CUDA graphs, and the collective sees the
        # same two gradient buckets every step.  Y and dX are copied to the host before their set comes round again.
        enc.set_buffer_pool(2)

        def copy_in(i):
            b = i & 1
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_free[b])
                xd[b].copy_(hX, non_blocking=True)
                dyd[b].copy_(hDY, non_blocking=True)
                ev_in[b].record(s_in)

        def copy_out(b, y, dx):
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_free[b])
                s_out.wait_event(ev_out[b])                    # previous copy out of these host buffers done
                hY.copy_(y, non_blocking=True)
                hDX.copy_(dx, non_blocking=True)
                ev_out[b].record(s_out)

        host_s = {'copies': 0.0, 'forward': 0.0, 'backward': 0.0, 'allreduce': 0.0}   # where the host's time per step goes
        clock = time.perf_counter

        def e2e_step(i):
            # the inputs of step i+1 start moving before the kernels of step i are enqueued, so the copy
            # runs beside this step's compute however far ahead of the GPU the host happens to be
            b = i & 1
            t0 = clock()
            copy_in(i + 1)
            cur.wait_event(ev_in[b])
            x = xd[b].detach().requires_grad_(True)
            t1 = clock()
            if works[b] is not None:                           # the bucket this backward writes (used two steps ago) is free again
                works[b].wait()
                works[b] = None
            cur.wait_event(ev_out[b])                          # ... and so are the Y / dX of that set (copied out)
            t2 = clock()
            y = enc(x)
            t3 = clock()
            y.backward(dyd[b])
            t4 = clock()
            ev_free[b].record(cur)
            if world > 1:
                # all twelve gradients are views into one bucket: one allreduce, asynchronous
                works[b] = dist.all_reduce(enc.grad_bucket(), op=dist.ReduceOp.SUM, async_op=True)
            t5 = clock()
            y.record_stream(s_out)
            x.grad.record_stream(s_out)
            copy_out(b, y.detach(), x.grad)
            keep[b] = (x, y)
            enc.zero_grad(set_to_none=True)
            t6 = clock()
            host_s['copies'] += (t1 - t0) + (t6 - t5)
            host_s['allreduce'] += (t2 - t1) + (t5 - t4)
            host_s['forward'] += t3 - t2
            host_s['backward'] += t4 - t3

        def copy_only_step(i):
            b = i & 1
            copy_in(i + 1)
            cur.wait_event(ev_in[b])
            ev_free[b].record(cur)
            copy_out(b, yd[b], xd[b])

        def e2e_drain():
            for w in works:
                if w is not None:
                    w.wait()
            cur.wait_stream(s_in)
            cur.wait_stream(s_out)

        def e2e_region(stepfn, first, n):
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            t_host = time.perf_counter()
            for i in range(first, first + n):
                stepfn(i)
            t_host = time.perf_counter() - t_host      # host time to issue the steps (no synchronisation inside)
            e2e_drain()
            e1.record()
            barrier()
            return max_over_ranks(e0.elapsed_time(e1)), t_host

        n_warm = max(3, args.warmup)
        copy_in(0)
        for i in range(n_warm):
            e2e_step(i)
        e2e_drain()
        # step i's inputs were copied during step i-1 (the first one during warm-up); every step issues
        # exactly one copy in and one copy out, so the timed region holds `steps` of each
        # Three regions of `steps` steps each, the fastest reported and all three listed: this leg runs at the
        # host's pace (Tensor.backward hands the pass to autograd's worker thread), and on a box that has just
        # booted a whole region has measured 4-5 ms per step where the next one measured 0.65.
        regions = []
        first = n_warm
        for rep in range(3):
            for k in host_s:
                host_s[k] = 0.0
            g0 = enc.graph_stats()
            r_ms, r_host = e2e_region(e2e_step, first, args.steps)
            g1 = enc.graph_stats()
            first += args.steps
            regions.append((r_ms, r_host, {k: round(1e3 * v / args.steps, 4) for k, v in host_s.items()},
                            g1[1] - g0[1], g1[0] - g0[0]))
        e2e_ms, t_host, host_ms, n_replays, n_captures = min(regions, key=lambda r: r[0])
        for i in range(first, first + 2):
            copy_only_step(i)
        e2e_drain()
        copy_ms, _ = e2e_region(copy_only_step, first + 2, args.steps)
        enc.set_buffer_pool(0)
        nbytes = hX.numel() * 2
        e2e = {'value': world * B * args.steps / (e2e_ms / 1e3), 'unit': UNIT,
               'h2d_bytes_per_step': 2 * nbytes, 'd2h_bytes_per_step': 2 * nbytes,
               'ms_per_step': e2e_ms / args.steps, 'host_issue_ms_per_step': 1e3 * t_host / args.steps,
               # the host's share per step by part (rank 0): input/output copies and bookkeeping, module forward,
               # Tensor.backward, waiting for and enqueueing the gradient allreduce
               'host_ms_per_step_by_part': host_ms,
               # passes replayed as CUDA graphs / captured anew inside the timed region (2 replays per step expected)
               'graph_replays': n_replays, 'graph_captures': n_captures,
               'regions_ms_per_step': [round(r[0] / args.steps, 4) for r in regions],
               # the same host<->device copies with no compute between them: what the host side of the box allows
               'copy_only_ms_per_step': copy_ms / args.steps,
               'over_max_of_copy_and_compute': round((e2e_ms / args.steps) / max(copy_ms / args.steps, ms_per_step), 3)}

    # ---- multi-GPU evidence, outside the timed regions ------------------------------------
    dp_check = strong = stack = None
    if world > 1 and not args.no_extras:
        dp_check = data_parallel_check(lb, reducer, grad_views, world, rank, dev, lay, args)
    if not args.no_extras:
        strong = strong_scaling_record(args, world, rank, dev, barrier, max_over_ranks)
        stack = stack_record(args, world, rank, dev, barrier, max_over_ranks)

    # ---- every fused operator alone at the kernel-sweep shapes (single-GPU run) ------------
    sweep = None
    if rank == 0 and world == 1 and not args.no_sweep:
        del lb
        torch.cuda.empty_cache()
        sweep = fused_kernel_sweep(dev, torch)

    # ---- CPU baseline (rank 0, N=1 only): bounded sample of the same workload ------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        sb = min(2, B)
        t = cpu_pass(sb, S)
        cpu = {'value': sb / t, 'unit': UNIT, 'cores': host_cores(), 'kind': 'port',
               'sample': f'{sb} of the {B} sequences (L={S}), one forward+backward of the numpy float64 '
                         f'port of substation/transformer.py ({t:.1f} s)'}

    if rank == 0:
        layer = {'sum_of_operator_us': round(sum_us, 1), 'sum_of_roofline_us': round(ideal_us, 1),
                 'frac_of_summed_roofline': round(ideal_us / sum_us, 3),
                 # the same ideal against the device time of a whole step (kernels overlap their
                 # neighbours' ramp-up and tail under programmatic dependent launch)
                 'roofline_us_over_step_us': round(ideal_us / (ms_per_step * 1e3), 3),
                 # the reference's own operator list (32 separate operators: 142*T*E + 14*S bytes of
                 # elementwise traffic, 72*E^2*T + 12*B*L^2*E flops) at the measured copy bandwidth and the
                 # tensor rate: burst peak against the short run, sustained peak against the sustained run
                 'reference_list_roofline_us': round(ref_list_us, 1),
                 'reference_list_roofline_burst_us': round(ref_list_burst_us, 1),
                 'reference_list_roofline_over_step': round(ref_list_us / (ms_per_step * 1e3), 3),
                 'reference_list_burst_roofline_over_step': round(ref_list_burst_us / (ms_per_step * 1e3), 3)}
        if sustained:
            layer['reference_list_roofline_over_sustained_step'] = round(ref_list_us / (sustained['ms_per_step'] * 1e3), 3)
        line = {
            'metric': METRIC, 'value': value, 'unit': UNIT, 'n_gpus': world, 'steps': args.steps,
            'warmup': args.warmup, 'ms_per_step': ms_per_step, 'higher_is_better': True, 'scaling': 'weak',
            'vs_baseline': None, 'dtype': 'f16', 'data': 'synthetic',
            'config': workload_config(args, args.layouts),
            'clocks': clocks, 'e2e': e2e, 'gpu_launches': launches, 'roofline': roof, 'cpu_baseline': cpu,
            'sustained': sustained, 'layer': layer, 'fp16_tflops_probe': probe, 'operators': ops,
            'dp_check': dp_check, 'strong': strong, 'stack': stack, 'fused_kernels': sweep,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def data_parallel_check(lb, reducer, grad_views, world, rank, dev, lay, args):
    """(a) the allreduced bucket against the fp32 sum of the gathered per-rank buckets; (b) at a small shape, the
    allreduced gradients of a batch sharded over the ranks against one GPU running the concatenated batch."""
    import torch
    import torch.distributed as dist
    from substation_b200 import layouts as L
    from substation_b200.data_parallel import shard_batch

    def rel_l2(a, b):
        return float(((a.double() - b.double()).norm() / b.double().norm().clamp_min(1e-30)).item())

    res = {}
    # (a) the bench's own shape
    reducer.drain()
    lb.run(grad_views[0])
    local = reducer.flat(0).clone()
    gathered = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(gathered, local)
    want = torch.zeros(local.numel(), dtype=torch.float32, device=dev)
    for g in gathered:
        want += g.float()
    reducer.reduce_async(0)
    reducer.drain()
    torch.cuda.synchronize(dev)
    res['allreduced_vs_fp32_sum_of_gathered'] = rel_l2(reducer.flat(0).float(), want)
    del gathered, want
    # (b) small shape: global batch 2*world at L=128, BERT-large widths
    b_loc, S = 2, 128
    Bg = b_loc * world
    table = L.validate(lay)
    if table['X'] != 'BJI' or any(table[n][0] != 'B' for n in ('DROP1MASK', 'DROP2MASK', 'DROP3MASK')) or \
            table['ATTN_DROP_MASK'][:2] != 'HB':
        res['sharded_vs_one_gpu'] = None     # slicing below assumes batch-major masks
        return res
    gen = torch.Generator(device=dev).manual_seed(4321)          # the same global batch on every rank
    Xg = torch.randn(Bg, S, E, device=dev, generator=gen).half()
    DYg = torch.randn(Bg, S, E, device=dev, generator=gen).half()
    mg = {'ATTN_DROP_MASK': (torch.rand(H, Bg, S, S, device=dev, generator=gen) >= P_DROP).to(torch.uint8),
          'DROP1MASK': (torch.rand(Bg, S, E, device=dev, generator=gen) >= P_DROP).to(torch.uint8),
          'DROP2MASK': (torch.rand(Bg, S, U, device=dev, generator=gen) >= P_DROP).to(torch.uint8),
          'DROP3MASK': (torch.rand(Bg, S, E, device=dev, generator=gen) >= P_DROP).to(torch.uint8)}
    lo, hi = shard_batch(Bg, world, rank)
    ml = {n: (m[:, lo:hi] if n == 'ATTN_DROP_MASK' else m[lo:hi]).contiguous() for n, m in mg.items()}
    small = LayerBench(hi - lo, S, lay, dev, rank, args.keep_all, profiling=False,
                       X=Xg[lo:hi].contiguous(), DY=DYg[lo:hi].contiguous(), masks=ml)
    bucket = torch.zeros(small.enc.arena_bytes('grads'), dtype=torch.uint8, device=dev)
    small.run(small.enc.views('grads', bucket))
    flat = bucket.view(torch.float16)
    dist.all_reduce(flat, op=dist.ReduceOp.SUM)
    worst = None
    if rank == 0:
        full = LayerBench(Bg, S, lay, dev, rank, args.keep_all, profiling=False, X=Xg, DY=DYg, masks=mg)
        fb = torch.zeros(full.enc.arena_bytes('grads'), dtype=torch.uint8, device=dev)
        fg = full.enc.views('grads', fb)
        full.run(fg)
        torch.cuda.synchronize(dev)
        sg = small.enc.views('grads', bucket)
        worst = max(rel_l2(sg[n], fg[n]) for n in fg if n != '__arena__')
    dist.barrier()
    res['sharded_vs_one_gpu'] = worst
    res['sharded_shape'] = f'global batch {Bg} (L={S}) as {b_loc} per rank; worst rel-L2 over the 12 gradients'
    res['tolerance'] = 1e-2
    return res


def strong_scaling_record(args, world, rank, dev, barrier, max_over_ranks, global_batch=96, S=128, steps=10):
    """Global batch 96 at L=128 (the small-sequence, large-batch configuration) split over the ranks: every rank runs
    96 / N sequences per step, gradients allreduced beside the next step.  With N > 1, rank 0 also times the whole
    batch alone so that the line carries both sides of the ratio."""
    import torch
    from substation_b200 import layouts as L
    from substation_b200.data_parallel import GradientBucketReducer, shard_batch
    lay = L.uniform_layouts()
    lo, hi = shard_batch(global_batch, world, rank)

    def measure(Bl, reduce):
        lb = LayerBench(Bl, S, lay, dev, rank, args.keep_all, profiling=False)
        red = GradientBucketReducer(lb.enc.arena_bytes('grads'), dev, buffers=2, verify=reduce) if reduce else None
        arenas = red.arenas if red else [torch.empty(lb.enc.arena_bytes('grads'), dtype=torch.uint8, device=dev)
                                         for _ in range(2)]
        views = [lb.enc.views('grads', a) for a in arenas]

        def step(i):
            if red:
                red.wait(i)
            lb.run(views[i & 1])
            if red:
                red.reduce_async(i)
        for i in range(4):
            step(i)
        if red:
            red.drain()
        if reduce:
            barrier()
        else:
            torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            step(i)
        if red:
            red.drain()
        e1.record()
        torch.cuda.synchronize(dev)
        ms = e0.elapsed_time(e1)
        del lb
        torch.cuda.empty_cache()
        return ms

    ms = max_over_ranks(measure(hi - lo, world > 1)) / steps
    rec = {'global_batch': global_batch, 'seq_len': S, 'per_gpu_batch': hi - lo, 'layouts': 'uniform',
           'ms_per_step': ms, 'value': global_batch / (ms / 1e3), 'unit': UNIT}
    if world > 1:
        one = measure(global_batch, False) / steps if rank == 0 else 0.0
        barrier()
        one = max_over_ranks(one)
        rec['one_gpu_ms_per_step'] = one
        rec['speedup_over_one_gpu'] = round(one / ms, 3)
    return rec


def stack_record(args, world, rank, dev, barrier, max_over_ranks, layers=24, steps=10):
    """24 layers with independent weights, per-GPU batch 8 at L=512: forward through all layers, backward through all
    layers, each layer's gradient bucket allreduced while the next layer's backward runs."""
    import torch
    from substation_b200.stack import EncoderStack
    lay = resolve_layouts(args.layouts)
    st = EncoderStack(layers, 8, 512, H, E, lay, dropout_p=P_DROP, device=dev, seed=1234)
    gen = torch.Generator(device=dev).manual_seed(100 + rank)
    X = torch.randn(st.acts[0].shape, device=dev, generator=gen).half()
    DY = torch.randn(st.acts[0].shape, device=dev, generator=gen).half()

    def step():
        st.forward(X)
        st.backward(DY)
    for _ in range(2):
        step()
    st.wait_gradients()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    st.wait_gradients()
    e1.record()
    barrier()
    ms = max_over_ranks(e0.elapsed_time(e1)) / steps
    rec = {'layers': layers, 'per_gpu_batch': 8, 'seq_len': 512, 'ms_per_step': ms, 'ms_per_layer': ms / layers,
           'value': world * 8 / (ms / 1e3), 'unit': UNIT, 'memory_gb': round(st.memory_bytes() / 2 ** 30, 2),
           'masks': 'in-kernel Philox'}
    if world > 1:
        # one more step, traced (outside the timed region): when each layer's backward and each bucket's allreduce
        # ended on this rank.  The reduction of layer l is hidden when it ends before the backward of layer l-1 does.
        st.forward(X)
        trace = []
        st.backward(DY, trace=trace)
        st.wait_gradients()
        torch.cuda.synchronize(dev)
        rows = st.overlap_trace(trace)
        hidden = sum(1 for a, b in zip(rows, rows[1:]) if a[2] is not None and a[2] <= b[1])
        rec['overlap_trace'] = {
            'columns': ['layer', 'backward_done_ms', 'allreduce_done_ms'], 'rank': rank, 'rows': rows,
            'reductions_hidden_behind_next_backward': hidden, 'of': len(rows) - 1,
            'exposed_after_last_backward_ms': None if rows[-1][2] is None else round(rows[-1][2] - rows[-1][1], 3)}
    del st
    torch.cuda.empty_cache()
    return rec


def run_stack(args):
    """--layers N > 1: a stack of N layers with independent weights (the 24-layer stack configuration at N=24);
    one step = forward through all layers + backward through all layers, each layer's gradient
    bucket allreduced while the next layer's backward runs."""
    import torch
    import torch.distributed as dist
    from substation_b200.stack import EncoderStack
    world, rank, local_rank, dev = dist_env(args)
    init_nccl(args, world, dev)
    lay = resolve_layouts(args.layouts)
    st = EncoderStack(args.layers, args.batch, args.seq, H, E, lay, dropout_p=P_DROP, device=dev, seed=1234)
    gen = torch.Generator(device=dev).manual_seed(100 + rank)
    X = torch.randn(st.acts[0].shape, device=dev, generator=gen).half()
    DY = torch.randn(st.acts[0].shape, device=dev, generator=gen).half()

    def step():
        st.forward(X)
        st.backward(DY)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(args.warmup):
        step()
    st.wait_gradients()
    sampler = ClockSampler(local_rank)
    barrier()
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    st.wait_gradients()
    e1.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    if rank == 0:
        cfg = workload_config(args, args.layouts)
        cfg['workload'] = (f'{args.layers}-layer stack of: ' + cfg['workload']).replace('seeded explicit masks', 'in-kernel Philox masks')
        cfg['layers'] = args.layers
        print(json.dumps({
            'metric': METRIC, 'value': world * args.batch * args.steps / (ms / 1e3), 'unit': UNIT, 'n_gpus': world,
            'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': ms / args.steps,
            'ms_per_layer': ms / args.steps / args.layers, 'higher_is_better': True, 'scaling': 'weak',
            'vs_baseline': None, 'dtype': 'f16', 'data': 'synthetic', 'config': cfg, 'clocks': clocks,
            'gpu_launches': sum(enc.kernel_count() for enc in st.layers) * args.steps, 'stack_memory_gb': round(st.memory_bytes() / 2 ** 30, 2)}))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=5)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--layouts', default='b200_b8_l512',
                    help='b200_b8_l512 (chosen by the layout search for these kernels), uniform, '
                         'b8_l512 / b96_l128 (the reference\'s shipped configurations) or a .json path')
    ap.add_argument('--batch', type=int, default=8)
    ap.add_argument('--seq', type=int, default=512)
    ap.add_argument('--comm-ctas', type=int, default=12,
                    help='SMs left to NCCL when N > 1 (every persistent grid of the library is sized for the rest)')
    ap.add_argument('--early-allreduce', type=int, default=0,
                    help='N > 1: sum the feed-forward gradients beside the attention half of backward (1) or the whole '
                         'bucket beside the next step (0)')
    ap.add_argument('--early-last', type=int, default=1,
                    help='N > 1: start the allreduce of the feed-forward gradients early on the last step of a timed region')
    ap.add_argument('--layers', type=int, default=1, help='>1: time a stack of layers (the 24-layer configuration uses 24)')
    ap.add_argument('--kernels', action='store_true', help='time every fused operator alone at the kernel-sweep shapes')
    ap.add_argument('--keep-all', type=int, default=0,
                    help='1: also store the nine intermediates nothing reads again (what enable_debug does)')
    ap.add_argument('--sustain-s', type=float, default=2.0, help='length of the sustained run in seconds (0: skip)')
    ap.add_argument('--no-e2e', action='store_true')
    ap.add_argument('--no-cpu', action='store_true')
    ap.add_argument('--no-anchors', action='store_true', help='skip the cuBLAS yardstick and the tensor-peak probe')
    ap.add_argument('--no-sweep', action='store_true', help='skip the fused-operator sweep')
    ap.add_argument('--no-extras', action='store_true', help='skip dp_check / strong / stack')
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == 'ours':
        args.warmup = 3
    if args.impl == 'reference':
        run_reference_arm(args)
    elif args.kernels:
        run_kernels(args)
    elif args.layers > 1:
        run_stack(args)
    else:
        run_ours(args)


if __name__ == '__main__':
    main()
