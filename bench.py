"""Benchmark of the encoder-layer hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--layouts b200_b8_l512|uniform|b8_l512|b96_l128] [--batch B] [--seq L]

One "step" = one BERT-large encoder layer forward+backward (B=8, L=512, H=16,
E=1024, fp16 storage / fp32 accumulation, dropout p=0.1 with seeded explicit
masks) on each GPU; with N>1 every rank runs its own batch of 8 (weak scaling)
and the layer's 12 parameter gradients are sum-allreduced over NCCL, overlapped
with the next step.  Rank 0 prints ONE JSON line.

value      sequences/s over all ranks, inputs resident in HBM, CUDA-event timed
e2e        same through the public ``Encoder`` module with host buffers:
           pinned-host X and dY copied in, Y and dX copied out, every step
roofline   the operator with the largest device time: algorithmic FLOPs (or
           bytes) / its mean duration, against MEASURED_PEAKS.json
cpu_baseline  the numpy port of the reference path (oracle/) timed on the host
--impl reference  that same numpy port as its own arm (rank 0 only)
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
# attention contractions are HBM-bound: minimum operand bytes (two [P,L] operands + one [L,L], or v.v.)
ATTN_BYTES = {
    'QKT': lambda B, L: 2 * H * B * (2 * P * L + L * L), 'gamma': lambda B, L: 2 * H * B * (2 * P * L + L * L),
    'dX1gamma': lambda B, L: 2 * H * B * (2 * P * L + L * L), 'dX2gamma': lambda B, L: 2 * H * B * (2 * P * L + L * L),
    'dX1QKT': lambda B, L: 2 * H * B * (2 * P * L + L * L), 'dX2QKT': lambda B, L: 2 * H * B * (2 * P * L + L * L),
}
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


# dram__bytes_read.sum + dram__bytes_write.sum of one launch at B=8, L=512, from the ncu --set full captures
# summarised in profiles/top_kernels_b8_l512_full_captures.md (part of each kernel's output is still in L2
# when it ends, so traffic can be below the algorithmic bytes)
NCU_DRAM_BYTES = {'QKT+softmax': 207.69e6, 'dX1gamma+bs': 200.28e6, 'gamma': 78.86e6, 'dX2gamma': 77.23e6,
                  'dX1QKT+dX2QKT': 87.78e6, 'bsb+blnrd1': 29.86e6, 'ebsb+blnrd2+baob': 51.58e6}


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


class ClockSampler:
    """nvidia-smi clock/throttle samples while the timed region runs."""
    Q = ('index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,'
         'clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
         'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')

    def __init__(self, gpu_index):
        self.proc, self.rows, self.idx = None, [], gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ['nvidia-smi', f'--query-gpu={self.Q}', '--format=csv,noheader,nounits', '-lms', '100',
                 '-i', str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['nvidia-smi unavailable']}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, smax, reasons = [], [], set()
        for line in out.strip().splitlines():
            c = [x.strip() for x in line.split(',')]
            if len(c) < 9:
                continue
            try:
                sm.append(float(c[1])); smax.append(float(c[2]))
            except ValueError:
                continue
            for name, val in zip(('hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap'), c[5:9]):
                if val.lower().startswith('active'):
                    reasons.add(name)
        return {'sm_mhz': statistics.median(sm) if sm else None,
                'sm_max_mhz': max(smax) if smax else None, 'samples': len(sm),
                'reasons': sorted(reasons)}


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
            'l2': 'per-step working set (~0.9 GB of intermediates) is larger than the 126 MB L2; no flush needed'}


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from substation_b200 import Encoder, layouts as L
    from substation_b200.data_parallel import GradientBucketReducer
    from tests.layer_harness import get_layouts

    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local_rank = int(os.environ.get('LOCAL_RANK', '0'))
    if world != args.gpus:
        raise SystemExit(f'--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run')
    if not torch.cuda.is_available():
        raise SystemExit('bench.py needs a CUDA device: the product path has no CPU fallback')
    torch.cuda.set_device(local_rank)
    dev = torch.device('cuda', local_rank)
    comm_ctas = 0
    if world > 1:
        # Few NCCL CTAs are enough for a 25 MB bucket over NVLink; the persistent contraction
        # kernels leave exactly those SMs free so that the allreduce runs beside them.
        comm_ctas = args.comm_ctas
        opts = None
        try:
            opts = dist.ProcessGroupNCCL.Options()
            opts.config.max_ctas = comm_ctas
            opts.config.min_ctas = min(4, comm_ctas)
        except Exception:
            opts = None
        dist.init_process_group('nccl', device_id=dev, pg_options=opts)
        from substation_b200 import ops as _ops
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        _ops.set_sm_budget(sms - comm_ctas)

    B, S = args.batch, args.seq
    lay = get_layouts(args.layouts)
    table = L.validate(lay)
    enc = Encoder('/tmp/substation_b200_unused', B, S, H, E, lay, torch.float16,
                  P_DROP, P_DROP, P_DROP, P_DROP, profiling=True, mask_mode='explicit',
                  keep_all_intermediates=bool(args.keep_all)).to(dev)
    fused_bytes = FUSED_BYTES if args.keep_all else FUSED_BYTES_SKIP
    gen = torch.Generator(device=dev).manual_seed(1234)        # same weights on every rank
    with torch.no_grad():
        for (name, layout), prm in zip(lay['params'], enc.params):
            if name in ('WKQV', 'WO', 'LINW1', 'LINW2'):
                prm.copy_((torch.randn(prm.shape, device=dev, generator=gen) * 0.02).half())
            elif name in ('S1', 'S2'):
                prm.fill_(1.0)
            else:
                prm.zero_()
    gen = torch.Generator(device=dev).manual_seed(100 + rank)  # different data per rank
    shape_x = L.shape_of(table['X'], enc.sizes)
    X = torch.randn(shape_x, device=dev, generator=gen).half()
    DY = torch.randn(shape_x, device=dev, generator=gen).half()
    masks = {}
    for n in L.MASKS:
        shp = L.shape_of(table[n], enc.sizes)
        masks[n] = (torch.rand(shp, device=dev, generator=gen) >= P_DROP).to(torch.uint8)
    enc.set_masks(masks)

    weights = [p.detach() for p in enc.params]
    fwd = enc._alloc(enc._fwd_plan, dev)
    fwd.update(masks)
    bwd = enc._alloc(enc._bwd_plan, dev)
    # double-buffered gradient buckets: the allreduce of step i overlaps step i+1
    reducer = GradientBucketReducer(enc.arena_bytes('grads'), dev, buffers=2)
    Y, DX = torch.empty_like(X), torch.empty_like(X)

    # The whole bucket is allreduced beside the next step.  With --early-allreduce 1 the gradients of the
    # feed-forward half, final in the middle of the backward pass, are allreduced beside the attention half of the
    # pass instead: measured slower (8 GPUs: 0.75 against 0.67 ms per step), the allreduce then competes with the
    # HBM-bound attention kernels rather than with the next step's tensor-bound projections.
    early = None
    if world > 1 and args.early_allreduce:
        ffn_event = torch.cuda.Event()
        enc.set_ffn_grads_event(ffn_event)
        early = (enc.early_grad_offset(), ffn_event)
    grad_views = [enc.views('grads', reducer.arenas[b]) for b in range(len(reducer.arenas))]

    def step(i):
        reducer.wait(i)                                   # this bucket's previous reduction has finished
        grads = grad_views[i % len(grad_views)]
        enc.forward_raw(X, weights, fwd, Y)
        enc.backward_raw(DY, grads, bwd, weights, fwd, X, DX)
        reducer.reduce_async(i, early=early)

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

    # ---- headline: K steps, device timed, per-operator events off -----------------------
    set_timing(False)
    for i in range(args.warmup):
        step(i)
    drain()
    sampler = ClockSampler(local_rank)
    barrier()
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(i)
    drain()
    e1.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    total_ms = max_over_ranks(e0.elapsed_time(e1))
    ms_per_step = total_ms / args.steps
    value = world * B * args.steps / (total_ms / 1e3)
    launches = None   # filled from the library's own count below

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
        else:
            by = fused_bytes[name](B, S)
            rec['gbs'] = round(by / us / 1e3, 1)
            rec['frac_hbm'] = round(by / us / 1e3 / hbm, 3)
            ideal = by / (hbm * 1e3)
        ideal_us += ideal
        ops[name] = rec
    sum_us = sum(r['us'] for r in ops.values())
    T_tok = B * S
    ref_list_us = ((142 * T_tok * E + 14 * H * B * S * S) / (hbm * 1e3) +
                   (72 * E * E * T_tok + 12 * B * S * S * E) / (tf_sustained * 1e6))
    top = max(ops, key=lambda n: ops[n]['us'])
    if top in GEMM_FLOPS and top not in ATTN_BYTES:
        roof = {'kernel': f'gemm_tc_kernel ({top})', 'bound': 'tensor', 'achieved': ops[top]['tflops'],
                'peak': tf_burst, 'unit': 'TFLOP/s', 'frac': round(ops[top]['tflops'] / tf_burst, 3)}
    else:
        roof = {'kernel': top, 'bound': 'hbm', 'achieved': ops[top]['gbs'], 'peak': hbm, 'unit': 'GB/s',
                'frac': round(ops[top]['gbs'] / hbm, 3)}
    # DRAM bytes (read + write) of one launch from the ncu capture of this workload; only known for B=8, L=512
    roof['traffic'] = NCU_DRAM_BYTES.get(top) if (B, S) == (8, 512) and args.keep_all else None
    roof['traffic_unit'] = 'bytes per launch (ncu dram__bytes_read.sum + dram__bytes_write.sum)'
    roof['algorithmic_bytes'] = (fused_bytes.get(top) or ATTN_BYTES.get(top, lambda b, l: None))(B, S)
    roof['peak_source'] = f'{peak_kind} (MEASURED_PEAKS.json: torch copy / cuBLAS bf16 burst)'
    roof['share_of_step'] = round(ops[top]['us'] / sum_us, 3)

    # ---- end to end through the public module with host buffers -------------------------
    e2e = None
    if not args.no_e2e:
        hX, hDY = X.cpu().pin_memory(), DY.cpu().pin_memory()
        hY, hDX = torch.empty_like(hX).pin_memory(), torch.empty_like(hX).pin_memory()

        # Three streams: host->device copies of step i+1 and device->host copies of step i-1 run
        # beside the compute of step i (PCIe is full duplex); every step still copies its own X and
        # dY in and its own Y and dX out, all inside the timed region.
        cur = torch.cuda.current_stream(dev)
        s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        xd = [torch.empty_like(X) for _ in range(2)]
        dyd = [torch.empty_like(X) for _ in range(2)]
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_free = [torch.cuda.Event() for _ in range(2)]       # compute no longer reads input buffer b
        ev_out = [torch.cuda.Event() for _ in range(2)]
        keep = [None, None]
        works = [None, None]
        for prm in enc.params:
            prm.requires_grad_(True)

        def copy_in(i):
            b = i & 1
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_free[b])
                xd[b].copy_(hX, non_blocking=True)
                dyd[b].copy_(hDY, non_blocking=True)
                ev_in[b].record(s_in)

        def e2e_step(i):
            # the inputs of step i+1 start moving before the kernels of step i are enqueued, so the copy
            # runs beside this step's compute however far ahead of the GPU the host happens to be
            b = i & 1
            copy_in(i + 1)
            cur.wait_event(ev_in[b])
            x = xd[b].detach().requires_grad_(True)
            y = enc(x)
            y.backward(dyd[b])
            ev_free[b].record(cur)
            if world > 1:
                # all twelve gradients are views into one bucket: one allreduce, asynchronous, waited for
                # two steps later (each step's backward gets a fresh bucket)
                bucket = enc.grad_bucket()
                lo, hi = bucket.data_ptr(), bucket.data_ptr() + bucket.numel() * 2
                if all(lo <= prm.grad.data_ptr() < hi for prm in enc.params):
                    if works[b] is not None:
                        works[b].wait()
                    works[b] = dist.all_reduce(bucket, op=dist.ReduceOp.SUM, async_op=True)
                else:
                    for prm in enc.params:
                        dist.all_reduce(prm.grad, op=dist.ReduceOp.SUM)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_free[b])
                s_out.wait_event(ev_out[b])                    # previous copy out of these host buffers done
                y.record_stream(s_out)
                x.grad.record_stream(s_out)
                hY.copy_(y.detach(), non_blocking=True)
                hDX.copy_(x.grad, non_blocking=True)
                ev_out[b].record(s_out)
            keep[b] = (x, y)
            enc.zero_grad(set_to_none=True)

        def e2e_drain():
            for w in works:
                if w is not None:
                    w.wait()
            cur.wait_stream(s_in)
            cur.wait_stream(s_out)

        n_warm = max(3, args.warmup)
        copy_in(0)
        for i in range(n_warm):
            e2e_step(i)
        e2e_drain()
        barrier()
        e0.record()
        t_host = time.perf_counter()
        # step i's inputs were copied during step i-1 (the first one during warm-up); every step issues
        # exactly one copy in and one copy out, so the timed region holds `steps` of each
        for i in range(n_warm, n_warm + args.steps):
            e2e_step(i)
        t_host = time.perf_counter() - t_host      # host time to issue the steps (no synchronisation inside)
        e2e_drain()
        e1.record()
        barrier()
        e2e_ms = max_over_ranks(e0.elapsed_time(e1))
        nbytes = hX.numel() * 2
        e2e = {'value': world * B * args.steps / (e2e_ms / 1e3), 'unit': UNIT,
               'h2d_bytes_per_step': 2 * nbytes, 'd2h_bytes_per_step': 2 * nbytes,
               'ms_per_step': e2e_ms / args.steps, 'host_issue_ms_per_step': 1e3 * t_host / args.steps}

    # ---- CPU baseline (rank 0, N=1 only): bounded sample of the same workload ------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        sb = min(2, B)
        t = cpu_pass(sb, S)
        cpu = {'value': sb / t, 'unit': UNIT, 'cores': host_cores(), 'kind': 'port',
               'sample': f'{sb} of the {B} sequences (L={S}), one forward+backward of the numpy float64 '
                         f'port of substation/transformer.py ({t:.1f} s)'}

    if rank == 0:
        line = {
            'metric': METRIC, 'value': value, 'unit': UNIT, 'n_gpus': world, 'steps': args.steps,
            'warmup': args.warmup, 'ms_per_step': ms_per_step, 'higher_is_better': True, 'scaling': 'weak',
            'vs_baseline': None, 'dtype': 'f16', 'data': 'synthetic',
            'config': workload_config(args, args.layouts),
            'clocks': clocks, 'e2e': e2e, 'gpu_launches': launches, 'roofline': roof, 'cpu_baseline': cpu,
            'layer': {'sum_of_operator_us': round(sum_us, 1), 'sum_of_roofline_us': round(ideal_us, 1),
                      'frac_of_summed_roofline': round(ideal_us / sum_us, 3),
                      # the same ideal against the device time of a whole step (kernels overlap their
                      # neighbours' ramp-up and tail under programmatic dependent launch)
                      'roofline_us_over_step_us': round(ideal_us / (ms_per_step * 1e3), 3),
                      # the reference's own operator list (32 separate operators: 142*T*E + 14*S bytes of
                      # elementwise traffic, 72*E^2*T + 12*B*L^2*E flops) at the measured copy bandwidth and the
                      # sustained tensor rate, which is the figure that applies inside a long step
                      'reference_list_roofline_us': round(ref_list_us, 1),
                      'reference_list_roofline_over_step': round(ref_list_us / (ms_per_step * 1e3), 3)},
            'operators': ops,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_stack(args):
    """--layers N > 1: a stack of N layers with independent weights (the 24-layer stack configuration at N=24);
    one step = forward through all layers + backward through all layers, each layer's gradient
    bucket allreduced while the next layer's backward runs."""
    import torch
    import torch.distributed as dist
    from substation_b200 import ops as _ops
    from substation_b200.stack import EncoderStack
    from tests.layer_harness import get_layouts
    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local_rank = int(os.environ.get('LOCAL_RANK', '0'))
    if world != args.gpus:
        raise SystemExit(f'--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run')
    torch.cuda.set_device(local_rank)
    dev = torch.device('cuda', local_rank)
    if world > 1:
        opts = dist.ProcessGroupNCCL.Options()
        opts.config.max_ctas = args.comm_ctas
        opts.config.min_ctas = min(4, args.comm_ctas)
        dist.init_process_group('nccl', device_id=dev, pg_options=opts)
        _ops.set_sm_budget(torch.cuda.get_device_properties(dev).multi_processor_count - args.comm_ctas)
    lay = get_layouts(args.layouts)
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
    ap.add_argument('--comm-ctas', type=int, default=4, help='SMs left to NCCL when N > 1')
    ap.add_argument('--early-allreduce', type=int, default=0,
                    help='N > 1: sum the feed-forward gradients beside the attention half of backward (1) or the whole '
                         'bucket beside the next step (0)')
    ap.add_argument('--layers', type=int, default=1, help='>1: time a stack of layers (config 5 uses 24)')
    ap.add_argument('--keep-all', type=int, default=0,
                    help='1: also store the nine intermediates nothing reads again (what enable_debug does)')
    ap.add_argument('--no-e2e', action='store_true')
    ap.add_argument('--no-cpu', action='store_true')
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == 'ours':
        args.warmup = 3
    if args.impl == 'reference':
        run_reference_arm(args)
    elif args.layers > 1:
        run_stack(args)
    else:
        run_ours(args)


if __name__ == '__main__':
    main()
