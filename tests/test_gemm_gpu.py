"""Contraction parity on the GPU: the tcgen05 kernel and the SIMT fallback against
numpy float64 matmul, over the eight operand-major combinations the reference maps to
cuBLAS op flags (pytorch_module/gemm.cuh:71-89), ragged extents, batching, and the
layer's own einsums under both shipped layout configurations."""

import numpy as np
import pytest
import torch

from oracle import encoder_oracle as orc
from tests.gpu_util import DEV, assert_close, get, h16

pytestmark = pytest.mark.gpu


def _ops():
    from substation_b200 import ops
    return ops


def _operand(rng, batch, rows, k, rows_major, pad=0):
    """fp16 operand [batch, rows, k] stored k-innermost (rows_major False) or
    rows-innermost (True); returns (float64 values, logical-order device view)."""
    a = h16(rng.normal(0, 1, (batch, rows, k)) / np.sqrt(k))
    if rows_major:
        st = torch.zeros(batch, k, rows + pad, dtype=torch.float16, device=DEV)
        st[..., :rows] = torch.from_numpy(a.transpose(0, 2, 1).copy()).to(DEV, torch.float16)
        view = st[..., :rows].permute(0, 2, 1)
    else:
        st = torch.zeros(batch, rows, k + pad, dtype=torch.float16, device=DEV)
        st[..., :k] = torch.from_numpy(a).to(DEV, torch.float16)
        view = st[..., :k]
    return a, view


SHAPES = [  # batch, M, N, K
    (1, 128, 256, 64), (1, 256, 512, 256), (3, 200, 136, 72), (2, 64, 512, 512), (4, 512, 64, 64),
    (1, 128, 128, 64 * 21), (2, 384, 320, 200), (1, 1024, 1024, 1024),
]


@pytest.mark.parametrize('batch,M,N,K', SHAPES)
@pytest.mark.parametrize('a_mn,b_mn,c_mn', [(a, b, c) for a in (0, 1) for b in (0, 1) for c in (0, 1)])
def test_tcgen05_all_operand_majors(batch, M, N, K, a_mn, b_mn, c_mn):
    ops = _ops()
    rng = np.random.default_rng(M * 7 + N * 3 + K + a_mn * 4 + b_mn * 2 + c_mn)
    pad = 8  # rows are not dense: strides differ from extents
    A, dA = _operand(rng, batch, M, K, bool(a_mn), pad)
    B, dB = _operand(rng, batch, N, K, bool(b_mn), pad)
    if c_mn:
        st = torch.full((batch, N, M + pad), float('nan'), dtype=torch.float16, device=DEV)
        dC = st[..., :M].permute(0, 2, 1)
    else:
        st = torch.full((batch, M, N + pad), float('nan'), dtype=torch.float16, device=DEV)
        dC = st[..., :N]
    used = ops.einsum('bmk,bnk->bmn', dA, dB, dC, alpha=0.5, impl='tcgen05')
    assert used == 'tcgen05'
    assert ops.device_error() == 0
    want = 0.5 * np.einsum('bmk,bnk->bmn', A, B)
    assert_close(dC, want, tol=2e-3, what=f'C a_mn={a_mn} b_mn={b_mn} c_mn={c_mn}')
    # the padding columns must be untouched
    assert torch.isnan(st[..., -pad:]).all()


@pytest.mark.parametrize('batch,M,N,K', [(1, 70, 50, 33), (3, 128, 64, 100), (2, 5, 7, 3)])
def test_simt_fallback_and_auto_dispatch(batch, M, N, K):
    ops = _ops()
    rng = np.random.default_rng(K)
    A, dA = _operand(rng, batch, M, K, False)
    B, dB = _operand(rng, batch, N, K, True)
    dC = torch.full((batch, M, N), float('nan'), dtype=torch.float16, device=DEV)
    assert ops.einsum('bmk,bnk->bmn', dA, dB, dC, impl='simt') == 'simt'
    want = np.einsum('bmk,bnk->bmn', A, B)
    assert_close(dC, want, tol=2e-3, what='simt')
    dC.fill_(float('nan'))
    used = ops.einsum('bmk,bnk->bmn', dA, dB, dC, impl='auto')
    assert used in ('tcgen05', 'simt')
    assert_close(dC, want, tol=2e-3, what='auto')


def test_tcgen05_rejects_what_tma_cannot_address():
    ops = _ops()
    from substation_b200._lib import SubstationError
    a = torch.zeros(1, 16, 33, dtype=torch.float16, device=DEV)   # row stride 66 bytes
    b = torch.zeros(1, 16, 33, dtype=torch.float16, device=DEV)
    c = torch.zeros(1, 16, 16, dtype=torch.float16, device=DEV)
    with pytest.raises(SubstationError) as e:
        ops.einsum('bmk,bnk->bmn', a, b, c, impl='tcgen05')
    assert e.value.status in (3, 5)
    assert ops.einsum('bmk,bnk->bmn', a, b, c, impl='auto') == 'simt'


def _layer_einsums(lay):
    """(name, spec in memory-order letters) for the 18 contractions of
    pytorch_module/encoder.cu:87-299 under layout table ``lay``."""
    kk = lay['KKQQVV'][1:]
    dkk = lay['DKKQQVV'][1:]
    r = lambda s: s.replace('J', 'K')
    return [
        ('QKV-fused', lay['X'], lay['WKQV'], lay['WKKWQQWVV']),
        ('QKT', r(kk), kk, lay['BETA']),
        ('gamma', r(kk), lay['ATTN_DROP'], lay['GAMMA']),
        ('out', lay['WO'], lay['GAMMA'], lay['ATT']),
        ('lin1', lay['SB1'], lay['LINW1'], lay['SB1_LINW1']),
        ('lin2', lay['DROP2'], lay['LINW2'], lay['DROP2_LINW2']),
        ('dXlin2', lay['DLIN2'], lay['LINW2'], lay['DDROP2']),
        ('dWlin2', lay['DLIN2'], lay['DROP2'], lay['LINW2']),
        ('dXlin1', lay['DLIN1'], lay['LINW1'], lay['DLIN1_LINW1']),
        ('dWlin1', lay['DLIN1'], lay['SB1'], lay['LINW1']),
        ('dWout', lay['GAMMA'], lay['DATT'], lay['WO']),
        ('dXout', lay['WO'], lay['DATT'], lay['DGAMMA']),
        ('dX1gamma', r(kk), lay['DGAMMA'], lay['DATTN_DROP']),
        ('dX2gamma', lay['DGAMMA'], lay['ATTN_DROP'], r(dkk)),
        ('dX1QKT', r(kk), lay['DBETA'], dkk),
        ('dX2QKT', kk, lay['DBETA'], r(dkk)),
        ('dXQKV-fused', lay['WKQV'], lay['DKKQQVV'], lay['DXATT']),
        ('dWQKV-fused', lay['X'], lay['DKKQQVV'], lay['WKQV']),
    ]


@pytest.mark.parametrize('which', ['uniform', 'b8_l512', 'b96_l128'])
def test_layer_einsums_run_on_tensor_cores(which):
    """Every contraction of the layer, with the operand layouts of each configuration,
    must qualify for the tcgen05 kernel and match numpy."""
    ops = _ops()
    from substation_b200 import layouts as L
    from tests.layer_harness import get_layouts
    lay = L.validate(get_layouts(which))
    sizes = L.sizes_map(2, 128, 2, 128)   # B=2, L=128, H=2, P=64
    rng = np.random.default_rng(1)
    for name, ad, bd, cd in _layer_einsums(lay):
        shp = lambda d: tuple(sizes[c] for c in d)
        ksz = np.prod([sizes[c] for c in ad if c in bd and c not in cd])
        A = h16(rng.normal(0, 1, shp(ad)) / np.sqrt(ksz))
        B = h16(rng.normal(0, 1, shp(bd)))
        dA = torch.from_numpy(A).to(DEV, torch.float16)
        dB = torch.from_numpy(B).to(DEV, torch.float16)
        dC = torch.full(shp(cd), float('nan'), dtype=torch.float16, device=DEV)
        spec = f'{ad.lower()},{bd.lower()}->{cd.lower()}'
        used = ops.einsum(spec, dA, dB, dC, impl='auto')
        assert used == 'tcgen05', f'{name} ({spec}) fell back to {used}'
        want = np.einsum(spec, A, B)
        assert_close(dC, want, tol=2e-3, what=f'{which}:{name} {spec}')
    assert ops.device_error() == 0


@pytest.mark.parametrize('M,N,K,c_mn', [(1024, 1024, 4096, 0), (3072, 1024, 4096, 0), (256, 512, 2048, 1),
                                        (384, 1000, 8192, 0)])
def test_split_k_with_workspace_matches_unsplit(M, N, K, c_mn):
    """Few output tiles and a long summed extent: with a workspace the kernel splits K over
    more SMs and reduces fp32 partials in a fixed order; results must match numpy and be
    reproducible bit for bit."""
    ops = _ops()
    rng = np.random.default_rng(M + N + K)
    A, dA = _operand(rng, 1, M, K, True)       # both operands token-major, as in the weight gradients
    B, dB = _operand(rng, 1, N, K, True)
    ws = torch.empty(64 << 20, dtype=torch.uint8, device=DEV)
    shape = (1, N, M) if c_mn else (1, M, N)
    outs = []
    for _ in range(2):
        st = torch.full(shape, float('nan'), dtype=torch.float16, device=DEV)
        dC = st.permute(0, 2, 1) if c_mn else st
        assert ops.einsum('bmk,bnk->bmn', dA, dB, dC, alpha=0.25, impl='tcgen05', workspace=ws) == 'tcgen05'
        outs.append(st.clone())
        want = 0.25 * np.einsum('bmk,bnk->bmn', A, B)
        assert_close(dC, want, tol=2e-3, what='split-K C')
    assert torch.equal(outs[0], outs[1])
    assert ops.device_error() == 0


def test_split_k_with_workspace_for_batched_problems():
    """Batched problems with few tiles keep the workspace form of split-K (fp32 partials, fixed-order reduce
    kernel): two batches of 256 x 256 over K = 4096, reproducible bit for bit."""
    ops = _ops()
    rng = np.random.default_rng(11)
    A, dA = _operand(rng, 2, 256, 4096, True)
    B, dB = _operand(rng, 2, 256, 4096, True)
    ws = torch.empty(64 << 20, dtype=torch.uint8, device=DEV)
    outs = []
    for _ in range(2):
        dC = torch.full((2, 256, 256), float('nan'), dtype=torch.float16, device=DEV)
        assert ops.einsum('bmk,bnk->bmn', dA, dB, dC, alpha=0.25, impl='tcgen05', workspace=ws) == 'tcgen05'
        assert_close(dC, 0.25 * np.einsum('bmk,bnk->bmn', A, B), tol=2e-3, what='batched split-K C')
        outs.append(dC)
    assert torch.equal(outs[0], outs[1])
    assert ops.device_error() == 0


@pytest.mark.parametrize('M,N,K', [(1024, 1024, 4096), (304, 520, 2080), (512, 768, 16384)])
@pytest.mark.parametrize('a_mn,b_mn', [(0, 0), (1, 1), (1, 0)])
def test_split_k_inside_a_cluster(M, N, K, a_mn, b_mn):
    """Few 256 x 256 tiles and a long K without a workspace: four CTA pairs per tile share K and add their
    partial accumulators up through distributed shared memory.  Ragged M and N, a K that does not divide into four
    equal parts, both operand majors; the result must match fp32 and repeat bit for bit."""
    ops = _ops()
    g = torch.Generator(device=DEV).manual_seed(M + N + K)
    A = (torch.randn(1, M, K, device=DEV, generator=g) / K ** 0.5).half()
    B = torch.randn(1, N, K, device=DEV, generator=g).half()
    dA = A.transpose(1, 2).contiguous().transpose(1, 2) if a_mn else A
    dB = B.transpose(1, 2).contiguous().transpose(1, 2) if b_mn else B
    ref = 0.5 * torch.einsum('bmk,bnk->bmn', A.float(), B.float())
    outs = []
    for _ in range(2):
        dC = torch.full((1, M, N), float('nan'), dtype=torch.float16, device=DEV)
        assert ops.einsum('bmk,bnk->bmn', dA, dB, dC, alpha=0.5, impl='tcgen05') == 'tcgen05'
        assert ops.device_error() == 0
        assert torch.isfinite(dC).all()
        assert ((dC.float() - ref).norm() / ref.norm()).item() < 1e-3
        outs.append(dC)
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize('M,N,K', [(4096, 4096, 1024), (2000, 1544, 520), (4096, 1024, 4096)])
@pytest.mark.parametrize('a_mn,b_mn,c_mn', [(0, 0, 0), (1, 0, 0), (0, 1, 0), (1, 1, 1)])
def test_paired_cta_kernel_on_large_problems(M, N, K, a_mn, b_mn, c_mn):
    """Problems with enough 256 x 256 tiles run on the two-CTA kernel (tcgen05.mma.cta_group::2);
    checked against an fp32 torch matmul (too large for the float64 oracle), ragged edges included."""
    ops = _ops()
    g = torch.Generator(device=DEV).manual_seed(M + K)
    A = (torch.randn(1, M, K, device=DEV, generator=g) / K ** 0.5).half()
    B = torch.randn(1, N, K, device=DEV, generator=g).half()
    dA = A.transpose(1, 2).contiguous().transpose(1, 2) if a_mn else A
    dB = B.transpose(1, 2).contiguous().transpose(1, 2) if b_mn else B
    st = torch.full((1, N, M) if c_mn else (1, M, N), float('nan'), dtype=torch.float16, device=DEV)
    dC = st.transpose(1, 2) if c_mn else st
    assert ops.einsum('bmk,bnk->bmn', dA, dB, dC, alpha=2.0, impl='tcgen05') == 'tcgen05'
    assert ops.device_error() == 0
    ref = 2.0 * torch.einsum('bmk,bnk->bmn', A.float(), B.float())
    assert torch.isfinite(dC).all()
    assert ((dC.float() - ref).norm() / ref.norm()).item() < 1e-3


def _rand(shape, scale=1.0, seed=0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(*shape, device=DEV, generator=g) * scale).half()


def test_fused_epilogue_bias_matches_einsum_then_input_biases():
    """QKV projection with the attention input biases in its epilogue (bias along the rows of the swapped
    problem) against sb_einsum followed by sb_attention_input_biases: bit-identical."""
    ops = _ops()
    B, J, I, Q, P, H = 4, 512, 256, 3, 64, 8
    x, w, bias = _rand((B, J, I), 1, 1), _rand((Q, P, H, I), 0.05, 2), _rand((Q, P, H), 0.5, 3)
    c, out2 = (torch.empty(Q, P, H, B, J, device=DEV, dtype=torch.float16) for _ in range(2))
    ops.einsum_fused('bji,qphi->qphbj', x, w, c, kind='bias', bias=bias, bias_dims='qph', out2=out2)
    c_ref, out_ref = torch.empty_like(c), torch.empty_like(c)
    ops.einsum('bji,qphi->qphbj', x, w, c_ref)
    ops.attention_input_biases(c_ref, bias, out_ref)
    assert ops.device_error() == 0
    assert torch.equal(c, c_ref) and torch.equal(out2, out_ref)
    want = np.einsum('bji,qphi->qphbj', get(x), get(w))
    assert_close(c, want, what='c')
    assert_close(out2, want + get(bias)[..., None, None], what='c + bias')


def test_fused_epilogue_residual_matches_einsum_then_encoder_input():
    ops = _ops()
    B, J, I, Q, P, H = 4, 512, 1280, 3, 64, 4
    w, d, resid = _rand((Q, P, H, I), 0.05, 4), _rand((Q, P, H, B, J), 1, 5), _rand((B, J, I), 1, 6)
    c, out2 = (torch.empty(B, J, I, device=DEV, dtype=torch.float16) for _ in range(2))
    ops.einsum_fused('qphi,qphbj->bji', w, d, c, kind='residual', resid=resid, out2=out2)
    c_ref, out_ref = torch.empty_like(c), torch.empty_like(c)
    ops.einsum('qphi,qphbj->bji', w, d, c_ref)
    ops.backward_encoder_input(c_ref, resid, out_ref)
    assert ops.device_error() == 0
    assert torch.equal(c, c_ref) and torch.equal(out2, out_ref)
    assert_close(c, np.einsum('qphi,qphbj->bji', get(w), get(d)), what='c')


@pytest.mark.parametrize('mode', ['explicit', 'philox'])
@pytest.mark.parametrize('activation', ['relu', 'gelu'])
def test_fused_epilogue_bias_activation_dropout_matches_separate_operator(mode, activation):
    ops = _ops()
    B, J, I, U = 4, 512, 256, 1280
    x, w, bias = _rand((B, J, I), 1, 7), _rand((I, U), 0.08, 8), _rand((U,), 0.5, 9)
    g = torch.Generator(device=DEV).manual_seed(10)
    mask = (torch.rand(B, J, U, device=DEV, generator=g) >= 0.1).to(torch.uint8)
    mask_ref = mask.clone()
    c, lin1, drop2 = (torch.empty(B, J, U, device=DEV, dtype=torch.float16) for _ in range(3))
    ops.einsum_fused('bji,iu->bju', x, w, c, kind='bias_act_dropout', bias=bias, bias_dims='u', mask=mask, out2=lin1,
                     out3=drop2, activation=activation, p=0.1, mode=mode, seed=21, offset=2, logical_dims='bju')
    c_ref, lin_ref, drop_ref = (torch.empty_like(c) for _ in range(3))
    ops.einsum('bji,iu->bju', x, w, c_ref)
    ops.bias_activation_dropout(c_ref, bias, mask_ref, lin_ref, drop_ref, activation=activation, p=0.1, mode=mode,
                                seed=21, offset=2)
    assert ops.device_error() == 0
    assert torch.equal(mask, mask_ref)
    if mode == 'philox':
        assert np.array_equal(get(mask).astype(np.uint8), orc.philox_mask((B, J, U), 0.1, 21, 2))
    assert torch.equal(c, c_ref) and torch.equal(lin1, lin_ref) and torch.equal(drop2, drop_ref)


def test_fused_epilogue_declines_small_problems():
    ops = _ops()
    from substation_b200._lib import SubstationError
    x, w, bias = _rand((2, 64, 128)), _rand((128, 256)), _rand((256,))
    c, out2 = (torch.empty(2, 64, 256, device=DEV, dtype=torch.float16) for _ in range(2))
    with pytest.raises(SubstationError) as e:
        ops.einsum_fused('bji,iu->bju', x, w, c, kind='bias', bias=bias, bias_dims='u', out2=out2)
    assert e.value.status == 3


@pytest.mark.parametrize('kind', ['bias', 'residual', 'bias_act_dropout'])
def test_fused_epilogue_can_discard_c(kind):
    """discard_c: the contraction's own output is not stored (it stays as the caller left it), the fused outputs
    keep their bits."""
    ops = _ops()
    B, J, I, U = 4, 512, 256, 1280
    x, w, bias, resid = _rand((B, J, I), 1, 7), _rand((I, U), 0.08, 8), _rand((U,), 0.5, 9), _rand((B, J, U), 1, 11)
    g = torch.Generator(device=DEV).manual_seed(10)
    mask = (torch.rand(B, J, U, device=DEV, generator=g) >= 0.1).to(torch.uint8)
    res = {}
    for discard in (False, True):
        c = torch.full((B, J, U), 7.0, device=DEV, dtype=torch.float16)
        out2, out3 = (torch.full((B, J, U), float('nan'), device=DEV, dtype=torch.float16) for _ in range(2))
        kw = dict(kind=kind, out2=out2, discard_c=discard)
        if kind != 'residual':
            kw.update(bias=bias, bias_dims='u')
        if kind == 'residual':
            kw.update(resid=resid)
        if kind == 'bias_act_dropout':
            kw.update(mask=mask, out3=out3, p=0.1)
        ops.einsum_fused('bji,iu->bju', x, w, c, **kw)
        res[discard] = (c, out2, out3)
    assert ops.device_error() == 0
    assert (res[True][0] == 7.0).all() and not (res[False][0] == 7.0).all()
    assert torch.equal(res[True][1], res[False][1])
    if kind == 'bias_act_dropout':
        assert torch.equal(res[True][2], res[False][2])


@pytest.mark.parametrize('bf16', [False, True])
def test_mma_peak_probe_runs_and_reports_its_flops(bf16):
    """The MMA-only launch the bench uses as the tensor-pipe yardstick: completes without a bounded wait running
    out, and a longer launch takes longer (the instructions are really issued)."""
    ops = _ops()
    times = []
    for k_blocks in (256, 4096):
        ops.mma_peak_probe(64, bf16)                 # warm-up
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        flops = ops.mma_peak_probe(k_blocks, bf16)
        e.record()
        torch.cuda.synchronize()
        assert flops == pytest.approx(flops // (k_blocks * 4 * 2 * 256 * 256 * 16) * k_blocks * 4 * 2 * 256 * 256 * 16)
        times.append((s.elapsed_time(e), flops))
    assert ops.device_error() == 0
    (t0, f0), (t1, f1) = times
    assert t1 > 4 * t0 and f1 == 16 * f0
    assert 100e12 < f1 / (t1 * 1e-3) < 3000e12, f'{f1 / (t1 * 1e-3) / 1e12:.0f} TFLOP/s is not a plausible tensor rate'


def test_bfloat16_build_contractions_and_epilogue():
    """bfloat16 operands go to the bf16 build of the library (the MMA instruction descriptor and the conversions are
    all that differs): paired-CTA contraction with a fused bias epilogue, a batched attention-shaped contraction, and
    the SIMT fall-back, against float64 einsums.  Tolerance 2e-2 (bf16 keeps 8 significant bits)."""
    ops = _ops()
    g = torch.Generator(device=DEV).manual_seed(3)
    rnd = lambda *s, std=1.0: (torch.randn(*s, device=DEV, generator=g) * std).to(torch.bfloat16)
    f64 = lambda t: t.double().cpu().numpy()
    B, J, I, U = 4, 512, 256, 1280
    x, w, bias = rnd(B, J, I), rnd(I, U, std=0.08), rnd(U, std=0.5)
    c, out2 = (torch.empty(B, J, U, device=DEV, dtype=torch.bfloat16) for _ in range(2))
    ops.einsum_fused('bji,iu->bju', x, w, c, kind='bias', bias=bias, bias_dims='u', out2=out2)
    want = np.einsum('bji,iu->bju', f64(x), f64(w))
    assert orc.rel_l2(f64(c), want) < 2e-2 and orc.rel_l2(f64(out2), want + f64(bias)) < 2e-2
    q, k = rnd(64, 2, 3, 256), rnd(64, 2, 3, 256)
    s = torch.empty(2, 3, 256, 256, device=DEV, dtype=torch.bfloat16)
    assert ops.einsum('phbk,phbj->hbjk', k, q, s, alpha=0.125) == 'tcgen05'
    assert orc.rel_l2(f64(s), 0.125 * np.einsum('phbk,phbj->hbjk', f64(k), f64(q))) < 2e-2
    a, b = rnd(37, 21), rnd(13, 21)
    o = torch.empty(37, 13, device=DEV, dtype=torch.bfloat16)
    ops.einsum('mk,nk->mn', a, b, o, impl='simt')
    assert orc.rel_l2(f64(o), f64(a) @ f64(b).T) < 2e-2
    with pytest.raises(TypeError):
        ops.einsum('mk,nk->mn', a, b.half(), o)
    assert ops.device_error() == 0
