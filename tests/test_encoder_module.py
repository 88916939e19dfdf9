"""CPU checks of the host-side mirror of pytorch_module/encoder.py: constructor
contract, parameter shapes and names, layout validation, state_dict round trip."""

import copy

import pytest
import torch

from substation_b200 import Encoder, layouts as L
from tests.layer_harness import get_layouts


@pytest.mark.parametrize('which', ['uniform', 'b8_l512', 'b96_l128'])
def test_constructor_mirrors_reference(which):
    lay = get_layouts(which)
    enc = Encoder('/tmp/unused', 2, 16, 4, 64, lay, torch.float16, 0.1, 0.2, 0.3, 0.4)
    assert (enc.batch_size, enc.max_seq_len, enc.num_heads, enc.embedding_size) == (2, 16, 4, 64)
    assert enc.proj_size == 16 and enc.intermediate_size == 256
    assert enc.softmax_dropout_probability == 0.1 and enc.residual2_dropout_probability == 0.4
    assert enc.layouts is lay and enc.debug == {}
    sizes = L.sizes_map(2, 16, 4, 64)
    assert [n for n, _ in enc.named_parameters()] == [n for n, _ in lay['params']]
    for (name, layout), prm in zip(lay['params'], enc.params):
        assert prm is getattr(enc, name)
        assert tuple(prm.shape) == tuple(sizes[c] for c in layout) and prm.dtype == torch.float16
        assert prm.float().abs().max() <= 2 ** -0.5 + 1e-3      # uniform(+-1/sqrt 2)
    fwd, bwd = enc.intermediate_bytes()
    assert fwd > 0 and bwd > 0


def test_state_dict_round_trip():
    lay = L.uniform_layouts()
    a = Encoder('/tmp/unused', 2, 8, 2, 16, lay, torch.float16, 0, 0, 0, 0)
    b = Encoder('/tmp/unused', 2, 8, 2, 16, lay, torch.float16, 0, 0, 0, 0)
    b.load_state_dict(a.state_dict())
    for x, y in zip(a.params, b.params):
        assert torch.equal(x, y)


def test_rejections():
    lay = L.uniform_layouts()
    with pytest.raises(NotImplementedError):
        Encoder('/tmp/unused', 2, 8, 2, 16, lay, torch.float64, 0, 0, 0, 0)
    with pytest.raises(ValueError):
        Encoder('/tmp/unused', 2, 8, 3, 16, lay, torch.float16, 0, 0, 0, 0)
    with pytest.raises(ValueError):
        Encoder('/tmp/unused', 2, 8, 2, 16, lay, torch.float16, 0, 0, 0, 0, activation='swish')
    bad = copy.deepcopy(lay)
    bad['forward_interm'][2] = ('BETA', 'HBJ')
    with pytest.raises(L.LayoutError):
        Encoder('/tmp/unused', 2, 8, 2, 16, bad, torch.float16, 0, 0, 0, 0)
    bad = copy.deepcopy(lay)
    bad['params'] = bad['params'][:-1]
    with pytest.raises(L.LayoutError):
        L.validate(bad)
    bad = copy.deepcopy(lay)
    bad['forward_interm'][0] = ('KKQQVV', 'PQHBJ')
    with pytest.raises(L.LayoutError):
        L.validate(bad)
    enc = Encoder('/tmp/unused', 2, 8, 2, 16, lay, torch.float16, 0, 0, 0, 0)
    with pytest.raises(ValueError):          # no CPU path
        enc(torch.zeros(2, 8, 16, dtype=torch.float16))
    with pytest.raises(ValueError):
        enc.set_masks({n: torch.zeros(1, dtype=torch.uint8) for n in L.MASKS})


def test_shipped_configurations_validate():
    for which in ('b8_l512', 'b96_l128'):
        t = L.validate(get_layouts(which))
        assert len(t) == 51 and t['X'] == t['SB2']


def test_early_gradient_part_is_a_suffix_of_the_bucket():
    """The gradients that are final before the attention half of backward form the tail of the bucket."""
    enc = Encoder('/tmp/unused', 2, 8, 2, 16, L.uniform_layouts(), torch.float16, 0, 0, 0, 0)
    plan, total = enc._grad_plan
    off = enc.early_grad_offset()
    names = [n for n, _, _, o, _ in plan if o >= off]
    assert names == ['BO', 'S1', 'B1', 'LINB1', 'LINW1', 'S2', 'B2', 'LINB2', 'LINW2']
    assert 0 < off < total and off % 2 == 0


def test_pointer_tables_are_remembered_per_arena():
    """With a buffer pool the same arenas return every step: their pointer tables are built once, hold the plan's
    offsets, follow the caller's masks, and are forgotten when the pool is set up again."""
    enc = Encoder('/tmp/unused', 2, 8, 2, 16, L.uniform_layouts(), torch.float16, 0, 0, 0, 0)
    plan, total = enc._fwd_plan
    a = torch.empty(max(total, 1), dtype=torch.uint8)
    b = torch.empty(max(total, 1), dtype=torch.uint8)
    t1 = enc._pooled_ptrs('fwd', plan, a, {})
    assert enc._pooled_ptrs('fwd', plan, a, {}) is t1
    t2 = enc._pooled_ptrs('fwd', plan, b, {})
    assert t2 is not t1
    for i, (_, _, _, off, _) in enumerate(plan):
        assert t1[i] == a.data_ptr() + off and t2[i] == b.data_ptr() + off
    name = plan[0][0]
    m = torch.empty(4, dtype=torch.uint8)
    t3 = enc._pooled_ptrs('fwd', plan, a, {name: m})
    assert t3 is not t1 and t3[0] == m.data_ptr() and t3[1] == t1[1]
    enc.set_buffer_pool(2)
    assert enc._pooled_ptrs('fwd', plan, a, {}) is not t1
