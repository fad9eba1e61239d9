"""Host-side shell: constructor/forward contract, buffer names, draw-once
projection, mask types -- everything that does not need a GPU."""
import copy
import math

import pytest
import torch

import fly_b200
from fly_b200 import FullMask, LengthMask, SBLocalAttention, TriangularCausalMask
from oracle import ref_bridge
from oracle import sblocal_oracle as so


def test_constructor_defaults_and_buffer_names():
    layer = SBLocalAttention(49, 64)
    assert layer.local_context == 49 and layer.causal is False and layer.softmax_eps == 0.0
    assert layer.feature_map.n_features == int(64 * math.log(64)) == 266
    sd = layer.state_dict()
    assert list(sd) == ['feature_map.projection_matrix']
    assert sd['feature_map.projection_matrix'].shape == (64, 266)       # placeholder before the first forward
    assert layer.feature_map._calls == -1
    assert isinstance(layer.dropout, torch.nn.Dropout)
    layer2 = SBLocalAttention(256, 64, 256, softmax_temp=147 ** -0.5, device='cpu', dtype=torch.float32)
    assert layer2.feature_map.softmax_temp == 147 ** -0.5


def test_projection_is_drawn_once_and_matches_the_seeded_draw():
    layer = SBLocalAttention(16, 32, 64)
    torch.manual_seed(5)
    layer.feature_map.new_feature_map('cpu')
    W1 = layer.feature_map.projection_matrix.clone()
    assert W1.shape == (32, 32)
    layer.feature_map.new_feature_map('cpu')
    layer.feature_map.new_feature_map('cpu')
    assert torch.equal(layer.feature_map.projection_matrix, W1)
    torch.manual_seed(5)
    assert torch.equal(W1, so.gaussian_orthogonal_random_matrix(32, 32))
    clone = copy.deepcopy(layer)
    assert torch.equal(clone.feature_map.projection_matrix, W1)
    assert 'feature_map.projection_matrix' in layer.state_dict()


@pytest.mark.skipif(not ref_bridge.reference_available(), reason='reference tree not present')
def test_same_seed_same_projection_as_reference_module():
    ref = ref_bridge.load_reference()
    torch.manual_seed(9)
    a = ref.SBLocalAttention(8, 16, 40)
    a.feature_map.new_feature_map('cpu')
    torch.manual_seed(9)
    b = SBLocalAttention(8, 16, 40)
    b.feature_map.new_feature_map('cpu')
    assert torch.equal(a.feature_map.projection_matrix, b.feature_map.projection_matrix)
    assert a.state_dict().keys() == b.state_dict().keys()


def test_cpu_tensors_raise_instead_of_falling_back():
    layer = SBLocalAttention(4, 8, 8).eval()
    q = torch.randn(1, 5, 1, 8)
    with pytest.raises(ValueError, match='CUDA'):
        layer(q, q, q)


def test_unbuilt_options_raise():
    q = torch.randn(1, 5, 1, 8)
    with pytest.raises(NotImplementedError):
        SBLocalAttention(4, 8, 8, causal=True)(q, q, q)
    with pytest.raises(ValueError, match='CUDA'):
        SBLocalAttention(4, 8, 8).eval()(q, q, q, need_weights=True)
    with pytest.raises(NotImplementedError):
        SBLocalAttention(4, 8, 8, attention_dropout=0.1).train()(q, q, q)
    mask = FullMask(torch.rand(5, 5) > 0.5)
    with pytest.raises(NotImplementedError):
        SBLocalAttention(4, 8, 8).eval()(q, q, q, attn_mask=mask)


def test_masks():
    lm = LengthMask(torch.tensor([3, 1, 5]), max_len=5)
    assert lm.bool_matrix.tolist() == [[1, 1, 1, 0, 0], [1, 0, 0, 0, 0], [1, 1, 1, 1, 1]]
    assert lm.lengths.tolist() == [3, 1, 5] and not lm.all_ones
    assert LengthMask(torch.tensor([5, 5]), max_len=5).all_ones
    fm = FullMask(4, 6)
    assert fm.shape == (4, 6) and bool(fm.all_ones)
    assert FullMask(N=3).shape == (3, 3)
    bm = FullMask(torch.tensor([[True, True, False], [True, False, False]]))
    assert bm.lengths.tolist() == [2, 1]
    assert bm.additive_matrix_finite[0].tolist() == [0.0, 0.0, float(torch.tensor(-1e24))]
    with pytest.raises(ValueError):
        FullMask(torch.tensor([[True, False, True]])).lengths
    with pytest.raises(ValueError):
        FullMask(torch.ones(2, 2))
    tm = TriangularCausalMask(4)
    assert tm.lower_triangular and tm.lengths.tolist() == [1, 2, 3, 4]


def test_package_exports():
    for name in ('SBLocalAttention', 'SBPerformerFeatures', 'gaussian_orthogonal_random_matrix', 'LengthMask'):
        assert hasattr(fly_b200, name)


def test_dropin_registers_the_reference_module_path():
    import importlib
    import sys
    from fly_b200 import dropin
    saved = {k: sys.modules.get(k) for k in ('src', 'src.models', 'src.models.attention', dropin.TARGET)}
    try:
        _check_dropin(dropin, importlib)
    finally:
        # leave the interpreter as found: other tests import the reference's own module under this name
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v
        parent = sys.modules.get('src.models.attention')
        if parent is not None and saved[dropin.TARGET] is None and hasattr(parent, 'sblocal_attention'):
            delattr(parent, 'sblocal_attention')


def _check_dropin(dropin, importlib):
    dropin.install()
    mod = importlib.import_module('src.models.attention.sblocal_attention')
    assert mod.SBLocalAttention is SBLocalAttention
    # what hydra.utils.instantiate does with a _target_ string: locate, then call with the config's kwargs
    path, _, name = 'src.models.attention.sblocal_attention.SBLocalAttention'.rpartition('.')
    cls = getattr(importlib.import_module(path), name)
    layer = cls(dim_heads=64, local_context=49, nb_features=24, softmax_temp=147 ** -0.5)
    assert isinstance(layer, SBLocalAttention) and layer.feature_map.n_features == 24
