"""Whole T2T-ViT-t-14 forward with SBLocal attention (window 256, 256 features) in both token-to-token stages.

Two links tie the CUDA model to the reference model:
  1. CPU, needs the reference tree: the unmodified reference `t2t_vit_t_14` (built through the import-only
     stand-ins under tests/shims) and `fly_b200.t2t_vit` with a CPU-oracle attention give the same logits from one
     `state_dict` (which carries both projection matrices).
  2. GPU: `fly_b200.t2t_vit` with `fly_b200.SBLocalAttention` on CUDA against the same wiring with the CPU-oracle
     attention, same weights and projections, 2 images of 3 x 224 x 224.
Random-init weights (seed 0) and N(0,1) images stand in for the ImageNet checkpoint and data, which are not
available offline.
"""
import importlib
import os
import sys

import pytest
import torch
import torch.nn as nn

from oracle import ref_bridge
from oracle import sblocal_oracle as so

SHIMS = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'shims')
W_CTX, N_FEAT = 256, 256


class OracleSBLocal(nn.Module):
    """CPU attention with the reference module's state layout (`feature_map.projection_matrix`), computed by the
    oracle restatement."""

    def __init__(self, softmax_temp, W=None):
        super().__init__()
        self.softmax_temp = softmax_temp
        self.feature_map = nn.Module()
        self.feature_map.register_buffer('projection_matrix', torch.zeros(N_FEAT // 2, 64) if W is None else W.clone())

    def forward(self, q, k, v):
        out, _ = so.sblocal_forward(q, k, v, self.feature_map.projection_matrix, W_CTX, self.softmax_temp)
        return out, None


def _oracle_model():
    from fly_b200 import t2t_vit
    mk = lambda softmax_temp: OracleSBLocal(softmax_temp)
    return t2t_vit.t2t_vit_t_14(mk, mk).eval()


@pytest.mark.skipif(not ref_bridge.reference_available(), reason='reference tree not present')
def test_wiring_matches_reference_model():
    ref_bridge.load_reference()
    if SHIMS not in sys.path:
        sys.path.append(SHIMS)          # behind site-packages: real packages win where they exist
    ref_mod = importlib.import_module('src.models.vit.t2t_vit')
    cfg = dict(_target_='src.models.attention.sblocal_attention.SBLocalAttention', dim_heads=64,
               local_context=W_CTX, nb_features=N_FEAT)
    torch.manual_seed(0)
    ref_model = ref_mod.t2t_vit_t_14(t2tattn1_cfg=cfg, t2tattn2_cfg=cfg).eval()
    img = torch.randn(1, 3, 224, 224)
    with torch.no_grad():
        ref_logits = ref_model(img)          # the first forward draws both projection matrices
        mine = _oracle_model()
        missing, unexpected = mine.load_state_dict(ref_model.state_dict(), strict=True)
        assert not missing and not unexpected
        assert mine.patch_embed.attention1.attn.attention_layer.softmax_temp == pytest.approx(147 ** -0.5)
        assert mine.patch_embed.attention2.attn.attention_layer.softmax_temp == pytest.approx(576 ** -0.5)
        logits = mine(img)
    assert logits.shape == (1, 1000)
    assert so.rel_err(logits, ref_logits) <= 1e-4


@pytest.mark.gpu
@pytest.mark.parametrize('compute_dtype,tol', [(None, 1e-3), (torch.bfloat16, 2e-2)])
def test_whole_model_logits_on_gpu(compute_dtype, tol, sbl_lib):
    from fly_b200 import t2t_vit
    torch.manual_seed(0)
    model = t2t_vit.t2t_vit_t_14(t2t_vit.sblocal_factory(W_CTX, N_FEAT), t2t_vit.sblocal_factory(W_CTX, N_FEAT)).eval()
    layers = [model.patch_embed.attention1.attn.attention_layer, model.patch_embed.attention2.attn.attention_layer]
    for layer in layers:
        layer.feature_map.new_feature_map('cpu')      # draw W once, on the host, as the reference's first forward does
        layer.compute_dtype = compute_dtype
    oracle = _oracle_model()
    oracle.load_state_dict(model.state_dict(), strict=True)
    img = torch.randn(2, 3, 224, 224)
    with torch.no_grad():
        ref_logits = oracle(img)
        logits = model.cuda()(img.cuda()).float().cpu()
    assert torch.isfinite(logits).all()
    assert so.rel_err(logits, ref_logits) <= tol
