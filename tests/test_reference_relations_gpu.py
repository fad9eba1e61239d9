"""The reference's own test of SBLocalAttention
(tests/models/attention/test_sblocal_attention.py:23-97), restated against the
B200 module on CUDA with the same shapes, parameter grid and tolerances: it
exercises need_weights / return_attn_unnormalized, a ragged LengthMask,
T != S, E = 21, D = 17 and odd feature counts.  Plus the stored dense attention
matrices of the reference (golden files)."""
import math
import os

import numpy as np
import pytest
import torch

from cases import CASES, make_inputs
from oracle import sblocal_oracle as so

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), 'golden')


@pytest.mark.parametrize('softmax_temp', [None, 1.0, 0.235])
@pytest.mark.parametrize('nb_features', [73, 26, 30000])
@pytest.mark.parametrize('local_context', [3, 4, 28, 33])
def test_output(local_context, nb_features, softmax_temp, sbl_lib):
    from fly_b200 import LengthMask, SBLocalAttention
    device = 'cuda'
    torch.manual_seed(2357)
    torch.cuda.manual_seed(2357)
    embed_dim, v_dim, num_heads, batch_size, q_seqlen, k_seqlen = 21, 17, 7, 18, 47, 39
    key_padding_mask = LengthMask(torch.randint(low=k_seqlen // 4, high=k_seqlen, size=(batch_size,), device=device),
                                  max_len=k_seqlen)
    layer = SBLocalAttention(local_context, embed_dim, nb_features, softmax_temp=softmax_temp,
                             attention_dropout=0.0).to(device)
    q = torch.randn(batch_size, q_seqlen, num_heads, embed_dim, device=device)
    k = torch.randn(batch_size, k_seqlen, num_heads, embed_dim, device=device)
    v = torch.randn(batch_size, k_seqlen, num_heads, v_dim, device=device)
    out, (A, A_un, A_lr_un) = layer(q, k, v, attn_mask=None, key_padding_mask=key_padding_mask, need_weights=True,
                                    return_attn_unnormalized=True)
    assert out.shape == (batch_size, q_seqlen, num_heads, v_dim)
    assert A.shape == (batch_size, num_heads, q_seqlen, k_seqlen)
    assert torch.all(A >= 0)
    row_sum = A.sum(dim=-1)
    assert torch.all(torch.isclose(row_sum, torch.ones_like(row_sum), atol=1e-2)
                     | torch.isclose(row_sum, torch.zeros_like(row_sum), atol=1e-2))
    assert torch.allclose(out, torch.einsum('bhts,bshd->bthd', A, v), rtol=1e-3, atol=1e-3)

    temperature = 1 / math.sqrt(embed_dim) if softmax_temp is None else softmax_temp
    A_full_un = torch.exp(torch.einsum('bthe,bshe->bhts', q * temperature, k))
    A_full_un.masked_fill_(~key_padding_mask.bool_matrix.view(batch_size, 1, 1, k_seqlen), 0.0)
    i = torch.arange(q_seqlen, device=device).view(1, 1, -1, 1)
    j = torch.arange(k_seqlen, device=device)
    idx = j - i
    local_mask = ((idx >= -(local_context // 2)) & (idx < (local_context + 1) // 2)
                  & (j < key_padding_mask.lengths.view(-1, 1, 1, 1)))
    local_mask = local_mask.expand_as(A_un)
    assert torch.allclose(A_un[local_mask], A_full_un[local_mask], rtol=1e-3, atol=1e-4)
    assert torch.allclose(A_un[~local_mask], A_lr_un[~local_mask], rtol=1e-3, atol=1e-4)
    rel_error = ((A_un - A_full_un) / A_full_un.clamp_min(1e-6)).abs().mean()
    if nb_features > 10000 and local_context > 10 and (softmax_temp is None or softmax_temp < 1.0):
        assert rel_error < 0.2


@pytest.mark.parametrize('name', [n for n, c in CASES.items() if c['weights']])
def test_dense_matrices_match_reference(name, sbl_lib):
    from fly_b200 import ops
    c = CASES[name]
    q, k, v, lengths = make_inputs(c)
    g = np.load(os.path.join(GOLDEN, name + '.npz'))
    t = lambda a: torch.from_numpy(a).cuda()
    pr = ops.Problem(t(q), t(k), t(v), t(g['W']), c['w'], c['tau'], c['eps'],
                     t(lengths) if lengths is not None else None, generic=True)
    ws = pr.workspace()
    out = pr.forward(workspace=ws)
    attn, un, lr = pr.attention_weights(unnormalized=True, workspace=ws)
    assert so.rel_err(out.cpu(), torch.from_numpy(g['out'])) <= 1e-4
    assert so.rel_err(attn.cpu(), torch.from_numpy(g['attn'])) <= 1e-4
    assert so.rel_err(un.cpu(), torch.from_numpy(g['attn_unnormalized'])) <= 1e-4
    assert so.rel_err(lr.cpu(), torch.from_numpy(g['attn_lowrank_unnormalized'])) <= 1e-4
