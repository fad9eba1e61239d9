"""CPU checks of the oracle itself: against the committed golden vectors
(outputs of the unmodified reference), against the reference module where its
tree is present, and through the relations the reference's own tests assert."""
import math
import os

import numpy as np
import pytest
import torch

from cases import CASES, make_inputs
from oracle import local_product as lp
from oracle import ref_bridge
from oracle import sblocal_oracle as so

GOLDEN = os.path.join(os.path.dirname(__file__), 'golden')
FAST = [n for n, c in CASES.items() if c['T'] <= 700]


def _case(name):
    c = CASES[name]
    q, k, v, lengths = make_inputs(c)
    g = np.load(os.path.join(GOLDEN, name + '.npz'))
    t = torch.from_numpy
    return c, t(q), t(k), t(v), (t(lengths) if lengths is not None else None), g


def test_every_case_has_a_golden_file():
    for name in CASES:
        assert os.path.exists(os.path.join(GOLDEN, name + '.npz')), name


@pytest.mark.parametrize('name', FAST)
def test_oracle_matches_golden(name):
    c, q, k, v, lengths, g = _case(name)
    out, extras = so.sblocal_forward(q, k, v, torch.from_numpy(g['W']), c['w'], c['tau'], c['eps'], lengths,
                                     need_weights=c['weights'], row_chunk=128)
    assert so.rel_err(out, torch.from_numpy(g['out'])) < 2e-6
    if c['weights']:
        for got, key in zip(extras, ('attn', 'attn_unnormalized', 'attn_lowrank_unnormalized')):
            assert so.rel_err(got, torch.from_numpy(g[key])) < 2e-6


@pytest.mark.parametrize('name', ['reftest_w28_nb73_tau0.235', 'bench_d64_w256_m256', 't_ne_s_nomask'])
def test_dense_closed_form_matches_golden(name):
    c, q, k, v, lengths, g = _case(name)
    out = so.sblocal_dense_closed_form(q, k, v, torch.from_numpy(g['W']), c['w'], c['tau'], lengths)
    assert so.rel_err(out.float(), torch.from_numpy(g['out'])) < 1e-5


def test_projection_matches_golden_draw():
    """The seeded W restatement reproduces the matrix the reference drew."""
    c, *_rest, g = _case('bench_d64_w256_m256')
    torch.manual_seed(c['seed'])
    W = so.gaussian_orthogonal_random_matrix(c['nb'] // 2, c['E'])
    assert torch.equal(W, torch.from_numpy(g['W']))


@pytest.mark.skipif(not ref_bridge.reference_available(), reason='reference tree not present')
@pytest.mark.parametrize('w,nb,tau,eps', [(3, 73, None, 0.0), (33, 26, 0.235, 0.0), (28, 26, 1.0, 1e-4)])
def test_oracle_matches_reference_module(w, nb, tau, eps):
    torch.manual_seed(2357)
    B, H, T, S, E, D = 4, 3, 47, 39, 21, 17
    q, k, v = torch.randn(B, T, H, E), torch.randn(B, S, H, E), torch.randn(B, S, H, D)
    lengths = torch.randint(S // 4, S, (B,))
    W = so.gaussian_orthogonal_random_matrix(nb // 2, E)
    ref_out, ref_attn = ref_bridge.reference_forward(q, k, v, W, w, tau, eps, lengths, need_weights=True)
    out, extras = so.sblocal_forward(q, k, v, W, w, tau, eps, lengths, need_weights=True, row_chunk=16)
    assert so.rel_err(out, ref_out) < 2e-6
    for a, b in zip(extras, ref_attn):
        assert so.rel_err(a, b) < 2e-6


@pytest.mark.parametrize('w', [3, 4, 28, 33])
@pytest.mark.parametrize('tau', [None, 1.0, 0.235])
def test_window_functions_equal_masked_full_attention(w, tau):
    """tests/models/attention/test_local_attention.py:49-99 restated: softmax
    over the window == full softmax restricted to -(w//2) <= s-i < (w+1)//2 and
    s < len_b, renormalised; rows with no valid key are zero."""
    torch.manual_seed(2357)
    B, H, T, S, E, D = 6, 3, 47, 39, 21, 17
    q, k, v = torch.randn(B, H, T, E), torch.randn(B, H, S, E), torch.randn(B, H, S, D)
    lengths = torch.randint(0, S, (B,))
    temp = tau or 1 / math.sqrt(E)
    QK = lp.local_dot_product(q, k, torch.zeros(T, S), lengths, w)
    A = torch.softmax(temp * QK, dim=-1)
    i = torch.arange(T).view(1, 1, T, 1)
    idx = i - w // 2 + torch.arange(w)
    valid = (idx >= 0) & (idx < lengths.view(B, 1, 1, 1))
    A = A.masked_fill(~valid, 0.0)
    out = lp.local_weighted_average(A, v)
    s = torch.arange(S).view(1, 1, 1, S)
    rel = s - i
    mask = (rel >= -(w // 2)) & (rel < (w + 1) // 2) & (s < lengths.view(B, 1, 1, 1))
    full = torch.softmax((temp * torch.einsum('bhte,bhse->bhts', q, k)).masked_fill(~mask, float('-inf')), -1)
    full = torch.nan_to_num(full, nan=0.0)
    dense = torch.zeros(B, H, T, S)
    dense.masked_scatter_(mask.expand(B, H, T, S), A.masked_select(valid.expand(B, H, T, w)))
    assert torch.allclose(dense, full, rtol=1e-5, atol=1e-7)
    assert torch.allclose(out, torch.einsum('bhts,bhsd->bhtd', full, v), rtol=1e-4, atol=1e-6)
    assert (QK[~valid.expand_as(QK)] == lp.INVALID_FILL).all()


@pytest.mark.parametrize('w,nb', [(4, 26), (33, 73)])
def test_reference_test_relations_hold(w, nb):
    """tests/models/attention/test_sblocal_attention.py:59-88 restated on the
    oracle: attention rows are >= 0 and sum to 0 or 1, out == A V, the
    unnormalised matrix is exp(tau q.k) inside the window and the Performer
    estimate outside."""
    torch.manual_seed(2357)
    B, H, T, S, E, D = 5, 3, 47, 39, 21, 17
    q, k, v = torch.randn(B, T, H, E), torch.randn(B, S, H, E), torch.randn(B, S, H, D)
    lengths = torch.randint(S // 4, S, (B,))
    W = so.gaussian_orthogonal_random_matrix(nb // 2, E)
    out, (A, A_un, A_lr) = so.sblocal_forward(q, k, v, W, w, None, 0.0, lengths, need_weights=True)
    assert torch.all(A >= 0)
    rs = A.sum(-1)
    assert torch.all(torch.isclose(rs, torch.ones_like(rs), atol=1e-2) | torch.isclose(rs, torch.zeros_like(rs), atol=1e-2))
    assert torch.allclose(out, torch.einsum('bhts,bshd->bthd', A, v), rtol=1e-3, atol=1e-3)
    full = torch.exp(torch.einsum('bthe,bshe->bhts', q / math.sqrt(E), k))
    s = torch.arange(S).view(1, 1, 1, S)
    full = full * (s < lengths.view(B, 1, 1, 1))
    rel = s - torch.arange(T).view(1, 1, T, 1)
    local = ((rel >= -(w // 2)) & (rel < (w + 1) // 2) & (s < lengths.view(B, 1, 1, 1))).expand_as(full)
    assert torch.allclose(A_un[local], full[local], rtol=1e-3, atol=1e-4)
    assert torch.allclose(A_un[~local], A_lr[~local], rtol=1e-3, atol=1e-4)
