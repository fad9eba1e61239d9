"""GPU parity: the CUDA path, called through the C ABI, against the committed
golden vectors (outputs of the unmodified reference) and against the CPU
oracle on fresh seeded inputs.

Tolerances (metric: max|out - ref| / max|ref| per tensor):
  fp32 storage  <= 1e-4     bf16 storage (fp32 accumulate)  <= 2e-2
"""
import os

import numpy as np
import pytest
import torch

from cases import CASES, make_inputs
from oracle import sblocal_oracle as so

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), 'golden')
TOL_F32 = 1e-4
TOL_BF16 = 2e-2


def _load(name):
    c = CASES[name]
    q, k, v, lengths = make_inputs(c)
    g = np.load(os.path.join(GOLDEN, name + '.npz'))
    t = lambda a: torch.from_numpy(a)
    return c, t(q), t(k), t(v), (t(lengths) if lengths is not None else None), t(g['W']), t(g['out']), g


@pytest.mark.parametrize('name', [n for n, c in CASES.items() if not c['bf16']])
def test_golden_fp32(name, sbl_lib):
    from fly_b200 import ops
    c, q, k, v, lengths, W, ref, _ = _load(name)
    out = ops.sblocal_forward(q.cuda(), k.cuda(), v.cuda(), W.cuda(), c['w'], c['tau'], c['eps'],
                              lengths.cuda() if lengths is not None else None)
    torch.cuda.synchronize()
    err = so.rel_err(out.cpu(), ref)
    assert torch.isfinite(out).all()
    assert err <= TOL_F32, f'{name}: rel err {err:.3e}'


@pytest.mark.parametrize('name', [n for n, c in CASES.items() if c['bf16']])
def test_golden_bf16(name, sbl_lib):
    from fly_b200 import ops
    c, q, k, v, lengths, W, ref, _ = _load(name)
    out = ops.sblocal_forward(q.cuda().bfloat16(), k.cuda().bfloat16(), v.cuda().bfloat16(), W.cuda(), c['w'],
                              c['tau'], c['eps'], lengths.cuda() if lengths is not None else None)
    torch.cuda.synchronize()
    assert out.dtype == torch.bfloat16
    err = so.rel_err(out.float().cpu(), ref)
    assert err <= TOL_BF16, f'{name}: rel err {err:.3e}'


@pytest.mark.parametrize('name', ['reftest_w4_nb26_tauNone', 'lra_eps_w32_nb32', 'bench_d64_ragged'])
def test_feature_maps_match_oracle(name, sbl_lib):
    """sbl_query_features / sbl_key_features against softmax_kernel."""
    from fly_b200 import ops
    c, q, k, v, lengths, W, _, _ = _load(name)
    tau = c['tau'] or c['E'] ** -0.5
    pr = ops.Problem(q.cuda(), k.cuda(), v.cuda(), W.cuda(), c['w'], c['tau'], c['eps'],
                     lengths.cuda() if lengths is not None else None)
    qp, qls = pr.query_features()
    kp, kls = pr.key_features()
    qp_ref, qls_ref = so.query_features(q.permute(0, 2, 1, 3), W, tau, c['eps'])
    kp_ref, kls_ref = so.key_features(k.permute(0, 2, 1, 3), W, tau, c['eps'])
    if lengths is not None:
        pad = torch.arange(c['S']).view(1, 1, -1, 1) >= lengths.view(-1, 1, 1, 1)
        kp_ref = kp_ref.masked_fill(pad, 0.0)
    assert torch.allclose(qp.cpu(), qp_ref, rtol=1e-4, atol=1e-6)
    assert torch.allclose(qls.cpu(), qls_ref.squeeze(-1), rtol=1e-5, atol=1e-5)
    assert torch.allclose(kls.cpu(), kls_ref.reshape(kls.shape), rtol=1e-5, atol=1e-5)
    assert torch.allclose(kp.cpu(), kp_ref, rtol=1e-4, atol=1e-6)


def test_staged_equals_fused(sbl_lib):
    """key_logscale -> key_summary -> band_forward equals sbl_forward, and the
    summary equals the oracle's phi(K)^T V and sum phi(K)."""
    from fly_b200 import ops
    c, q, k, v, lengths, W, ref, _ = _load('bench_d64_ragged')
    args = (q.cuda(), k.cuda(), v.cuda(), W.cuda(), c['w'], c['tau'], c['eps'], lengths.cuda())
    fused = ops.Problem(*args).forward().clone()
    pr = ops.Problem(*args)
    beta = pr.key_logscale()
    kv, ksum = pr.key_summary(beta)
    staged = pr.band_forward(beta, kv, ksum)
    assert torch.equal(fused, staged)
    kp, _ = so.key_features(k.permute(0, 2, 1, 3), W, c['E'] ** -0.5)
    pad = torch.arange(c['S']).view(1, 1, -1, 1) >= lengths.view(-1, 1, 1, 1)
    kp = kp.masked_fill(pad, 0.0)
    kv_ref = torch.einsum('bhsm,bhsd->bhmd', kp, v.permute(0, 2, 1, 3))
    assert so.rel_err(kv.cpu(), kv_ref) < 1e-5
    assert so.rel_err(ksum.cpu(), kp.sum(-2)) < 1e-5


@pytest.mark.parametrize('chunks', [2, 3])
def test_sequence_shards_on_one_gpu(chunks, sbl_lib):
    """The sequence-sharded protocol, emulated serially on one device: every
    shard sees only its rows plus the window halo; the key log-scales are
    max-combined and the summaries added, as the collectives would."""
    from fly_b200 import ops
    c, q, k, v, lengths, W, ref, _ = _load('bench_d64_w256_m256')
    q, k, v, W = q.cuda(), k.cuda(), v.cuda(), W.cuda()
    N, w = c['T'], c['w']
    bounds = [N * i // chunks for i in range(chunks + 1)]
    probs = []
    for g in range(chunks):
        lo, hi = bounds[g], bounds[g + 1]
        klo, khi = max(0, lo - w // 2), min(N, hi - 1 - w // 2 + w)
        out = torch.empty(q.shape[0], hi - lo, q.shape[2], v.shape[3], device='cuda')
        probs.append(ops.Problem(q[:, lo:hi], k[:, klo:khi], v[:, klo:khi], W, w, c['tau'], c['eps'], None, out,
                                 q_pos0=lo, k_pos0=klo, S_total=N, sum_range=(lo - klo, hi - klo)))
    ws = [torch.empty(p.workspace_bytes, dtype=torch.uint8, device='cuda') for p in probs]
    beta = torch.stack([p.key_logscale(workspace=x) for p, x in zip(probs, ws)]).amax(0)
    parts = [p.key_summary(beta, workspace=x) for p, x in zip(probs, ws)]
    kv = torch.stack([a for a, _ in parts]).sum(0)
    ksum = torch.stack([b for _, b in parts]).sum(0)
    outs = [p.band_forward(beta, kv, ksum, workspace=x) for p, x in zip(probs, ws)]
    out = torch.cat(outs, dim=1)
    assert so.rel_err(out.cpu(), ref) <= TOL_F32


@pytest.mark.parametrize('dtype,tol', [(torch.float32, TOL_F32), (torch.bfloat16, TOL_BF16)])
def test_fresh_inputs_vs_oracle_strided(dtype, tol, sbl_lib):
    """Seeded inputs never seen by the golden files, passed as the strided
    views the T2T caller produces (chunk of a fused qkv tensor)."""
    from fly_b200 import ops
    torch.manual_seed(77)
    B, N, H, E, w, r = 2, 600, 2, 64, 256, 128
    qkv = (torch.randn(B, N, 3, H, E) / E ** 0.25)
    if dtype == torch.bfloat16:
        qkv = qkv.bfloat16().float()
    q, k, v = qkv.unbind(2)
    W = so.gaussian_orthogonal_random_matrix(r, E)
    ref, _ = so.sblocal_forward(q, k, v, W, w)
    dq = qkv.cuda().to(dtype)
    out = ops.sblocal_forward(dq[:, :, 0], dq[:, :, 1], dq[:, :, 2], W.cuda(), w)
    assert so.rel_err(out.float().cpu(), ref) <= tol
