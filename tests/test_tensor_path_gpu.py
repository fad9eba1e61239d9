"""The bf16 tensor-core kernels (E = D = 64, m = 256 and E = D = 128, m = 512) against the CPU oracle
run in fp32 on the same bf16-rounded inputs.  Bound: max|out - ref| / max|ref|
<= 2e-2.  Every call is followed by sbl_check_status, which fails if a
device-side bounded wait ran out."""
import pytest
import torch

from oracle import sblocal_oracle as so

pytestmark = pytest.mark.gpu
TOL_BF16 = 2e-2


def _inputs(B, T, S, H, seed, scale=None, E=64):
    g = torch.Generator().manual_seed(seed)
    scale = scale or E ** 0.25
    q = (torch.randn(B, T, H, E, generator=g) / scale).bfloat16()
    k = (torch.randn(B, S, H, E, generator=g) / scale).bfloat16()
    v = (torch.randn(B, S, H, E, generator=g) / scale).bfloat16()
    torch.manual_seed(seed)
    W = so.gaussian_orthogonal_random_matrix(2 * E, E)
    return q, k, v, W


def _run(q, k, v, W, w, tau=None, lengths=None):
    from fly_b200 import ops
    pr = ops.Problem(q.cuda(), k.cuda(), v.cuda(), W.cuda(), w, tau, 0.0,
                     lengths.cuda() if lengths is not None else None)
    out = pr.forward()
    pr.check_status()
    return out.float().cpu()


def test_very_wide_window_takes_the_generic_kernels(sbl_lib):
    """d = 64 with a window of more than 2048 keys is outside the tensor-core band kernel's per-tile plan: the
    problem must run the generic kernels (no status words) and still match the oracle."""
    from fly_b200 import ops
    q, k, v, W = _inputs(1, 3000, 3000, 1, seed=3)
    pr = ops.Problem(q.cuda(), k.cuda(), v.cuda(), W.cuda(), 2500)
    assert pr.status_offset is None
    ref, _ = so.sblocal_forward(q.float(), k.float(), v.float(), W, 2500)
    assert so.rel_err(pr.forward().float().cpu(), ref) <= TOL_BF16
    # the widest window the tensor-core kernel takes
    pr = ops.Problem(q.cuda(), k.cuda(), v.cuda(), W.cuda(), 2048)
    assert pr.status_offset is not None
    ref, _ = so.sblocal_forward(q.float(), k.float(), v.float(), W, 2048)
    out = pr.forward().float().cpu()
    pr.check_status()
    assert so.rel_err(out, ref) <= TOL_BF16


def test_library_reports_tensor_path(sbl_lib):
    assert sbl_lib.sbl_has_tensor_path() == 1


@pytest.mark.parametrize('T,S,w', [(640, 640, 256), (1000, 1000, 256), (130, 130, 256), (777, 777, 33),
                                   (512, 512, 100), (300, 300, 257), (64, 64, 8), (500, 380, 128),
                                   (380, 500, 128), (1, 1, 4)])
def test_shapes(T, S, w, sbl_lib):
    q, k, v, W = _inputs(2, T, S, 2, seed=T + S + w)
    ref, _ = so.sblocal_forward(q.float(), k.float(), v.float(), W, w)
    out = _run(q, k, v, W, w)
    assert torch.isfinite(out).all()
    assert so.rel_err(out, ref) <= TOL_BF16


@pytest.mark.parametrize('tau', [147 ** -0.5, 576 ** -0.5, 0.3])
def test_temperatures(tau, sbl_lib):
    q, k, v, W = _inputs(1, 700, 700, 3, seed=5)
    ref, _ = so.sblocal_forward(q.float(), k.float(), v.float(), W, 256, tau)
    assert so.rel_err(_run(q, k, v, W, 256, tau), ref) <= TOL_BF16


def test_ragged_lengths(sbl_lib):
    q, k, v, W = _inputs(4, 600, 600, 2, seed=9)
    lengths = torch.tensor([600, 150, 411, 1])
    ref, _ = so.sblocal_forward(q.float(), k.float(), v.float(), W, 256, None, 0.0, lengths)
    assert so.rel_err(_run(q, k, v, W, 256, None, lengths), ref) <= TOL_BF16


def test_larger_logits(sbl_lib):
    """Inputs ~N(0,1)/1.5: logits with 3.5x the variance of the benchmark
    distribution, so a wider dynamic range of exact weights and features.
    (At N(0,1) inputs with d = 64 the bf16 features alone cost 2-4e-2; that
    regime is served by the fp32 path.)"""
    q, k, v, W = _inputs(2, 400, 400, 2, seed=13, scale=1.5)
    ref, _ = so.sblocal_forward(q.float(), k.float(), v.float(), W, 64)
    assert so.rel_err(_run(q, k, v, W, 64), ref) <= TOL_BF16


def test_summary_matches_oracle(sbl_lib):
    from fly_b200 import ops
    q, k, v, W = _inputs(2, 900, 900, 2, seed=21)
    pr = ops.Problem(q.cuda(), k.cuda(), v.cuda(), W.cuda(), 256)
    beta = pr.key_logscale()
    kv, ksum = pr.key_summary(beta)
    pr.check_status()
    kp, beta_ref = so.key_features(k.float().permute(0, 2, 1, 3), W, 64 ** -0.5)
    # the library's beta comes from the bf16-rounded projection; any beta is a valid stabiliser
    assert torch.allclose(beta.cpu(), beta_ref.reshape(beta.shape), atol=5e-2)
    scale = torch.exp(beta_ref.reshape(2, 2) - beta.cpu())
    kv_ref = torch.einsum('bhsm,bhsd->bhmd', kp, v.float().permute(0, 2, 1, 3)) * scale[..., None, None]
    assert so.rel_err(kv.cpu(), kv_ref) < 1e-2
    assert so.rel_err(ksum.cpu(), kp.sum(-2) * scale[..., None]) < 1e-2


@pytest.mark.parametrize('chunks', [2, 3])
def test_sequence_shards_on_one_gpu(chunks, sbl_lib):
    from fly_b200 import ops
    q, k, v, W = _inputs(1, 1200, 1200, 2, seed=31)
    w = 256
    ref, _ = so.sblocal_forward(q.float(), k.float(), v.float(), W, w)
    q, k, v, W = q.cuda(), k.cuda(), v.cuda(), W.cuda()
    N = 1200
    bounds = [N * i // chunks // 8 * 8 for i in range(chunks)] + [N]
    probs = []
    for g in range(chunks):
        lo, hi = bounds[g], bounds[g + 1]
        klo, khi = max(0, lo - w // 2), min(N, hi - 1 - w // 2 + w)
        out = torch.empty(1, hi - lo, 2, 64, device='cuda', dtype=torch.bfloat16)
        probs.append(ops.Problem(q[:, lo:hi], k[:, klo:khi], v[:, klo:khi], W, w, None, 0.0, None, out,
                                 q_pos0=lo, k_pos0=klo, S_total=N, sum_range=(lo - klo, hi - klo)))
    ws = [torch.empty(p.workspace_bytes, dtype=torch.uint8, device='cuda') for p in probs]
    beta = torch.stack([p.key_logscale(workspace=x) for p, x in zip(probs, ws)]).amax(0)
    parts = [p.key_summary(beta, workspace=x) for p, x in zip(probs, ws)]
    kv = torch.stack([a for a, _ in parts]).sum(0)
    ksum = torch.stack([b for _, b in parts]).sum(0)
    outs = [p.band_forward(beta, kv, ksum, workspace=x) for p, x in zip(probs, ws)]
    for p, x in zip(probs, ws):
        p.check_status(workspace=x)
    out = torch.cat(outs, dim=1).float().cpu()
    assert so.rel_err(out, ref) <= TOL_BF16


def test_strided_output_is_clipped(sbl_lib):
    """The output tile goes out through one bulk tensor store per 128 queries: a caller-provided output that is a
    strided view (every other row of a larger buffer, T not a multiple of 128) must receive exactly its T rows and
    nothing else may be touched."""
    from fly_b200 import ops
    B, T, H, E, w = 2, 333, 2, 64, 256
    q, k, v, W = _inputs(B, T, T, H, seed=21)
    ref, _ = so.sblocal_forward(q.float(), k.float(), v.float(), W, w)
    sentinel = 7.0
    big = torch.full((B, 2 * T + 5, H, E), sentinel, dtype=torch.bfloat16, device='cuda')
    out_view = big[:, 0:2 * T:2]                      # rows 0, 2, ..., 2T-2
    pr = ops.Problem(q.cuda(), k.cuda(), v.cuda(), W.cuda(), w, None, 0.0, None, out_view)
    out = pr.forward()
    pr.check_status()
    assert out.data_ptr() == out_view.data_ptr()
    assert so.rel_err(out.float().cpu(), ref) <= TOL_BF16
    untouched = torch.ones(2 * T + 5, dtype=torch.bool)
    untouched[0:2 * T:2] = False
    assert (big[:, untouched.cuda()] == sentinel).all()


def test_bounded_wait_runs_out_and_context_survives(sbl_lib):
    """Every device-side wait has an iteration limit.  The self-test kernel waits on a barrier nothing arrives on:
    the call must come back with SBL_ERR_DEVICE_STATUS and the recorded wait site, and the next forward on the
    same device must work."""
    ws = torch.zeros(256, dtype=torch.uint8, device='cuda')
    rc = sbl_lib.sbl_selftest_wait_timeout(ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream)
    assert rc == -5, rc                                # SBL_ERR_DEVICE_STATUS
    assert b'wait site 99' in sbl_lib.sbl_last_error()
    q, k, v, W = _inputs(1, 256, 256, 1, seed=3)
    ref, _ = so.sblocal_forward(q.float(), k.float(), v.float(), W, 256)
    assert so.rel_err(_run(q, k, v, W, 256), ref) <= TOL_BF16


def test_bf16_compute_for_fp32_inputs(sbl_lib):
    """compute_dtype = bfloat16 on the module: fp32 inputs of a supported shape run on the tensor-core kernels and
    come back as fp32, within the bf16 bound; without it the same inputs stay within the fp32 bound."""
    from fly_b200 import SBLocalAttention
    torch.manual_seed(11)
    B, N, H, E = 2, 784, 1, 64
    q, k, v = [(torch.randn(B, N, H, E) / E ** 0.25) for _ in range(3)]
    layer = SBLocalAttention(256, E, 256, softmax_temp=576 ** -0.5).cuda().eval()
    with torch.no_grad():
        out32, _ = layer(q.cuda(), k.cuda(), v.cuda())
        W = layer.feature_map.projection_matrix.float().cpu()
        ref, _ = so.sblocal_forward(q, k, v, W, 256, 576 ** -0.5)
        assert so.rel_err(out32.cpu(), ref) <= 1e-4
        layer.compute_dtype = torch.bfloat16
        out16, _ = layer(q.cuda(), k.cuda(), v.cuda())
    assert out16.dtype == torch.float32
    assert so.rel_err(out16.cpu(), ref) <= TOL_BF16
    assert not torch.equal(out16, out32)               # it did take the other path


def test_long_sequence_tensor_vs_generic(sbl_lib):
    """N = 131072 (the sequence length of the sharded configuration) on one device: the tensor-core kernels against
    the generic fp32-math kernels on the same bf16 inputs (the CPU oracle would take minutes at this size; the
    generic kernels are tied to it by the other tests)."""
    from fly_b200 import ops
    B, N, H, w = 1, 131072, 2, 256
    q, k, v, W = _inputs(B, N, N, H, seed=31)
    q, k, v, W = q.cuda(), k.cuda(), v.cuda(), W.cuda()
    fast = ops.Problem(q, k, v, W, w)
    out = fast.forward()
    fast.check_status()
    slow = ops.Problem(q, k, v, W, w, generic=True)
    ref = slow.forward()
    torch.cuda.synchronize()
    assert torch.isfinite(out).all()
    assert so.rel_err(out.float().cpu(), ref.float().cpu()) <= TOL_BF16
    # and directly against the CPU oracle on sampled row blocks (start, middle, the ragged end of the sequence)
    qc, kc, vc, Wc = q.float().cpu(), k.float().cpu(), v.float().cpu(), W.cpu()
    for t0 in (0, 65000, N - 700):
        t1 = min(N, t0 + 700)
        want, _ = so.sblocal_forward(qc, kc, vc, Wc, w, row_range=(t0, t1))
        got = out[:, t0:t1].float().cpu()
        assert so.rel_err(got, want[:, t0:t1]) <= TOL_BF16


@pytest.mark.parametrize('name,B,H,N,seed', [('B4_H12_N4096', 4, 12, 4096, 1), ('B2_H16_N16384', 2, 16, 16384, 2)])
def test_benchmark_shapes_against_oracle(name, B, H, N, seed, sbl_lib):
    """The two (batch x head)-sharded benchmark configurations at their full shapes, seeds and input scale; the
    whole batch runs on the GPU, the CPU oracle checks the first and the last (batch, head) unit."""
    g = torch.Generator().manual_seed(seed)
    q, k, v = ((torch.randn(B, N, H, 64, generator=g) / 64 ** 0.25).bfloat16() for _ in range(3))
    torch.manual_seed(seed)
    W = so.gaussian_orthogonal_random_matrix(128, 64)
    out = _run(q, k, v, W, 256)
    assert torch.isfinite(out).all()
    for b, h in ((0, 0), (B - 1, H - 1)):
        unit = lambda t: t[b:b + 1, :, h:h + 1].float()
        ref, _ = so.sblocal_forward(unit(q), unit(k), unit(v), W, 256, row_chunk=1024)
        assert so.rel_err(out[b:b + 1, :, h:h + 1], ref) <= TOL_BF16


@pytest.mark.parametrize('factor,expect', [(2.0, 'ok'), (4.0, 'precision'), (6.0, 'ok')])
def test_scaled_inputs(factor, expect, sbl_lib):
    """Queries and keys `factor` times the benchmark scale (logits factor^2 times larger).  Up to twice the scale
    the tensor-core kernels stay inside the bf16 bound.  Around 3-4 times their accuracy degrades before their range
    ends: for a few query rows the in-window low-rank estimate is a few huge, mutually cancelling terms, tens of
    times the exact in-window mass, and features, KV and D = E - P rounded to bf16 leave errors relative to those
    terms (9e-2 at 4x).  The kernels see this (the row sums of D and of E are at hand) and report it as "precision".
    At 6x the exact part dominates again and the result is inside the bound.  The kernels never rescale an
    accumulator, so their range is finite too: past it the call reports the numeric range (next test).  Here: a
    call that reports nothing is inside the bf16 bound; the fp32-math kernels are inside it on all of these inputs."""
    from fly_b200 import ops, _cabi
    q, k, v, W = _inputs(1, 512, 512, 2, seed=17)
    q, k = (q.float() * factor).bfloat16(), (k.float() * factor).bfloat16()
    ref, _ = so.sblocal_forward(q.float(), k.float(), v.float(), W, 256)
    gen = ops.Problem(q.cuda(), k.cuda(), v.cuda(), W.cuda(), 256, generic=True).forward().float().cpu()
    assert so.rel_err(gen, ref) <= TOL_BF16
    pr = ops.Problem(q.cuda(), k.cuda(), v.cuda(), W.cuda(), 256)
    out = pr.forward().float().cpu()
    if expect == 'precision':
        with pytest.raises(_cabi.SblError, match='precision'):
            pr.check_status()
        assert torch.isfinite(out).all()
        assert so.rel_err(out, ref) <= 0.2      # degraded, not garbage
        return
    pr.check_status()
    assert so.rel_err(out, ref) <= TOL_BF16


def test_out_of_range_logits_are_reported(sbl_lib):
    """Inputs 24 times the benchmark scale drive exponentials out of the fp32 range in the tensor-core kernels:
    sbl_check_status must report it, the module must raise on its next call, and the generic kernels (which
    follow the reference's logsumexp form) must still match the oracle."""
    from fly_b200 import SBLocalAttention, ops, _cabi
    q, k, v, W = _inputs(1, 512, 512, 2, seed=17)
    q, k = (q.float() * 24).bfloat16(), (k.float() * 24).bfloat16()
    pr = ops.Problem(q.cuda(), k.cuda(), v.cuda(), W.cuda(), 256)
    pr.forward()
    with pytest.raises(_cabi.SblError, match='numeric range'):
        pr.check_status()
    ref, _ = so.sblocal_forward(q.float(), k.float(), v.float(), W, 256)
    gen = ops.Problem(q.cuda(), k.cuda(), v.cuda(), W.cuda(), 256, generic=True).forward().float().cpu()
    assert so.rel_err(gen, ref) <= TOL_BF16
    layer = SBLocalAttention(256, 64, 256).cuda().eval()
    layer.feature_map.new_feature_map('cuda')
    layer.feature_map.projection_matrix.copy_(W)
    with torch.no_grad():
        layer(q.cuda(), k.cuda(), v.cuda())
        torch.cuda.synchronize()
        with pytest.raises(_cabi.SblError, match='range'):
            layer(q.cuda(), k.cuda(), v.cuda())
    # the watch has reported the first call; drain what the second one queued so later tests start clean
    torch.cuda.synchronize()
    try:
        ops.status_watch.poll()
    except _cabi.SblError:
        pass


# ---- head dim 128, m = 512 (projection of 256 rows): the second shape of the tensor-core path ----

def test_head_dim_128_takes_the_tensor_path(sbl_lib):
    from fly_b200 import ops
    q, k, v, W = _inputs(1, 256, 256, 1, seed=1, E=128)
    pr = ops.Problem(q.cuda(), k.cuda(), v.cuda(), W.cuda(), 512)
    assert pr.status_offset is not None      # only the tensor-core kernels keep status words


@pytest.mark.parametrize('T,S,w', [(1100, 1100, 512), (640, 640, 512), (1000, 1000, 256), (130, 130, 512),
                                   (777, 777, 33), (512, 512, 100), (300, 300, 257), (64, 64, 8), (500, 380, 128),
                                   (380, 500, 128), (1, 1, 4), (2000, 2000, 1024)])
def test_shapes_d128(T, S, w, sbl_lib):
    q, k, v, W = _inputs(2, T, S, 2, seed=T + S + w, E=128)
    ref, _ = so.sblocal_forward(q.float(), k.float(), v.float(), W, w)
    out = _run(q, k, v, W, w)
    assert torch.isfinite(out).all()
    assert so.rel_err(out, ref) <= TOL_BF16


def test_ragged_lengths_d128(sbl_lib):
    q, k, v, W = _inputs(4, 900, 900, 2, seed=9, E=128)
    lengths = torch.tensor([900, 150, 611, 1])
    ref, _ = so.sblocal_forward(q.float(), k.float(), v.float(), W, 512, None, 0.0, lengths)
    assert so.rel_err(_run(q, k, v, W, 512, None, lengths), ref) <= TOL_BF16


def test_summary_matches_oracle_d128(sbl_lib):
    from fly_b200 import ops
    q, k, v, W = _inputs(2, 900, 900, 2, seed=21, E=128)
    pr = ops.Problem(q.cuda(), k.cuda(), v.cuda(), W.cuda(), 512)
    beta = pr.key_logscale()
    kv, ksum = pr.key_summary(beta)
    pr.check_status()
    kp, beta_ref = so.key_features(k.float().permute(0, 2, 1, 3), W, 128 ** -0.5)
    # the library's beta is the one-pass bound from the key norms: any beta >= the maximum is a valid stabiliser
    assert (beta.cpu() >= beta_ref.reshape(beta.shape) - 5e-2).all()
    scale = torch.exp(beta_ref.reshape(2, 2) - beta.cpu())
    kv_ref = torch.einsum('bhsm,bhsd->bhmd', kp, v.float().permute(0, 2, 1, 3)) * scale[..., None, None]
    assert so.rel_err(kv.cpu(), kv_ref) < 1e-2
    assert so.rel_err(ksum.cpu(), kp.sum(-2) * scale[..., None]) < 1e-2


@pytest.mark.parametrize('chunks', [2, 3])
def test_sequence_shards_on_one_gpu_d128(chunks, sbl_lib):
    from fly_b200 import ops
    q, k, v, W = _inputs(1, 1500, 1500, 2, seed=31, E=128)
    w, N = 512, 1500
    ref, _ = so.sblocal_forward(q.float(), k.float(), v.float(), W, w)
    q, k, v, W = q.cuda(), k.cuda(), v.cuda(), W.cuda()
    bounds = [N * i // chunks // 8 * 8 for i in range(chunks)] + [N]
    probs = []
    for g in range(chunks):
        lo, hi = bounds[g], bounds[g + 1]
        klo, khi = max(0, lo - w // 2), min(N, hi - 1 - w // 2 + w)
        out = torch.empty(1, hi - lo, 2, 128, device='cuda', dtype=torch.bfloat16)
        probs.append(ops.Problem(q[:, lo:hi], k[:, klo:khi], v[:, klo:khi], W, w, None, 0.0, None, out,
                                 q_pos0=lo, k_pos0=klo, S_total=N, sum_range=(lo - klo, hi - klo)))
    ws = [torch.empty(p.workspace_bytes, dtype=torch.uint8, device='cuda') for p in probs]
    beta = torch.stack([p.key_logscale(workspace=x) for p, x in zip(probs, ws)]).amax(0)
    parts = [p.key_summary(beta, workspace=x) for p, x in zip(probs, ws)]
    kv = torch.stack([a for a, _ in parts]).sum(0)
    ksum = torch.stack([b for _, b in parts]).sum(0)
    outs = [p.band_forward(beta, kv, ksum, workspace=x) for p, x in zip(probs, ws)]
    for p, x in zip(probs, ws):
        p.check_status(workspace=x)
    out = torch.cat(outs, dim=1).float().cpu()
    assert so.rel_err(out, ref) <= TOL_BF16


def test_long_sequence_d128_sampled_rows(sbl_lib):
    """B1 H2 N = 16384 at the d = 128 / w = 512 / m = 512 head shape: whole output finite, and rows of three
    windows (start, middle, end) against the oracle restricted to those rows."""
    N, w = 16384, 512
    q, k, v, W = _inputs(1, N, N, 2, seed=77, E=128)
    out = _run(q, k, v, W, w)
    assert torch.isfinite(out).all()
    for t0 in (0, 8000, N - 300):
        ref, _ = so.sblocal_forward(q.float(), k.float(), v.float(), W, w, row_range=(t0, t0 + 300))
        assert so.rel_err(out[:, t0:t0 + 300], ref[:, t0:t0 + 300]) <= TOL_BF16


def test_strided_views_and_clipped_output_d128(sbl_lib):
    """d = 128: q, k, v as strided views of one packed projection (B, N, 3, H, E) and a caller-provided output that is
    every other row of a larger buffer with T not a multiple of 128: exactly the T rows are written."""
    from fly_b200 import ops
    B, T, H, E, w = 1, 333, 2, 128, 512
    g = torch.Generator().manual_seed(5)
    qkv = (torch.randn(B, T, 3, H, E, generator=g) / E ** 0.25).bfloat16()
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    torch.manual_seed(5)
    W = so.gaussian_orthogonal_random_matrix(256, E)
    ref, _ = so.sblocal_forward(q.float(), k.float(), v.float(), W, w)
    qkv_d = qkv.cuda()
    sentinel = 7.0
    big = torch.full((B, 2 * T + 5, H, E), sentinel, dtype=torch.bfloat16, device='cuda')
    out_view = big[:, 0:2 * T:2]
    pr = ops.Problem(qkv_d[:, :, 0], qkv_d[:, :, 1], qkv_d[:, :, 2], W.cuda(), w, None, 0.0, None, out_view)
    assert pr.status_offset is not None
    out = pr.forward()
    pr.check_status()
    assert so.rel_err(out.float().cpu(), ref) <= TOL_BF16
    untouched = torch.ones(2 * T + 5, dtype=torch.bool)
    untouched[0:2 * T:2] = False
    assert (big[:, untouched.cuda()] == sentinel).all()


@pytest.mark.parametrize('tau', [0.3, 0.03])
def test_temperatures_d128(tau, sbl_lib):
    q, k, v, W = _inputs(1, 700, 700, 3, seed=5, E=128)
    ref, _ = so.sblocal_forward(q.float(), k.float(), v.float(), W, 512, tau)
    assert so.rel_err(_run(q, k, v, W, 512, tau), ref) <= TOL_BF16


def test_bf16_compute_for_fp32_inputs_d128(sbl_lib):
    """compute_dtype = bfloat16 on the module at the second tensor-core shape (d = 128, 512 features)."""
    from fly_b200 import SBLocalAttention
    torch.manual_seed(12)
    B, N, H, E = 1, 900, 2, 128
    q, k, v = [(torch.randn(B, N, H, E) / E ** 0.25) for _ in range(3)]
    layer = SBLocalAttention(512, E, 512).cuda().eval()
    with torch.no_grad():
        out32, _ = layer(q.cuda(), k.cuda(), v.cuda())
        W = layer.feature_map.projection_matrix.float().cpu()
        ref, _ = so.sblocal_forward(q, k, v, W, 512)
        assert so.rel_err(out32.cpu(), ref) <= 1e-4
        layer.compute_dtype = torch.bfloat16
        out16, _ = layer(q.cuda(), k.cuda(), v.cuda())
    assert out16.dtype == torch.float32
    assert so.rel_err(out16.cpu(), ref) <= TOL_BF16
    assert not torch.equal(out16, out32)
