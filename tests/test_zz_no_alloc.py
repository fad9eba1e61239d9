"""The allocation-free key log-scale entry point.

Some hosts may not allocate GPU memory once they are running (all memory was
claimed by an arena at start-up, or cudaMalloc is banned in the serving loop
because it stalls the device), so they cannot pass the workspace the regular
entry points need.  `sbl_key_logscale_static` keeps its scratch in a fixed
array inside the library.  This test calls it through the C ABI twice in a row
on different inputs -- the second call finds the first call's data in the
shared array -- and compares each result with `sbl_key_logscale`, which uses a
caller-provided workspace.  It also checks the size limit.  The file name
sorts last so a failing run has already executed every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _static_logscale(lib, prob):
    B, H = prob.shape[:2]
    beta = torch.full((B, H), float('nan'), device=prob.device)
    with torch.cuda.device(prob.device):
        stream = torch.cuda.current_stream(prob.device).cuda_stream
        rc = lib.sbl_key_logscale_static(ctypes.byref(prob.params), beta.data_ptr(), stream)
    return rc, beta


def test_static_scratch_matches_workspace_version(sbl_lib):
    from fly_b200 import ops
    from oracle import sblocal_oracle as so
    torch.manual_seed(11)
    for (B, S, H, E, r, tau, dtype) in [(2, 300, 3, 64, 128, None, torch.float32),
                                         (3, 77, 2, 21, 13, 0.235, torch.float32),
                                         (2, 300, 3, 32, 64, None, torch.bfloat16)]:   # shapes both entry points run on the same kernels
        k = torch.randn(B, S, H, E, device='cuda').to(dtype)
        W = so.gaussian_orthogonal_random_matrix(r, E).cuda()
        prob = ops.Problem(k, k, k, W, 4, tau)
        expected = prob.key_logscale()
        rc, got = _static_logscale(sbl_lib, prob)
        assert rc == 0, sbl_lib.sbl_static_last_error().decode()
        torch.cuda.synchronize()
        assert torch.allclose(got, expected, rtol=1e-5, atol=1e-5)
        ref = so.key_features(k.float().cpu().permute(0, 2, 1, 3), W.cpu(), tau or E ** -0.5)[1]
        assert torch.allclose(got.cpu(), ref.reshape(B, H), rtol=1e-4, atol=1e-4)


def test_static_scratch_rejects_oversized_projection(sbl_lib):
    from fly_b200 import ops, _cabi
    k = torch.randn(1, 16, 1, 128, device='cuda')
    W = torch.randn(300, 128, device='cuda')          # 38400 floats > 32768
    prob = ops.Problem(k, k, k, W, 4)
    rc, _ = _static_logscale(sbl_lib, prob)
    assert rc == _cabi.SBL_ERR_UNSUPPORTED
    assert b'exceeds' in sbl_lib.sbl_static_last_error()


def test_static_scratch_on_the_tensor_core_shape(sbl_lib):
    """bf16, E = 64, r = 128 is the one shape where `sbl_key_logscale` takes another route (tensor cores, on the
    projection rounded to bf16) than the static call (fp32 projection, generic kernel): the two agree only to
    bf16 accuracy there, and the static call agrees with the generic-path `sbl_key_logscale` exactly."""
    from fly_b200 import ops
    from oracle import sblocal_oracle as so
    torch.manual_seed(12)
    k = (torch.randn(2, 500, 2, 64, device='cuda') / 64 ** 0.25).bfloat16()
    W = so.gaussian_orthogonal_random_matrix(128, 64).cuda()
    for _ in range(2):                                     # two calls in a row share the array
        rc, got = _static_logscale(sbl_lib, ops.Problem(k, k, k, W, 256))
        assert rc == 0, sbl_lib.sbl_static_last_error().decode()
        torch.cuda.synchronize()
        generic = ops.Problem(k, k, k, W, 256, generic=True).key_logscale()
        assert torch.allclose(got, generic, rtol=1e-5, atol=1e-5)
        tensor = ops.Problem(k, k, k, W, 256).key_logscale()
        assert torch.allclose(got, tensor, atol=5e-2)


def test_static_scratch_checks_reserved_fields(sbl_lib):
    from fly_b200 import ops, _cabi
    k = torch.randn(1, 16, 1, 32, device='cuda')
    prob = ops.Problem(k, k, k, torch.randn(8, 32, device='cuda'), 4)
    prob.params.reserved[1] = 7
    rc, _ = _static_logscale(sbl_lib, prob)
    assert rc == _cabi.SBL_ERR_INVALID_ARGUMENT
