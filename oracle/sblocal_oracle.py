"""CPU restatement of the reference's SBLocal attention forward.

TEST INFRASTRUCTURE ONLY -- never imported by the product package.  Parity
status: pinned (see `oracle/__init__.py`).

Every function names the reference lines it follows (paths relative to the
HazyResearch/fly tree).  The arithmetic is done with torch CPU ops in the
dtype of the inputs (fp32 by default, fp64 for a tighter yardstick), in the
same order as the reference, but chunked over query rows so that the
(B,H,T,w) and (B,H,T,m) intermediates of long sequences fit in host memory.
"""
import math

import torch

from .local_product import local_dot_product, local_weighted_average


def gaussian_orthogonal_random_matrix(nrows, ncols, scaling=0, dtype=None):
    """src/models/attention/projection_utils.py:8-28 -- blocks of Haar
    orthogonal rows (QR of Gaussian blocks, sign-fixed), rows rescaled by the
    norms of fresh Gaussian vectors (scaling=0) or by sqrt(ncols) (scaling=1).
    Consumes the global torch CPU generator exactly as the reference does."""
    nblocks = int(math.ceil(nrows / ncols))
    blocks = torch.randn((nblocks, ncols, ncols), device='cpu')            # :12
    q, r = torch.linalg.qr(blocks)                                          # :13
    q = q * torch.diagonal(r, dim1=-2, dim2=-1).sign().unsqueeze(1)         # :15
    q = q.to(dtype=dtype) if dtype is not None else q                       # :16
    g_ortho = q.transpose(1, 2).reshape(nblocks * ncols, ncols)[:nrows]     # :19-20
    if scaling == 0:
        mult = torch.randn((nrows, ncols), dtype=dtype).norm(dim=1)         # :23
        return mult.unsqueeze(1) * g_ortho                                  # :24
    if scaling == 1:
        return math.sqrt(ncols) * g_ortho                                   # :26
    raise ValueError(f'Invalid scaling {scaling}')                          # :28


def feature_dash(x, W, tau):
    """src/models/attention/feature_maps_sb.py:62-69 -- u = x (sqrt(tau) W)^T,
    dash = [u, -u], diag = tau |x|^2 / 2."""
    c = math.sqrt(tau)
    u = torch.einsum('...id,jd->...ij', x, c * W.to(x.dtype))               # :64
    diag = x.square().sum(dim=-1, keepdim=True) / 2 * (c ** 2)              # :65
    return torch.cat([u, -u], dim=-1), diag                                 # :69


def query_features(q, W, tau, eps=0.0):
    """feature_maps_sb.py:70-75 -- q' = exp(dash - rowmax) + eps/sqrt(m),
    log scale = -diag + rowmax - ln(m)/2.  q: (..., T, E)."""
    dash, diag = feature_dash(q, W, tau)
    m = dash.shape[-1]
    rowmax = torch.amax(dash, dim=-1, keepdim=True)
    log_scale = -diag + rowmax - math.log(m) / 2                            # :71
    return torch.exp(dash - rowmax) + eps / math.sqrt(m), log_scale         # :73-75


def key_log_features(k, W, tau):
    """feature_maps_sb.py:77 -- dash - diag - ln(m)/2 before the stabiliser."""
    dash, diag = feature_dash(k, W, tau)
    m = dash.shape[-1]
    return dash - diag - math.log(m) / 2


def key_features(k, W, tau, eps=0.0):
    """feature_maps_sb.py:76-81 -- k' = exp(kd - beta) + eps/sqrt(m) with
    beta = max over (s, f) per leading index.  k: (..., S, E)."""
    kd = key_log_features(k, W, tau)
    m = kd.shape[-1]
    beta = torch.amax(kd, dim=(-1, -2), keepdim=True)                       # :78
    return torch.exp(kd - beta) + eps / math.sqrt(m), beta                  # :79-81


def sblocal_forward(query, key, value, W, local_context, softmax_temp=None, softmax_eps=0.0,
                    key_lengths=None, need_weights=False, row_chunk=512, row_range=None):
    """src/models/attention/sblocal_attention.py:43-137 (non-causal, no
    attn_mask, dropout off).

    query (B,T,H,E), key (B,S,H,E), value (B,S,H,D), W (r,E), key_lengths
    (B,) or None.  Returns (out (B,T,H,D), extras) where extras is None or,
    with need_weights, the tuple the reference returns under
    return_attn_unnormalized=True (attn, attn*e^{log_norm}, attn'*e^{pls}).
    row_range=(t0, t1): compute only those query rows (all keys still enter the
    global summary); the other rows of `out` are left uninitialised.  For spot
    checks of long sequences.
    """
    B, T, H, E = query.shape
    _, S, _, D = value.shape
    w = int(local_context)
    tau = softmax_temp or 1 / math.sqrt(E)                                  # :59
    dt = query.dtype
    lengths = (torch.full((B,), S, dtype=torch.long) if key_lengths is None
               else key_lengths.to(torch.long))                             # :66-70
    q = query.permute(0, 2, 1, 3).contiguous()                              # :73-75
    k = key.permute(0, 2, 1, 3).contiguous()
    v = value.permute(0, 2, 1, 3).contiguous()

    k_prime, beta = key_features(k, W, tau, softmax_eps)                    # :79
    pad = torch.arange(S).view(1, 1, S, 1) >= lengths.view(B, 1, 1, 1)
    k_prime = k_prime.masked_fill(pad, 0.0)                                 # :83-85
    ksum = k_prime.sum(dim=-2)                                              # scatterbrain_utils.py:20
    kv = torch.einsum('...nm,...nd->...md', k_prime, v)                     # scatterbrain_utils.py:49

    out = torch.empty(B, H, T, D, dtype=dt)
    zeros_mask = None
    extras = None
    if need_weights:
        attn = torch.zeros(B, H, T, S, dtype=dt)
        attn_un = torch.zeros(B, H, T, S, dtype=dt)
        attn_lr = torch.zeros(B, H, T, S, dtype=dt)
    r_lo, r_hi = (0, T) if row_range is None else row_range
    for t0 in range(r_lo, r_hi, row_chunk):
        t1 = min(r_hi, t0 + row_chunk)
        n = t1 - t0
        qc = q[:, :, t0:t1]
        q_prime, q_ls = query_features(qc, W, tau, softmax_eps)             # :78
        pls = q_ls + beta                                                   # :81
        Z = torch.einsum('...nm,...m->...n', q_prime, ksum)                 # :87
        lr = torch.einsum('...nm,...md->...nd', q_prime, kv)                # :88
        # Keys any row of this chunk can see: [t0 - w//2, t1 - 1 - w//2 + w).
        s0 = max(0, t0 - w // 2)
        s1 = min(S, t1 - 1 - w // 2 + w)
        if s1 <= s0:           # no key of the sequence falls in any window
            s0, s1 = 0, 1
        # Shift so that the window ops can run on the key slice: row r of the
        # chunk (global i = t0 + r) sees slice index idx - s0; the restated
        # window functions use idx = r' - w//2 + j with r' = r + (t0 - s0).
        shift = t0 - s0
        qpad = torch.zeros(B, H, shift + n, E, dtype=dt)
        qpad[:, :, shift:] = qc
        qppad = torch.zeros(B, H, shift + n, q_prime.shape[-1], dtype=dt)
        qppad[:, :, shift:] = q_prime
        lens_local = (lengths - s0).clamp(min=0, max=s1 - s0)
        if zeros_mask is None or zeros_mask.shape != (shift + n, s1 - s0):
            zeros_mask = torch.zeros(shift + n, s1 - s0, dtype=dt)          # :63
        QK = tau * local_dot_product(qpad, k[:, :, s0:s1], zeros_mask, lens_local, w)[:, :, shift:]   # :90-93
        dp = local_dot_product(qppad, k_prime[:, :, s0:s1], zeros_mask, lens_local, w)[:, :, shift:]  # :94-97
        i = torch.arange(t0, t1).view(1, 1, n, 1)
        j = torch.arange(w)
        idx = i - w // 2 + j                                                # :102
        valid = (idx >= 0) & (idx < lengths.view(B, 1, 1, 1))               # :103-104
        dp = dp.masked_fill(~valid, 0.0)                                    # :105
        assert torch.all(dp >= 0)                                           # :106
        lse = torch.logsumexp(QK, dim=-1, keepdim=True)                     # :109
        dps = dp.sum(dim=-1, keepdim=True)                                  # :110
        lr_log_norm = torch.log((Z.unsqueeze(-1) - dps).clamp_min(1e-24)) + pls   # :111-112
        log_norm = torch.logaddexp(lse, lr_log_norm)                        # :113
        prime_scale = torch.exp(pls - log_norm)                             # :115
        dots = torch.exp(QK - log_norm) - dp * prime_scale                  # :119
        dpad = torch.zeros(B, H, shift + n, w, dtype=dt)
        dpad[:, :, shift:] = dots
        out_local = local_weighted_average(dpad, v[:, :, s0:s1])[:, :, shift:]    # :121
        out[:, :, t0:t1] = out_local + lr * prime_scale                     # :122
        if need_weights:                                                    # :124-136
            attn_prime = torch.einsum('...im,...jm->...ij', q_prime, k_prime)
            ks = torch.arange(S)
            rel = ks.view(1, 1, 1, S) - i
            local_mask = ((rel >= -(w // 2)) & (rel < (w + 1) // 2)
                          & (ks.view(1, 1, 1, S) < lengths.view(B, 1, 1, 1)))
            local_mask = local_mask.expand(B, H, n, S)
            a_local = torch.zeros(B, H, n, S, dtype=dt)
            a_local.masked_scatter_(local_mask, dots.masked_select(valid.expand(B, H, n, w)))
            a = a_local + attn_prime * prime_scale
            attn[:, :, t0:t1] = a
            attn_un[:, :, t0:t1] = a * torch.exp(log_norm)
            attn_lr[:, :, t0:t1] = attn_prime * torch.exp(pls)
    if need_weights:
        extras = (attn, attn_un, attn_lr)
    return out.permute(0, 2, 1, 3), extras


def sblocal_dense_closed_form(query, key, value, W, local_context, softmax_temp=None,
                              key_lengths=None):
    """Independent second statement (eps = 0): exact exp(tau q.k) inside the
    window, Performer estimate phi(q).phi(k) outside, one shared normaliser.
    Follows what tests/models/attention/test_sblocal_attention.py:69-88 assert
    about the unnormalised attention matrix.  O(T*S) memory: small cases only,
    computed in float64."""
    B, T, H, E = query.shape
    S = key.shape[1]
    w = int(local_context)
    tau = softmax_temp or 1 / math.sqrt(E)
    q = query.permute(0, 2, 1, 3).double()
    k = key.permute(0, 2, 1, 3).double()
    v = value.permute(0, 2, 1, 3).double()
    Wd = W.double()
    lengths = (torch.full((B,), S, dtype=torch.long) if key_lengths is None
               else key_lengths.to(torch.long))
    c = math.sqrt(tau)
    m = 2 * Wd.shape[0]

    def phi_log(x):
        u = torch.einsum('...id,jd->...ij', x, c * Wd)
        return torch.cat([u, -u], -1) - tau * x.square().sum(-1, keepdim=True) / 2 - math.log(m) / 2

    lq, lk = phi_log(q), phi_log(k)
    # log of phi(q).phi(k) via a stable log-sum-exp over the feature axis
    lowrank = torch.logsumexp(lq.unsqueeze(-2) + lk.unsqueeze(-3), dim=-1).exp()   # (B,H,T,S)
    exact = torch.exp(tau * torch.einsum('bhte,bhse->bhts', q, k))
    i = torch.arange(T).view(1, 1, T, 1)
    s = torch.arange(S).view(1, 1, 1, S)
    rel = s - i
    in_len = s < lengths.view(B, 1, 1, 1)
    in_win = (rel >= -(w // 2)) & (rel < (w + 1) // 2)
    A = torch.where(in_win, exact, lowrank) * in_len
    out = torch.einsum('bhts,bhsd->bhtd', A, v) / A.sum(-1, keepdim=True)
    return out.permute(0, 2, 1, 3)


def rel_err(out, ref):
    """Parity metric used throughout: max|out - ref| / max|ref| per tensor
    (element-wise relative error is ill-posed here: many outputs are ~0)."""
    out = out.double()
    ref = ref.double()
    return ((out - ref).abs().max() / ref.abs().max().clamp_min(1e-300)).item()
