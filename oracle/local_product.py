"""CPU restatement of the two banded-window functions the reference imports
from the third-party package `fast_transformers.local_product`
(idiap/fast-transformers; un-vendored and un-pinned in the reference:
Dockerfile:106-111 clones the default branch, version hints 0.3.0/0.4.0).

TEST INFRASTRUCTURE ONLY -- never imported by the product package.

The semantics restated here are the ones the reference itself pins:
  * call sites      src/models/attention/sblocal_attention.py:90-97,121
                    src/models/attention/local_attention.py:68-74,91
  * index formula   sblocal_attention.py:100-104  (idx = i - w//2 + j)
  * fill value      sblocal_attention.py:98       (-1e24 at invalid slots)
  * window/length   tests/models/attention/test_local_attention.py:92-99
                    (-(w//2) <= s - i < (w+1)//2 and s < len_b)

local_dot_product(Q, K, mask, lengths, w)[b,h,i,j]
    = Q[b,h,i,:] . K[b,h,idx,:] + mask[i,idx]   if 0 <= idx < lengths[b]
    = -1e24                                      otherwise,  idx = i - w//2 + j
local_weighted_average(A, V)[b,h,i,:]
    = sum_j A[b,h,i,j] * V[b,h,idx,:]            over 0 <= idx < S
"""
import torch

INVALID_FILL = -1e24


def _window_index(T, w, device):
    i = torch.arange(T, device=device).view(T, 1)
    j = torch.arange(w, device=device).view(1, w)
    return i - w // 2 + j                      # (T, w)


def local_dot_product(queries, keys, attn_mask, key_lengths, local_context, row_chunk=1024):
    """queries (B,H,T,E), keys (B,H,S,E), attn_mask (T,S) additive,
    key_lengths (B,) int64 -> (B,H,T,w)."""
    B, H, T, E = queries.shape
    S = keys.shape[2]
    w = int(local_context)
    out = queries.new_empty(B, H, T, w)
    lengths = key_lengths.to(torch.long).view(B, 1, 1, 1)
    for t0 in range(0, T, row_chunk):
        t1 = min(T, t0 + row_chunk)
        idx = _window_index(T, w, queries.device)[t0:t1]          # (t,w)
        safe = idx.clamp(0, S - 1)
        kg = keys[:, :, safe.reshape(-1), :].view(B, H, t1 - t0, w, E)
        dots = torch.einsum('bhte,bhtwe->bhtw', queries[:, :, t0:t1], kg)
        rows = torch.arange(t0, t1, device=queries.device).view(-1, 1).expand_as(safe)
        dots = dots + attn_mask[rows, safe].to(dots.dtype)
        valid = (idx >= 0).view(1, 1, t1 - t0, w) & (idx.view(1, 1, t1 - t0, w) < lengths)
        out[:, :, t0:t1] = torch.where(valid, dots, dots.new_full((), INVALID_FILL))
    return out


def local_weighted_average(attention, values, row_chunk=1024):
    """attention (B,H,T,w), values (B,H,S,D) -> (B,H,T,D)."""
    B, H, T, w = attention.shape
    S, D = values.shape[2], values.shape[3]
    out = values.new_empty(B, H, T, D)
    for t0 in range(0, T, row_chunk):
        t1 = min(T, t0 + row_chunk)
        idx = _window_index(T, w, attention.device)[t0:t1]
        inside = ((idx >= 0) & (idx < S)).view(1, 1, t1 - t0, w)
        safe = idx.clamp(0, S - 1)
        vg = values[:, :, safe.reshape(-1), :].view(B, H, t1 - t0, w, D)
        a = torch.where(inside, attention[:, :, t0:t1], attention.new_zeros(()))
        out[:, :, t0:t1] = torch.einsum('bhtw,bhtwd->bhtd', a, vg)
    return out
