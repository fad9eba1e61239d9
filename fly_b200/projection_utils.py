"""Seeded orthogonal Gaussian projection for the Performer feature map.

Produces the same matrix as the reference's
src/models/attention/projection_utils.py:8-28 for the same global torch seed:
the QR blocks are drawn from the CPU generator, the row norms from the target
device's generator, in that order.  It runs once per module (first forward);
the matrix it returns is handed to the CUDA kernels unchanged.
"""
import math

import torch


def gaussian_orthogonal_random_matrix(nrows, ncols, scaling=0, device=None, dtype=None):
    nblocks = int(math.ceil(nrows / ncols))
    gauss = torch.randn((nblocks, ncols, ncols), device='cpu')
    q, r = torch.linalg.qr(gauss)
    # Haar-uniform Q: flip each column by the sign of R's diagonal
    q = q * torch.diagonal(r, dim1=-2, dim2=-1).sign().unsqueeze(-2)
    q = q.to(device=device, dtype=dtype)
    rows = q.transpose(-1, -2).reshape(nblocks * ncols, ncols)[:nrows]
    if scaling == 0:
        norms = torch.randn((nrows, ncols), device=device, dtype=dtype).norm(dim=1)
        return norms.unsqueeze(-1) * rows
    if scaling == 1:
        return math.sqrt(ncols) * rows
    raise ValueError(f'Invalid scaling {scaling}')
