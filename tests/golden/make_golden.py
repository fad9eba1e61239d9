"""Generates tests/golden/*.npz by running the UNMODIFIED reference
`SBLocalAttention` on CPU (through oracle/ref_bridge.py, which supplies the
two absent third-party window functions).  Run in the build container:

    python tests/golden/make_golden.py

Each file holds the projection W the reference drew (seeded), the reference's
output, and for a few cases the dense attention matrices of the
need_weights/return_attn_unnormalized path.  Inputs are not stored: they are
regenerated from the seed in tests/golden/cases.py.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, HERE)

from cases import CASES, make_inputs          # noqa: E402
from oracle import ref_bridge                 # noqa: E402


def main():
    ref = ref_bridge.load_reference()
    for name, c in CASES.items():
        q, k, v, lengths = make_inputs(c)
        tq, tk, tv = torch.from_numpy(q), torch.from_numpy(k), torch.from_numpy(v)
        torch.manual_seed(c['seed'])
        mod = ref.SBLocalAttention(c['w'], c['E'], c['nb'], softmax_temp=c['tau'],
                                   softmax_eps=c['eps'])
        mask = None
        if lengths is not None:
            mask = ref.LengthMask(torch.from_numpy(lengths), max_len=c['S'])
        with torch.no_grad():
            out, attn = mod(tq, tk, tv, key_padding_mask=mask, need_weights=c['weights'],
                            return_attn_unnormalized=c['weights'])
        W = mod.feature_map.projection_matrix       # drawn on that first forward
        arrays = dict(W=W.numpy().copy(), out=out.contiguous().numpy().copy())
        if c['weights']:
            arrays['attn'] = attn[0].numpy().copy()
            arrays['attn_unnormalized'] = attn[1].numpy().copy()
            arrays['attn_lowrank_unnormalized'] = attn[2].numpy().copy()
        np.savez_compressed(os.path.join(HERE, name + '.npz'), **arrays)
        print(f'{name}: W{tuple(W.shape)} out{tuple(out.shape)} |out|max={out.abs().max():.4g}')


if __name__ == '__main__':
    main()
