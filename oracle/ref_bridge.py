"""Runs the reference's own `SBLocalAttention` on CPU, in the build container
only (the reference tree is not present on GPU machines).

TEST INFRASTRUCTURE ONLY.  The reference imports two functions from the
third-party `fast_transformers.local_product` extension, which is not
installed; `oracle/local_product.py` is registered under that module name
before the reference module is imported.  Used by `tests/golden/make_golden.py`
to produce the committed golden vectors and by the CPU tests that check the
restatement in `oracle/sblocal_oracle.py` against the reference itself.
"""
import importlib
import os
import sys
import types

def reference_root():
    """Where the reference tree lives: the SBL_REFERENCE_ROOT environment variable, else a directory
    `reference` beside the repository."""
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    return os.environ.get('SBL_REFERENCE_ROOT') or os.path.join(os.path.dirname(here), 'reference')


def reference_available(root=None):
    root = root or reference_root()
    return os.path.isfile(os.path.join(root, 'src', 'models', 'attention', 'sblocal_attention.py'))


def load_reference(root=None):
    """Returns a namespace with the reference's SBLocalAttention, LengthMask,
    FullMask, FullAttention and LocalAttention classes."""
    root = root or reference_root()
    if not reference_available(root):
        raise FileNotFoundError(f'reference tree not found at {root}')
    from . import local_product as lp
    if 'fast_transformers.local_product' not in sys.modules:
        pkg = types.ModuleType('fast_transformers')
        pkg.__path__ = []
        sub = types.ModuleType('fast_transformers.local_product')
        sub.local_dot_product = lp.local_dot_product
        sub.local_weighted_average = lp.local_weighted_average
        pkg.local_product = sub
        sys.modules['fast_transformers'] = pkg
        sys.modules['fast_transformers.local_product'] = sub
    if root not in sys.path:
        sys.path.insert(0, root)
    ns = types.SimpleNamespace()
    ns.SBLocalAttention = importlib.import_module(
        'src.models.attention.sblocal_attention').SBLocalAttention
    ns.LocalAttention = importlib.import_module(
        'src.models.attention.local_attention').LocalAttention
    ns.FullAttention = importlib.import_module(
        'src.models.attention.full_attention').FullAttention
    masking = importlib.import_module('src.models.modules.masking')
    ns.LengthMask, ns.FullMask = masking.LengthMask, masking.FullMask
    ns.gaussian_orthogonal_random_matrix = importlib.import_module(
        'src.models.attention.projection_utils').gaussian_orthogonal_random_matrix
    return ns


def reference_forward(query, key, value, W, local_context, softmax_temp=None, softmax_eps=0.0,
                      key_lengths=None, need_weights=False, root=None):
    """One forward of the unmodified reference module with projection W
    installed (the reference draws W on its first forward only,
    feature_maps_sb.py:129-146; the draw is made and then overwritten)."""
    import torch
    ref = load_reference(root)
    E = query.shape[-1]
    mod = ref.SBLocalAttention(local_context, E, nb_features=2 * W.shape[0],
                               softmax_temp=softmax_temp, softmax_eps=softmax_eps,
                               dtype=query.dtype)
    rng = torch.get_rng_state()
    mod.feature_map.new_feature_map('cpu')          # consumes the one and only draw
    torch.set_rng_state(rng)
    mod.feature_map.projection_matrix.copy_(W.to(query.dtype))
    mask = None
    if key_lengths is not None:
        mask = ref.LengthMask(key_lengths.to(torch.long), max_len=key.shape[1])
    with torch.no_grad():
        out, attn = mod(query, key, value, key_padding_mask=mask, need_weights=need_weights,
                        return_attn_unnormalized=need_weights)
    return out, attn
