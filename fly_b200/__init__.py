"""sblocal_b200: the forward of Scatterbrain's SBLocal attention as
hand-written sm_100a CUDA kernels behind a C ABI, with a Python shell that
mirrors the reference module's interface."""
from .masking import BaseMask, FullMask, LengthMask, TriangularCausalMask
from .projection_utils import gaussian_orthogonal_random_matrix
from .feature_maps_sb import SBPerformerFeatures
from .sblocal_attention import SBLocalAttention

__all__ = ['SBLocalAttention', 'SBPerformerFeatures', 'gaussian_orthogonal_random_matrix',
           'BaseMask', 'FullMask', 'LengthMask', 'TriangularCausalMask']
