"""Drop-in for the reference's `SBLocalAttention`
(src/models/attention/sblocal_attention.py:15-137): banded exact softmax
attention plus a Performer low-rank estimate outside the band, jointly
normalised.  Same constructor and `forward` signature; the forward runs as
hand-written sm_100a CUDA kernels behind the C ABI of include/sblocal_b200.h.

Forward only.  There is no CPU path: CPU tensors raise.  Not built (raise
NotImplementedError): causal=True (the reference marks it unchecked, :61),
an attn_mask that masks anything (the reference's own assert at :106 rejects
it), dropout in training mode.
"""
import torch
import torch.nn as nn

from . import ops
from .feature_maps_sb import SBPerformerFeatures


class _ForwardOnly(torch.autograd.Function):
    @staticmethod
    def forward(ctx, query, key, value, W, local_context, softmax_temp, softmax_eps, key_lengths):
        return ops.sblocal_forward(query, key, value, W, local_context, softmax_temp, softmax_eps, key_lengths,
                                   watch=True)

    @staticmethod
    def backward(ctx, *grads):
        raise NotImplementedError('sblocal_b200 implements the forward pass only')


class SBLocalAttention(nn.Module):
    """Arguments as in the reference (sblocal_attention.py:29-31):
    local_context, dim_heads, nb_features=None (-> int(d ln d)),
    ortho_scaling=0, causal=False, softmax_temp=None (-> 1/sqrt(E)),
    attention_dropout=0.0, softmax_eps=0.0, device=None, dtype=None."""

    def __init__(self, local_context, dim_heads, nb_features=None, ortho_scaling=0,
                 causal=False, softmax_temp=None, attention_dropout=0.0, softmax_eps=0.0,
                 device=None, dtype=None):
        factory_kwargs = {'device': device, 'dtype': dtype}
        super().__init__()
        self.feature_map = SBPerformerFeatures(dim_heads, nb_features, ortho_scaling=ortho_scaling,
                                               softmax_temp=softmax_temp, eps=softmax_eps,
                                               **factory_kwargs)
        self.local_context = local_context
        self.causal = causal
        self.softmax_temp = softmax_temp
        self.dropout = nn.Dropout(attention_dropout)
        self.softmax_eps = softmax_eps
        # Not in the reference.  None: compute in the inputs' dtype (fp32 inputs take the fp32-math kernels,
        # 1e-4 of the reference).  torch.bfloat16: fp32 inputs of a shape the tensor-core kernels support
        # (E = D = 64, 256 features, eps = 0) are rounded to bf16, run there, and the output is returned in fp32
        # (2e-2 of the reference, several times faster).  Set it on the module; the constructor is unchanged.
        self.compute_dtype = None

    def forward(self, query, key, value, attn_mask=None, key_padding_mask=None, need_weights=False,
                return_attn_unnormalized=False):
        """query (B,T,H,E), key (B,S,H,E), value (B,S,H,D); masks are mask
        objects (fly_b200.masking or the reference's).  Returns
        (out (B,T,H,D), None)."""
        # A device-side problem of an earlier forward (a wait that ran out, logits beyond the bf16 kernels' range)
        # surfaces here, without a host synchronisation: only status copies that have already landed are read.
        ops.status_watch.poll()
        if self.causal:
            raise NotImplementedError('causal SBLocal attention is not built')
        if self.training and self.dropout.p > 0:
            raise NotImplementedError('attention dropout in training mode is not built')
        if attn_mask is not None and not bool(attn_mask.all_ones):
            raise NotImplementedError('attn_mask must be None or all ones')
        key_lengths = None
        if key_padding_mask is not None and not bool(key_padding_mask.all_ones):
            key_lengths = key_padding_mask.lengths
        self.feature_map.new_feature_map(query.device)
        W = self.feature_map.projection_matrix
        out_dtype = None
        if (self.compute_dtype == torch.bfloat16 and query.dtype == torch.float32 and not need_weights
                and (query.shape[-1], value.shape[-1], W.shape[0]) in ((64, 64, 128), (128, 128, 256))
                and self.softmax_eps == 0):
            out_dtype = query.dtype
            query, key, value = query.bfloat16(), key.bfloat16(), value.bfloat16()
        args = (query, key, value, W, self.local_context, self.softmax_temp, self.softmax_eps, key_lengths)
        if need_weights:
            # dense (B,H,T,S) matrices, fp32 (sblocal_attention.py:124-136): the generic kernels keep phi(Q) and
            # phi(K) in the workspace for this; meant for tests and inspection, O(T*S) memory
            prob = ops.Problem(*args, generic=True)
            ws = prob.workspace()
            out = prob.forward(workspace=ws)
            attn = prob.attention_weights(unnormalized=return_attn_unnormalized, workspace=ws)
            return out, attn
        if torch.is_grad_enabled() and any(t.requires_grad for t in (query, key, value)):
            out = _ForwardOnly.apply(*args)
        else:
            out = ops.sblocal_forward(*args, watch=True)
        if out_dtype is not None:
            out = out.to(out_dtype)
        return out, None
