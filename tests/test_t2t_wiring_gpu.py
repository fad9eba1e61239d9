"""The call pattern of the reference's T2T attention wrapper
(src/models/modules/token_transformer.py:39-63): a fused qkv Linear, chunk and
reshape to (B, N, 1, 64) views, attention_layer(q, k, v) called positionally,
the value skip connection.  Run on CUDA with the B200 module and compared with
the same wrapper around the CPU oracle, at both T2T stage temperatures."""
import pytest
import torch

from oracle import sblocal_oracle as so

pytestmark = pytest.mark.gpu


class T2TAttentionLike(torch.nn.Module):
    def __init__(self, dim, in_dim, attention_layer):
        super().__init__()
        self.in_dim = in_dim
        self.qkv = torch.nn.Linear(dim, in_dim * 3, bias=False)
        self.proj = torch.nn.Linear(in_dim, in_dim)
        self.attention_layer = attention_layer

    def forward(self, x):
        B, N, _ = x.shape
        q, k, v = self.qkv(x).chunk(3, dim=-1)
        q, k, v = (t.reshape(B, N, 1, self.in_dim) for t in (q, k, v))
        out, _ = self.attention_layer(q, k, v)
        out = out.reshape(B, N, self.in_dim)
        return v.squeeze(2) + self.proj(out)


@pytest.mark.parametrize('dim,N', [(147, 3136), (576, 784)])
def test_t2t_stage(dim, N, sbl_lib):
    from fly_b200 import SBLocalAttention
    torch.manual_seed(0)
    tau = dim ** -0.5                       # token_transformer.py:26-27: scale comes from the INPUT width
    layer = SBLocalAttention(256, 64, 256, softmax_temp=tau)
    block = T2TAttentionLike(dim, 64, layer).eval()
    x = torch.randn(2, N, dim)
    layer.feature_map.new_feature_map('cpu')
    W = layer.feature_map.projection_matrix.clone()

    class OracleLayer:
        def __call__(self, q, k, v):
            return so.sblocal_forward(q, k, v, W, 256, tau)[0], None

    with torch.no_grad():
        ref_block = T2TAttentionLike(dim, 64, OracleLayer())
        ref_block.qkv, ref_block.proj = block.qkv, block.proj
        ref = ref_block(x)
        got = block.cuda()(x.cuda()).cpu()
    assert so.rel_err(got, ref) <= 1e-4
