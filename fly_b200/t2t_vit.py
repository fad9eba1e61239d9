"""The caller either side of the SBLocal forward in the T2T-ViT-t-14 configuration:
token-to-token stages (Unfold -> LayerNorm -> qkv Linear -> attention -> proj + v skip -> MLP),
and the plain ViT backbone behind them.  Used by the whole-model parity test and
by `bench.py --workload t2t_vit_t14_b64`; the attention layer is injected, so
the same wiring runs with `fly_b200.SBLocalAttention` on a GPU or with any
module that has the reference's forward(query, key, value) -> (out, attn).

Restates, with parameter names kept so that a `state_dict` of the reference
model loads unchanged:
  T2T_module.forward            src/models/modules/t2t.py:61-82
  Token_transformer / T2TAttention  src/models/modules/token_transformer.py:20-86
  Block / AttentionSimple       src/models/modules/vision_common.py:16-105
  T2T_ViT / t2t_vit_t_14        src/models/vit/t2t_vit.py:54-128,197-206
The reference scales the T2T attention by (input width / heads)^-0.5
(token_transformer.py:26-27): 147^-0.5 in stage 1 and 576^-0.5 in stage 2, not
64^-0.5; the injected attention receives that value as `softmax_temp`.
"""
import math

import torch
import torch.nn as nn
import torch.nn.functional as F


class Mlp(nn.Module):
    def __init__(self, width, hidden):
        super().__init__()
        self.fc1 = nn.Linear(width, hidden)
        self.fc2 = nn.Linear(hidden, width)

    def forward(self, x):
        return self.fc2(F.gelu(self.fc1(x)))


class T2TAttention(nn.Module):
    """qkv projection to `in_dim`, injected attention over (B, N, heads, in_dim/heads), output projection, and
    the skip connection through v (the input has another width, token_transformer.py:60-62)."""

    def __init__(self, dim, in_dim, num_heads, make_attention):
        super().__init__()
        self.num_heads = num_heads
        self.qkv = nn.Linear(dim, in_dim * 3, bias=False)
        self.proj = nn.Linear(in_dim, in_dim)
        self.attention_layer = make_attention(softmax_temp=(dim // num_heads) ** -0.5)

    def forward(self, x):
        B, N, _ = x.shape
        q, k, v = self.qkv(x).chunk(3, dim=-1)
        heads = lambda t: t.reshape(B, N, self.num_heads, -1)      # strided views of the packed projection
        out, _ = self.attention_layer(heads(q), heads(k), heads(v))
        return v + self.proj(out.reshape(B, N, -1))


class TokenTransformer(nn.Module):
    def __init__(self, dim, in_dim, num_heads, make_attention):
        super().__init__()
        self.norm1 = nn.LayerNorm(dim)
        self.attn = T2TAttention(dim, in_dim, num_heads, make_attention)
        self.norm2 = nn.LayerNorm(in_dim)
        self.mlp = Mlp(in_dim, in_dim)          # mlp_ratio 1.0 in the T2T stages

    def forward(self, x):
        x = self.attn(self.norm1(x))
        return x + self.mlp(self.norm2(x))


class T2TModule(nn.Module):
    """224x224 image -> 56x56 = 3136 tokens of width 147 -> attention -> 28x28 = 784 tokens of width 576 ->
    attention -> 14x14 = 196 tokens -> Linear to the backbone width."""

    def __init__(self, embed_dim, token_dim, make_attention1, make_attention2, in_chans=3):
        super().__init__()
        self.soft_split0 = nn.Unfold(kernel_size=7, stride=4, padding=2)
        self.soft_split1 = nn.Unfold(kernel_size=3, stride=2, padding=1)
        self.soft_split2 = nn.Unfold(kernel_size=3, stride=2, padding=1)
        self.attention1 = TokenTransformer(in_chans * 49, token_dim, 1, make_attention1)
        self.attention2 = TokenTransformer(token_dim * 9, token_dim, 1, make_attention2)
        self.project = nn.Linear(token_dim * 9, embed_dim)

    @staticmethod
    def _to_image(tokens):
        B, N, C = tokens.shape
        side = math.isqrt(N)
        return tokens.transpose(1, 2).reshape(B, C, side, side)

    def forward(self, img):
        x = self.attention1(self.soft_split0(img).transpose(1, 2))
        x = self.attention2(self.soft_split1(self._to_image(x)).transpose(1, 2))
        return self.project(self.soft_split2(self._to_image(x)).transpose(1, 2))


class DenseAttention(nn.Module):
    """Packed-qkv softmax attention of the backbone blocks (vision_common.py:54-80)."""

    def __init__(self, dim, num_heads):
        super().__init__()
        self.num_heads = num_heads
        self.qkv = nn.Linear(dim, dim * 3, bias=False)
        self.proj = nn.Linear(dim, dim)

    def forward(self, x):
        B, N, C = x.shape
        q, k, v = self.qkv(x).reshape(B, N, 3, self.num_heads, C // self.num_heads).permute(2, 0, 3, 1, 4)
        out = F.scaled_dot_product_attention(q, k, v)
        return self.proj(out.transpose(1, 2).reshape(B, N, C))


class Block(nn.Module):
    def __init__(self, dim, num_heads, mlp_ratio):
        super().__init__()
        self.norm1 = nn.LayerNorm(dim)
        self.attn = DenseAttention(dim, num_heads)
        self.norm2 = nn.LayerNorm(dim)
        self.mlp = Mlp(dim, int(dim * mlp_ratio))

    def forward(self, x):
        x = x + self.attn(self.norm1(x))
        return x + self.mlp(self.norm2(x))


class _SinusoidalPositions(nn.Module):
    def __init__(self, width, max_len):
        super().__init__()
        pos = torch.arange(0.0, max_len).unsqueeze(1)
        div = torch.exp(-math.log(10000.0) * torch.arange(0.0, width, 2.0) / width)
        pe = torch.empty(max_len, width)
        pe[:, 0::2] = torch.sin(pos * div)
        pe[:, 1::2] = torch.cos(pos * div)
        self.register_buffer('pe', pe.unsqueeze(0))

    def forward(self, x):
        return x + self.pe[:, :x.size(1)]


class T2TViT(nn.Module):
    """T2T-ViT with transformer token stages; `make_attention1/2(softmax_temp=...)` build the two T2T attention
    layers.  Inference wiring only (dropout and stochastic depth are identities in eval mode and are left out)."""

    def __init__(self, make_attention1, make_attention2, embed_dim=384, depth=14, num_heads=6, mlp_ratio=3.0,
                 token_dim=64, num_classes=1000, img_size=224):
        super().__init__()
        self.patch_embed = T2TModule(embed_dim, token_dim, make_attention1, make_attention2)
        self.cls_token = nn.Parameter(torch.zeros(1, 1, embed_dim))
        self.pos_embed = _SinusoidalPositions(embed_dim, (img_size // 16) ** 2 + 1)
        self.blocks = nn.Sequential(*[Block(embed_dim, num_heads, mlp_ratio) for _ in range(depth)])
        self.norm = nn.LayerNorm(embed_dim)
        self.head = nn.Linear(embed_dim, num_classes)
        nn.init.trunc_normal_(self.cls_token, std=0.02)
        for mod in self.modules():
            if isinstance(mod, nn.Linear):
                nn.init.trunc_normal_(mod.weight, std=0.02)
                if mod.bias is not None:
                    nn.init.zeros_(mod.bias)

    def forward(self, img):
        x = self.patch_embed(img)
        x = torch.cat((self.cls_token.expand(x.shape[0], -1, -1), x), dim=1)
        x = self.norm(self.blocks(self.pos_embed(x)))
        return self.head(x[:, 0])


def t2t_vit_t_14(make_attention1, make_attention2, **kwargs):
    """The configuration of src/models/vit/t2t_vit.py:197-206: width 384, 14 blocks, 6 heads, mlp_ratio 3."""
    return T2TViT(make_attention1, make_attention2, embed_dim=384, depth=14, num_heads=6, mlp_ratio=3.0, **kwargs)


def sblocal_factory(local_context=256, nb_features=256, dim_heads=64):
    """make_attention callable that builds this package's CUDA SBLocalAttention."""
    from .sblocal_attention import SBLocalAttention
    return lambda softmax_temp: SBLocalAttention(local_context, dim_heads, nb_features, softmax_temp=softmax_temp)
