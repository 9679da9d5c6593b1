"""A routed multi-layer Relation LM: the parameter container of the stateful decode path.

The reference project ships dense (all-pairs) models only; its sparse decode driver is not
public.  This module defines the smallest model whose decode step is exactly the
composition the reference's operators were written for, built from the reference's own
layer definitions:

* embeddings, input scale and sinusoidal positions as ``RelationLexLM``
  (src/relation_lm/models/relation_lm.py:12-18, 86-91, 130-131 of the reference project);
* one shared ``memory = LayerNorm(x)`` and a residual ``hidden`` stream passed through
  ``layers`` single-anchor relation layers, as ``StackedRelationLayers``
  (src/relation_lm/models/stacked_relation.py:23-124, 152-182);
* one ``DistilledBlockRouter`` parameter set per layer
  (src/relation_lm/routing/block_router.py:21-48);
* final LayerNorm, tied token head and boundary head (relation_lm.py:121-124, 204-207).

``decode_weights`` repacks the parameters the way the decode operators consume them: the six
memory-side projections of every layer stacked into one packed matrix
(src/relation_lm/inference/packed_cache.py:10-17 gives the column order), the query-side
projections into one ``[256, d]`` matrix per layer (anchor query, anchor router query and the
128-channel partner base of relation_select.py:165-193), and the first relation-MLP layer
factorised (relation_reduce.py:23-57).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
from torch import Tensor, nn


@dataclass
class RoutedRelationConfig:
    vocab_size: int = 16_000
    boundary_vocab_size: int = 256
    d_model: int = 512
    layers: int = 6
    gate_dim: int = 64
    relation_dim: int = 128
    ff_mult: int = 4
    k_max: int = 8
    max_context: int = 512
    block_size: int = 32
    local_window: int = 64
    top_blocks: int = 2
    strict_valid: bool = False
    router_heads: int = 4
    router_head_dim: int = 16
    relative_buckets: int = 16
    norm_eps: float = 1.0e-5
    mix_logit_init: float = -1.5

    @property
    def hidden_dim(self) -> int:
        return self.ff_mult * self.d_model

    @property
    def packed_width(self) -> int:
        """anchor key 64 | partner key 64 | operand R | partner-anchor 128 | two router keys 64."""
        return 384 + self.relation_dim


def sinusoidal_positions(length: int, width: int) -> Tensor:
    position = torch.arange(length, dtype=torch.float32)[:, None]
    scale = torch.exp(torch.arange(0, width, 2, dtype=torch.float32) * (-math.log(10000.0) / width))
    table = torch.zeros(length, width)
    table[:, 0::2] = torch.sin(position * scale)
    table[:, 1::2] = torch.cos(position * scale[: table[:, 1::2].shape[1]])
    return table


class RouterParameters(nn.Module):
    """Per-layer block-router parameters (names as in the reference's ``DistilledBlockRouter``)."""

    def __init__(self, cfg: RoutedRelationConfig) -> None:
        super().__init__()
        width = cfg.router_heads * cfg.router_head_dim
        self.anchor_q = nn.Linear(cfg.d_model, width, bias=False)
        self.anchor_k = nn.Linear(cfg.d_model, width, bias=False)
        self.partner_q = nn.Linear(2 * cfg.d_model, width, bias=False)
        self.partner_k = nn.Linear(cfg.d_model, width, bias=False)
        self.anchor_gamma = nn.Parameter(torch.zeros(cfg.router_heads))
        self.partner_gamma = nn.Parameter(torch.zeros(cfg.router_heads))
        self.anchor_bias = nn.Parameter(torch.zeros(cfg.router_heads, cfg.relative_buckets))
        self.partner_bias = nn.Parameter(torch.zeros(cfg.router_heads, cfg.relative_buckets))
        self.anchor_conv_weight = nn.Parameter(torch.zeros(width, 3))
        self.partner_conv_weight = nn.Parameter(torch.zeros(width, 3))


class RoutedRelationLayer(nn.Module):
    """One anchor + K partners relation layer (names as in the reference's ``RelationBlock``)."""

    def __init__(self, cfg: RoutedRelationConfig) -> None:
        super().__init__()
        d = cfg.d_model
        self.input_norm = nn.LayerNorm(d, eps=cfg.norm_eps)
        self.anchor_query = nn.Linear(d, cfg.gate_dim, bias=False)
        self.anchor_key = nn.Linear(d, cfg.gate_dim, bias=False)
        self.partner_query = nn.Linear(2 * d, cfg.gate_dim, bias=False)
        self.partner_key = nn.Linear(d, cfg.gate_dim, bias=False)
        self.operand_projection = nn.Linear(d, cfg.relation_dim, bias=False)
        self.relation_mlp = nn.Sequential(
            nn.Linear(4 * cfg.relation_dim, cfg.hidden_dim),
            nn.GELU(),
            nn.Linear(cfg.hidden_dim, d),
            nn.LayerNorm(d, eps=cfg.norm_eps),
        )
        self.mix_logit = nn.Parameter(torch.tensor(float(cfg.mix_logit_init)))
        self.router = RouterParameters(cfg)


class RoutedRelationLM(nn.Module):
    def __init__(self, cfg: RoutedRelationConfig, seed: int = 0) -> None:
        super().__init__()
        if cfg.gate_dim != 64 or cfg.router_heads * cfg.router_head_dim != 64:
            raise ValueError("the decode kernels are built for gate width 64 and a 4 x 16 router")
        if cfg.max_context % cfg.block_size != 0:
            raise ValueError("max_context must be a multiple of block_size")
        self.config = cfg
        d = cfg.d_model
        self.token_embedding = nn.Embedding(cfg.vocab_size, d)
        self.boundary_embedding = nn.Embedding(cfg.boundary_vocab_size, d)
        self.input_scale = math.sqrt(d / 2.0)
        self.register_buffer("position_embedding", sinusoidal_positions(cfg.max_context, d),
                             persistent=False)
        self.memory_norm = nn.LayerNorm(d, eps=cfg.norm_eps)
        self.blocks = nn.ModuleList(RoutedRelationLayer(cfg) for _ in range(cfg.layers))
        self.final_norm = nn.LayerNorm(d, eps=cfg.norm_eps)
        self.boundary_output = nn.Linear(d, cfg.boundary_vocab_size)
        self.reset_parameters(seed)

    def reset_parameters(self, seed: int) -> None:
        """Seeded random init: Xavier-uniform matrices, N(0, 0.1^2) conv taps, N(0, 1) router
        gamma / bias tables and embeddings, small random biases and LayerNorm affines so that
        no term of the decode step is trivially zero."""
        g = torch.Generator(device="cpu").manual_seed(int(seed))
        with torch.no_grad():
            for name, p in self.named_parameters():
                if name.endswith("conv_weight"):
                    p.copy_(torch.randn(p.shape, generator=g) * 0.1)
                elif name.endswith("gamma") or (name.endswith("_bias") and p.dim() == 2):
                    p.copy_(torch.randn(p.shape, generator=g))
                elif "embedding" in name:
                    p.copy_(torch.randn(p.shape, generator=g) * (0.5 if "token" in name else 0.1))
                elif name.endswith("mix_logit"):
                    p.fill_(float(self.config.mix_logit_init))
                elif p.dim() == 2:
                    bound = math.sqrt(6.0 / (p.size(0) + p.size(1)))
                    p.copy_((torch.rand(p.shape, generator=g) * 2 - 1) * bound)
                elif "norm" in name or name.endswith("relation_mlp.3.weight") or name.endswith("relation_mlp.3.bias"):
                    base = 1.0 if name.endswith("weight") else 0.0
                    p.copy_(base + torch.randn(p.shape, generator=g) * 0.05)
                else:
                    p.copy_(torch.randn(p.shape, generator=g) * 0.02)

    def parameter_count(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def decode_weights(self, device, dtype) -> dict[str, Tensor]:
        """Parameters in the layout the stateful decode step consumes (see module docstring)."""
        cfg = self.config
        d = cfg.d_model
        packed, query, wa, wp, wm, b1, w2, b2 = [], [], [], [], [], [], [], []
        for block in self.blocks:
            r = block.router
            partner_anchor = torch.cat((block.partner_query.weight[:, d:], r.partner_q.weight[:, d:]), 0)
            packed.append(torch.cat((block.anchor_key.weight, block.partner_key.weight,
                                     block.operand_projection.weight, partner_anchor,
                                     r.anchor_k.weight, r.partner_k.weight), 0))
            query.append(torch.cat((block.anchor_query.weight, r.anchor_q.weight,
                                    block.partner_query.weight[:, :d], r.partner_q.weight[:, :d]), 0))
            first = block.relation_mlp[0]
            a_raw, p_raw, product, diff = first.weight.split(cfg.relation_dim, dim=1)
            wa.append(a_raw + diff)
            wp.append(p_raw - diff)
            wm.append(product)
            b1.append(first.bias)
            w2.append(block.relation_mlp[2].weight)
            b2.append(block.relation_mlp[2].bias)

        def stack(items, dt=dtype):
            return torch.stack([x.detach() for x in items]).to(device=device, dtype=dt).contiguous()

        f32 = torch.float32
        blocks = self.blocks
        return {
            "token_embedding": self.token_embedding.weight.detach().to(device, dtype).contiguous(),
            "boundary_embedding": self.boundary_embedding.weight.detach().to(device, dtype).contiguous(),
            "position_embedding": self.position_embedding.to(device, f32).contiguous(),
            "memory_norm_w": self.memory_norm.weight.detach().to(device, f32),
            "memory_norm_b": self.memory_norm.bias.detach().to(device, f32),
            "w_packed": torch.cat([x.detach() for x in packed], 0).to(device, dtype).contiguous(),
            "w_query": stack(query),
            "anchor_weight": stack(wa), "partner_weight": stack(wp), "product_weight": stack(wm),
            "first_bias": stack(b1),
            "w2": stack(w2), "b2": stack(b2),
            "input_norm_w": stack([b.input_norm.weight for b in blocks], f32),
            "input_norm_b": stack([b.input_norm.bias for b in blocks], f32),
            "relation_norm_w": stack([b.relation_mlp[3].weight for b in blocks], f32),
            "relation_norm_b": stack([b.relation_mlp[3].bias for b in blocks], f32),
            "mix": stack([torch.sigmoid(b.mix_logit) for b in blocks], f32),
            "anchor_gamma": stack([b.router.anchor_gamma for b in blocks], f32),
            "partner_gamma": stack([b.router.partner_gamma for b in blocks], f32),
            "anchor_bias": stack([b.router.anchor_bias for b in blocks], f32),
            "partner_bias": stack([b.router.partner_bias for b in blocks], f32),
            "anchor_conv_weight": stack([b.router.anchor_conv_weight for b in blocks], f32),
            "partner_conv_weight": stack([b.router.partner_conv_weight for b in blocks], f32),
            "final_norm_w": self.final_norm.weight.detach().to(device, f32),
            "final_norm_b": self.final_norm.bias.detach().to(device, f32),
            "boundary_w": self.boundary_output.weight.detach().to(device, dtype).contiguous(),
            "boundary_b": self.boundary_output.bias.detach().to(device, dtype).contiguous(),
        }
