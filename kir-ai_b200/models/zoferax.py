"""The Zoferax decoder put together from parts.

Embedding rows times a constant plus a sinusoidal position vector; layers that norm a sub-layer's OUTPUT
(``out_norm`` blocks: h += norm1(mixer(h)); h += norm2(ffn(h))); attention without rotation whose q, k and v carry
biases, whose queries and keys are normed over the whole projection, whose values have a width of their own and
whose score factor is a constant of the configuration; a layer may read an earlier layer's keys and values
(``kv_from``) and then has no k and v tensors; the feed-forward, where a layer has one, is a mixture of small
relu^2 experts; a final norm and an output head of its own.

Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.{q,k,v,o}``, biases ``.q.b`` and so on, norm
weights ``.q.norm`` and ``.k.norm``, ``l<i>.mlp.router``, ``l<i>.mlp.e<j>.{up,down}``, ``final.norm``, ``head``.
"""
from __future__ import annotations

import torch

from ..config.zoferax import ZoferaxConfig
from ..parts import Block, Embedding, GQAttention, OutputHead, RMSNorm, RoutedExperts
from .plan import LayerCall, ModelPlan

_ATTENTION_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm",
                    "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b"}
_EXPERT_NAMES = {"router": "router", "up": "e{e}.up", "down": "e{e}.down"}


def build_zoferax_plan(cfg: ZoferaxConfig) -> ModelPlan:
    blocks, order, cache_of_layer = [], [], {}
    for index, layer in enumerate(cfg.layers):
        base = f"l{index}."
        m = layer.mixer
        shares = m.kv_from is not None
        attention = GQAttention(
            base + "mix.", cfg.width, m.heads, m.kv_heads, m.dim, None, scale=m.scale, value_dim=m.vdim, bias=True,
            qk_norm_eps=cfg.norm_eps, qk_norm_over="projection", reads_only=shares, names=_ATTENTION_NAMES,
            out_dtype=torch.float32,
        )
        ffn = norm2 = None
        if layer.mlp is not None:
            ffn = RoutedExperts(base + "mlp.", cfg.width, layer.mlp.ff, layer.mlp.experts, layer.mlp.top,
                                activation="relu2", names=_EXPERT_NAMES, out_dtype=torch.float32)
            norm2 = RMSNorm(base + "norm2", cfg.width, cfg.norm_eps)
        blocks.append(Block(RMSNorm(base + "norm1", cfg.width, cfg.norm_eps), attention, norm2, ffn, arrangement="out_norm"))
        if shares:
            order.append(LayerCall(block=index, cache=cache_of_layer[m.kv_from], write=False))
        else:
            cache_of_layer[index] = len(cache_of_layer)
            order.append(LayerCall(block=index, cache=cache_of_layer[index], write=True))
    return ModelPlan(
        embedding=Embedding("embed", cfg.vocab, cfg.width, scale=cfg.embedding_scale, sinusoid_base=cfg.SINUSOID_BASE),
        blocks=blocks,
        order=order,
        final_norm=RMSNorm("final.norm", cfg.width, cfg.norm_eps),
        head=OutputHead("head", cfg.vocab, cfg.width),
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        max_positions=None,
    ).validate()
