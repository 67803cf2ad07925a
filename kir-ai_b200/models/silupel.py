"""The Silupel decoder put together from parts.

Embedding rows as they are; pre-norm layers x <- x + mixer(shift(norm1(x))), x <- x + ff(norm2(x)) with layer norms
that have a weight and no bias, and a token shift on what the mixer reads (each layer run keeps the previous token's
normed row per request); three kinds of mixer, in whatever order the configuration lists them: a minGRU recurrence,
grouped-query attention (biases, a rotated part of each head with stretched long wavelengths, a factor per head, a
soft cap, a chunked mask, a sigmoid gate on the heads' outputs, an output bias) and latent attention (one small cached
row per token for all heads); a dense gated feed-forward with the tanh form of gelu, or none; a stretch of layers may
run several times in a row with the same weights, every run with a cache and state of its own; the model's norm, then
an output head of its own.

Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.shift``, ``l<i>.mix.*`` (minGRU: ``z``, ``z.b``, ``x``,
``x.b``, ``g``, ``o``; attention: ``q``, ``k``, ``v``, ``o`` with ``.b`` biases, ``temp``, ``g``; latent attention:
``dq``, ``dq.norm``, ``uq``, ``dkv``, ``dkv.norm``, ``uk``, ``uv``, ``o``), ``l<i>.mlp.{gate,up,down}``, ``final.norm``,
``head``.
"""
from __future__ import annotations

from ..config.silupel import SilupelConfig
from ..parts import (Block, Embedding, GatedMLP, GQAttention, LatentAttention, LayerNorm, MinGRU, OutputHead, RotaryEmbedding,
                     TokenShift)
from .plan import LayerCall, ModelPlan

_ATTENTION_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b"}
_MLP_NAMES = {"gate": "gate", "up": "up", "down": "down"}


def _rotary(head_dim: int, rot) -> RotaryEmbedding:
    scaling = None
    if rot.scaling is not None:
        scaling = {"factor": rot.scaling.factor, "low": rot.scaling.low, "high": rot.scaling.high, "original": rot.scaling.original}
    return RotaryEmbedding(head_dim, rot.base, rot.dims, scaling=scaling, precise=True)


def mixer_for_layer(cfg: SilupelConfig, layer, prefix: str):
    """The mixer of one configured layer, its tensors under ``prefix``."""
    m = layer.mixer
    if layer.kind == "mingru":
        return MinGRU(prefix, cfg.width, m.width)
    if layer.kind == "attention":
        return GQAttention(prefix, cfg.width, m.heads, m.kv_heads, m.dim, _rotary(m.dim, m.rot), scale=m.scale, value_dim=m.vdim,
                           bias=True, names=_ATTENTION_NAMES, head_factor="temp", softcap=m.softcap, chunk=m.chunk, gate="g",
                           out_bias="o.b")
    return LatentAttention(prefix, cfg.width, m.heads, m.dim, m.rot_dim, m.vdim, m.q_rank, m.kv_rank, m.scale, cfg.norm_eps,
                           _rotary(m.rot_dim, m.rot))


def build_silupel_plan(cfg: SilupelConfig) -> ModelPlan:
    blocks = []
    for index, layer in enumerate(cfg.layers):
        base = f"l{index}."
        ffn = norm2 = None
        if layer.mlp is not None:
            ffn = GatedMLP(base + "mlp.", cfg.width, layer.mlp.ff, "gelu_tanh", names=_MLP_NAMES)
            norm2 = LayerNorm(base + "norm2", cfg.width, cfg.norm_eps)
        blocks.append(Block(LayerNorm(base + "norm1", cfg.width, cfg.norm_eps), mixer_for_layer(cfg, layer, base + "mix."), norm2, ffn,
                            arrangement="pre_norm", shift=TokenShift(base + "shift", cfg.width)))
    # every run of a layer has a cache layer for its mixer and one for its token shift
    order, next_cache = [], 0
    for index in cfg.layer_runs():
        order.append(LayerCall(block=index, cache=next_cache, write=True, shift_cache=next_cache + 1))
        next_cache += 2
    return ModelPlan(
        embedding=Embedding("embed", cfg.vocab, cfg.width),
        blocks=blocks,
        order=order,
        final_norm=LayerNorm("final.norm", cfg.width, cfg.norm_eps),
        head=OutputHead("head", cfg.vocab, cfg.width),
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        max_positions=None,
    ).validate()
