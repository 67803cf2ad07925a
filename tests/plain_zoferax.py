"""A plain, slow statement of the Zoferax decoder: whole sequences, no cache, one function per mechanism.

Everything here is 32-bit torch on whatever device the inputs live on, written from the design's equations
and sharing nothing with the framework's parts or kernels.  ``weights`` is a dict name -> tensor, ``config``
the parsed config.json.

Notation: T tokens, E model width, H query heads, G key/value heads, dk the query/key size of a head and dv
its value size.
"""
from __future__ import annotations

import math

import torch


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def scaled_embedding(table: torch.Tensor, tokens: torch.Tensor, scale: float) -> torch.Tensor:
    return table[tokens].float() * scale


def sinusoid_positions(positions: torch.Tensor, width: int, base: float = 10000.0) -> torch.Tensor:
    """[T, width]: column 2i is sin(p * base^(-2i/width)), column 2i + 1 the cosine of the same angle."""
    out = torch.zeros(positions.numel(), width, dtype=torch.float32)
    for t, p in enumerate(positions.tolist()):
        for i in range((width + 1) // 2):
            angle = p * base ** (-2.0 * i / width)
            out[t, 2 * i] = math.sin(angle)
            if 2 * i + 1 < width:
                out[t, 2 * i + 1] = math.cos(angle)
    return out


def projection(x: torch.Tensor, weight: torch.Tensor, bias=None) -> torch.Tensor:
    y = x @ weight.float().t()
    return y + bias.float() if bias is not None else y


def keys_and_values(x, weights, prefix: str, eps: float):
    """The keys (after the norm over the whole projection) and values that a layer with own projections makes."""
    k = projection(x, weights[prefix + "k"], weights[prefix + "k.b"])
    k = rms_unit(k, eps) * weights[prefix + "k.norm"].float()
    v = projection(x, weights[prefix + "v"], weights[prefix + "v.b"])
    return k, v


def causal_attention(q, k, v, heads: int, kv_heads: int, dk: int, dv: int, scale: float) -> torch.Tensor:
    """q [T, H dk], k [T, G dk], v [T, G dv] of one sequence -> [T, H dv]; row i attends rows 0..i."""
    T = q.shape[0]
    out = torch.zeros(T, heads * dv, dtype=torch.float32)
    per = heads // kv_heads
    for h in range(heads):
        g = h // per
        qh, kh, vh = q[:, h * dk:(h + 1) * dk], k[:, g * dk:(g + 1) * dk], v[:, g * dv:(g + 1) * dv]
        for i in range(T):
            s = (kh[: i + 1] @ qh[i]) * scale
            w = torch.softmax(s, dim=0)
            out[i, h * dv:(h + 1) * dv] = w @ vh[: i + 1]
    return out


def attention_mixer(x, weights, prefix: str, mixer: dict, eps: float, shared_kv=None):
    """Returns (output [T, E], (k, v)).  ``shared_kv`` is another layer's (k, v) for a layer that has none."""
    H, G, dk, dv = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    q = projection(x, weights[prefix + "q"], weights[prefix + "q.b"])
    q = rms_unit(q, eps) * weights[prefix + "q.norm"].float()
    k, v = shared_kv if shared_kv is not None else keys_and_values(x, weights, prefix, eps)
    mixed = causal_attention(q, k, v, H, G, dk, dv, mixer["scale"])
    return projection(mixed, weights[prefix + "o"]), (k, v)


def relu_squared(z: torch.Tensor) -> torch.Tensor:
    return torch.relu(z) ** 2


def router_margins(logits: torch.Tensor, top: int) -> torch.Tensor:
    """How far each row is from another choice of experts: the gap between the last chosen logit and the first one left
    out, relative to the row's largest logit in size (infinite when every expert is chosen)."""
    if top >= logits.shape[-1]:
        return torch.full(logits.shape[:-1], float("inf"))
    ordered = torch.sort(logits, dim=-1, descending=True).values
    return (ordered[..., top - 1] - ordered[..., top]) / logits.abs().max(dim=-1).values.clamp_min(1e-30)


def routed_experts(x, weights, prefix: str, experts: int, top: int, margins=None) -> torch.Tensor:
    """Each row goes through its ``top`` experts with the largest router logits; their outputs are mixed with
    the softmax over those chosen logits alone.  ``margins`` (a list) receives this call's ``router_margins``."""
    logits = projection(x, weights[prefix + "router"])
    if margins is not None:
        margins.append(router_margins(logits, top))
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        chosen = torch.topk(logits[t], top).indices
        mix = torch.softmax(logits[t, chosen], dim=0)
        for weight, e in zip(mix.tolist(), chosen.tolist()):
            hidden = relu_squared(projection(x[t], weights[f"{prefix}e{e}.up"]))
            out[t] += weight * projection(hidden, weights[f"{prefix}e{e}.down"])
    return out


def forward(config: dict, weights: dict, tokens, keep_layers: bool = False, margins=None):
    """Logits [T, vocab] of one whole sequence (and, with ``keep_layers``, the stream after every layer).  ``margins``
    (a list) receives one tensor [T] of router margins per layer with experts."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    E, eps = config["width"], config["norm"]["eps"]
    x = scaled_embedding(weights["embed"], tokens, config["embedding"]["scale"])
    x = x + sinusoid_positions(torch.arange(tokens.numel()), E)
    kept, streams = {}, []
    for index, layer in enumerate(config["layers"]):
        base = f"l{index}."
        if layer["type"] != "attention":
            raise ValueError(f"unknown layer type {layer['type']!r}")
        mixer = layer["mixer"]
        source = mixer.get("kv_from")
        y, kept[index] = attention_mixer(x, weights, base + "mix.", mixer, eps, kept[source] if source is not None else None)
        x = x + rms_unit(y, eps) * weights[base + "norm1"].float()
        mlp = layer.get("mlp")
        if mlp is not None:
            if mlp["kind"] != "moe":
                raise ValueError(f"unknown feed-forward kind {mlp['kind']!r}")
            y = routed_experts(x, weights, base + "mlp.", mlp["router"]["experts"], mlp["router"]["top"], margins)
            x = x + rms_unit(y, eps) * weights[base + "norm2"].float()
        streams.append(x.clone())
    logits = projection(rms_unit(x, eps) * weights["final.norm"].float(), weights["head"])
    return (logits, torch.stack(streams)) if keep_layers else logits
