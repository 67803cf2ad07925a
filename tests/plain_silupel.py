"""A plain, slow implementation of the Silupel decoder: whole sequences, no cache, one function per mechanism,
64-bit arithmetic on the CPU.  It shares no code with the framework; model folders are read with the plain reader
of ``plain_qwen3``.

Notation: T tokens, E the model width, x the residual stream [T, E], n the normed rows a mixer reads.
"""
import math

import torch

F = torch.float64


def layer_norm(x, w, eps):
    """(x - mean) / sqrt(var + eps) * w over the last axis; var is the mean squared deviation."""
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * w


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def token_shift(n, mu, before=None):
    """n_t + (n_{t-1} - n_t) * mu with the rows as they were before the replacement; ``before`` is the row ahead of
    the first one (zeros at a sequence's start)."""
    first = torch.zeros_like(n[:1]) if before is None else before.reshape(1, -1)
    previous = torch.cat([first, n[:-1]], dim=0)
    return n + (previous - n) * mu


def rotary_frequencies(rot):
    """f_i = base^(-2i / dims), long wavelengths stretched where ``scaling`` says so."""
    dims = rot["dims"]
    out = []
    for i in range(dims // 2):
        f = rot["base"] ** (-2.0 * i / dims)
        sc = rot.get("scaling")
        if sc:
            wavelength = 2.0 * math.pi / f
            if wavelength > sc["original"] / sc["low"]:
                f = f / sc["factor"]
            elif wavelength >= sc["original"] / sc["high"]:
                s = (sc["original"] / wavelength - sc["low"]) / (sc["high"] - sc["low"])
                f = (1.0 - s) * f / sc["factor"] + s * f
        out.append(f)
    return torch.tensor(out, dtype=F)


def rotate(x, positions, rot, first=0):
    """Rotates columns [first, first + dims) of x [T, heads, d]: column i of the first half with column i + dims/2."""
    dims = rot["dims"]
    half = dims // 2
    # the angle is a 32-bit product of a 32-bit position and a 32-bit frequency in the design
    freq = rotary_frequencies(rot).to(torch.float32)
    angle = (positions.to(torch.float32)[:, None] * freq[None, :]).to(F)
    cos, sin = angle.cos()[:, None, :], angle.sin()[:, None, :]
    u, v = x[..., first : first + half], x[..., first + half : first + dims]
    y = x.clone()
    y[..., first : first + half] = u * cos - v * sin
    y[..., first + half : first + dims] = v * cos + u * sin
    return y


def softmax_rows(scores, visible):
    scores = scores.masked_fill(~visible, float("-inf"))
    return torch.softmax(scores, dim=-1)


def mingru(n, w, m, prefix):
    T = n.shape[0]
    z = torch.sigmoid(n @ w[prefix + "z"].T + w[prefix + "z.b"])
    u = n @ w[prefix + "x"].T + w[prefix + "x.b"]
    candidate = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    state = torch.zeros(m["width"], dtype=F)
    rows = []
    for t in range(T):
        state = (1.0 - z[t]) * state + z[t] * candidate[t]
        rows.append(state)
    g = n @ w[prefix + "g"].T
    return (torch.stack(rows) * g * torch.sigmoid(g)) @ w[prefix + "o"].T


def attention(n, w, m, prefix, probabilities=None):
    T = n.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    positions = torch.arange(T)
    q = (n @ w[prefix + "q"].T + w[prefix + "q.b"]).view(T, H, d)
    k = (n @ w[prefix + "k"].T + w[prefix + "k.b"]).view(T, G, d)
    v = (n @ w[prefix + "v"].T + w[prefix + "v.b"]).view(T, G, dv)
    q, k = rotate(q, positions, m["rot"]), rotate(k, positions, m["rot"])
    per = H // G
    heads = []
    for h in range(H):
        scores = (q[:, h] @ k[:, h // per].T) * m["scale"] * w[prefix + "temp"][h]
        if m.get("softcap"):
            scores = m["softcap"] * torch.tanh(scores / m["softcap"])
        i, j = positions[:, None], positions[None, :]
        visible = j <= i
        if m.get("mask"):
            size = m["mask"]["size"]
            visible = visible & ((i // size) == (j // size))
        p = softmax_rows(scores, visible)
        if probabilities is not None:
            probabilities.append(p)
        heads.append(p @ v[:, h // per])
    mixed = torch.cat(heads, dim=1) * torch.sigmoid(n @ w[prefix + "g"].T)
    return mixed @ w[prefix + "o"].T + w[prefix + "o.b"]


def latent_attention(n, w, m, prefix, eps, probabilities=None):
    T = n.shape[0]
    H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    positions = torch.arange(T)
    q_latent = rms_norm(n @ w[prefix + "dq"].T, w[prefix + "dq.norm"], eps)
    q = (q_latent @ w[prefix + "uq"].T).view(T, H, d + r)
    down = n @ w[prefix + "dkv"].T
    latent = rms_norm(down[:, :rank], w[prefix + "dkv.norm"], eps)
    shared = rotate(down[:, rank:].reshape(T, 1, r), positions, m["rot"])[:, 0]
    q = rotate(q, positions, m["rot"], first=d)
    keys = (latent @ w[prefix + "uk"].T).view(T, H, d)
    values = (latent @ w[prefix + "uv"].T).view(T, H, dv)
    visible = positions[None, :] <= positions[:, None]
    heads = []
    for h in range(H):
        scores = (q[:, h, :d] @ keys[:, h].T + q[:, h, d:] @ shared.T) * m["scale"]
        p = softmax_rows(scores, visible)
        if probabilities is not None:
            probabilities.append(p)
        heads.append(p @ values[:, h])
    return torch.cat(heads, dim=1) @ w[prefix + "o"].T


def feed_forward(n, w, prefix):
    return (gelu_tanh(n @ w[prefix + "gate"].T) * (n @ w[prefix + "up"].T)) @ w[prefix + "down"].T


def layer_runs(config):
    count = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return list(range(count))
    start = loop.get("start", 0)
    return list(range(start)) + list(range(start, loop["stop"])) * loop["times"] + list(range(loop["stop"], count))


def forward(config, weights, tokens, keep_layers=False):
    """Logits [T, vocab] (float32) of a whole sequence; with ``keep_layers`` also the stream after every layer run."""
    w = {name: t.to(F) for name, t in weights.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][torch.as_tensor(list(tokens), dtype=torch.long)]
    kept = []
    for index in layer_runs(config):
        layer, base = config["layers"][index], f"l{index}."
        n = token_shift(layer_norm(x, w[base + "norm1"], eps), w[base + "shift"])
        if layer["type"] == "mingru":
            x = x + mingru(n, w, layer["mixer"], base + "mix.")
        elif layer["type"] == "attention":
            x = x + attention(n, w, layer["mixer"], base + "mix.")
        else:
            x = x + latent_attention(n, w, layer["mixer"], base + "mix.", eps)
        if layer["mlp"] is not None:
            x = x + feed_forward(layer_norm(x, w[base + "norm2"], eps), w, base + "mlp.")
        kept.append(x.to(torch.float32))
    logits = (layer_norm(x, w["final.norm"], eps) @ w["head"].T).to(torch.float32)
    return (logits, torch.stack(kept)) if keep_layers else logits
