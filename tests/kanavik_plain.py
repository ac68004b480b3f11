"""The Kanavik decoder stated plainly from its equations: float64, one function per mechanism,
whole sequences token by token or with explicit masks, nothing of the package imported.

``forward(config, weights, tokens)`` gives the logits of every position of one sequence and the
residual stream after every layer; the engine's tests compare against it.

Embedding plus a learned vector per position.  A layer is pre-norm with a residual multiplier m:
``x += m mixer(c1(norm1 x)); x += m ff(c2(norm2 x))`` where ``c(h) = h + conv(h)`` is a short causal
convolution over time on each channel; then a per-layer token input (a slice of a second embedding
table, gated by a projection of x, projected back, divided by its root mean square) and a learned
weighted sum over the embedding output and the results of all layers so far.  The mixer runs two
branches on the same input: softmax attention (grouped heads, a linear distance bias, the heads'
scores mixed by a matrix before the softmax, a sliding window, a sink in the denominator) and a
gated linear recurrence with block-diagonal gates.  The feed-forward is gated with the tanh form
of GELU.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms_norm(x, weight, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps) * weight


def causal_conv(h, weight, bias=None):
    """h [T, C], weight [C, taps]: out_t = sum_j weight[:, j] h_(t - taps + 1 + j), zeros before t = 0."""
    length, taps = h.shape[0], weight.shape[1]
    out = torch.zeros_like(h)
    for t in range(length):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += weight[:, j] * h[s]
    if bias is not None:
        out = out + bias
    return out


def distance_slopes(heads, dtype=F64):
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)], dtype=dtype)


def talking_sink_attention(h, w, m):
    """Left branch.  h [T, width] -> [T, width]."""
    length = h.shape[0]
    heads, kv_heads, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    size = (m.get("mask") or {}).get("size")
    q = (h @ w["q"].T).view(length, heads, dim)
    k = (h @ w["k"].T).view(length, kv_heads, dim)
    v = (h @ w["v"].T).view(length, kv_heads, vdim)
    per = heads // kv_heads
    slopes = distance_slopes(heads, h.dtype)
    out = torch.zeros(length, heads, vdim, dtype=h.dtype)
    group = torch.arange(heads) // per                              # key/value head of each query head
    for i in range(length):
        first = 0 if size is None else max(0, i - size + 1)
        distance = (i - torch.arange(first, i + 1)).to(h.dtype)         # i - j for every visible j
        raw = torch.einsum("hd,jhd->hj", q[i], k[first:i + 1][:, group]) * m["scale"]
        raw = raw - slopes[:, None] * distance[None, :]
        mixed = w["talk"] @ raw                                     # [H, keys]: score_h <- sum_g T[h, g] score_g
        top = torch.maximum(mixed.max(dim=1).values, w["sink"])
        e = torch.exp(mixed - top[:, None])
        p = e / (e.sum(dim=1) + torch.exp(w["sink"] - top))[:, None]   # the sink counts once, has no value
        out[i] = torch.einsum("hj,jhv->hv", p, v[first:i + 1][:, group])
    return out.reshape(length, heads * vdim) @ w["o"].T


def gated_linear_recurrence(h, w, m):
    """Right branch.  h [T, width] -> [T, width]."""
    length = h.shape[0]
    width, blocks = m["width"], m["blocks"]
    y = gelu_tanh(h @ w["y"].T + w["y.b"])
    u = causal_conv(h @ w["x"].T + w["x.b"], w["conv"], w["conv.b"])
    part = width // blocks
    softplus = torch.log1p(torch.exp(w["lam"]))
    state = torch.zeros(width, dtype=h.dtype)
    out = torch.zeros(length, width, dtype=h.dtype)
    for t in range(length):
        r = torch.zeros(width, dtype=h.dtype)
        i = torch.zeros(width, dtype=h.dtype)
        for b in range(blocks):
            ub = u[t, b * part:(b + 1) * part]
            r[b * part:(b + 1) * part] = torch.sigmoid(w["ra"][b] @ ub + w["ra.b"][b])
            i[b * part:(b + 1) * part] = torch.sigmoid(w["ri"][b] @ ub + w["ri.b"][b])
        a = torch.exp(-8.0 * r * softplus)
        state = a * state + torch.sqrt(1.0 - a * a) * i * u[t]
        out[t] = state * y[t]
    return out @ w["o"].T


def parallel_mixer(h, w, m):
    left = talking_sink_attention(h, _sub(w, "left."), m["left"])
    right = gated_linear_recurrence(h, _sub(w, "right."), m["right"])
    return m["left_scale"] * left + m["right_scale"] * right


def gated_feed_forward(h, w):
    return (gelu_tanh(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def token_side_input(x, tokens, table, layer, dim, w, eps):
    e = table[tokens][:, layer * dim:(layer + 1) * dim]
    g = gelu_tanh(x @ w["gate"].T) * e
    y = g @ w["proj"].T
    return y / torch.sqrt(y.pow(2).mean(-1, keepdim=True) + eps) * w["norm"]


def _sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(config, weights, tokens, after="average", dtype=F64):
    """Logits [T, vocab] and the residual stream after every layer [layers, T, width] (``after``:
    ``average``: what goes on to the next layer; ``result``: before the weighted sum).  ``dtype``: the
    arithmetic; float32 shows how far plain rounding alone moves a row (how well it is conditioned)."""
    w = {k: v.to(dtype) for k, v in weights.items()}
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    length = tokens.shape[0]
    eps = float(config["norm"]["eps"])
    m = float(config.get("residual_mult", 1.0))
    side = config.get("token_side")
    canon = config.get("canon")
    x = w["embed"][tokens] + w["pos"][:length]
    history = [x]
    stream = []
    for index, layer in enumerate(config["layers"]):
        lw = _sub(w, f"l{index}.")
        h = rms_norm(x, lw["norm1"], eps)
        if canon:
            h = h + causal_conv(h, lw["canon1"])
        x = x + m * parallel_mixer(h, _sub(lw, "mix."), layer["mixer"])
        if layer.get("mlp") is not None:
            h = rms_norm(x, lw["norm2"], eps)
            if canon:
                h = h + causal_conv(h, lw["canon2"])
            x = x + m * gated_feed_forward(h, _sub(lw, "mlp."))
        if side:
            x = x + m * token_side_input(x, tokens, w["side.embed"], index, side["dim"], _sub(lw, "side."), eps)
        history.append(x)
        if after == "result":
            stream.append(x)
        x = sum(lw["dwa"][j] * history[j] for j in range(index + 2))
        if after == "average":
            stream.append(x)
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    return logits, torch.stack(stream)


def tensor_shapes(config):
    width, vocab = config["width"], config["vocab"]
    side = config.get("token_side")
    canon = config.get("canon")
    layers = config["layers"]
    shapes = {"embed": (vocab, width), "pos": (config["max_positions"], width), "final.norm": (width,),
              "head": (vocab, width)}
    if side:
        shapes["side.embed"] = (vocab, side["dim"] * len(layers))
    for index, layer in enumerate(layers):
        p = f"l{index}."
        left, right = layer["mixer"]["left"], layer["mixer"]["right"]
        shapes[p + "norm1"] = (width,)
        shapes[p + "mix.left.q"] = (left["heads"] * left["dim"], width)
        shapes[p + "mix.left.k"] = (left["kv_heads"] * left["dim"], width)
        shapes[p + "mix.left.v"] = (left["kv_heads"] * left["vdim"], width)
        shapes[p + "mix.left.talk"] = (left["heads"], left["heads"])
        shapes[p + "mix.left.sink"] = (left["heads"],)
        shapes[p + "mix.left.o"] = (width, left["heads"] * left["vdim"])
        rw, blocks = right["width"], right["blocks"]
        for name in ("y", "x"):
            shapes[p + f"mix.right.{name}"] = (rw, width)
            shapes[p + f"mix.right.{name}.b"] = (rw,)
        shapes[p + "mix.right.conv"] = (rw, right["conv"])
        shapes[p + "mix.right.conv.b"] = (rw,)
        for name in ("ra", "ri"):
            shapes[p + f"mix.right.{name}"] = (blocks, rw // blocks, rw // blocks)
            shapes[p + f"mix.right.{name}.b"] = (blocks, rw // blocks)
        shapes[p + "mix.right.lam"] = (rw,)
        shapes[p + "mix.right.o"] = (width, rw)
        if layer.get("mlp") is not None:
            ff = layer["mlp"]["ff"]
            shapes[p + "norm2"] = (width,)
            shapes[p + "mlp.gate"] = (ff, width)
            shapes[p + "mlp.up"] = (ff, width)
            shapes[p + "mlp.down"] = (width, ff)
        if canon:
            shapes[p + "canon1"] = (width, canon["taps"])
            if layer.get("mlp") is not None:
                shapes[p + "canon2"] = (width, canon["taps"])
        shapes[p + "dwa"] = (index + 2,)
        if side:
            shapes[p + "side.gate"] = (side["dim"], width)
            shapes[p + "side.proj"] = (width, side["dim"])
            shapes[p + "side.norm"] = (width,)
    return shapes


def random_model(config, seed):
    """Random bfloat16 weights that keep activations of order one and let every mechanism count."""
    generator = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        leaf = name.split(".", 1)[1] if name.startswith("l") and name[1].isdigit() else name
        if leaf in ("norm1", "norm2", "side.norm") or name == "final.norm":
            t = 1.0 + 0.1 * torch.randn(shape, generator=generator)
        elif leaf == "dwa":
            t = torch.randn(shape, generator=generator) * 0.2
            t[-1] += 1.0
        elif leaf in ("canon1", "canon2", "mix.right.conv"):
            t = torch.randn(shape, generator=generator) * 0.4
        elif leaf == "mix.left.talk":
            t = torch.eye(shape[0]) + 0.3 * torch.randn(shape, generator=generator)
        elif leaf == "mix.left.sink":
            t = torch.randn(shape, generator=generator)
        elif leaf == "mix.right.lam":
            t = torch.randn(shape, generator=generator) * 1.5 - 2.0
        elif leaf.endswith(".b"):
            t = torch.randn(shape, generator=generator) * 0.3
        elif name in ("embed", "pos", "side.embed"):
            t = torch.randn(shape, generator=generator)
            if name == "pos":
                t = t * 0.5
        else:
            t = torch.randn(shape, generator=generator) * (float(shape[-1]) ** -0.5)
        out[name] = t.to(torch.bfloat16)
    return out
