"""The Rekodra decoder stated plainly from its equations: float64, one function per mechanism,
whole sequences token by token or with explicit masks, nothing of the package imported.

``forward(config, weights, tokens)`` gives the logits of every position of one sequence and the
residual stream after every run of a layer; the engine's tests compare against it.

Scaled token embedding; pre-norm layers ``x += mixer(norm1 x); x += ff(norm2 x)``; a span of
layers may run several times in a row with the same weights, and before every repeat the
embedding output is added to the stream again.  Two mixers: causal softmax attention whose
values are its unnormalised keys, with a norm over the whole query and key rows, a rotation of
part of every head and a sink in the denominator; and a pair of branches on one input, windowed
softmax attention with a per-head norm of queries and keys beside a matrix memory with
exponential gates and a running maximum, joined as the mean of the two branches' normed
outputs.  The feed-forward routes every token to a few of many small gated experts (softmax
scores, a selection bias, groups of neighbours, experts that hand their input through) beside a
shared expert with a gate of its own.  Final norm, output matrix tied to the embedding table,
logits times a constant.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64
#: the number added to the matrix memory's denominator
MEMORY_EPS = 1e-6


def rms_norm(x, weight, eps):
    y = x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def silu(z):
    return z * torch.sigmoid(z)


def rotate_halves(x, positions, base, dims):
    """x [T, heads, dim]: dimension i of the first ``dims`` is paired with i + dims / 2."""
    half = dims // 2
    frequencies = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=x.dtype)
    angle = torch.as_tensor(positions, dtype=x.dtype)[:, None, None] * frequencies
    cos, sin = torch.cos(angle), torch.sin(angle)
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., dims:]], dim=-1)


def masked_softmax_attention(q, k, v, scale, visible, sink=None):
    """q [T, H, d], k [T, G, d], v [T, G, e]; ``visible(i, j)`` says whether query i sees key j;
    ``sink`` [H] joins every denominator once, with no value."""
    length, heads = q.shape[0], q.shape[1]
    group = torch.arange(heads) // (heads // k.shape[1])           # key/value head of each query head
    out = torch.zeros(length, heads, v.shape[2], dtype=q.dtype)
    for i in range(length):
        keys = torch.tensor([j for j in range(length) if visible(i, j)])
        scores = torch.einsum("hd,jhd->hj", q[i], k[keys][:, group]) * scale
        top = scores.max(dim=1).values
        if sink is not None:
            top = torch.maximum(top, sink)
        e = torch.exp(scores - top[:, None])
        total = e.sum(dim=1)
        if sink is not None:
            total = total + torch.exp(sink - top)                  # counts once, brings no value
        out[i] = torch.einsum("hj,jhv->hv", e / total[:, None], v[keys][:, group])
    return out


def sink_attention(h, w, m, eps):
    """The ``attention`` mixer."""
    length = h.shape[0]
    heads, kv_heads, dim = m["heads"], m["kv_heads"], m["dim"]
    q_raw, k_raw = h @ w["q"].T, h @ w["k"].T
    v = k_raw.view(length, kv_heads, dim)                      # the values: the keys as projected
    q = rms_norm(q_raw, w["q.norm"], eps).view(length, heads, dim)
    k = rms_norm(k_raw, w["k.norm"], eps).view(length, kv_heads, dim)
    rot = m.get("rot")
    if rot is not None:
        positions = list(range(length))
        q = rotate_halves(q, positions, float(rot["base"]), int(rot["dims"]))
        k = rotate_halves(k, positions, float(rot["base"]), int(rot["dims"]))
    mixed = masked_softmax_attention(q, k, v, m["scale"], lambda i, j: j <= i, w["sink"])
    return mixed.reshape(length, -1) @ w["o"].T


def windowed_attention(h, w, m, eps):
    """The left branch of the ``parallel`` mixer."""
    length = h.shape[0]
    heads, kv_heads, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    size = (m.get("mask") or {}).get("size")
    q = rms_norm((h @ w["q"].T).view(length, heads, dim), w["q.norm"], eps)
    k = rms_norm((h @ w["k"].T).view(length, kv_heads, dim), w["k.norm"], eps)
    v = (h @ w["v"].T).view(length, kv_heads, vdim)
    mixed = masked_softmax_attention(q, k, v, m["scale"],
                                     lambda i, j: j <= i and (size is None or i - j < size))
    return mixed.reshape(length, -1) @ w["o"].T


def matrix_memory(h, w, m, eps, state=None):
    """The right branch: per head a matrix S [dim, vdim], a vector n [dim] and a running maximum
    of the gates' logarithms, which starts at zero."""
    length = h.shape[0]
    heads, dim, vdim, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (h @ w["q"].T).view(length, heads, dim) * dim ** -0.5
    k = (h @ w["k"].T).view(length, heads, dim)
    v = (h @ w["v"].T).view(length, heads, vdim)
    log_in = cap * torch.tanh((h @ w["i"].T + w["i.b"]) / cap)                                    # [T, heads]
    log_keep = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w["f"].T + w["f.b"]) / cap))
    memory = torch.zeros(heads, dim, vdim, dtype=h.dtype)
    normaliser = torch.zeros(heads, dim, dtype=h.dtype)
    top = torch.zeros(heads, dtype=h.dtype)
    out = torch.zeros(length, heads, vdim, dtype=h.dtype)
    for t in range(length):
        for a in range(heads):
            new_top = torch.maximum(log_keep[t, a] + top[a], log_in[t, a])
            keep = torch.exp(log_keep[t, a] + top[a] - new_top)
            take = torch.exp(log_in[t, a] - new_top)
            memory[a] = keep * memory[a] + take * torch.outer(k[t, a], v[t, a])
            normaliser[a] = keep * normaliser[a] + take * k[t, a]
            top[a] = new_top
            below = torch.maximum(torch.abs(normaliser[a] @ q[t, a]), torch.exp(-new_top)) + MEMORY_EPS
            out[t, a] = (memory[a].T @ q[t, a]) / below
    out = rms_norm(out, None, eps).reshape(length, heads * vdim) * w["norm"]
    return (out * torch.sigmoid(h @ w["g"].T)) @ w["o"].T


def parallel_mixer(h, w, m, eps):
    left = windowed_attention(h, _sub(w, "left."), m["left"], eps)
    right = matrix_memory(h, _sub(w, "right."), m["right"], eps)
    return 0.5 * (rms_norm(left, w["left.out"], eps) + rms_norm(right, w["right.out"], eps))


def gated_expert(h, w):
    return (silu(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def route(scores, correction, top, groups=None):
    """The chosen experts of one token, best first.  ``scores`` [E]; the choice goes by
    ``scores + correction``, limited to the ``keep`` groups of neighbours whose best choice score
    is largest."""
    choice = scores + correction
    allowed = torch.ones_like(choice, dtype=torch.bool)
    if groups is not None:
        count, keep = int(groups["count"]), int(groups["keep"])
        per = choice.shape[0] // count
        best = choice.view(count, per).max(dim=1).values
        kept = torch.topk(best, keep).indices
        allowed = torch.zeros(count, per, dtype=torch.bool)
        allowed[kept] = True
        allowed = allowed.reshape(-1)
    choice = torch.where(allowed, choice, torch.full_like(choice, -math.inf))
    return torch.topk(choice, top).indices.tolist()


def routed_feed_forward(h, w, mlp, margins=None):
    """h [T, width].  ``margins``: a list that receives, per token, how far the last chosen
    expert's choice score lies above the first one left out (a close call flips in lower precision)."""
    router = mlp["router"]
    experts, identity, top = int(router["experts"]), int(router.get("identity", 0)), int(router["top"])
    scores = torch.softmax(h @ w["router"].T, dim=-1)                 # over experts and identity experts
    correction = w["correction"] if "correction" in w else torch.zeros(experts + identity, dtype=h.dtype)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = route(scores[t], correction, top, router.get("groups"))
        if margins is not None:
            margins.append(_margin(scores[t] + correction, chosen, router.get("groups")))
        for e in chosen:
            if e >= experts:
                out[t] += scores[t, e] * h[t]                            # an identity expert
            else:
                out[t] += scores[t, e] * gated_expert(h[t], _sub(w, f"e{e}."))
    shared = mlp.get("shared")
    if shared is not None:
        s = _sub(w, "shared.")
        out = out + gated_expert(h, s) * torch.sigmoid(h @ s["sg"].T)
    return out


def _margin(choice, chosen, groups):
    allowed = torch.ones_like(choice, dtype=torch.bool)
    if groups is not None:
        per = choice.shape[0] // int(groups["count"])
        kept = {e // per for e in chosen}
        best = choice.view(-1, per).max(dim=1).values
        inside = sorted(best[list(kept)].tolist())
        outside = sorted((best[g].item() for g in range(best.shape[0]) if g not in kept), reverse=True)
        group_margin = inside[0] - outside[0] if outside and len(kept) == int(groups["keep"]) else math.inf
        allowed = torch.tensor([e // per in kept for e in range(choice.shape[0])])
    else:
        group_margin = math.inf
    rest = [choice[e].item() for e in range(choice.shape[0]) if allowed[e] and e not in chosen]
    last = min(choice[e].item() for e in chosen)
    return min(group_margin, last - max(rest) if rest else math.inf)


def _sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def schedule(config):
    """The layers in the order they run, each with the number of its pass through the loop
    (0 outside the loop and in its first pass)."""
    count = len(config["layers"])
    loop = config.get("loop")
    if loop is None:
        return [(i, 0) for i in range(count)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, 0) for i in range(start)]
    for p in range(times):
        runs += [(i, p) for i in range(start, stop)]
    return runs + [(i, 0) for i in range(stop, count)]


def forward(config, weights, tokens, dtype=F64, margins=None):
    """Logits ``[T, vocab]`` and the residual stream after every run of a layer ``[runs, T, width]``."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = float(config["norm"]["eps"])
    first = w["embed"][torch.tensor(tokens)] * float(config["embedding"]["scale"])
    x = first.clone()
    loop = config.get("loop")
    after = []
    for index, p in schedule(config):
        layer = config["layers"][index]
        if p > 0 and index == int(loop["start"]):
            x = x + first                                   # once a repeat, ahead of its first layer
        lw = _sub(w, f"l{index}.")
        h = rms_norm(x, lw["norm1"], eps)
        if layer["type"] == "parallel":
            x = x + parallel_mixer(h, _sub(lw, "mix."), layer["mixer"], eps)
        elif layer["type"] == "attention":
            x = x + sink_attention(h, _sub(lw, "mix."), layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            h = rms_norm(x, lw["norm2"], eps)
            x = x + routed_feed_forward(h, _sub(lw, "mlp."), layer["mlp"], margins)
        after.append(x.clone())
    x = rms_norm(x, w["final.norm"], eps)
    return (x @ w["embed"].T) * float(config["logit_scale"]), torch.stack(after)


# ---------------------------------------------------------------------------
def tensor_shapes(config):
    width, shapes = config["width"], {"embed": (config["vocab"], config["width"]), "final.norm": (config["width"],)}
    for index, layer in enumerate(config["layers"]):
        p, m = f"l{index}.", layer["mixer"]
        shapes[p + "norm1"] = (width,)
        if layer["type"] == "parallel":
            a, r = m["left"], m["right"]
            shapes.update({
                p + "mix.left.q": (a["heads"] * a["dim"], width), p + "mix.left.k": (a["kv_heads"] * a["dim"], width),
                p + "mix.left.v": (a["kv_heads"] * a["vdim"], width), p + "mix.left.q.norm": (a["dim"],),
                p + "mix.left.k.norm": (a["dim"],), p + "mix.left.o": (width, a["heads"] * a["vdim"]),
                p + "mix.right.q": (r["heads"] * r["dim"], width), p + "mix.right.k": (r["heads"] * r["dim"], width),
                p + "mix.right.v": (r["heads"] * r["vdim"], width), p + "mix.right.g": (r["heads"] * r["vdim"], width),
                p + "mix.right.o": (width, r["heads"] * r["vdim"]), p + "mix.right.norm": (r["heads"] * r["vdim"],),
                p + "mix.right.i": (r["heads"], width), p + "mix.right.i.b": (r["heads"],),
                p + "mix.right.f": (r["heads"], width), p + "mix.right.f.b": (r["heads"],),
                p + "mix.left.out": (width,), p + "mix.right.out": (width,),
            })
        else:
            shapes.update({
                p + "mix.q": (m["heads"] * m["dim"], width), p + "mix.k": (m["kv_heads"] * m["dim"], width),
                p + "mix.q.norm": (m["heads"] * m["dim"],), p + "mix.k.norm": (m["kv_heads"] * m["dim"],),
                p + "mix.sink": (m["heads"],), p + "mix.o": (width, m["heads"] * m["vdim"]),
            })
        mlp = layer.get("mlp")
        if mlp is not None:
            shapes[p + "norm2"] = (width,)
            router, ff = mlp["router"], mlp["expert"]["ff"]
            total = router["experts"] + router.get("identity", 0)
            for e in range(router["experts"]):
                shapes.update({p + f"mlp.e{e}.gate": (ff, width), p + f"mlp.e{e}.up": (ff, width),
                               p + f"mlp.e{e}.down": (width, ff)})
            shapes[p + "mlp.router"] = (total, width)
            shapes[p + "mlp.correction"] = (total,)
            if mlp.get("shared") is not None:
                sff = mlp["shared"]["ff"]
                shapes.update({p + "mlp.shared.gate": (sff, width), p + "mlp.shared.up": (sff, width),
                               p + "mlp.shared.down": (width, sff), p + "mlp.shared.sg": (1, width)})
    return shapes


def random_model(config, seed):
    """Random bfloat16 weights that keep activations of order one: matrices N(0, 1/in), norm weights
    around one, routers wide enough that scores spread, gate biases that let the memory forget."""
    generator = torch.Generator().manual_seed(seed)
    weights = {}
    for name, shape in tensor_shapes(config).items():
        leaf = name.split(".")[-1]
        if name.endswith(("norm1", "norm2", ".norm", ".out", "final.norm")) and len(shape) == 1:
            t = 1.0 + 0.1 * torch.randn(shape, generator=generator)
        elif leaf == "sink":
            t = 0.5 * torch.randn(shape, generator=generator)
        elif leaf == "correction":
            t = 0.05 * torch.randn(shape, generator=generator)
        elif name.endswith((".i.b", ".f.b")):
            t = torch.randn(shape, generator=generator) + (2.0 if name.endswith(".f.b") else 0.0)
        elif leaf == "router":
            t = 3.0 * torch.randn(shape, generator=generator) * shape[-1] ** -0.5
        elif name == "embed":
            t = torch.randn(shape, generator=generator)
        else:
            t = torch.randn(shape, generator=generator) * shape[-1] ** -0.5
        weights[name] = t.to(torch.bfloat16)
    return weights
