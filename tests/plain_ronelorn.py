"""A plain, slow statement of the Ronelorn design in float64 on the CPU: one function per mechanism, one
sequence at a time, every query a Python loop over what it may see.  It shares no code with the library:
the tests compare the library's kernels, cache and step function against it.

``weights`` maps tensor names to tensors, ``config`` is the dictionary of a config.json.  Every function takes
a whole sequence ``[T, ...]`` and starts from empty state; ``forward`` returns the logits of every position and
the stream after every layer.
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def _w(weights, name):
    return weights[name].to(F)


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z):
    return z * sigmoid(z)


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def block_norm(x, weights, name, eps):
    """The layers' norm: its weight is stored around zero."""
    return unit_rms(x, eps) * (1.0 + _w(weights, name))


def turn(x, positions, dims, base, divide=1.0, back=False):
    """x [T, heads, d]: the first ``dims`` coordinates of every head turned by the row's position, coordinate i
    with i + dims / 2, pair i by the angle position * base^(-2 i / dims) / divide (``back``: by minus that)."""
    if not dims:
        return x
    half = dims // 2
    freq = torch.tensor([float(base) ** (-2.0 * i / dims) / divide for i in range(half)], dtype=F)
    angle = torch.as_tensor(positions, dtype=F)[:, None] * freq[None, :]
    if back:
        angle = -angle
    c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def tokens_seen(i, size, keep_first):
    """Positions a query at i sees as tokens: its window, and the kept first tokens that have left it."""
    return [j for j in range(i + 1) if i - j < size or j < keep_first]


def runs_seen(i, size, pool):
    """Runs of ``pool`` tokens that lie wholly before the window of a query at i."""
    if not pool:
        return []
    return [b for b in range((i + 1) // pool + 1) if b * pool + pool - 1 <= i - size]


def softmax_over_seen(q, k, v, scale, size, keep_first=0, pool=0, softcap=None, sink=False):
    """q [T, H, D], k [T, G, D], v [T, G, V] as the cache would hold them -> [T, H, V].  One softmax over the
    tokens a query sees and the means of the runs it sees; ``sink``: one is added to the denominator."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=F)
    for i in range(T):
        js, bs = tokens_seen(i, size, keep_first), runs_seen(i, size, pool)
        for h in range(H):
            g = h // (H // G)
            keys = [k[b * pool:(b + 1) * pool, g].mean(0) for b in bs] + [k[j, g] for j in js]
            vals = [v[b * pool:(b + 1) * pool, g].mean(0) for b in bs] + [v[j, g] for j in js]
            s = torch.stack(keys) @ q[i, h] * scale
            if softcap:
                s = softcap * torch.tanh(s / softcap)
            e = torch.exp(s - s.max())
            denom = e.sum() + (math.exp(-float(s.max())) if sink else 0.0)
            out[i, h] = (e / denom) @ torch.stack(vals)
    return out


# ---- mixers ---------------------------------------------------------------------------------------
def attention(h, weights, p, m, eps):
    """Norm of q and k per head, rotation of q and k with scaled frequencies, values turned over their whole
    width and the heads' sums turned back, capped scores, window with pooled runs."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot, pos = m["rot"], list(range(T))
    q = unit_rms((h @ _w(weights, p + ".q").T).reshape(T, H, D), eps) * _w(weights, p + ".q.norm")
    k = unit_rms((h @ _w(weights, p + ".k").T).reshape(T, G, D), eps) * _w(weights, p + ".k.norm")
    v = (h @ _w(weights, p + ".v").T).reshape(T, G, V)
    divide = float((rot.get("scaling") or {}).get("factor", 1.0))
    q, k = turn(q, pos, rot["dims"], rot["base"], divide), turn(k, pos, rot["dims"], rot["base"], divide)
    v = turn(v, pos, V, rot["base"])
    o = softmax_over_seen(q, k, v, m["scale"], m["mask"]["size"], 0, m["mask"].get("pool") or 0, m.get("softcap"))
    o = turn(o, pos, V, rot["base"], back=True)
    return o.reshape(T, H * V) @ _w(weights, p + ".o").T


def attention_2(h, weights, p, m, eps):
    """Norm of q and k over the whole projection, rotation of q and k, window with kept first tokens, a sink."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot, pos = m["rot"], list(range(T))
    q = (unit_rms(h @ _w(weights, p + ".q").T, eps) * _w(weights, p + ".q.norm")).reshape(T, H, D)
    k = (unit_rms(h @ _w(weights, p + ".k").T, eps) * _w(weights, p + ".k.norm")).reshape(T, G, D)
    v = (h @ _w(weights, p + ".v").T).reshape(T, G, V)
    q, k = turn(q, pos, rot["dims"], rot["base"]), turn(k, pos, rot["dims"], rot["base"])
    o = softmax_over_seen(q, k, v, m["scale"], m["mask"]["size"], m["mask"].get("keep_first") or 0, sink=True)
    return o.reshape(T, H * V) @ _w(weights, p + ".o").T


def min_gru(h, weights, p, m):
    z = sigmoid(h @ _w(weights, p + ".z").T + _w(weights, p + ".z.b"))
    u = h @ _w(weights, p + ".x").T + _w(weights, p + ".x.b")
    cand = torch.where(u >= 0, u + 0.5, sigmoid(u))
    gate = silu(h @ _w(weights, p + ".g").T)
    state, rows = torch.zeros(m["width"], dtype=F), []
    for t in range(h.shape[0]):
        state = (1.0 - z[t]) * state + z[t] * cand[t]
        rows.append(state * gate[t])
    return torch.stack(rows) @ _w(weights, p + ".o").T


def dense(h, weights, p):
    return torch.relu(h @ _w(weights, p + ".up").T) ** 2 @ _w(weights, p + ".down").T


MIXERS = {"attention": attention, "attention_2": attention_2}


def forward(tokens, weights, config):
    """(logits [T, vocab], [the stream after every layer])."""
    eps, mult = config["norm"]["eps"], config.get("residual_mult", 1.0)
    x = _w(weights, "embed")[torch.as_tensor(tokens)] * (config.get("embedding") or {}).get("scale", 1.0)
    streams = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{layer.get('weights_of', i) if layer.get('weights_of') is not None else i}"
        h = block_norm(x, weights, p + ".norm1", eps)
        if layer["type"] == "mingru":
            y = min_gru(h, weights, p + ".mix", layer["mixer"])
        else:
            y = MIXERS[layer["type"]](h, weights, p + ".mix", layer["mixer"], eps)
        x = x + mult * y
        if layer.get("mlp"):
            x = x + mult * dense(block_norm(x, weights, p + ".norm2", eps), weights, p + ".mlp")
        streams.append(x.clone())
    return block_norm(x, weights, "final.norm", eps) @ _w(weights, "head").T, streams
