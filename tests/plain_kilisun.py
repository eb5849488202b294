"""A plain, slow statement of the Kilisun design in float64 on the CPU: one function per mechanism, one
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


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x, weights, name, eps):
    """The model's and the layers' norm: the weight is stored around zero."""
    return unit_rms(x, eps) * (1.0 + _w(weights, name))


def short_conv(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    T, taps = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            src = t - taps + 1 + j
            if src >= 0:
                y[t] += w[:, j] * u[src]
    return y


def head_norm(x, w, eps):
    """x [T, heads, d]: every head divided by its root mean square, times the one weight vector."""
    return unit_rms(x, eps) * w


def turn(x, dims, base):
    """x [T, heads, d]: the first ``dims`` coordinates turned by the row's position, i with i + dims / 2."""
    if not dims:
        return x
    half = dims // 2
    freq = torch.tensor([float(base) ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    angle = torch.arange(x.shape[0], dtype=F)[:, None] * freq[None, :]
    c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def temperature(p, coef, every):
    return 1.0 + coef * math.log(math.floor((p + 1) / every) + 1)


def softmax_over(q, keys, values, visible, scale, softcap=None):
    """One query [d] over the visible positions of keys [T, d] and values [T, v]."""
    s = (keys[visible] @ q) * scale
    if softcap:
        s = softcap * torch.tanh(s / softcap)
    w = torch.softmax(s, dim=0)
    return w @ values[visible]


def conv_attention(h, weights, p, m, eps):
    """The mixer ``attention``: keys are the values, a short convolution behind the projections of q and k, norms
    per head, a query temperature by position, causal softmax, a gate per head."""
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    T = h.shape[0]
    q = h @ _w(weights, f"{p}.q").T
    k = h @ _w(weights, f"{p}.k").T
    q = short_conv(q, _w(weights, f"{p}.q.conv"))
    k = short_conv(k, _w(weights, f"{p}.k.conv"))
    v = k.reshape(T, G, D)
    qn = head_norm(q.reshape(T, H, D), _w(weights, f"{p}.q.norm"), eps)
    kn = head_norm(k.reshape(T, G, D), _w(weights, f"{p}.k.norm"), eps)
    gate = sigmoid(h @ _w(weights, f"{p}.g").T)              # [T, H]
    out = torch.zeros((T, H, m["vdim"]), dtype=F)
    for i in range(T):
        tau = temperature(i, m["q_temp"]["coef"], m["q_temp"]["every"])
        vis = list(range(i + 1))
        for a in range(H):
            g = a // (H // G)
            out[i, a] = softmax_over(qn[i, a] * tau, kn[:, g], v[:, g], vis, m["scale"]) * gate[i, a]
    return out.reshape(T, -1) @ _w(weights, f"{p}.o").T


def diff_keys_values(h, weights, p, m, eps):
    """What a layer of ``attention_2`` keeps per token: keys [T, G, 2, D] after norm and rotation, values [T, G, V]."""
    G, D, V = m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    k = (h @ _w(weights, f"{p}.k").T).reshape(T, G * 2, D)
    k = turn(head_norm(k, _w(weights, f"{p}.k.norm"), eps), m["rot"]["dims"], m["rot"]["base"])
    v = (h @ _w(weights, f"{p}.v").T).reshape(T, G, V)
    return k.reshape(T, G, 2, D), v


def diff_attention(h, weights, p, m, eps, kv=None):
    """The mixer ``attention_2``: two maps per head over the same values within a window, the second taken off the
    first with one factor a layer, then a norm without weight.  ``kv``: another layer's keys and values."""
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    if kv is None:
        kv = diff_keys_values(h, weights, p, m, eps)
    keys, values = kv
    q = (h @ _w(weights, f"{p}.q").T).reshape(T, H * 2, D)
    q = turn(head_norm(q, _w(weights, f"{p}.q.norm"), eps), m["rot"]["dims"], m["rot"]["base"]).reshape(T, H, 2, D)
    lam = math.exp(float((_w(weights, f"{p}.lq1") * _w(weights, f"{p}.lk1")).sum())) \
        - math.exp(float((_w(weights, f"{p}.lq2") * _w(weights, f"{p}.lk2")).sum())) + m["diff"]
    out = torch.zeros((T, H, V), dtype=F)
    for i in range(T):
        vis = [j for j in range(i + 1) if i - j < m["mask"]["size"]]
        for a in range(H):
            g = a // (H // G)
            a1 = softmax_over(q[i, a, 0], keys[:, g, 0], values[:, g], vis, m["scale"], m.get("softcap"))
            a2 = softmax_over(q[i, a, 1], keys[:, g, 1], values[:, g], vis, m["scale"], m.get("softcap"))
            o = a1 - lam * a2
            out[i, a] = unit_rms(o, eps) * (1.0 - m["diff"])
    return out.reshape(T, -1) @ _w(weights, f"{p}.o").T


def gated_unit(h, weights, p, limit):
    """g = min(gate, limit), u = clamp(up, +-limit), down(g sigmoid(1.702 g) (u + 1))."""
    g = torch.clamp(h @ _w(weights, f"{p}.gate").T, max=limit)
    u = torch.clamp(h @ _w(weights, f"{p}.up").T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ _w(weights, f"{p}.down").T


def route(h, weights, p, r):
    """Per token the chosen experts and their weights: sigmoid scores, a correction for the choice only, experts
    of the best groups only (a group's score: its two largest choice scores), weights not renormalized."""
    s = sigmoid(h @ _w(weights, f"{p}.router").T)               # [T, E]
    choice = s + _w(weights, f"{p}.correction")
    E, top = r["experts"], r["top"]
    n_groups, keep = r["groups"]["count"], r["groups"]["keep"]
    per = E // n_groups
    chosen, weight = [], []
    for t in range(h.shape[0]):
        c = choice[t].clone()
        gs = [float(torch.topk(c[g * per:(g + 1) * per], min(2, per)).values.sum()) for g in range(n_groups)]
        best = sorted(range(n_groups), key=lambda g: (-gs[g], g))[:keep]
        for g in range(n_groups):
            if g not in best:
                c[g * per:(g + 1) * per] = -math.inf
        idx = sorted(range(E), key=lambda e: (-float(c[e]), e))[:top]
        chosen.append(idx)
        weight.append([float(s[t, e]) * r["scale"] for e in idx])
    return chosen, weight


def experts(h, weights, p, mlp):
    chosen, weight = route(h, weights, p, mlp["router"])
    out = torch.zeros((h.shape[0], _w(weights, f"{p}.e0.down").shape[0]), dtype=F)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t], weight[t]):
            out[t] += w * gated_unit(h[t:t + 1], weights, f"{p}.e{e}", mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        gate = sigmoid(h @ _w(weights, f"{p}.shared.sg").T)      # [T, 1]
        out = out + gate * gated_unit(h, weights, f"{p}.shared", mlp["shared"]["limit"])
    return out


def feed_forward(h, weights, p, mlp):
    if mlp["kind"] == "dense":
        return gated_unit(h, weights, p, mlp["limit"])
    return experts(h, weights, p, mlp)


def forward(config, weights, tokens):
    """(logits [T, vocab], the stream after every layer [layers, T, width])."""
    eps = config["norm"]["eps"]
    x = offset_norm(_w(weights, "embed")[torch.as_tensor(tokens)], weights, "embed.norm", eps)
    kept, streams = {}, []
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}", layer["mixer"]
        h = offset_norm(x, weights, f"{p}.norm1", eps)
        if layer["type"] == "attention":
            y = conv_attention(h, weights, f"{p}.mix", m, eps)
        else:
            src = m.get("kv_from")
            if src is None:
                kept[i] = diff_keys_values(h, weights, f"{p}.mix", m, eps)
            y = diff_attention(h, weights, f"{p}.mix", m, eps, kv=kept[i if src is None else src])
        x = x + offset_norm(y, weights, f"{p}.norm1b", eps)
        if layer.get("mlp") is not None:
            h = offset_norm(x, weights, f"{p}.norm2", eps)
            x = x + offset_norm(feed_forward(h, weights, f"{p}.mlp", layer["mlp"]), weights, f"{p}.norm2b", eps)
        streams.append(x.clone())
    logits = offset_norm(x, weights, "final.norm", eps) @ _w(weights, "embed").T
    return logits, torch.stack(streams)
