"""The tests' own small configurations of the Kilisun design, and weights for them.

They differ from one another in every size and in the order of the layers: query heads over fewer, as many and a
single kv head; value rows narrower than, as wide as and wider than key rows; rotated coordinates fewer than and equal
to the head's, and none; capped and uncapped scores; windows shorter than, equal to and longer than a cache page,
down to one token; layers that read another layer's keys with a shorter and with a longer window than the layer that
writes them; convolutions of one, two and more taps; a query temperature that steps every token and every few
tokens; experts in one group and in several, of which one or more are kept, one to three a token, with and without a
shared expert; dense feed-forwards and layers without one.  Matrices are drawn wide so that weights are far from
uniform."""
import copy

import torch


def conv(heads, kv_heads, dim, taps, coef, every, scale=None):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "conv": taps,
                      "q_temp": {"coef": coef, "every": every}, "scale": scale if scale is not None else dim ** -0.5}}


def diff(heads, kv_heads, dim, vdim, size, rot_dims, base, offset, softcap=None, scale=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": size},
         "rot": {"base": base, "dims": rot_dims}, "diff": offset, "scale": scale if scale is not None else dim ** -0.5}
    if softcap:
        m["softcap"] = softcap
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention_2", "mixer": m}


def reader(layers, j, size=None, heads=None):
    """A layer that reads layer j's keys and values, with a window (and a number of query heads) of its own."""
    layer = copy.deepcopy(layers[j])
    layer["mixer"]["kv_from"] = j
    if size is not None:
        layer["mixer"]["mask"]["size"] = size
    if heads is not None:
        layer["mixer"]["heads"] = heads
    return layer


def dense(layer, ff, limit):
    layer = copy.deepcopy(layer)
    layer["mlp"] = None if ff is None else {"kind": "dense", "ff": ff, "limit": limit}
    return layer


def moe(layer, experts, top, groups, keep, ff, limit, scale, shared=None):
    layer = copy.deepcopy(layer)
    layer["mlp"] = {"kind": "moe", "expert": {"ff": ff, "limit": limit},
                    "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": groups, "keep": keep}}}
    if shared is not None:
        layer["mlp"]["shared"] = {"ff": shared[0], "limit": shared[1]}
    return layer


def model(vocab, width, eps, layers):
    return {"architecture": "Kilisun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


# odd sizes that no fast kernel takes; a reader with a longer window than its writer; experts in four groups
_a = [moe(diff(6, 3, 10, 14, 9, 6, 300.0, 0.3, softcap=7.0, scale=0.4), 12, 3, 4, 2, 18, 1.2, 1.5, shared=(22, 0.9)),
      dense(conv(6, 2, 12, 4, 0.4, 5, scale=0.35), 30, 2.0),
      dense(diff(4, 4, 6, 6, 21, 0, 50.0, 0.7), None, 1.0)]
A = model(97, 44, 1e-5, _a + [moe(reader(_a, 0, size=30), 6, 1, 1, 1, 12, 0.8, 0.7), dense(conv(5, 5, 8, 2, 0.2, 1), 26, 1.1)])

# round sizes, which every fast kernel takes; a reader with a shorter window and other query heads than its writer
_b = [dense(conv(8, 2, 64, 5, 0.25, 32), 128, 1.75),
      moe(diff(4, 2, 64, 128, 100, 32, 10000.0, 0.5, softcap=30.0), 8, 2, 4, 2, 64, 1.25, 1.75, shared=(64, 1.5)),
      moe(diff(2, 1, 128, 64, 70, 128, 5000.0, 0.2), 16, 4, 4, 3, 64, 2.5, 1.0)]
B = model(256, 128, 1e-6, _b + [dense(reader(_b, 1, size=40, heads=8), 256, 3.0), dense(conv(8, 1, 128, 2, 0.5, 7), None, 1.0),
                                moe(reader(_b, 1), 8, 3, 1, 1, 128, 1.0, 0.5, shared=(128, 2.0))])

# what another model might make equal or one: a single head, a window of one token and of exactly a page, a
# convolution of one tap, one expert a token out of two, a factor offset of zero, no shared expert, no feed-forward
C = model(50, 32, 1e-4,
          [dense(diff(1, 1, 16, 8, 1, 16, 20.0, 0.0), 16, 0.5),
           moe(conv(1, 1, 16, 1, 1.0, 3), 2, 1, 2, 1, 8, 1.0, 1.0),
           dense(diff(2, 1, 8, 24, 64, 4, 1000.0, 0.9, softcap=2.0), None, 1.0),
           dense(conv(3, 1, 8, 16, 0.0, 2), 40, 4.0)])

# head sizes between the tensor-core kernel's tile sizes; several readers of one entry; a reader right behind its writer
_d = [moe(diff(6, 2, 40, 80, 150, 40, 7000.0, 0.4, softcap=25.0), 8, 2, 4, 2, 32, 1.3, 2.5, shared=(48, 1.5))]
D = model(300, 192, 1e-6, _d + [moe(reader(_d, 0, size=64), 4, 2, 2, 2, 64, 1.0, 1.0, shared=(32, 1.0)),
                                dense(conv(6, 3, 96, 3, 0.3, 40), 96, 1.5),
                                dense(reader(_d, 0, size=200), 64, 2.0)])

CONFIGS = {"A": (A, 31, 0.3), "B": (B, 32, 0.2), "C": (C, 33, 0.4), "D": (D, 34, 0.2)}


def build(name_or_cfg, seed=0, std=0.3):
    """(typed configuration, weight store, the weights by name)."""
    from supersonic_b200.config import config_from_dict
    from supersonic_b200.weights import random_store
    if isinstance(name_or_cfg, str):
        name_or_cfg, seed, std = CONFIGS[name_or_cfg]
    cfg = config_from_dict(name_or_cfg)
    store = random_store(cfg, seed, std=std)
    plain = {n: store.get(n) for n in store.names()}
    return cfg, store, plain


def changed(plain, **changes):
    """(weight store, weights by name) with some tensors replaced; ``__`` in a keyword stands for a dot."""
    from supersonic_b200.weights import WeightStore
    t = dict(plain)
    for k, v in changes.items():
        name = k.replace("__", ".")
        t[name] = v.to(t[name].dtype)
    return WeightStore.from_tensors(t), t


def decisive(plain, factor=8.0):
    """(weight store, weights by name) with the routers' corrections spread ``factor`` times as wide.  Random routers
    leave several tokens in a hundred with two experts (or two groups) within a hundredth of each other; bfloat16
    then picks the other one for some of them, the plain statement's logits there are no longer the answer, and
    through the keys such a token leaves neither are those behind it.  Wider corrections keep the choice a function
    of the token (the scores still order the experts within their reach) and leave margins that rounding cannot
    cross."""
    return changed(plain, **{n.replace(".", "__"): t.float() * factor for n, t in plain.items() if n.endswith(".correction")})
