"""The tests' own small configurations of the Ronelorn design, and weights for them.

They differ from one another in every size and in the order of the layers: query heads over fewer, as many and
a single kv head; value rows narrower than, as wide as and wider than key rows; rotated coordinates fewer than
and equal to the head's; with and without frequency scaling and score cap; windows shorter than, equal to and
longer than a cache page, down to one token; runs that divide a page and runs that cross page borders, shorter
than, equal to and longer than the window; kept first tokens from one to more than a page; recurrent widths
other than the model's; layers without feed-forward; layers that run with another layer's tensors; embedding
scale and residual factor equal to one and not.  Matrices are drawn wide so that weights are far from uniform."""
import copy

import torch


def pooled(heads, kv_heads, dim, vdim, size, pool, rot_dims, base, factor=None, softcap=None, scale=None):
    rot = {"base": base, "dims": rot_dims}
    if factor:
        rot["scaling"] = {"factor": factor}
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": size, "pool": pool},
         "rot": rot, "scale": scale if scale is not None else dim ** -0.5}
    if softcap:
        m["softcap"] = softcap
    return {"type": "attention", "mixer": m}


def kept(heads, kv_heads, dim, vdim, size, keep_first, rot_dims, base, scale=None):
    return {"type": "attention_2",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                      "mask": {"size": size, "keep_first": keep_first}, "rot": {"base": base, "dims": rot_dims},
                      "scale": scale if scale is not None else dim ** -0.5}}


def gru(width):
    return {"type": "mingru", "mixer": {"width": width}}


def with_mlp(layer, ff):
    layer = copy.deepcopy(layer)
    layer["mlp"] = None if ff is None else {"kind": "dense", "ff": ff}
    return layer


def again(layers, j):
    """An entry that runs with layer j's tensors."""
    layer = copy.deepcopy(layers[j])
    layer["weights_of"] = j
    return layer


def model(vocab, width, eps, embed_scale, mult, layers):
    return {"architecture": "Ronelorn", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "embedding": {"scale": embed_scale}, "residual_mult": mult, "layers": layers}


_a = [with_mlp(pooled(4, 2, 16, 24, 20, 4, 8, 1000.0, factor=4.0, softcap=12.0, scale=0.3), 40),
      with_mlp(gru(36), None),
      with_mlp(kept(6, 3, 12, 8, 17, 3, 12, 500.0, scale=0.25), 56)]
A = model(101, 48, 1e-5, 3.0, 0.4, _a + [again(_a, 0), with_mlp(gru(20), 24)])

_b = [with_mlp(kept(3, 3, 16, 16, 9, 70, 4, 77.0), None),
      with_mlp(pooled(2, 1, 24, 10, 64, 3, 24, 300.0), 33),
      with_mlp(gru(64), 16)]
B = model(77, 40, 3e-6, 1.0, 1.0, _b + [again(_b, 0)])

# sizes that no fast kernel takes: odd widths and head sizes, a window of one token, runs as long as and longer than
# the window, two rotated coordinates
C = model(61, 50, 1e-4, 0.7, 0.9,
          [with_mlp(pooled(5, 5, 10, 6, 7, 7, 2, 50.0, factor=1.5), 9),
           with_mlp(kept(6, 1, 6, 14, 1, 1, 6, 30.0), 11),
           with_mlp(gru(7), None),
           with_mlp(pooled(3, 1, 8, 8, 5, 9, 8, 10.0, softcap=3.0), None)])

# round sizes, which every fast kernel takes
D = model(256, 128, 1e-6, 2.0, 0.5,
          [with_mlp(pooled(4, 2, 64, 128, 100, 16, 32, 10000.0, factor=2.0, softcap=20.0), 256),
           with_mlp(kept(8, 4, 128, 64, 130, 5, 64, 5000.0), 128),
           with_mlp(gru(256), None),
           with_mlp(pooled(8, 1, 128, 64, 64, 8, 128, 700.0), 64),
           with_mlp(kept(2, 2, 64, 64, 40, 66, 16, 100.0), 128)])

# another order: a recurrent layer first; recurrent and kept-token layers that run again with their tensors on state
# and pages of their own; no kept token at all; runs of one token (every token behind the window stays visible as
# its own run); a rotation over the whole head and none; head sizes between the tensor-core kernel's tile sizes
_e = [with_mlp(gru(96), 192),
      with_mlp(kept(4, 1, 40, 24, 33, 0, 40, 900.0), None),
      with_mlp(pooled(6, 2, 96, 48, 50, 1, 96, 5000.0, factor=3.0, softcap=50.0), 64)]
E = model(200, 96, 1e-5, 9.8, 0.25, _e + [again(_e, 0), again(_e, 1), with_mlp(pooled(2, 2, 32, 32, 70, 64, 0, 10.0), 40)])

CONFIGS = {"A": (A, 21, 0.3), "B": (B, 22, 0.35), "C": (C, 23, 0.4), "D": (D, 24, 0.2), "E": (E, 25, 0.3)}


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
