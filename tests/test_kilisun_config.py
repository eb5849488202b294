"""The Kilisun configuration on the CPU: its reader and refusals, the parts and the schedule it builds, what the
cache is asked for, and the plain statement's own masks and routing."""
import copy

import pytest
import torch

import plain_kilisun as pk
import tiny_kilisun as tk
from supersonic_b200.config import ConfigError, config_from_dict


def test_reads_and_writes_back():
    for name, (d, _, _) in tk.CONFIGS.items():
        cfg = config_from_dict(d)
        assert cfg.to_dict() == config_from_dict(cfg.to_dict()).to_dict(), name
        assert cfg.architectures == ["Kilisun"] and cfg.vocab_size == d["vocab"] and cfg.hidden_size == d["width"]
        assert cfg.num_hidden_layers == len(d["layers"])


@pytest.mark.parametrize("change,message", [
    (lambda d: d["layers"][0].update(type="mamba"), "not known"),
    (lambda d: d["layers"][0]["mixer"].update(heads=5), "kv heads"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda d: d["layers"][0]["mixer"]["mask"].update(size=0), "positive"),
    (lambda d: d["layers"][1]["mixer"].update(vdim=20), "vdim must equal dim"),
    (lambda d: d["layers"][1]["mixer"].update(conv=0), "taps"),
    (lambda d: d["layers"][1]["mixer"].update(kv_from=0), "attention_2"),
    (lambda d: d["layers"][3]["mixer"].update(kv_from=4), "earlier layer"),
    (lambda d: d["layers"][3]["mixer"].update(kv_from=1), "keeps no keys"),
    (lambda d: d["layers"][3]["mixer"].update(dim=12), "differs"),
    (lambda d: d["layers"][0]["mlp"]["router"].update(top=7), "cannot come from"),
    (lambda d: d["layers"][0]["mlp"]["router"]["groups"].update(count=5), "groups"),
    (lambda d: d["layers"][1]["mlp"].update(kind="glu"), "not known"),
    (lambda d: d["layers"][1]["mlp"].pop("limit"), "missing"),
    (lambda d: d.pop("norm"), "missing"),
])
def test_refusals(change, message):
    d = copy.deepcopy(tk.A)
    change(d)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(d)


def test_schedule_and_cache_reach():
    cfg = config_from_dict(tk.A)
    spec = cfg.build_spec()
    assert [(s.layer, s.cache, s.writes_cache) for s in spec.schedule] == \
        [(0, 0, True), (1, 1, True), (2, 2, True), (3, 0, False), (4, 4, True)]
    # the entry of layer 0 keeps tokens for its reader's longer window; both say so
    assert cfg.cache_reach(0) == 30
    assert spec.blocks[0].mixer.params["window"] == 9 and spec.blocks[0].mixer.params["cache_window"] == 30
    assert spec.blocks[3].mixer.params["window"] == 30 and not spec.blocks[3].mixer.params["own_kv"]
    assert "k" not in spec.blocks[3].mixer.weights and "v" not in spec.blocks[3].mixer.weights
    from supersonic_b200.cache import KvNeed, StateNeed
    from supersonic_b200.parts import MIXERS
    cls = MIXERS["window_attention"]
    writer, reader_ = cls.cache_need_from(spec.blocks[0].mixer.params), cls.cache_need_from(spec.blocks[3].mixer.params)
    assert writer == reader_ == KvNeed(3, 20, 30, value_dim=14)          # two maps of 10 in a key row
    conv = cls.cache_need_from(spec.blocks[1].mixer.params)
    assert conv == {"tokens": KvNeed(2, 12, None, value_dim=12), "conv": StateNeed(3 * (6 + 2) * 12)}
    # several readers, one of them with a shorter window than the writer
    d = config_from_dict(tk.D)
    assert d.cache_reach(0) == 200 and [d.kv_source(i) for i in range(4)] == [0, 0, 2, 0]


def test_tensor_shapes_and_random_weights():
    cfg, store, plain = tk.build("A")
    shapes = cfg.tensor_shapes()
    assert set(shapes) == set(store.names())
    assert shapes["l0.mix.q"] == [6 * 2 * 10, 44] and shapes["l0.mix.k"] == [3 * 2 * 10, 44] and shapes["l0.mix.v"] == [3 * 14, 44]
    assert "l3.mix.k" not in shapes and "l3.mix.v" not in shapes and "l3.mix.k.norm" not in shapes
    assert shapes["l1.mix.q.conv"] == [72, 4] and shapes["l1.mix.g"] == [6, 44] and "l1.mix.v" not in shapes
    assert shapes["l0.mlp.shared.sg"] == [1, 44] and shapes["l0.mlp.correction"] == [12] and "l3.mlp.shared.gate" not in shapes
    assert "l2.norm2" not in shapes and "l2.norm1b" in shapes
    assert float(plain["l0.norm1"].float().abs().max()) < 1.0            # stored around zero
    assert float(plain["l1.mix.q.conv"].float().abs().max()) > 0.3       # taps of order one


def test_plain_route_keeps_to_the_best_groups():
    cfg, _, plain = tk.build("A")
    h = torch.randn(40, 44, dtype=torch.float64, generator=torch.Generator().manual_seed(1))
    r = tk.A["layers"][0]["mlp"]["router"]
    chosen, weight = pk.route(h, plain, "l0.mlp", r)
    s = pk.sigmoid(h @ plain["l0.mlp.router"].double().T)
    for t in range(40):
        groups = {e // 3 for e in chosen[t]}
        assert len(chosen[t]) == 3 and len(set(chosen[t])) == 3 and len(groups) <= 2
        for e, w in zip(chosen[t], weight[t]):
            assert abs(w - 1.5 * float(s[t, e])) < 1e-12                  # the score without the correction, not renormalized


def test_plain_masks():
    """A window of n tokens sees the token itself and the n - 1 before it; the convolution reads taps - 1 tokens back."""
    cfg, _, plain = tk.build("C")
    toks = [3, 9, 27, 31, 4, 4, 18, 40, 2, 11]
    a, _ = pk.forward(tk.C, plain, toks)
    b, _ = pk.forward(tk.C, plain, toks[:6])
    assert float((a[:6] - b).abs().max()) < 1e-9                          # causal
    u = torch.randn(9, 5, dtype=torch.float64)
    w = torch.randn(5, 3, dtype=torch.float64)
    y = pk.short_conv(u, w)
    assert torch.allclose(y[0], w[:, 2] * u[0]) and torch.allclose(y[4], w[:, 0] * u[2] + w[:, 1] * u[3] + w[:, 2] * u[4])
    assert abs(pk.temperature(0, 0.5, 1) - (1.0 + 0.5 * 0.6931471805599453)) < 1e-12
    assert pk.temperature(3, 0.5, 5) == 1.0 and pk.temperature(4, 0.5, 5) > 1.0
