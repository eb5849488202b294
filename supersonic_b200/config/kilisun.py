"""Typed configuration of the ``Kilisun`` architecture.

Its config.json is nested.  Top level: ``vocab``, ``width``, ``norm.eps`` and ``layers``, a list with one entry per
layer: ``type`` (``attention`` or ``attention_2``), ``mixer`` (that mixer's sizes and constants) and ``mlp`` (null,
``{"kind": "dense", "ff", "limit"}`` or ``{"kind": "moe", "router": {"experts", "top", "scale", "groups": {"count",
"keep"}}, "expert": {"ff", "limit"}, "shared": {"ff", "limit"} or absent}``).

``build_spec`` turns that into parts.  The embedding's rows pass an RMS norm (``embed.norm``).  A layer is a
``sandwich`` block, x <- x + norm1b(mixer(norm1(x))), then x <- x + norm2b(ff(norm2(x))), with ``rmsnorm`` norms whose
weights are stored around zero (``unit_offset``).  The mixers are both ``window_attention``:

* ``attention``: causal over all earlier tokens, no rotation; the values are the keys as projected; a short causal
  convolution (``conv`` taps) behind the projections of q and k; a norm of q and k per head; a query temperature
  that grows with the position (``q_temp``); a sigmoid gate per head on the result;
* ``attention_2``: differential attention inside a sliding window ``mask.size``: two score maps per head over the
  same values, normed per head and map, the first ``rot.dims`` coordinates rotated, scores capped by ``softcap``;
  ``diff`` is the offset of the factor the second map is taken off with.  With ``kv_from``: j the layer has no key
  and value tensors and reads the cache entry of layer j (which keeps tokens for the longest window of its readers).

The feed-forward is a gated unit with the clamped activation (``swiglu`` with ``activation``), or ``experts`` of such
units with the ``sigmoid_groups`` router and a gated shared expert.  The head is the embedding table.  Tensor names:
``embed``, ``embed.norm``, ``final.norm`` and per layer i ``l<i>.norm1``, ``norm1b``, ``norm2``, ``norm2b``,
``l<i>.mix.*``, ``l<i>.mlp.*``.  The design has no position limit; the cache bounds a sequence.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import torch

from .base import BlockSpec, ConfigError, ModelSpec, PartSpec, ScheduleEntry
from .ronelorn import _need, _positive

ARCHITECTURE = "Kilisun"
MIXERS = ("attention", "attention_2")
NO_POSITION_LIMIT = 1 << 20
GATE_SLOPE_ACTIVATION = "clamped_swish"      # g' sigmoid(1.702 g') (u' + 1) with g', u' clamped by the layer's limit


def _number(d, key, where: str, positive: bool = True) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or (positive and not v > 0):
        raise ConfigError(f"{where}.{key} must be a {'positive ' if positive else ''}number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class KilisunConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: List[Dict[str, Any]] = field(default_factory=list)
    eos_token_ids: List[int] = field(default_factory=list)
    model_type: str = "kilisun"

    # ---- reading -----------------------------------------------------
    @staticmethod
    def from_dict(d: Dict[str, Any]) -> "KilisunConfig":
        _need(d, ("vocab", "width", "layers", "norm"), "config.json")
        _need(d["norm"], ("eps",), "norm")
        eos = d.get("eos_token_id")
        cfg = KilisunConfig(
            vocab=int(d["vocab"]), width=int(d["width"]), norm_eps=float(d["norm"]["eps"]),
            layers=copy.deepcopy(list(d["layers"])),
            eos_token_ids=[] if eos is None else [int(eos)] if isinstance(eos, int) else [int(e) for e in eos])
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("vocab and width must be positive")
        if not self.norm_eps > 0:
            raise ConfigError("norm.eps must be positive")
        if not self.layers:
            raise ConfigError("layers must name at least one layer")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            _need(layer, ("type", "mixer"), where)
            m, kind = layer["mixer"], layer["type"]
            if kind not in MIXERS:
                raise ConfigError(f"{where}.type {kind!r} is not known (known: {list(MIXERS)})")
            _need(m, ("heads", "kv_heads", "dim", "vdim", "scale"), where + ".mixer")
            _positive(m, ("heads", "kv_heads", "dim", "vdim"), where + ".mixer")
            _number(m, "scale", where + ".mixer")
            if m["heads"] % m["kv_heads"]:
                raise ConfigError(f"{where}.mixer: {m['heads']} heads over {m['kv_heads']} kv heads")
            if kind == "attention":
                _need(m, ("conv", "q_temp"), where + ".mixer")
                if not isinstance(m["conv"], int) or isinstance(m["conv"], bool) or m["conv"] < 1 or m["conv"] > 16:
                    raise ConfigError(f"{where}.mixer.conv must be 1 to 16 taps, got {m['conv']!r}")
                _need(m["q_temp"], ("coef", "every"), where + ".mixer.q_temp")
                _number(m["q_temp"], "coef", where + ".mixer.q_temp", positive=False)
                _positive(m["q_temp"], ("every",), where + ".mixer.q_temp")
                if m["vdim"] != m["dim"]:
                    raise ConfigError(f"{where}.mixer: the values are the keys, so vdim must equal dim")
                if m.get("kv_from") is not None:
                    raise ConfigError(f"{where}.mixer.kv_from: only a layer of attention_2 reads another layer's keys")
            else:
                _need(m, ("mask", "rot", "diff"), where + ".mixer")
                _need(m["mask"], ("size",), where + ".mixer.mask")
                _positive(m["mask"], ("size",), where + ".mixer.mask")
                _need(m["rot"], ("base", "dims"), where + ".mixer.rot")
                dims = m["rot"]["dims"]
                if not isinstance(dims, int) or isinstance(dims, bool) or dims < 0 or dims % 2 or dims > m["dim"]:
                    raise ConfigError(f"{where}.mixer.rot.dims must be even and at most dim, got {dims!r}")
                _number(m["rot"], "base", where + ".mixer.rot")
                _number(m, "diff", where + ".mixer", positive=False)
                if m.get("softcap") is not None:
                    _number(m, "softcap", where + ".mixer")
                src = m.get("kv_from")
                if src is not None:
                    if not isinstance(src, int) or isinstance(src, bool) or not 0 <= src < i:
                        raise ConfigError(f"{where}.mixer.kv_from must name an earlier layer, got {src!r}")
                    other = self.layers[src]
                    if other["type"] != "attention_2" or other["mixer"].get("kv_from") is not None:
                        raise ConfigError(f"{where}.mixer.kv_from names layer {src}, which keeps no keys of this kind")
                    om = other["mixer"]
                    if any(om[k] != m[k] for k in ("kv_heads", "dim", "vdim")) or om["rot"] != m["rot"]:
                        raise ConfigError(f"{where} reads the keys of layer {src} but differs from it in heads or rotation")
            self._validate_mlp(layer.get("mlp"), where + ".mlp")
        for e in self.eos_token_ids:
            if not 0 <= e < self.vocab:
                raise ConfigError(f"eos_token_id {e} is outside the vocabulary")

    @staticmethod
    def _validate_mlp(mlp, where: str) -> None:
        if mlp is None:
            return
        kind = mlp.get("kind") if isinstance(mlp, dict) else None
        if kind == "dense":
            _need(mlp, ("ff", "limit"), where)
            _positive(mlp, ("ff",), where)
            _number(mlp, "limit", where)
        elif kind == "moe":
            _need(mlp, ("router", "expert"), where)
            r = mlp["router"]
            _need(r, ("experts", "top"), where + ".router")
            _positive(r, ("experts", "top"), where + ".router")
            groups = r.get("groups") or {"count": 1, "keep": 1}
            _need(groups, ("count", "keep"), where + ".router.groups")
            _positive(groups, ("count", "keep"), where + ".router.groups")
            if r["experts"] % groups["count"] or groups["keep"] > groups["count"]:
                raise ConfigError(f"{where}.router: {r['experts']} experts in {groups['count']} groups, {groups['keep']} kept")
            if r["top"] > groups["keep"] * (r["experts"] // groups["count"]):
                raise ConfigError(f"{where}.router: {r['top']} experts a token cannot come from {groups['keep']} groups")
            if r.get("scale") is not None:
                _number(r, "scale", where + ".router")
            for part in ("expert", "shared"):
                if mlp.get(part) is not None:
                    _need(mlp[part], ("ff", "limit"), f"{where}.{part}")
                    _positive(mlp[part], ("ff",), f"{where}.{part}")
                    _number(mlp[part], "limit", f"{where}.{part}")
        else:
            raise ConfigError(f"{where}.kind {kind!r} is not known (known: 'dense', 'moe')")

    # ---- writing -----------------------------------------------------
    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": ARCHITECTURE, "layers": copy.deepcopy(self.layers),
                             "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # ---- what other parts of the framework ask ---------------------------------------
    @property
    def architectures(self) -> List[str]:
        return [ARCHITECTURE]

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @property
    def max_position_embeddings(self) -> int:
        return NO_POSITION_LIMIT

    def kv_source(self, i: int) -> int:
        """The layer whose cache entry layer i reads."""
        src = self.layers[i]["mixer"].get("kv_from")
        return i if src is None else int(src)

    def cache_reach(self, i: int) -> int:
        """How far back the cache entry of layer i keeps tokens: the longest window among the layers that read it."""
        return max(int(l["mixer"]["mask"]["size"]) for j, l in enumerate(self.layers)
                   if l["type"] == "attention_2" and self.kv_source(j) == i)

    # ---- the architecture as parts ----------------------------------
    def _norm(self, name: str) -> PartSpec:
        return PartSpec(kind="rmsnorm", params={"size": self.width, "eps": self.norm_eps, "unit_offset": True},
                        weights={"weight": name})

    def _mixer(self, i: int):
        W, eps = self.width, self.norm_eps
        layer, p = self.layers[i], f"l{i}.mix"
        m = layer["mixer"]
        params = {"hidden_size": W, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "dim": m["dim"],
                  "value_dim": m["vdim"], "scale": float(m["scale"]), "norm_eps": eps, "qk_norm": "head"}
        weights = {"q": f"{p}.q", "o": f"{p}.o", "q_norm": f"{p}.q.norm"}
        if layer["type"] == "attention":
            params.update(window=None, values="keys", conv=int(m["conv"]), head_gate=True,
                          query_temperature={"coef": float(m["q_temp"]["coef"]), "every": int(m["q_temp"]["every"])})
            weights.update(k=f"{p}.k", k_norm=f"{p}.k.norm", g=f"{p}.g", q_conv=f"{p}.q.conv", k_conv=f"{p}.k.conv")
            return PartSpec(kind="window_attention", params=params, weights=weights), None
        rot, src = m["rot"], self.kv_source(i)
        position = None
        if rot["dims"] > 0:
            position = PartSpec(kind="rotary", params={
                "head_dim": m["dim"], "rotary_dim": rot["dims"], "theta": float(rot["base"]),
                "max_positions": NO_POSITION_LIMIT, "pairing": "halves", "scaling": None})
        params.update(window=int(m["mask"]["size"]), cache_window=self.cache_reach(src), score_maps=2,
                      map_offset=float(m["diff"]), own_kv=src == i,
                      softcap=None if m.get("softcap") is None else float(m["softcap"]))
        weights.update({r: f"{p}.{r}" for r in ("lq1", "lk1", "lq2", "lk2")})
        if src == i:
            weights.update(k=f"{p}.k", v=f"{p}.v", k_norm=f"{p}.k.norm")
        return PartSpec(kind="window_attention", params=params, weights=weights), position

    def _feed_forward(self, i: int) -> Optional[PartSpec]:
        mlp, p, W = self.layers[i].get("mlp"), f"l{i}.mlp", self.width
        if mlp is None:
            return None

        def act(limit):
            return {"kind": GATE_SLOPE_ACTIVATION, "limit": float(limit)}
        if mlp["kind"] == "dense":
            return PartSpec(kind="swiglu", params={"hidden_size": W, "intermediate_size": mlp["ff"],
                                                   "activation": act(mlp["limit"])},
                            weights={"gate": f"{p}.gate", "up": f"{p}.up", "down": f"{p}.down"})
        r = mlp["router"]
        groups = r.get("groups") or {"count": 1, "keep": 1}
        E = int(r["experts"])
        weights = {"weight": f"{p}.router", "correction": f"{p}.correction"}
        for e in range(E):
            weights.update({f"gate.{e}": f"{p}.e{e}.gate", f"up.{e}": f"{p}.e{e}.up", f"down.{e}": f"{p}.e{e}.down"})
        shared = None
        if mlp.get("shared") is not None:
            shared = {"intermediate_size": mlp["shared"]["ff"], "activation": act(mlp["shared"]["limit"]), "gate": True}
            weights.update({f"shared.{r_}": f"{p}.shared.{r_}" for r_ in ("gate", "up", "down", "sg")})
        return PartSpec(kind="experts", params={
            "hidden_size": W, "n_experts": E, "top": int(r["top"]), "expert_size": mlp["expert"]["ff"],
            "activation": act(mlp["expert"]["limit"]), "shared": shared,
            "router": {"kind": "sigmoid_groups", "groups": int(groups["count"]), "keep": int(groups["keep"]),
                       "scale": float(r.get("scale") or 1.0)}}, weights=weights)

    def build_spec(self) -> ModelSpec:
        W = self.width
        blocks = []
        for i, layer in enumerate(self.layers):
            p = f"l{i}"
            mixer, position = self._mixer(i)
            ff = self._feed_forward(i)
            out = {"mixer_out": f"{p}.norm1b"}
            if ff is not None:
                out["feed_forward_out"] = f"{p}.norm2b"
            blocks.append(BlockSpec(kind="sandwich", mixer=mixer, feed_forward=ff, mixer_norm=self._norm(f"{p}.norm1"),
                                    feed_forward_norm=None if ff is None else self._norm(f"{p}.norm2"), position=position,
                                    params={"size": W, "eps": self.norm_eps, "unit_offset": True}, weights=out))
        schedule = [ScheduleEntry(layer=i, cache=self.kv_source(i), writes_cache=self.kv_source(i) == i)
                    for i in range(len(self.layers))]
        spec = ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=W, max_positions=NO_POSITION_LIMIT,
            embedding=PartSpec(kind="embedding", params={"vocab_size": self.vocab, "hidden_size": W,
                                                         "norm": {"eps": self.norm_eps, "unit_offset": True}},
                               weights={"weight": "embed", "norm": "embed.norm"}),
            blocks=blocks, schedule=schedule, final_norm=self._norm("final.norm"),
            head=PartSpec(kind="linear_head", params={"vocab_size": self.vocab, "hidden_size": W},
                          weights={"weight": "embed"}),
            stop_token_ids=list(self.eos_token_ids))
        spec.validate()
        return spec

    def tensor_shapes(self) -> Dict[str, List[int]]:
        W = self.width
        shapes: Dict[str, List[int]] = {"embed": [self.vocab, W], "embed.norm": [W], "final.norm": [W]}
        for i, layer in enumerate(self.layers):
            p, m = f"l{i}", layer["mixer"]
            q = p + ".mix"
            H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            shapes[f"{p}.norm1"], shapes[f"{p}.norm1b"] = [W], [W]
            shapes[f"{q}.q.norm"] = [D]
            shapes[f"{q}.o"] = [W, H * V]
            if layer["type"] == "attention":
                shapes[f"{q}.q"], shapes[f"{q}.k"], shapes[f"{q}.k.norm"] = [H * D, W], [G * D, W], [D]
                shapes[f"{q}.g"] = [H, W]
                shapes[f"{q}.q.conv"], shapes[f"{q}.k.conv"] = [H * D, m["conv"]], [G * D, m["conv"]]
            else:
                shapes[f"{q}.q"] = [H * 2 * D, W]
                for r in ("lq1", "lk1", "lq2", "lk2"):
                    shapes[f"{q}.{r}"] = [D]
                if self.kv_source(i) == i:
                    shapes[f"{q}.k"], shapes[f"{q}.v"], shapes[f"{q}.k.norm"] = [G * 2 * D, W], [G * V, W], [D]
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            shapes[f"{p}.norm2"], shapes[f"{p}.norm2b"] = [W], [W]
            f = p + ".mlp"

            def unit(prefix, ff):
                shapes[f"{prefix}.gate"], shapes[f"{prefix}.up"], shapes[f"{prefix}.down"] = [ff, W], [ff, W], [W, ff]
            if mlp["kind"] == "dense":
                unit(f, mlp["ff"])
            else:
                E = mlp["router"]["experts"]
                for e in range(E):
                    unit(f"{f}.e{e}", mlp["expert"]["ff"])
                shapes[f"{f}.router"], shapes[f"{f}.correction"] = [E, W], [E]
                if mlp.get("shared") is not None:
                    unit(f"{f}.shared", mlp["shared"]["ff"])
                    shapes[f"{f}.shared.sg"] = [1, W]
        return shapes

    def is_norm_tensor(self, name: str) -> bool:
        return name.endswith((".q.norm", ".k.norm"))

    def special_random_tensor(self, name: str, seed: int, device, std: float) -> Optional[torch.Tensor]:
        """Random values for what is neither a matrix nor a plain norm weight: norms stored around zero, the
        router's corrections, the vectors behind the maps' factor, and convolution taps of order one."""
        from ..weights.random_fill import fnv1a64
        last = name.rsplit(".", 1)[-1]
        spread = {"norm1": 0.1, "norm1b": 0.1, "norm2": 0.1, "norm2b": 0.1, "correction": 0.1, "lq1": 0.1, "lk1": 0.1,
                  "lq2": 0.1, "lk2": 0.1, "conv": 0.5}.get(last)
        if name in ("final.norm", "embed.norm"):
            spread = 0.1
        if spread is None or name.endswith((".q.norm", ".k.norm")):
            return None
        shape = self.tensor_shapes()[name]
        g = torch.Generator().manual_seed((seed * 0x9E3779B1 + fnv1a64(name)) % (1 << 62))
        t = spread * torch.randn(shape, generator=g)
        return t.to(torch.bfloat16).contiguous().to(device)

    def parameter_count(self) -> int:
        total = 0
        for shape in self.tensor_shapes().values():
            n = 1
            for s in shape:
                n *= s
            total += n
        return total
