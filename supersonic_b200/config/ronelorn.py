"""Typed configuration of the ``Ronelorn`` architecture.

Its config.json is nested.  Top level: ``vocab``, ``width``, ``norm.eps``, ``embedding.scale`` (the embedding's rows are
multiplied by it), ``residual_mult`` (every sublayer's output is multiplied by it before it joins the stream) and
``layers``, a list with one entry per layer: ``type`` (``attention``, ``attention_2`` or ``mingru``), ``mixer`` (that
mixer's sizes and constants), ``mlp`` (null, or ``{"kind": "dense", "ff"}``) and optionally ``weights_of``: j, which
says that the layer has no tensors of its own and runs with layer j's (mixer, feed-forward and norms) on a cache
entry of its own.

``build_spec`` turns that into parts.  A layer is a ``pre_norm`` block, x <- x + m mixer(norm1(x)), then
x <- x + m ff(norm2(x)), with ``rmsnorm`` norms whose weights are stored around zero (``unit_offset``) and the
``dense`` feed-forward down(relu(up(h))^2).  The mixers:

* ``attention``: ``window_attention`` with a norm of q and k per head, rotation of the first ``rot.dims`` coordinates
  (frequencies divided by ``rot.scaling.factor``), values turned over their whole width by ``rot.base`` without
  scaling, scores capped by ``softcap``, and beyond the window ``mask.size`` one pooled row per run of ``mask.pool``
  tokens;
* ``attention_2``: ``window_attention`` with a norm of q and k over the whole projection, rotation, no value
  rotation, the first ``mask.keep_first`` tokens kept visible beyond the window, and a sink of score 0;
* ``mingru``: ``min_gru`` of ``width`` channels.

A layer with ``weights_of`` is a second stop of the schedule at the named layer's block.  Tensor names: ``embed``,
``final.norm``, ``head`` and per layer i with tensors of its own ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``,
``l<i>.mlp.up``, ``l<i>.mlp.down``.  The design has no position limit; the cache bounds a sequence.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import torch

from .base import BlockSpec, ConfigError, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "Ronelorn"
MIXERS = ("attention", "attention_2", "mingru")
NO_POSITION_LIMIT = 1 << 20


def _need(d, keys, where: str) -> None:
    if not isinstance(d, dict):
        raise ConfigError(f"{where} must be an object")
    missing = [k for k in keys if k not in d]
    if missing:
        raise ConfigError(f"{where} is missing {missing}")


def _positive(d, keys, where: str) -> None:
    for k in keys:
        if not (isinstance(d[k], int) and not isinstance(d[k], bool) and d[k] > 0):
            raise ConfigError(f"{where}.{k} must be a positive integer, got {d[k]!r}")


def _count(d, key, where: str) -> int:
    """An optional count: absent or null is 0."""
    v = d.get(key)
    if v is None:
        return 0
    if not isinstance(v, int) or isinstance(v, bool) or v < 0:
        raise ConfigError(f"{where}.{key} must be a non-negative integer, got {v!r}")
    return v


@dataclass(frozen=True)
class RonelornConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    residual_mult: float
    layers: List[Dict[str, Any]] = field(default_factory=list)
    eos_token_ids: List[int] = field(default_factory=list)
    model_type: str = "ronelorn"

    # ---- reading -----------------------------------------------------
    @staticmethod
    def from_dict(d: Dict[str, Any]) -> "RonelornConfig":
        _need(d, ("vocab", "width", "layers", "norm"), "config.json")
        _need(d["norm"], ("eps",), "norm")
        eos = d.get("eos_token_id")
        cfg = RonelornConfig(
            vocab=int(d["vocab"]), width=int(d["width"]), norm_eps=float(d["norm"]["eps"]),
            embedding_scale=float((d.get("embedding") or {}).get("scale", 1.0)),
            residual_mult=float(d.get("residual_mult", 1.0)), layers=copy.deepcopy(list(d["layers"])),
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
            if kind in ("attention", "attention_2"):
                _need(m, ("heads", "kv_heads", "dim", "vdim", "scale", "mask", "rot"), where + ".mixer")
                _positive(m, ("heads", "kv_heads", "dim", "vdim"), where + ".mixer")
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"{where}.mixer: {m['heads']} heads over {m['kv_heads']} kv heads")
                _need(m["mask"], ("size",), where + ".mixer.mask")
                _positive(m["mask"], ("size",), where + ".mixer.mask")
                _count(m["mask"], "pool", where + ".mixer.mask")
                _count(m["mask"], "keep_first", where + ".mixer.mask")
                _need(m["rot"], ("base", "dims"), where + ".mixer.rot")
                dims = m["rot"]["dims"]
                if not isinstance(dims, int) or dims < 0 or dims % 2 or dims > m["dim"]:
                    raise ConfigError(f"{where}.mixer.rot.dims must be even and at most dim, got {dims!r}")
                if m["rot"].get("scaling"):
                    _need(m["rot"]["scaling"], ("factor",), where + ".mixer.rot.scaling")
                    if not float(m["rot"]["scaling"]["factor"]) > 0:
                        raise ConfigError(f"{where}.mixer.rot.scaling.factor must be positive")
                if kind == "attention" and m["vdim"] % 2:
                    raise ConfigError(f"{where}.mixer.vdim must be even: values are turned in pairs")
                if m.get("softcap") is not None and not float(m["softcap"]) > 0:
                    raise ConfigError(f"{where}.mixer.softcap must be positive")
            elif kind == "mingru":
                _need(m, ("width",), where + ".mixer")
                _positive(m, ("width",), where + ".mixer")
            else:
                raise ConfigError(f"{where}.type {kind!r} is not known (known: {list(MIXERS)})")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind", "dense") != "dense":
                    raise ConfigError(f"{where}.mlp.kind {mlp.get('kind')!r} is not known (known: 'dense')")
                _need(mlp, ("ff",), where + ".mlp")
                _positive(mlp, ("ff",), where + ".mlp")
            src = layer.get("weights_of")
            if src is not None:
                if not isinstance(src, int) or isinstance(src, bool) or not 0 <= src < len(self.layers) or src == i:
                    raise ConfigError(f"{where}.weights_of must name another layer, got {src!r}")
                other = self.layers[src]
                if other.get("weights_of") is not None:
                    raise ConfigError(f"{where}.weights_of names layer {src}, which has no tensors of its own")
                if other["type"] != kind or other["mixer"] != m or other.get("mlp") != mlp:
                    raise ConfigError(f"{where} uses the tensors of layer {src} but differs from it")
        for e in self.eos_token_ids:
            if not 0 <= e < self.vocab:
                raise ConfigError(f"eos_token_id {e} is outside the vocabulary")

    # ---- writing -----------------------------------------------------
    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": ARCHITECTURE, "embedding": {"scale": self.embedding_scale},
                             "layers": copy.deepcopy(self.layers), "norm": {"eps": self.norm_eps},
                             "residual_mult": self.residual_mult, "vocab": self.vocab, "width": self.width}
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

    def owner(self, i: int) -> int:
        """The layer whose tensors layer i runs with."""
        src = self.layers[i].get("weights_of")
        return i if src is None else int(src)

    # ---- the architecture as parts ----------------------------------
    def _norm(self, name: str) -> PartSpec:
        return PartSpec(kind="rmsnorm", params={"size": self.width, "eps": self.norm_eps, "unit_offset": True},
                        weights={"weight": name})

    def _mixer(self, i: int):
        W, eps, mult = self.width, self.norm_eps, self.residual_mult
        layer, p = self.layers[i], f"l{i}.mix"
        m, kind = layer["mixer"], layer["type"]
        if kind == "mingru":
            return PartSpec(kind="min_gru", params={"hidden_size": W, "width": m["width"], "out_scale": mult},
                            weights={"z": f"{p}.z", "z_bias": f"{p}.z.b", "x": f"{p}.x", "x_bias": f"{p}.x.b",
                                     "g": f"{p}.g", "o": f"{p}.o"}), None
        rot, mask = m["rot"], m["mask"]
        scaling = rot.get("scaling") or None
        position = None
        if rot["dims"] > 0:
            # linear scaling: every frequency divided by the factor, which is the same as every position divided by it
            position = PartSpec(kind="rotary", params={
                "head_dim": m["dim"], "rotary_dim": rot["dims"], "theta": float(rot["base"]),
                "max_positions": NO_POSITION_LIMIT, "pairing": "halves",
                "scaling": None if not scaling else {"kind": "linear", "factor": float(scaling["factor"])}})
        params = {"hidden_size": W, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "dim": m["dim"],
                  "value_dim": m["vdim"], "scale": float(m["scale"]), "window": int(mask["size"]),
                  "keep_first": int(mask.get("keep_first") or 0), "pool": int(mask.get("pool") or 0),
                  "norm_eps": eps, "out_scale": mult}
        if kind == "attention":
            params.update(qk_norm="head", sink=False,
                          softcap=None if m.get("softcap") is None else float(m["softcap"]),
                          value_rotation={"theta": float(rot["base"]), "pairing": "halves"})
        else:
            params.update(qk_norm="row", sink=True, softcap=None, value_rotation=None)
        return PartSpec(kind="window_attention", params=params,
                        weights={"q": f"{p}.q", "k": f"{p}.k", "v": f"{p}.v", "o": f"{p}.o", "q_norm": f"{p}.q.norm",
                                 "k_norm": f"{p}.k.norm"}), position

    def build_spec(self) -> ModelSpec:
        W = self.width
        blocks, block_of = [], {}
        for i, layer in enumerate(self.layers):
            if self.owner(i) != i:
                continue
            p = f"l{i}"
            mixer, position = self._mixer(i)
            mlp = layer.get("mlp")
            ff = None if mlp is None else PartSpec(
                kind="dense", params={"hidden_size": W, "intermediate_size": mlp["ff"], "activation": "relu_squared",
                                      "out_scale": self.residual_mult},
                weights={"up": f"{p}.mlp.up", "down": f"{p}.mlp.down"})
            block_of[i] = len(blocks)
            blocks.append(BlockSpec(kind="pre_norm", mixer=mixer, feed_forward=ff, mixer_norm=self._norm(f"{p}.norm1"),
                                    feed_forward_norm=None if ff is None else self._norm(f"{p}.norm2"),
                                    position=position))
        schedule = [ScheduleEntry(layer=block_of[self.owner(i)], cache=i) for i in range(len(self.layers))]
        emb = {"vocab_size": self.vocab, "hidden_size": W}
        if self.embedding_scale != 1.0:
            emb["scale"] = self.embedding_scale
        spec = ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=W, max_positions=NO_POSITION_LIMIT,
            embedding=PartSpec(kind="embedding", params=emb, weights={"weight": "embed"}),
            blocks=blocks, schedule=schedule, final_norm=self._norm("final.norm"),
            head=PartSpec(kind="linear_head", params={"vocab_size": self.vocab, "hidden_size": W},
                          weights={"weight": "head"}),
            stop_token_ids=list(self.eos_token_ids))
        spec.validate()
        return spec

    def tensor_shapes(self) -> Dict[str, List[int]]:
        W = self.width
        shapes: Dict[str, List[int]] = {"embed": [self.vocab, W], "final.norm": [W], "head": [self.vocab, W]}
        for i, layer in enumerate(self.layers):
            if self.owner(i) != i:
                continue
            p, m = f"l{i}", layer["mixer"]
            q = p + ".mix"
            shapes[f"{p}.norm1"] = [W]
            if layer["type"] == "mingru":
                C = m["width"]
                for r in ("z", "x", "g"):
                    shapes[f"{q}.{r}"] = [C, W]
                shapes[f"{q}.z.b"], shapes[f"{q}.x.b"], shapes[f"{q}.o"] = [C], [C], [W, C]
            else:
                H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
                shapes[f"{q}.q"], shapes[f"{q}.k"], shapes[f"{q}.v"] = [H * D, W], [G * D, W], [G * V, W]
                whole = layer["type"] == "attention_2"
                shapes[f"{q}.q.norm"], shapes[f"{q}.k.norm"] = [H * D if whole else D], [G * D if whole else D]
                shapes[f"{q}.o"] = [W, H * V]
            mlp = layer.get("mlp")
            if mlp is not None:
                shapes[f"{p}.norm2"] = [W]
                shapes[f"{p}.mlp.up"], shapes[f"{p}.mlp.down"] = [mlp["ff"], W], [W, mlp["ff"]]
        return shapes

    def is_norm_tensor(self, name: str) -> bool:
        return name.endswith((".q.norm", ".k.norm"))

    def special_random_tensor(self, name: str, seed: int, device, std: float) -> Optional[torch.Tensor]:
        """Random values for what is neither a matrix nor a plain norm weight: block norms stored around zero, and
        gate biases of order one."""
        from ..weights.random_fill import fnv1a64
        last = name.rsplit(".", 1)[-1]
        if last not in ("norm1", "norm2", "b") and name != "final.norm":
            return None
        shape = self.tensor_shapes()[name]
        g = torch.Generator().manual_seed((seed * 0x9E3779B1 + fnv1a64(name)) % (1 << 62))
        t = (0.5 if last == "b" else 0.1) * torch.randn(shape, generator=g)
        return t.to(torch.bfloat16).contiguous().to(device)

    def parameter_count(self) -> int:
        total = 0
        for shape in self.tensor_shapes().values():
            n = 1
            for s in shape:
                n *= s
            total += n
        return total
