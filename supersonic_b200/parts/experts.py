"""Feed-forward experts: y(x) = sum_k w_k E_(e_k)(x) over the ``top`` experts (e_k, w_k) a router picks for the
token out of ``n_experts``, plus E_shared(x) if the layer has a shared expert.

An expert is a gated unit without biases, E(x) = Wdown (silu(Wgate x) * (Wup x)), or with ``activation`` another
inner step (see the ``swiglu`` feed-forward).  Routers are registered by name and fill two arrays per step, the
chosen experts and their weights:

* ``table``: nothing is learned and nothing is computed from x: row ``token id`` of an integer table
  [vocab, top] names the token's experts (distinct within a row), all with weight 1 / top.
* ``sigmoid_groups``: scores s = sigmoid(W x) in float32; experts are chosen by s + correction (a stored vector),
  but only among the experts of the ``keep`` best of ``groups`` equal groups of neighbours, a group's score being
  the sum of its two largest choice scores; the weights are the chosen experts' s times ``scale``, not renormalized.

A shared expert runs for every token; with ``shared.gate`` its result is multiplied by sigmoid(w_sg . x), one number
per token.

The step's (token, choice) pairs are sorted by expert on the device, the experts' matrix
products run group by group from that order, and a token's outputs are summed in the order of
its choices, so nothing depends on what else is in the step and the launch sizes depend on the
number of tokens alone (the step can be captured in a graph).
"""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc.kernel_sets import as_tensor
from .registry import BuildContext, register_feed_forward

ROUTERS: Dict[str, type] = {}


def register_router(name: str):
    def deco(cls):
        ROUTERS[name] = cls
        return cls
    return deco


@register_router("table")
class TableRouter:
    """params: ``vocab_size``; weights: ``table`` [vocab, top] int32.

    Interface of a router: ``route(ctx, x, expert_of, pair_weight)`` fills the int32 ``expert_of`` and the
    float32 ``pair_weight`` (both [tokens, top]) for the step's tokens, whose normed activations are ``x``."""

    def __init__(self, params, weights, build: BuildContext, n_experts: int, top: int):
        self.n_experts, self.top = n_experts, top
        table = build.weights.stored(weights["table"])
        if table.dtype != torch.int32 or tuple(table.shape) != (int(params["vocab_size"]), top):
            raise ValueError(f"{weights['table']}: expected int32 [{params['vocab_size']}, {top}], "
                             f"found {table.dtype} {tuple(table.shape)}")
        lo, hi = int(table.min()), int(table.max())
        if lo < 0 or hi >= n_experts:
            raise ValueError(f"{weights['table']} names experts {lo}..{hi}; there are {n_experts}")
        self.table = table.contiguous()

    def route(self, ctx, x, expert_of, pair_weight):
        ctx.kernels.route_table(ctx.batch.token_ids, self.table, self.n_experts, expert_of, pair_weight)


@register_router("sigmoid_groups")
class SigmoidGroupRouter:
    """params: ``groups`` (1), ``keep`` (all groups), ``scale`` (1.0); weights: ``weight`` [experts, hidden],
    ``correction`` [experts] (optional).  The logits are a product of their own with a float32 result (in the
    bfloat16 path: bfloat16 operands, whose products are exact in float32, summed in float32).  ``add_row`` (called
    by the part that owns the router) lets one more row ride along in that product; its sigmoid per token is
    written by the router's kernel."""

    def __init__(self, params, weights, build: BuildContext, n_experts: int, top: int):
        self.n_experts, self.top = n_experts, top
        self.groups = int(params.get("groups") or 1)
        self.keep = int(params.get("keep") or self.groups)
        self.scale = float(params.get("scale", 1.0))
        if n_experts % self.groups or not 1 <= self.keep <= self.groups:
            raise ValueError(f"sigmoid_groups: {n_experts} experts in {self.groups} groups, {self.keep} kept")
        if top > self.keep * (n_experts // self.groups):
            raise ValueError(f"sigmoid_groups: {top} experts a token cannot come from {self.keep} groups of "
                             f"{n_experts // self.groups}")
        self.rows = [build.weights.as_dtype(weights["weight"], build.dtype)]
        if self.rows[0].dim() != 2 or self.rows[0].shape[0] != n_experts:
            raise ValueError(f"{weights['weight']} has shape {tuple(self.rows[0].shape)}, expected [{n_experts}, hidden]")
        self.correction = None
        if weights.get("correction"):
            self.correction = build.weights.stored(weights["correction"]).float().contiguous()
            if tuple(self.correction.shape) != (n_experts,):
                raise ValueError(f"{weights['correction']} has shape {tuple(self.correction.shape)}, expected ({n_experts},)")
        self.extra_col = None
        self._pack()

    def _pack(self):
        w = torch.cat(self.rows, dim=0)
        pad = (-w.shape[0]) % 8                  # rows of the product's result stay a multiple of 8 wide
        if pad:
            w = torch.cat([w, torch.zeros((pad, w.shape[1]), dtype=w.dtype, device=w.device)], dim=0)
        self.weight = w.contiguous()

    def add_row(self, row: torch.Tensor) -> None:
        self.rows.append(row.reshape(1, -1).to(self.rows[0].dtype))
        self.extra_col = self.n_experts
        self._pack()

    def route(self, ctx, x, expert_of, pair_weight, extra_out=None):
        logits = torch.empty((x.shape[0], self.weight.shape[0]), dtype=torch.float32, device=x.device)
        ctx.kernels.linear(x, self.weight, logits)
        ctx.kernels.route_sigmoid_groups(logits, self.n_experts, self.correction, self.groups, self.keep, self.scale,
                                         expert_of, pair_weight, self.extra_col if extra_out is not None else None, extra_out)


@register_feed_forward("experts")
class Experts:
    """params: ``hidden_size``, ``n_experts``, ``top``, ``expert_size``, ``activation`` (None, or as the ``swiglu``
    feed-forward's), ``router`` ({"kind": ..., its own parameters}), ``shared`` (None or {"intermediate_size": ...,
    "activation": ..., "gate": bool}); weights: ``gate.<e>``, ``up.<e>``, ``down.<e>`` for every expert e, the router's
    own, and ``shared.gate`` / ``shared.up`` / ``shared.down`` (with a gate ``shared.sg`` [1, hidden])."""

    takes_lazy_input = True

    def __init__(self, params, weights, build: BuildContext):
        self.hidden, self.E = int(params["hidden_size"]), int(params["n_experts"])
        self.top, self.inter = int(params["top"]), int(params["expert_size"])
        w, dt = build.weights, build.dtype
        first, second = [], []
        for e in range(self.E):
            gate, up, down = (w.as_dtype(weights[f"{r}.{e}"], dt) for r in ("gate", "up", "down"))
            for name, t, want in ((f"gate.{e}", gate, (self.inter, self.hidden)), (f"up.{e}", up, (self.inter, self.hidden)),
                                  (f"down.{e}", down, (self.hidden, self.inter))):
                if tuple(t.shape) != want:
                    raise ValueError(f"{weights[name]} has shape {tuple(t.shape)}, expected {want}")
            first.append(torch.cat([gate, up], dim=0))
            second.append(down)
        self.w_gate_up = torch.stack(first).contiguous()       # [E, 2 * inter, hidden]: gate rows, then up rows
        self.w_down = torch.stack(second).contiguous()         # [E, hidden, inter]
        router = dict(params["router"])
        if router.get("kind") not in ROUTERS:
            raise KeyError(f"unknown router {router.get('kind')!r}; registered: {sorted(ROUTERS)}")
        self.router = ROUTERS[router["kind"]](router, weights, build, self.E, self.top)
        from .feed_forward import SwiGLU, gated_activation_of
        self.act = gated_activation_of(params.get("activation"))
        self.shared, self.shared_gate = None, False
        if params.get("shared"):
            sh = params["shared"]
            self.shared = SwiGLU({"hidden_size": self.hidden, "intermediate_size": int(sh["intermediate_size"]),
                                  "activation": sh.get("activation")},
                                 {r: weights[f"shared.{r}"] for r in ("gate", "up", "down")}, build)
            if sh.get("gate"):
                sg = w.stored(weights["shared.sg"]).reshape(-1)
                if sg.numel() != self.hidden:
                    raise ValueError(f"{weights['shared.sg']} has {sg.numel()} values, expected {self.hidden}")
                if not hasattr(self.router, "add_row"):
                    raise ValueError(f"experts: the router {router['kind']!r} reads no activations, so it cannot take the "
                                     "shared expert's gate along")
                self.router.add_row(sg)          # the router's product reads the token anyway: it takes this row too
                self.shared_gate = True
        self.dtype = dt

    @staticmethod
    def activation_elements(params) -> int:
        """Elements per token while the part runs: per choice gate, up, their product and the expert's output
        (float32: counted twice); the shared expert's rows."""
        shared = 3 * int(params["shared"]["intermediate_size"]) if params.get("shared") else 0
        return int(params["top"]) * (3 * int(params["expert_size"]) + 2 * int(params["hidden_size"])) + shared

    def forward(self, ctx, x, residual):
        T, dev, top = residual.shape[0], residual.device, self.top
        xt = as_tensor(x)
        P = T * top
        expert_of = torch.empty((T, top), dtype=torch.int32, device=dev)
        pair_weight = torch.empty((T, top), dtype=torch.float32, device=dev)
        shared_scale = None
        if self.shared_gate:
            shared_scale = torch.empty(T, dtype=torch.float32, device=dev)
            self.router.route(ctx, xt, expert_of, pair_weight, extra_out=shared_scale)
        else:
            self.router.route(ctx, xt, expert_of, pair_weight)
        tile_rows = ctx.kernels.expert_tile_rows
        max_tiles = P // tile_rows + min(self.E, P)
        ints = torch.empty(self.E + 1 + P + 2 * max_tiles + 1, dtype=torch.int32, device=dev)
        groups = {"tile_rows": tile_rows, "max_tiles": max_tiles, "offsets": ints[: self.E + 1],
                  "order": ints[self.E + 1: self.E + 1 + P],
                  "tile_expert": ints[self.E + 1 + P: self.E + 1 + P + max_tiles],
                  "tile_row0": ints[self.E + 1 + P + max_tiles: self.E + 1 + P + 2 * max_tiles], "meta": ints[-1:]}
        ctx.kernels.group_by_expert(expert_of, self.E, groups)
        z = torch.empty((P, self.inter), dtype=self.dtype, device=dev)
        if self.act is None:
            ctx.kernels.expert_gate_up(xt, top, self.w_gate_up, z, groups)
        else:
            ctx.kernels.expert_gate_up(xt, top, self.w_gate_up, z, groups, act=self.act)
        y = torch.empty((P, self.hidden), dtype=torch.float32, device=dev)
        ctx.kernels.grouped_linear(z, False, top, self.w_down, y, True, groups)
        ctx.kernels.expert_combine(residual, y, pair_weight, top)
        if self.shared is not None:
            if shared_scale is None:
                self.shared.forward(ctx, x, residual)
            else:
                self.shared.forward(ctx, x, residual, row_scale=shared_scale)
