"""Feed-forwards.  ``swiglu``: down( silu(gate(x)) * up(x) ), silu(g) = g / (1 + exp(-g)),
added to the residual (crates/runner/src/prefill_engine.rs:3226-3366;
kernels/full_attention_cuda.cuh:1995-2010).  Gate and up run as one matrix product
over row-concatenated weights; ``activation`` names another inner step of the gated unit.  ``dense``: out_scale * down( act(up(x)) ) with a named activation."""
from __future__ import annotations

import torch

from .registry import BuildContext, register_feed_forward


def gated_activation_of(spec):
    """(kind, limit) of a gated unit's inner step from its parameter, None for silu(g) u."""
    if not spec or spec.get("kind", "silu") == "silu":
        return None
    from ..csrc.ops import GATE_KINDS_FF
    if spec["kind"] not in GATE_KINDS_FF:
        raise ValueError(f"gated unit: activation {spec['kind']!r} is not known (known: {sorted(GATE_KINDS_FF)})")
    limit = float(spec.get("limit", 0.0))
    if spec["kind"] == "clamped_swish" and not limit > 0:
        raise ValueError("gated unit: the clamped activation needs a positive limit")
    return spec["kind"], limit


@register_feed_forward("swiglu")
class SwiGLU:
    """params: ``hidden_size``, ``intermediate_size``, ``activation`` (None: silu(g) u; ``{"kind": "clamped_swish",
    "limit": L}``: with g' = min(g, L) and u' = clamp(u, -L, L), g' sigmoid(1.702 g') (u' + 1)); weights: ``gate``,
    ``up``, ``down``.

    Interface of a feed-forward: ``forward(ctx, x, residual)`` reads the normed
    activations ``x`` [T, hidden] and adds its output into ``residual`` (float32).
    """

    takes_lazy_input = True

    def __init__(self, params, weights, build: BuildContext):
        self.hidden, self.inter = int(params["hidden_size"]), int(params["intermediate_size"])
        w = build.weights
        gate, up = w.as_dtype(weights["gate"], build.dtype), w.as_dtype(weights["up"], build.dtype)
        self.w_down = w.as_dtype(weights["down"], build.dtype)
        for name, t, want in ((weights["gate"], gate, (self.inter, self.hidden)),
                              (weights["up"], up, (self.inter, self.hidden)),
                              (weights["down"], self.w_down, (self.hidden, self.inter))):
            if tuple(t.shape) != want:
                raise ValueError(f"{name} has shape {tuple(t.shape)}, expected {want}")
        self.w_gate_up, self.layout = build.kernels.pack_gate_up(gate, up)
        self.act = gated_activation_of(params.get("activation"))
        self.dtype = build.dtype

    @staticmethod
    def activation_elements(params) -> int:
        """Elements per token this part holds while it runs: gate and up, and their product."""
        return 3 * int(params["intermediate_size"])

    def forward(self, ctx, x, residual, row_scale=None):
        """``row_scale``: one float32 factor per token on the unit's result (applied to the inner rows, which the
        last product maps linearly)."""
        z = torch.empty((residual.shape[0], self.inter), dtype=self.dtype, device=residual.device)
        if self.act is None and row_scale is None:
            ctx.kernels.gate_up_swiglu(x, self.w_gate_up, self.layout, z)
        else:
            ctx.kernels.gate_up_swiglu(x, self.w_gate_up, self.layout, z, act=self.act, row_scale=row_scale)
        ctx.kernels.linear(z, self.w_down, residual, accumulate=True)


@register_feed_forward("dense")
class DenseFeedForward:
    """params: ``hidden_size``, ``intermediate_size``, ``activation`` (``relu_squared``: relu(u)^2; ``gelu_tanh``;
    ``silu``), ``out_scale`` (1.0: what the sublayer's output is multiplied by before it joins the stream; applied
    to the activation's float32 result, before its one rounding); weights: ``up``, ``down``."""

    takes_lazy_input = True

    def __init__(self, params, weights, build: BuildContext):
        self.hidden, self.inter = int(params["hidden_size"]), int(params["intermediate_size"])
        self.activation = str(params.get("activation", "relu_squared"))
        from ..csrc.ops import ACTIVATIONS
        if self.activation not in ACTIVATIONS:
            raise ValueError(f"dense feed-forward: activation {self.activation!r} is not known (known: {sorted(ACTIVATIONS)})")
        self.out_scale = float(params.get("out_scale", 1.0))
        w = build.weights
        self.w_up = w.as_dtype(weights["up"], build.dtype)
        self.w_down = w.as_dtype(weights["down"], build.dtype)
        for name, t, want in ((weights["up"], self.w_up, (self.inter, self.hidden)),
                              (weights["down"], self.w_down, (self.hidden, self.inter))):
            if tuple(t.shape) != want:
                raise ValueError(f"{name} has shape {tuple(t.shape)}, expected {want}")
        self.dtype = build.dtype

    @staticmethod
    def activation_elements(params) -> int:
        return 2 * int(params["intermediate_size"])

    def forward(self, ctx, x, residual):
        z = torch.empty((residual.shape[0], self.inter), dtype=self.dtype, device=residual.device)
        ctx.kernels.linear_activation(x, self.w_up, z, self.activation, self.out_scale)
        ctx.kernels.linear(z, self.w_down, residual, accumulate=True)
