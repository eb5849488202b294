"""Norms.  ``rmsnorm``: y = x * rsqrt(mean(x^2) + eps) * w, statistics in float32,
one rounding at the end (kernels/full_attention_cuda.cuh:2826-2873; the weight is
used as ``w``, not ``1 + w``: crates/runner/src/llama31_engine.rs:89).  ``dynamic_tanh``:
y = tanh(alpha * x) * w + b, which takes no statistics of x at all."""
from __future__ import annotations

import torch

from .registry import BuildContext, register_norm


@register_norm("rmsnorm")
class RMSNorm:
    """params: ``size``, ``eps``, ``unit_offset`` (False; True: the weight is stored around zero and the norm
    multiplies by 1 + w, the sum taken in float32 and kept so); weights: ``weight`` [size].

    Interface of a norm: ``__call__(ctx, x, rows=None) -> tensor`` where ``x`` is the
    float32 residual stream ``[T, size]`` and the result has the activation dtype;
    ``rows`` (int32) picks rows of ``x`` instead of taking all.
    """

    fusable_rms = True     # kernels may apply this norm (weight, eps) inside a matrix product

    def __init__(self, params, weights, build: BuildContext):
        self.size, self.eps = int(params["size"]), float(params["eps"])
        w = build.weights.stored(weights["weight"])
        # 32-bit weights stay 32-bit; in the float32 path everything is 32-bit
        self.weight = w.float() if build.dtype == torch.float32 else w
        if params.get("unit_offset"):
            self.weight = (w.float() + 1.0).contiguous()
        if tuple(self.weight.shape) != (self.size,):
            raise ValueError(f"rmsnorm weight has shape {tuple(self.weight.shape)}, expected ({self.size},)")
        self.dtype = build.dtype

    @property
    def weight_f32(self):
        """The multiplier in float32, for kernels that take this norm inside another operation."""
        if getattr(self, "_weight_f32", None) is None:
            self._weight_f32 = self.weight if self.weight.dtype == torch.float32 else self.weight.float()
        return self._weight_f32

    def __call__(self, ctx, x, rows=None):
        n = x.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, self.size), dtype=self.dtype, device=x.device)
        ctx.kernels.rmsnorm(x, self.weight, self.eps, out, rows)
        return out


@register_norm("rmsnorm_scalar")
class ScalarRMSNorm(RMSNorm):
    """y = x * rsqrt(mean(x^2) + eps) * g with one gain g for all coordinates.

    params: ``size``, ``eps``; weights: ``weight``, a tensor of a single number.  The gain is spread
    over a vector when the part is built, so every kernel that takes ``rmsnorm`` (also those that
    fold the norm into a matrix product) takes this norm unchanged.
    """

    def __init__(self, params, weights, build: BuildContext):
        self.size, self.eps = int(params["size"]), float(params["eps"])
        g = build.weights.stored(weights["weight"])
        if g.numel() != 1:
            raise ValueError(f"{weights['weight']} has shape {tuple(g.shape)}, expected a single number")
        g = g.reshape(1).expand(self.size).contiguous()
        self.weight = g.float() if build.dtype == torch.float32 else g
        self.dtype = build.dtype


@register_norm("dynamic_tanh")
class DynamicTanh:
    """y = tanh(alpha * x) * w + b, element by element: no mean, no variance, no eps.

    params: ``size``; weights: ``weight`` [size], ``bias`` [size], ``alpha`` (a single number).  The three are
    kept in float32 (they are read once per element); the result has the activation type.
    """

    fusable_rms = False    # not a root-mean-square norm: kernels that fold one into a product must not take it

    def __init__(self, params, weights, build: BuildContext):
        self.size = int(params["size"])
        w = build.weights
        self.weight = w.stored(weights["weight"]).float().contiguous()
        self.bias = w.stored(weights["bias"]).float().contiguous()
        self.alpha = w.stored(weights["alpha"]).float().reshape(-1).contiguous()
        if tuple(self.weight.shape) != (self.size,) or tuple(self.bias.shape) != (self.size,) or self.alpha.numel() != 1:
            raise ValueError(f"{weights['weight']}: weight and bias of ({self.size},) and a single alpha expected, got "
                             f"{tuple(self.weight.shape)}, {tuple(self.bias.shape)}, {tuple(self.alpha.shape)}")
        self.dtype = build.dtype

    def __call__(self, ctx, x, rows=None):
        n = x.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, self.size), dtype=self.dtype, device=x.device)
        ctx.kernels.dynamic_tanh(x, self.alpha, self.weight, self.bias, out, rows)
        return out

    def with_shift(self, ctx, x, mu, last, second=None):
        """This norm of ``x`` with a token shift behind it (``mu`` [1, size], ``last``: the per-slot row that carries a
        sequence's last normed row), and the norm ``second`` (another of this kind, or None) of the same ``x``, in
        one pass: returns (shifted, second's output or None)."""
        mixed = torch.empty((x.shape[0], self.size), dtype=self.dtype, device=x.device)
        other = torch.empty_like(mixed) if second is not None else None
        ctx.kernels.tanh_norm_shift(x, (self.alpha, self.weight, self.bias),
                                    None if second is None else (second.alpha, second.weight, second.bias), mu, last,
                                    ctx.batch, mixed, other)
        return mixed, other
