"""Softmax attention over a sliding window, with what may stay visible beyond it.

For a token at position p with normed input h, query head g of H and its kv head g // (H / G):

    q_g = rot_p(norm(Wq h)),   k = rot_p(norm(Wk h)),   v = vrot_p(Wv h)
    s_gj = (q_g . k_j) * scale,      then, with a cap c,   s_gj <- c * tanh(s_gj / c)
    w_gj = exp(s_gj) / (sum over the visible j' of exp(s_gj') + sink),      out_g = vrot_(-p)(sum_j w_gj v_j)
    result = out_scale * Wo [out_1 ... out_H]

Visible to position p, with window W, F kept first tokens and runs of P tokens:

    the tokens j with p - W < j <= p,
    the tokens j < F that have left the window (they keep their own positions),
    one pooled row per run b = 0, 1, ... of P tokens that lies wholly before the window ((b + 1) P <= p - W + 1):
    its key is the mean of the run's P keys as the cache holds them, its value the mean of their values.

A token that has left the window while its run is not yet wholly before it is not visible.  ``norm`` is an RMS norm
of q and of k with a plain weight: per head over ``dim`` with one weight vector for all heads (``"head"``), or over
the whole projection of all heads at once with a weight of that size (``"row"``).  ``rot`` turns the first
coordinates of q and k (the position encoding of the block); ``vrot`` turns every value over its whole width by
its own position, so that a value enters a head's sum by its distance to the query.  ``sink``: a key of score 0
that has no value (exp(0) = 1 is added to the denominator).  Scores, weights, norms and rotations are float32.

Pooled rows live in a store of their own with one row per finished run (``KvNeed.tokens_per_row``): the step
that brings a run's last token writes the row, so a decode step reads W + p / P rows instead of p.
"""
from __future__ import annotations

import torch

from ..cache import PAGE_SHIFT, KvNeed
from .registry import POSITION_ENCODINGS, BuildContext, lookup, register_mixer


@register_mixer("window_attention")
class WindowAttention:
    """params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``dim``, ``value_dim``, ``scale``, ``window`` (None: all
    earlier tokens), ``keep_first`` (0), ``pool`` (0: no pooled runs), ``softcap`` (None), ``sink`` (False),
    ``qk_norm`` (``"head"``, ``"row"`` or None), ``norm_eps``, ``value_rotation`` (None, or ``{"theta", "pairing"}``),
    ``out_scale`` (1.0); weights: ``q``, ``k``, ``v``, ``o`` and with a norm ``q_norm``, ``k_norm``."""

    def __init__(self, params, weights, build: BuildContext):
        self.hidden = int(params["hidden_size"])
        self.n_q, self.n_kv = int(params["num_heads"]), int(params["num_kv_heads"])
        self.dim, self.vdim = int(params["dim"]), int(params["value_dim"])
        self.scale, self.eps = float(params["scale"]), float(params.get("norm_eps", 1e-6))
        self.window = int(params["window"]) if params.get("window") else None
        self.keep_first, self.pool = int(params.get("keep_first") or 0), int(params.get("pool") or 0)
        self.softcap = float(params["softcap"]) if params.get("softcap") else None
        self.sink = bool(params.get("sink", False))
        self.qk_norm = params.get("qk_norm")
        self.out_scale = float(params.get("out_scale", 1.0))
        if self.n_q % self.n_kv:
            raise ValueError(f"{self.n_q} query heads do not split over {self.n_kv} kv heads")
        if self.qk_norm not in (None, "head", "row"):
            raise ValueError(f"window_attention: qk_norm {self.qk_norm!r} is not known ('head', 'row' or None)")
        if self.pool and not self.window:
            raise ValueError("window_attention: pooled runs stand for what has left a window; no window is given")
        w, dt = build.weights, build.dtype
        q, k, v = (w.as_dtype(weights[r], dt) for r in ("q", "k", "v"))
        self.w_o = w.as_dtype(weights["o"], dt)
        want = {"q": (self.n_q * self.dim, self.hidden), "k": (self.n_kv * self.dim, self.hidden),
                "v": (self.n_kv * self.vdim, self.hidden), "o": (self.hidden, self.n_q * self.vdim)}
        for r, t in (("q", q), ("k", k), ("v", v), ("o", self.w_o)):
            if tuple(t.shape) != want[r]:
                raise ValueError(f"{weights[r]} has shape {tuple(t.shape)}, expected {want[r]}")
        self.w_qkv = torch.cat([q, k, v], dim=0).contiguous()
        self.w_q = self.w_qkv[: self.n_q * self.dim]
        self.q_norm = self.k_norm = None
        if self.qk_norm:
            self.q_norm = w.stored(weights["q_norm"]).float().contiguous()
            self.k_norm = w.stored(weights["k_norm"]).float().contiguous()
            sizes = (self.dim, self.dim) if self.qk_norm == "head" else (self.n_q * self.dim, self.n_kv * self.dim)
            if (self.q_norm.numel(), self.k_norm.numel()) != sizes or self.q_norm.dim() != 1 or self.k_norm.dim() != 1:
                raise ValueError(f"{weights['q_norm']} / {weights['k_norm']}: expected {sizes[0]} and {sizes[1]} weights")
        self.value_position = None
        vr = params.get("value_rotation")
        if vr:
            if self.vdim % 2:
                raise ValueError("window_attention: rotated values need an even value width")
            self.value_position = lookup(POSITION_ENCODINGS, "rotary", "position encoding")(
                {"head_dim": self.vdim, "rotary_dim": self.vdim, "theta": float(vr["theta"]),
                 "max_positions": int(vr.get("max_positions", 1 << 30)), "pairing": vr.get("pairing", "halves"),
                 "scaling": None}, {}, build)
        self.dtype = dt

    @staticmethod
    def _needs(n_kv, dim, vdim, window, keep_first, pool):
        # the step that finishes a run reads the run's tokens back from the cache: they stay for a run's length at least
        reach = None if not window else max(int(window), int(pool or 0))
        tokens = KvNeed(n_kv, dim, reach, value_dim=vdim, keep_first=int(keep_first or 0) if reach else 0)
        if not pool:
            return tokens
        return {"tokens": tokens, "pooled": KvNeed(n_kv, dim, None, value_dim=vdim, tokens_per_row=int(pool))}

    def cache_need(self):
        return self._needs(self.n_kv, self.dim, self.vdim, self.window, self.keep_first, self.pool)

    @staticmethod
    def cache_need_from(params):
        return WindowAttention._needs(int(params["num_kv_heads"]), int(params["dim"]), int(params["value_dim"]),
                                      params.get("window"), params.get("keep_first"), params.get("pool"))

    @staticmethod
    def activation_elements(params) -> int:
        H, G = int(params["num_heads"]), int(params["num_kv_heads"])
        return (H + G) * int(params["dim"]) + (H + G) * int(params["value_dim"])

    def forward(self, ctx, x, residual, cache_id, writes_cache, position):
        T, dev, k = ctx.batch.n_tokens, residual.device, ctx.kernels
        kv = ctx.cache.kv((cache_id, "tokens") if self.pool else cache_id)
        pooled = ctx.cache.kv((cache_id, "pooled")) if self.pool else None
        width = self.n_q * self.dim + (self.n_kv * (self.dim + self.vdim) if writes_cache else 0)
        qkv = torch.empty((T, width), dtype=self.dtype, device=dev)
        k.linear(x, self.w_qkv if writes_cache else self.w_q, qkv)
        pooled_there = k.qkv_prepare(qkv, self.q_norm, self.k_norm, self.qk_norm, self.eps, position, self.value_position, kv,
                                     ctx.batch, self.n_q, self.n_kv, self.dim, self.vdim, PAGE_SHIFT, writes_cache,
                                     pooled_kv=pooled if writes_cache else None, pool=self.pool)
        if self.pool and writes_cache and not pooled_there:
            k.pool_rows(kv, pooled, ctx.batch, self.n_kv, self.dim, self.vdim, PAGE_SHIFT, self.pool)
        heads = torch.empty((T, self.n_q * self.vdim), dtype=self.dtype, device=dev)
        k.window_attention(qkv, kv, pooled, ctx.batch, heads, self.n_q, self.n_kv, self.dim, self.vdim, PAGE_SHIFT,
                           self.window, self.keep_first, self.pool, self.scale, self.softcap,
                           True if self.sink else None, self.value_position, self.out_scale)
        k.linear(heads, self.w_o, residual, accumulate=True)
