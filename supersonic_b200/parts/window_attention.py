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

Further options, each usable without the others:

* ``conv`` = taps: a short causal convolution over time on every channel of the projected q and k, straight behind
  the projection and before the norm, y_t = sum_j w[:, j] u_(t - taps + 1 + j) with zeros before the sequence's
  start; the last taps - 1 projected rows are per-sequence state beside the keys.
* ``values`` = ``"keys"``: there is no value projection; a token's value is its key as it leaves the projection (and
  the convolution), before the norm.
* ``query_temperature`` = {coef, every}: the queries at position p are multiplied by
  1 + coef ln(floor((p + 1) / every) + 1).
* ``head_gate``: head g's result is multiplied by sigmoid(Wg h)_g, one number per head and token, read from the same
  input as the projections.
* ``score_maps`` = 2 with ``map_offset`` = d (differential attention): q and k hold two maps per head, laid out head
  by head as [map 1 | map 2], each normed and rotated like a head; both maps weigh the same values, and with
  lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + d (one number for the layer) the head's result is
  o = a1 - lambda a2, then o / sqrt(mean(o^2) + eps) * (1 - d).
* ``own_kv`` = False: the mixer has no key and value tensors; its stop of the schedule reads the cache entry another
  layer wrote (keys as cached: normed and rotated), with its own queries, window and everything else.
* ``cache_window``: how far back the cache entry keeps tokens, where a reader of the entry has a longer window.

Pooled rows live in a store of their own with one row per finished run (``KvNeed.tokens_per_row``): the step
that brings a run's last token writes the row, so a decode step reads W + p / P rows instead of p.
"""
from __future__ import annotations

import math

import torch

from ..cache import PAGE_SHIFT, KvNeed, StateNeed
from .registry import POSITION_ENCODINGS, BuildContext, lookup, register_mixer


@register_mixer("window_attention")
class WindowAttention:
    """params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``dim``, ``value_dim``, ``scale``, ``window`` (None: all
    earlier tokens), ``keep_first`` (0), ``pool`` (0: no pooled runs), ``softcap`` (None), ``sink`` (False),
    ``qk_norm`` (``"head"``, ``"row"`` or None), ``norm_eps``, ``value_rotation`` (None, or ``{"theta", "pairing"}``),
    ``out_scale`` (1.0), ``conv`` (0), ``values`` (``"projection"`` or ``"keys"``), ``query_temperature`` (None),
    ``head_gate`` (False), ``score_maps`` (1 or 2), ``map_offset``, ``own_kv`` (True), ``cache_window``; weights: ``q``,
    ``k``, ``v``, ``o``, with a norm ``q_norm``, ``k_norm``, with a convolution ``q_conv``, ``k_conv`` [channels, taps],
    with a gate ``g`` [heads, hidden], with two maps ``lq1``, ``lk1``, ``lq2``, ``lk2`` [dim]."""

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
        self.taps = int(params.get("conv") or 0)
        self.values = params.get("values") or "projection"
        self.maps = int(params.get("score_maps") or 1)
        self.own_kv = bool(params.get("own_kv", True))
        self.head_gate = bool(params.get("head_gate", False))
        qt = params.get("query_temperature")
        self.q_temp = (float(qt["coef"]), int(qt["every"])) if qt else None
        self.cache_window = self._reach(self.window, params.get("cache_window"))
        if self.n_q % self.n_kv:
            raise ValueError(f"{self.n_q} query heads do not split over {self.n_kv} kv heads")
        if self.qk_norm not in (None, "head", "row"):
            raise ValueError(f"window_attention: qk_norm {self.qk_norm!r} is not known ('head', 'row' or None)")
        if self.pool and not self.window:
            raise ValueError("window_attention: pooled runs stand for what has left a window; no window is given")
        if self.values not in ("projection", "keys"):
            raise ValueError(f"window_attention: values {self.values!r} is not known ('projection' or 'keys')")
        if self.values == "keys" and (self.vdim != self.dim or self.maps != 1):
            raise ValueError("window_attention: values that are the keys have the keys' width, and one score map")
        if self.maps not in (1, 2) or (self.maps == 2 and (self.pool or self.qk_norm == "row" or self.sink or self.head_gate)):
            raise ValueError("window_attention: one score map, or two without pooled runs, row norms, a sink or a head gate")
        if self.taps < 0 or (self.taps and not self.own_kv):
            raise ValueError("window_attention: a convolution needs keys of its own behind it")
        if self.q_temp and self.q_temp[1] < 1:
            raise ValueError("window_attention: the query temperature's period must be at least one token")
        w, dt = build.weights, build.dtype
        H, G, M, D, V = self.n_q, self.n_kv, self.maps, self.dim, self.vdim
        q = w.as_dtype(weights["q"], dt)
        self.w_o = w.as_dtype(weights["o"], dt)
        want = {"q": (H * M * D, self.hidden), "k": (G * M * D, self.hidden), "v": (G * V, self.hidden),
                "o": (self.hidden, H * V), "g": (H, self.hidden)}

        def checked(role, t):
            if tuple(t.shape) != want[role]:
                raise ValueError(f"{weights[role]} has shape {tuple(t.shape)}, expected {want[role]}")
            return t
        checked("q", q); checked("o", self.w_o)
        if M == 2:
            # a map's heads side by side: rows [kv head][map][head of the group], so that the heads which share a
            # map's keys form one group of query heads over one key head, as in grouped-query attention
            R = H // G
            q = q.view(G, R, M, D, self.hidden).permute(0, 2, 1, 3, 4).reshape(H * M * D, self.hidden)
        rows = [q]
        if self.own_kv:
            rows.append(checked("k", w.as_dtype(weights["k"], dt)))
            if self.values == "projection":
                rows.append(checked("v", w.as_dtype(weights["v"], dt)))
        self.kv_cols = sum(r.shape[0] for r in rows[1:])
        gate_rows = []
        if self.head_gate:
            g = checked("g", w.as_dtype(weights["g"], dt))
            pad = (-H) % 8                   # rows of the projection's result stay a multiple of 8 wide
            gate_rows = [g] + ([torch.zeros((pad, self.hidden), dtype=dt, device=g.device)] if pad else [])
        self.gate_cols = sum(r.shape[0] for r in gate_rows)
        # [q | k | v | gate]; a stop that does not write the cache projects [q | gate] only
        self.w_qkv = torch.cat(rows + gate_rows, dim=0).contiguous()
        if not self.kv_cols or not self.gate_cols:
            self.w_q = self.w_qkv[: H * M * D + (0 if self.kv_cols else self.gate_cols)]
        else:
            self.w_q = None                  # built if such a stop ever runs
        self._q_rows, self._gate_rows = q, gate_rows
        self.q_norm = self.k_norm = None
        if self.qk_norm:
            self.q_norm = w.stored(weights["q_norm"]).float().contiguous()
            sizes = [D if self.qk_norm == "head" else H * D]
            norms = [self.q_norm]
            if self.own_kv:
                self.k_norm = w.stored(weights["k_norm"]).float().contiguous()
                sizes.append(D if self.qk_norm == "head" else G * D)
                norms.append(self.k_norm)
            else:
                self.k_norm = self.q_norm    # never applied: the stop does not write keys
            if [n.numel() for n in norms] != sizes or any(n.dim() != 1 for n in norms):
                raise ValueError(f"{weights['q_norm']} / {weights.get('k_norm')}: expected {sizes} weights")
        self.conv_w = None
        if self.taps:
            cq, ck = (w.stored(weights[r]).float() for r in ("q_conv", "k_conv"))
            if tuple(cq.shape) != (H * M * D, self.taps) or tuple(ck.shape) != (G * M * D, self.taps):
                raise ValueError(f"{weights['q_conv']} / {weights['k_conv']}: expected [{H * M * D}, {self.taps}] and "
                                 f"[{G * M * D}, {self.taps}]")
            self.conv_w = torch.cat([cq, ck], dim=0).contiguous()
        self.lam = None
        if M == 2:
            lq1, lk1, lq2, lk2 = (w.stored(weights[r]).double().cpu() for r in ("lq1", "lk1", "lq2", "lk2"))
            if any(tuple(t.shape) != (D,) for t in (lq1, lk1, lq2, lk2)):
                raise ValueError(f"{weights['lq1']} and its like: expected ({D},) each")
            self.map_offset = float(params["map_offset"])
            self.lam = math.exp(float((lq1 * lk1).sum())) - math.exp(float((lq2 * lk2).sum())) + self.map_offset
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
    def _reach(window, cache_window):
        if not window:
            return None
        return max(int(window), int(cache_window or 0))

    @staticmethod
    def _needs(n_kv, dim, vdim, window, keep_first, pool, maps=1, taps=0, conv_channels=0):
        # the step that finishes a run reads the run's tokens back from the cache: they stay for a run's length at least
        reach = None if not window else max(int(window), int(pool or 0))
        tokens = KvNeed(n_kv, dim * maps, reach, value_dim=vdim, keep_first=int(keep_first or 0) if reach else 0)
        if not pool and taps < 2:
            return tokens
        needs = {"tokens": tokens}
        if pool:
            needs["pooled"] = KvNeed(n_kv, dim, None, value_dim=vdim, tokens_per_row=int(pool))
        if taps > 1:
            needs["conv"] = StateNeed((taps - 1) * conv_channels)
        return needs

    def cache_need(self):
        return self._needs(self.n_kv, self.dim, self.vdim, self.cache_window, self.keep_first, self.pool, self.maps,
                           self.taps, (self.n_q + self.n_kv) * self.maps * self.dim)

    @staticmethod
    def cache_need_from(params):
        maps, taps = int(params.get("score_maps") or 1), int(params.get("conv") or 0)
        H, G, D = int(params["num_heads"]), int(params["num_kv_heads"]), int(params["dim"])
        return WindowAttention._needs(G, D, int(params["value_dim"]),
                                      WindowAttention._reach(params.get("window"), params.get("cache_window")),
                                      params.get("keep_first"), params.get("pool"), maps, taps, (H + G) * maps * D)

    @staticmethod
    def activation_elements(params) -> int:
        H, G = int(params["num_heads"]), int(params["num_kv_heads"])
        maps = int(params.get("score_maps") or 1)
        conv = 2 if params.get("conv") else 1
        return conv * (H + G) * maps * int(params["dim"]) + (H * maps + G) * int(params["value_dim"]) + 2 * H

    def _read_weight(self):
        """[q | gate] for a stop that reads another stop's keys."""
        if self.w_q is None:
            self.w_q = torch.cat([self._q_rows] + self._gate_rows, dim=0).contiguous()
        return self.w_q

    def forward(self, ctx, x, residual, cache_id, writes_cache, position):
        T, dev, k = ctx.batch.n_tokens, residual.device, ctx.kernels
        if writes_cache and not self.own_kv:
            raise ValueError("window_attention: a mixer without keys of its own cannot write a cache entry")
        named = bool(self.pool or self.taps > 1)
        kv = ctx.cache.kv((cache_id, "tokens") if named else cache_id)
        pooled = ctx.cache.kv((cache_id, "pooled")) if self.pool else None
        H, G, M, D, V = self.n_q, self.n_kv, self.maps, self.dim, self.vdim
        if M > 1:
            # the entry's key rows [kv head][64][maps x dim] are used as [kv head x map][64][dim]: a map is a key head
            kc = kv[0]
            kv = (kc.view(kc.shape[0], G * M, kc.shape[2], D),) + tuple(kv[1:])
        q_cols = H * M * D
        weight = self.w_qkv if writes_cache else self._read_weight()
        kv_cols = self.kv_cols if writes_cache else 0
        qkv = torch.empty((T, weight.shape[0]), dtype=self.dtype, device=dev)
        k.linear(x, weight, qkv)
        if self.taps:
            if not writes_cache:
                raise ValueError("window_attention: a convolution keeps state: its stop must write its cache entry")
            conv = torch.empty_like(qkv)
            # a single tap keeps nothing from earlier tokens: it scales every channel
            tail = ctx.cache.state((cache_id, "conv")) if self.taps > 1 else self.conv_w[:1, :0]
            k.causal_conv(qkv, None, self.conv_w, None, tail, ctx.batch, conv,
                          pass_cols=qkv.shape[1] - self.conv_w.shape[0])
            qkv = conv
        v_off = q_cols if self.values == "keys" else None
        pooled_there = k.qkv_prepare(qkv, self.q_norm, self.k_norm, self.qk_norm, self.eps, position, self.value_position, kv,
                                     ctx.batch, H * M, G * M, D, V, PAGE_SHIFT, writes_cache,
                                     pooled_kv=pooled if writes_cache else None, pool=self.pool, v_off=v_off,
                                     q_temp=self.q_temp, n_v=G)
        if self.pool and writes_cache and not pooled_there:
            k.pool_rows(kv, pooled, ctx.batch, G, D, V, PAGE_SHIFT, self.pool)
        gate = qkv[:, q_cols + kv_cols: q_cols + kv_cols + H] if self.head_gate else None
        heads = torch.empty((T, H * M * V), dtype=self.dtype, device=dev)
        k.window_attention(qkv, kv, pooled, ctx.batch, heads, H * M, G * M, D, V, PAGE_SHIFT,
                           self.window, self.keep_first, self.pool, self.scale, self.softcap,
                           True if self.sink else None, self.value_position, self.out_scale if M == 1 else 1.0,
                           v_share=M, gate=gate)
        if M > 1:
            merged = torch.empty((T, H * V), dtype=self.dtype, device=dev)
            k.map_difference(heads, merged, H, G, V, self.lam, self.eps, (1.0 - self.map_offset) * self.out_scale)
            heads = merged
        k.linear(heads, self.w_o, residual, accumulate=True)
