"""Recurrent mixers whose memory is a fixed-size float32 state per sequence.

``real_gated_recurrence`` (a vector state per channel).  With the normed input h of a token:

    y = gelu_tanh(Wy h + by),    x = Wx h + bx
    u = conv(x)                               a causal convolution per channel over a few taps (no activation)
    r = sigmoid(Ra_b u_b + ra_b),  i = sigmoid(Ri_b u_b + ri_b)      per block b of the channels, square matrices
    a = exp(-8 * r * softplus(lambda))
    S_t = a S_(t-1) + sqrt(1 - a^2) * i * u                          S_(-1) = 0
    result = Wo (S_t * y)

``delta_rule`` (a matrix state [dim, dim] per head), with r, k, v = Wr h, Wk h, Wv h per head:

    w = exp(-c * sigmoid(Ww2 tanh(Ww1 h) + w0))        decay per key channel, c = ``decay_scale``
    a = sigmoid(Wa h + ab)                             removal rate per key channel
    u = k / sqrt(sum(k^2) + unit_eps)                  the head's unit key
    S_t = diag(w) S_(t-1) - (a * u)(u^T S_(t-1)) + k v^T,      o = S_t^T r
    result = Wo [rms(o_head) * norm * sigmoid(Wg h)]

``time_mixing`` (a matrix state per head), where each of r, k, v, g, w reads its own mix of the token's and the
previous token's input, m_s = h_t + (h_(t-1) - h_t) * mu_s:

    r, k, v = Wr m_r, Wk m_k, Wv m_v;   gate = silu(Wg m_g);   w = exp(-exp(Ww2 tanh(Ww1 m_w) + w0))
    o = (S_(t-1) + diag(bonus) k v^T)^T r,      S_t = diag(w) S_(t-1) + k v^T
    result = Wo [rms(o_head) * norm * gate]

``min_gru`` (a vector state per channel whose gates read the current token alone):

    z = sigmoid(Wz h + bz),    u = Wx h + bx,    cand = u + 1/2 where u >= 0, sigmoid(u) where u < 0
    S_t = (1 - z) S_(t-1) + z cand                                   S_(-1) = 0
    result = out_scale * Wo (S_t * silu(Wg h))

Decays, gates of the recurrences, unit keys, the states and o are float32 whatever the activation type; the
matrix products and the convolution run in the activation type.
"""
from __future__ import annotations

import math

import torch

from ..cache import StateNeed
from .registry import BuildContext, register_mixer


def _shapes(got, want, names):
    for role, shape in want.items():
        if tuple(got[role].shape) != tuple(shape):
            raise ValueError(f"{names[role]} has shape {tuple(got[role].shape)}, expected {tuple(shape)}")


@register_mixer("real_gated_recurrence")
class RealGatedRecurrence:
    """params: ``hidden_size``, ``width`` (channels), ``taps``, ``blocks``; weights: ``y``, ``y_bias``, ``x``,
    ``x_bias``, ``conv`` [channels, taps], ``conv_bias``, ``ra`` / ``ri`` [blocks, b, b], ``ra_bias`` / ``ri_bias``
    [blocks, b], ``lam`` [channels], ``o``."""

    def __init__(self, params, weights, build: BuildContext):
        self.hidden, self.C = int(params["hidden_size"]), int(params["width"])
        self.taps, self.nb = int(params["taps"]), int(params["blocks"])
        from ..csrc.ops import CONV_MAX_TAPS
        if self.C % self.nb or self.taps < 1 or self.taps > CONV_MAX_TAPS:
            raise ValueError(f"real_gated_recurrence: {self.C} channels in {self.nb} blocks, {self.taps} taps "
                             f"(up to {CONV_MAX_TAPS})")
        self.bs = self.C // self.nb
        w, dt = build.weights, build.dtype
        C, nb, bs = self.C, self.nb, self.bs
        got = {r: w.as_dtype(weights[r], dt) for r in ("y", "x", "ra", "ri", "o")}
        got.update({r: w.stored(weights[r]).float().contiguous()
                    for r in ("y_bias", "x_bias", "conv", "conv_bias", "ra_bias", "ri_bias", "lam")})
        _shapes(got, {"y": (C, self.hidden), "x": (C, self.hidden), "o": (self.hidden, C), "ra": (nb, bs, bs),
                      "ri": (nb, bs, bs), "y_bias": (C,), "x_bias": (C,), "conv": (C, self.taps), "conv_bias": (C,),
                      "ra_bias": (nb, bs), "ri_bias": (nb, bs), "lam": (C,)}, weights)
        self.w_in = torch.cat([got["y"], got["x"]], dim=0).contiguous()            # one product: [y | x]
        self.w_gates = torch.cat([got["ra"], got["ri"]], dim=1).contiguous()       # per block: [r rows | i rows]
        self.w_o = got["o"]
        self.y_bias, self.x_bias = got["y_bias"], got["x_bias"]
        self.conv, self.conv_bias = got["conv"], got["conv_bias"]
        self.bias_r, self.bias_i = got["ra_bias"].reshape(C).contiguous(), got["ri_bias"].reshape(C).contiguous()
        self.rate = (-8.0 * torch.nn.functional.softplus(got["lam"])).contiguous()  # log a = rate * r
        self.dtype = dt

    def cache_need(self):
        return self.cache_need_from({"width": self.C, "taps": self.taps})

    @staticmethod
    def cache_need_from(params):
        C, taps = int(params["width"]), int(params["taps"])
        return {"state": StateNeed(C), "tail": StateNeed((taps - 1) * C)}

    @staticmethod
    def activation_elements(params) -> int:
        return 8 * int(params["width"])

    def forward(self, ctx, x, residual, cache_id, writes_cache, position):
        if not writes_cache:
            raise ValueError("a recurrent mixer cannot read another layer's state without advancing it")
        C, T, dev = self.C, ctx.batch.n_tokens, residual.device
        proj = torch.empty((T, 2 * C), dtype=self.dtype, device=dev)
        ctx.kernels.linear(x, self.w_in, proj)
        u = torch.empty((T, C), dtype=self.dtype, device=dev)
        ctx.kernels.causal_conv(proj[:, C:], self.x_bias, self.conv, self.conv_bias,
                                ctx.cache.state((cache_id, "tail")), ctx.batch, u)
        gates = torch.empty((T, 2 * C), dtype=torch.float32, device=dev)
        ctx.kernels.head_linear(u.view(T, self.nb, self.bs), self.w_gates, gates.view(T, self.nb, 2 * self.bs))
        y = torch.empty((T, C), dtype=self.dtype, device=dev)
        ctx.kernels.gated_unit_scan(gates, self.bias_r, self.bias_i, self.rate, u, proj[:, :C], self.y_bias,
                                    ctx.cache.state((cache_id, "state")), ctx.batch, y, self.bs)
        ctx.kernels.linear(y, self.w_o, residual, accumulate=True)


@register_mixer("delta_rule")
class DeltaRule:
    """params: ``hidden_size``, ``num_heads``, ``dim``, ``decay_rank``, ``norm_eps``, ``decay_scale`` (default
    exp(-1/2)), ``unit_eps`` (default 1e-6); weights: ``r``, ``k``, ``v``, ``g``, ``a``, ``a_bias``, ``w1``, ``w2``,
    ``w0``, ``norm`` [heads x dim], ``o``."""

    def __init__(self, params, weights, build: BuildContext):
        self.hidden, self.H, self.dim = int(params["hidden_size"]), int(params["num_heads"]), int(params["dim"])
        self.rank, self.eps = int(params["decay_rank"]), float(params["norm_eps"])
        self.decay_scale = float(params.get("decay_scale", math.exp(-0.5)))
        self.unit_eps = float(params.get("unit_eps", 1e-6))
        from ..csrc.ops import SCAN_MAX_DIM
        if self.dim > SCAN_MAX_DIM:
            raise ValueError(f"delta_rule: {self.dim} key channels a head; the recurrence kernel holds up to {SCAN_MAX_DIM}")
        w, dt = build.weights, build.dtype
        HD, W, r = self.H * self.dim, self.hidden, self.rank
        got = {role: w.as_dtype(weights[role], dt) for role in ("r", "k", "v", "g", "a", "w1", "w2", "o")}
        got.update({role: w.stored(weights[role]).float().contiguous() for role in ("a_bias", "w0")})
        norm = w.stored(weights["norm"])
        got["norm"] = norm.float() if dt == torch.float32 else norm
        _shapes(got, {"r": (HD, W), "k": (HD, W), "v": (HD, W), "g": (HD, W), "a": (HD, W), "w1": (r, W), "w2": (HD, r),
                      "o": (W, HD), "a_bias": (HD,), "w0": (HD,), "norm": (HD,)}, weights)
        self.w_in = torch.cat([got[x] for x in ("r", "k", "v", "g", "a", "w1")], dim=0).contiguous()
        self.r_off, self.k_off, self.v_off, self.g_off, self.a_off, self.z_off = (i * HD for i in range(6))
        self.w2, self.w_o, self.a_bias, self.w0, self.norm_w = got["w2"], got["o"], got["a_bias"], got["w0"], got["norm"].contiguous()
        self.dtype = dt

    def cache_need(self):
        return StateNeed(self.H * self.dim * self.dim)

    @staticmethod
    def cache_need_from(params):
        return StateNeed(int(params["num_heads"]) * int(params["dim"]) ** 2)

    @staticmethod
    def activation_elements(params) -> int:
        return 14 * int(params["num_heads"]) * int(params["dim"]) + int(params["decay_rank"])

    def forward(self, ctx, x, residual, cache_id, writes_cache, position):
        if not writes_cache:
            raise ValueError("a recurrent mixer cannot read another layer's state without advancing it")
        H, d, HD = self.H, self.dim, self.H * self.dim
        T, dev, k = ctx.batch.n_tokens, residual.device, ctx.kernels
        proj = torch.empty((T, self.w_in.shape[0]), dtype=self.dtype, device=dev)
        k.linear(x, self.w_in, proj)
        k.tanh_(proj[:, self.z_off:])
        z = torch.empty((T, HD), dtype=torch.float32, device=dev)
        k.linear(proj[:, self.z_off:], self.w2, z)
        y = torch.empty((T, HD), dtype=self.dtype, device=dev)
        if k.matrix_state_step(proj, self.r_off, self.k_off, self.v_off, self.g_off, self.a_off, z, self.w0, "exp_sigmoid",
                               self.decay_scale, self.a_bias, self.unit_eps, "delta", None, ctx.cache.state(cache_id),
                               ctx.batch, self.norm_w, self.eps, "sigmoid", y, H, d, d):
            k.linear(y, self.w_o, residual, accumulate=True)       # a decode step: decays, walk, norm and gate in one launch
            return
        unit = torch.empty((T, 2 * HD), dtype=torch.float32, device=dev)
        k.state_scan_prepare(z, self.w0, "exp_sigmoid", self.decay_scale, H, d, proj, self.k_off, self.a_off,
                             self.a_bias, self.unit_eps, unit, log_decay=self.dtype == torch.float32)
        o = torch.empty((T, HD), dtype=torch.float32, device=dev)
        k.matrix_state_scan(proj, self.r_off, self.k_off, self.v_off, z, "delta", ctx.cache.state(cache_id), ctx.batch,
                            o, H, d, d, unit=unit)
        k.head_norm_gate(o, self.norm_w, self.eps, proj[:, self.g_off:], y, H, d, gate_kind="sigmoid")
        k.linear(y, self.w_o, residual, accumulate=True)


@register_mixer("time_mixing")
class TimeMixing:
    """params: ``hidden_size``, ``num_heads``, ``dim``, ``decay_rank``, ``norm_eps``; weights: ``mu_r``, ``mu_k``,
    ``mu_v``, ``mu_g``, ``mu_w`` [hidden], ``r``, ``k``, ``v``, ``g``, ``w1``, ``w2``, ``w0``, ``bonus`` [heads, dim],
    ``norm`` [heads x dim], ``o``.  Keeps the state matrices and the last token's input per sequence."""

    MIXES = ("r", "k", "v", "g", "w")

    def __init__(self, params, weights, build: BuildContext):
        self.hidden, self.H, self.dim = int(params["hidden_size"]), int(params["num_heads"]), int(params["dim"])
        self.rank, self.eps = int(params["decay_rank"]), float(params["norm_eps"])
        from ..csrc.ops import SCAN_MAX_DIM
        if self.dim > SCAN_MAX_DIM:
            raise ValueError(f"time_mixing: {self.dim} key channels a head; the recurrence kernel holds up to {SCAN_MAX_DIM}")
        w, dt = build.weights, build.dtype
        HD, W, r = self.H * self.dim, self.hidden, self.rank
        got = {role: w.as_dtype(weights[role], dt) for role in ("r", "k", "v", "g", "w1", "w2", "o")}
        got.update({role: w.stored(weights[role]).float().contiguous()
                    for role in ("w0", "bonus") + tuple("mu_" + s for s in self.MIXES)})
        norm = w.stored(weights["norm"])
        got["norm"] = norm.float() if dt == torch.float32 else norm
        want = {"r": (HD, W), "k": (HD, W), "v": (HD, W), "g": (HD, W), "w1": (r, W), "w2": (HD, r), "o": (W, HD),
                "w0": (HD,), "bonus": (self.H, self.dim), "norm": (HD,)}
        want.update({"mu_" + s: (W,) for s in self.MIXES})
        _shapes(got, want, weights)
        self.mu = torch.stack([got["mu_" + s] for s in self.MIXES]).contiguous()
        self.w = [got[s] for s in ("r", "k", "v", "g", "w1")]
        self.r_off, self.k_off, self.v_off, self.g_off, self.z_off = (i * HD for i in range(5))
        self.w2, self.w_o, self.w0, self.bonus, self.norm_w = got["w2"], got["o"], got["w0"], got["bonus"], got["norm"].contiguous()
        self.dtype = dt

    def cache_need(self):
        return {"state": StateNeed(self.H * self.dim * self.dim), "last": StateNeed(self.hidden)}

    @staticmethod
    def cache_need_from(params):
        return {"state": StateNeed(int(params["num_heads"]) * int(params["dim"]) ** 2),
                "last": StateNeed(int(params["hidden_size"]))}

    @staticmethod
    def activation_elements(params) -> int:
        return 5 * int(params["hidden_size"]) + 10 * int(params["num_heads"]) * int(params["dim"]) + int(params["decay_rank"])

    def forward(self, ctx, x, residual, cache_id, writes_cache, position):
        if not writes_cache:
            raise ValueError("a recurrent mixer cannot read another layer's state without advancing it")
        H, d, HD = self.H, self.dim, self.H * self.dim
        T, dev, k = ctx.batch.n_tokens, residual.device, ctx.kernels
        mixes = torch.empty((len(self.MIXES), T, self.hidden), dtype=self.dtype, device=dev)
        k.shift_mix(x, self.mu, ctx.cache.state((cache_id, "last")), ctx.batch, mixes)
        proj = torch.empty((T, 4 * HD + self.rank), dtype=self.dtype, device=dev)
        for i, wm in enumerate(self.w):                      # every product reads a mix of its own
            k.linear(mixes[i], wm, proj[:, i * HD: i * HD + wm.shape[0]])
        k.tanh_(proj[:, self.z_off:])
        z = torch.empty((T, HD), dtype=torch.float32, device=dev)
        k.linear(proj[:, self.z_off:], self.w2, z)
        y = torch.empty((T, HD), dtype=self.dtype, device=dev)
        if k.matrix_state_step(proj, self.r_off, self.k_off, self.v_off, self.g_off, 0, z, self.w0, "double_exp", 1.0, None,
                               0.0, "bonus", self.bonus, ctx.cache.state((cache_id, "state")), ctx.batch, self.norm_w,
                               self.eps, "silu", y, H, d, d):
            k.linear(y, self.w_o, residual, accumulate=True)
            return
        k.state_scan_prepare(z, self.w0, "double_exp", 1.0, H, d, log_decay=self.dtype == torch.float32)
        o = torch.empty((T, HD), dtype=torch.float32, device=dev)
        k.matrix_state_scan(proj, self.r_off, self.k_off, self.v_off, z, "bonus", ctx.cache.state((cache_id, "state")),
                            ctx.batch, o, H, d, d, bonus=self.bonus)
        k.head_norm_gate(o, self.norm_w, self.eps, proj[:, self.g_off:], y, H, d, gate_kind="silu")
        k.linear(y, self.w_o, residual, accumulate=True)


@register_mixer("min_gru")
class MinGRU:
    """params: ``hidden_size``, ``width`` (channels), ``out_scale`` (1.0); weights: ``z``, ``z_bias``, ``x``, ``x_bias``,
    ``g``, ``o``.  The three input products run as one over [z | x | g]."""

    def __init__(self, params, weights, build: BuildContext):
        self.hidden, self.C = int(params["hidden_size"]), int(params["width"])
        self.out_scale = float(params.get("out_scale", 1.0))
        w, dt = build.weights, build.dtype
        got = {r: w.as_dtype(weights[r], dt) for r in ("z", "x", "g", "o")}
        got.update({r: w.stored(weights[r]).float().contiguous() for r in ("z_bias", "x_bias")})
        C = self.C
        _shapes(got, {"z": (C, self.hidden), "x": (C, self.hidden), "g": (C, self.hidden), "o": (self.hidden, C),
                      "z_bias": (C,), "x_bias": (C,)}, weights)
        self.w_in = torch.cat([got["z"], got["x"], got["g"]], dim=0).contiguous()
        self.w_o = got["o"]
        self.z_bias, self.x_bias = got["z_bias"], got["x_bias"]
        self.dtype = dt

    def cache_need(self):
        return StateNeed(self.C)

    @staticmethod
    def cache_need_from(params):
        return StateNeed(int(params["width"]))

    @staticmethod
    def activation_elements(params) -> int:
        return 4 * int(params["width"])

    def forward(self, ctx, x, residual, cache_id, writes_cache, position):
        if not writes_cache:
            raise ValueError("min_gru keeps state: its stop of the schedule must write its cache entry")
        T, dev, k = ctx.batch.n_tokens, residual.device, ctx.kernels
        proj = torch.empty((T, 3 * self.C), dtype=self.dtype, device=dev)
        k.linear(x, self.w_in, proj)
        y = torch.empty((T, self.C), dtype=self.dtype, device=dev)
        k.mingru_scan(proj, self.z_bias, self.x_bias, ctx.cache.state(cache_id), ctx.batch, y, self.C, self.out_scale)
        k.linear(y, self.w_o, residual, accumulate=True)
