"""Block arrangements.  ``pre_norm``: h += mixer(norm(h)); h += feed_forward(norm(h)),
the residual stream kept and summed in float32 (crates/runner/src/prefill_engine.rs:1116-1222).
``sandwich``: h += norm_b(mixer(norm_a(h))); h += norm_d(feed_forward(norm_c(h))): a sublayer's result passes a
norm of its own before it joins the stream.
``parallel``: h += mixer(n) + feed_forward(n) with the one n = norm(h), or with a norm each (both of the
same h); optionally the mixer's input is mixed with the previous token's (token shift), and optionally the
layer is followed by a learned weighted sum over the results of all layers so far."""
from __future__ import annotations

import torch

from ..cache import StateNeed
from ..csrc.kernel_sets import NormedInput
from .registry import register_block


@register_block("pre_norm")
class PreNormBlock:
    """Interface of a block: ``forward(ctx, residual, cache_id, writes_cache)`` updates the
    float32 residual stream ``[T, hidden]`` in place."""

    def __init__(self, mixer, feed_forward, mixer_norm, feed_forward_norm, position):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm
        self.position = position

    @staticmethod
    def _give(x, part):
        """Parts that set ``takes_lazy_input`` get the norm unapplied (a NormedInput) so that
        their kernels may fold it in; all others get the normed activations."""
        return x if getattr(part, "takes_lazy_input", False) else x.tensor()

    def forward(self, ctx, residual, cache_id, writes_cache):
        x = NormedInput(ctx, residual, self.mixer_norm)
        ctx.stage = "mixer"           # names the running part for stage timings; nothing depends on it
        self.mixer.forward(ctx, self._give(x, self.mixer), residual, cache_id, writes_cache, self.position)
        if self.feed_forward is None:
            return
        x2 = NormedInput(ctx, residual, self.feed_forward_norm)
        ctx.stage = "feed_forward"
        self.feed_forward.forward(ctx, self._give(x2, self.feed_forward), residual)


@register_block("sandwich")
class SandwichBlock:
    """x <- x + norm_1b(mixer(norm_1(x))), then x <- x + norm_2b(feed_forward(norm_2(x))): RMS norms before and
    behind each sublayer (the feed-forward may be absent).

    ``params``: ``size``, ``eps``, ``unit_offset`` (the norms behind the sublayers multiply by 1 + w); tensors
    ``mixer_out`` and ``feed_forward_out`` [size].  The sublayers add their products into a float32 row of zeros per
    token (one buffer for the whole step, which the kernel that norms it and adds it to the stream zeroes again
    behind its read); the same kernel takes the feed-forward's entry norm of the new stream, where that is an RMS
    norm, so that between the two sublayers the stream is read once."""

    def __init__(self, mixer, feed_forward, mixer_norm, feed_forward_norm, position, params=None, weights=None, build=None):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm, self.position = mixer_norm, feed_forward_norm, position
        params, weights = params or {}, weights or {}
        self.size, self.eps = int(params["size"]), float(params["eps"])
        offset = 1.0 if params.get("unit_offset") else 0.0

        def multiplier(role):
            w = build.weights.stored(weights[role]).float()
            if tuple(w.shape) != (self.size,):
                raise ValueError(f"{weights[role]} has shape {tuple(w.shape)}, expected ({self.size},)")
            return (w + offset).contiguous()
        self.mixer_out = multiplier("mixer_out")
        self.feed_forward_out = multiplier("feed_forward_out") if feed_forward is not None else None
        self.dtype = build.dtype
        self.fused_entry = feed_forward is not None and getattr(feed_forward_norm, "fusable_rms", False)

    _give = staticmethod(PreNormBlock._give)

    def forward(self, ctx, residual, cache_id, writes_cache):
        branch = ctx.streams
        if not (isinstance(branch, torch.Tensor) and branch.shape == residual.shape and branch.dtype == torch.float32):
            branch = ctx.streams = torch.zeros_like(residual)         # zero again behind every use
        x = NormedInput(ctx, residual, self.mixer_norm)
        ctx.stage = "mixer"
        self.mixer.forward(ctx, self._give(x, self.mixer), branch, cache_id, writes_cache, self.position)
        if self.feed_forward is None:
            ctx.kernels.rms_add(residual, branch, self.mixer_out, self.eps, clear=True)
            return
        ctx.stage = "feed_forward"
        if self.fused_entry:
            x2 = torch.empty(residual.shape, dtype=self.dtype, device=residual.device)
            ctx.kernels.rms_add(residual, branch, self.mixer_out, self.eps, clear=True, next_norm=self.feed_forward_norm,
                                next_out=x2)
        else:
            ctx.kernels.rms_add(residual, branch, self.mixer_out, self.eps, clear=True)
            x2 = self._give(NormedInput(ctx, residual, self.feed_forward_norm), self.feed_forward)
        self.feed_forward.forward(ctx, x2, branch)
        ctx.kernels.rms_add(residual, branch, self.feed_forward_out, self.eps, clear=True)


@register_block("parallel")
class ParallelBlock:
    """x <- x + mixer(n) + feed_forward(n), n = norm(x): one norm, read by both sublayers (the
    feed-forward may be absent).  With a second norm: x <- x + mixer(norm_1(x)) + feed_forward(norm_2(x)), both
    norms taken of the x that enters the layer.

    ``params["token_shift"] = {"size": width}`` with the tensor ``shift`` [width]: the mixer reads
    n_t + (n_(t-1) - n_t) * shift instead of n_t, where n_(t-1) is the previous token's normed row as it was
    before this replacement (zeros for a sequence's first token).  The last row of a step is kept per
    sequence: the block then asks the cache for ``{"mixer": the mixer's need, "shift": a row of width
    floats}``, and the mixer gets the cache id ``(cache_id, "mixer")``.

    ``params["depth_average"] = {"index": i, "layers": L}`` adds a weighted sum over depth.  Call R_0 what the
    embedding gives and R_(n+1) = s_n + mixer(norm(s_n)) + feed_forward(norm(s_n)) the raw result of layer n,
    where s_n is the stream that enters it; then s_(i+1) = sum_{j = 0 .. i+1} a_i[j] R_j with layer i's own
    i + 2 numbers a_i (``depth_weights``).  The R_j of a step are planes of one float32 stack ``ctx.streams``
    [L + 2, T, width]: plane i + 1 holds s_i, the sublayers add into it in place (which makes it R_(i+1)), and
    the weighted sum is written into plane i + 2, which the block returns as the stream from then on.
    """

    def __init__(self, mixer, feed_forward, mixer_norm, feed_forward_norm, position, params=None,
                 weights=None, build=None):
        self.mixer, self.feed_forward, self.mixer_norm, self.position = mixer, feed_forward, mixer_norm, position
        self.feed_forward_norm = feed_forward_norm
        self.shift = (params or {}).get("token_shift")
        if self.shift is not None:
            self.shift_size = int(self.shift["size"])
            mu = build.weights.stored(weights["shift"]).float().reshape(1, -1).contiguous()
            if tuple(mu.shape) != (1, self.shift_size):
                raise ValueError(f"{weights['shift']} has shape {tuple(mu.shape[1:])}, expected ({self.shift_size},)")
            self.shift_mu = mu
        self.depth = (params or {}).get("depth_average")
        if self.depth is not None:
            self.index, self.layers = int(self.depth["index"]), int(self.depth["layers"])
            w = build.weights.stored(weights["depth_weights"]).float().contiguous()
            if tuple(w.shape) != (self.index + 2,):
                raise ValueError(f"{weights['depth_weights']} has shape {tuple(w.shape)}, expected ({self.index + 2},)")
            self.depth_weights = w
            self.one = torch.ones(1, dtype=torch.float32, device=build.device)

    _give = staticmethod(PreNormBlock._give)

    def cache_need(self):
        """What the block's stop of the schedule keeps per sequence: the mixer's need, and with token shift a
        row of its own beside it."""
        need = self.mixer.cache_need()
        if self.shift is None:
            return need
        return {"mixer": need, "shift": StateNeed(self.shift_size)}

    @staticmethod
    def cache_need_from(params, mixer_need):
        shift = (params or {}).get("token_shift")
        return mixer_need if shift is None else {"mixer": mixer_need, "shift": StateNeed(int(shift["size"]))}

    def forward(self, ctx, residual, cache_id, writes_cache):
        if self.depth is not None:
            if self.index == 0:
                T, width = residual.shape
                ctx.streams = torch.empty((self.layers + 2, T, width), dtype=torch.float32, device=residual.device)
                ctx.kernels.stream_mix(residual.unsqueeze(0), self.one, 1, ctx.streams[0])
                ctx.kernels.stream_mix(residual.unsqueeze(0), self.one, 1, ctx.streams[1])
            elif ctx.streams is None:
                raise RuntimeError("a depth-averaging layer ran before the first one of its step")
            residual = ctx.streams[self.index + 1]
        fused = self.shift is not None and hasattr(self.mixer_norm, "with_shift") and \
            (self.feed_forward is None or type(self.feed_forward_norm) is type(self.mixer_norm))
        if fused:
            # both norms and the shift read the entering stream once (a norm kind that offers this form)
            if not writes_cache:
                raise ValueError("a block with token shift keeps state: its stop must write its cache entry")
            ctx.stage = "mixer"
            mixed, n2 = self.mixer_norm.with_shift(ctx, residual, self.shift_mu, ctx.cache.state((cache_id, "shift")),
                                                   self.feed_forward_norm if self.feed_forward is not None else None)
            self.mixer.forward(ctx, mixed, residual, (cache_id, "mixer"), writes_cache, self.position)
            if self.feed_forward is not None:
                ctx.stage = "feed_forward"
                self.feed_forward.forward(ctx, n2, residual)
            return self._after(ctx)
        x = NormedInput(ctx, residual, self.mixer_norm)
        x2 = x
        if self.feed_forward is not None and self.feed_forward_norm is not None:
            # the second norm reads the stream as it enters the layer: taken before the mixer adds to it
            x2 = NormedInput(ctx, residual, self.feed_forward_norm)
            x2.tensor()
        ctx.stage = "mixer"
        if self.shift is not None:
            if not writes_cache:
                raise ValueError("a block with token shift keeps state: its stop must write its cache entry")
            n = x.tensor()
            mixed = torch.empty((1,) + tuple(n.shape), dtype=n.dtype, device=n.device)
            ctx.kernels.shift_mix(n, self.shift_mu, ctx.cache.state((cache_id, "shift")), ctx.batch, mixed)
            self.mixer.forward(ctx, mixed[0], residual, (cache_id, "mixer"), writes_cache, self.position)
        else:
            self.mixer.forward(ctx, self._give(x, self.mixer), residual, cache_id, writes_cache, self.position)
        if self.feed_forward is not None:
            ctx.stage = "feed_forward"
            self.feed_forward.forward(ctx, self._give(x2, self.feed_forward), residual)
        return self._after(ctx)

    def _after(self, ctx):
        if self.depth is None:
            return None
        out = ctx.streams[self.index + 2]
        ctx.kernels.stream_mix(ctx.streams, self.depth_weights, self.index + 2, out)
        return out
