"""Token embedding: h[t] = E[id_t], widened into the float32 residual stream
(kernels/full_attention_cuda.cuh:2012-2034).  ``pair_embedding`` adds a second row chosen by a hash of
the token and the one before it."""
from __future__ import annotations

import torch

from ..cache import StateNeed
from .registry import BuildContext, register_embedding


@register_embedding("embedding")
class Embedding:
    """params: ``vocab_size``, ``hidden_size``, ``scale`` (optional: the rows are multiplied by it in float32),
    ``norm`` (optional, ``{"eps", "unit_offset"}``: the rows pass an RMS norm on their way into the stream, in the
    same kernel); weights: ``weight`` [vocab, hidden], with a norm ``norm`` [hidden]."""

    def __init__(self, params, weights, build: BuildContext):
        self.vocab, self.hidden = int(params["vocab_size"]), int(params["hidden_size"])
        self.scale = float(params.get("scale", 1.0))
        self.norm_weight = None
        if params.get("norm"):
            w = build.weights.stored(weights["norm"]).float()
            if tuple(w.shape) != (self.hidden,):
                raise ValueError(f"{weights['norm']} has shape {tuple(w.shape)}, expected ({self.hidden},)")
            self.norm_weight = (w + (1.0 if params["norm"].get("unit_offset") else 0.0)).contiguous()
            self.norm_eps = float(params["norm"]["eps"])
        self.table = build.weights.as_dtype(weights["weight"], build.dtype, share=True)
        if tuple(self.table.shape) != (self.vocab, self.hidden):
            raise ValueError(f"{weights['weight']} has shape {tuple(self.table.shape)}, "
                             f"expected {(self.vocab, self.hidden)}")

    def __call__(self, ctx, token_ids):
        out = torch.empty((token_ids.shape[0], self.hidden), dtype=torch.float32, device=token_ids.device)
        if self.norm_weight is not None:
            ctx.kernels.embed_norm(token_ids, self.table, self.norm_weight, self.norm_eps, out, self.scale)
        else:
            ctx.kernels.embed(token_ids, self.table, out, self.scale)
        return out


@register_embedding("pair_embedding")
class PairEmbedding:
    """h[t] = E[id_t] + P[row_t] with row_t = (id_(t-1) * mul_prev + id_t * mul_cur) mod buckets, and row
    ``buckets`` (the table's last) for a sequence's first token.

    params: ``vocab_size``, ``hidden_size``, ``buckets``, ``mul_prev``, ``mul_cur``; weights: ``weight``
    [vocab, hidden], ``pair`` [buckets + 1, hidden].  The token before a step's first one is part of the
    sequence's state: an int32 per slot (id + 1; 0 for none), asked of the cache with ``cache_need()``.
    """

    cache_key = "embedding"

    def __init__(self, params, weights, build: BuildContext):
        self.vocab, self.hidden = int(params["vocab_size"]), int(params["hidden_size"])
        self.buckets = int(params["buckets"])
        self.mul_prev, self.mul_cur = int(params["mul_prev"]), int(params["mul_cur"])
        if self.buckets < 1:
            raise ValueError("pair_embedding: at least one bucket")
        self.table = build.weights.as_dtype(weights["weight"], build.dtype, share=True)
        self.pair = build.weights.as_dtype(weights["pair"], build.dtype)
        if tuple(self.table.shape) != (self.vocab, self.hidden) or tuple(self.pair.shape) != (self.buckets + 1, self.hidden):
            raise ValueError(f"{weights['weight']} / {weights['pair']} have shapes {tuple(self.table.shape)} / "
                             f"{tuple(self.pair.shape)}, expected {(self.vocab, self.hidden)} / "
                             f"{(self.buckets + 1, self.hidden)}")

    def cache_need(self):
        return StateNeed(1, "int32")

    @staticmethod
    def cache_need_from(params):
        return StateNeed(1, "int32")

    def __call__(self, ctx, token_ids):
        out = torch.empty((token_ids.shape[0], self.hidden), dtype=torch.float32, device=token_ids.device)
        ctx.kernels.pair_embed(token_ids, self.table, self.pair, ctx.cache.state(self.cache_key), ctx.batch, out,
                               self.buckets, self.mul_prev, self.mul_cur)
        return out
