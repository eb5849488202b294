"""Kernel sets: the operations parts call, bound to one family of kernels.

``PlainKernels`` runs every operation with the plain kernels (float32 arithmetic,
fixed summation order): it is the whole float32 path and also works with bfloat16
storage.  Faster sets derive from it and replace one operation at a time, each
checked against the plain one.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ops


class NormedInput:
    """The input of a mixer or feed-forward: ``norm(residual)``, not yet computed.

    ``tensor()`` runs the norm kernel (once) and gives the activations; a kernel set that
    can apply the norm inside its matrix product reads ``residual``, ``weight`` and
    ``eps`` instead and never materialises them."""

    def __init__(self, ctx, residual, norm):
        self.ctx, self.residual, self.norm = ctx, residual, norm
        self._tensor = None

    @property
    def fusable(self) -> bool:
        return getattr(self.norm, "fusable_rms", False)

    @property
    def weight(self):
        return self.norm.weight

    @property
    def eps(self) -> float:
        return self.norm.eps

    @property
    def n_rows(self) -> int:
        return self.residual.shape[0]

    def tensor(self) -> torch.Tensor:
        if self._tensor is None:
            self._tensor = self.norm(self.ctx, self.residual)
        return self._tensor


def as_tensor(x) -> torch.Tensor:
    return x.tensor() if isinstance(x, NormedInput) else x


class PlainKernels:
    name = "plain"
    capturable = False      # the float32 path launches every step eagerly: each launch's status is looked at
    pdl = False             # no launch is a programmatic dependent of the one before
    PDL_MAX_ROWS = 128      # ... and in a set that does chain its launches, only those of small steps are: the blocks of a
                            # dependent kernel become resident while a long kernel before it still runs, and a prompt of
                            # 2,048 tokens whose recurrences take a millisecond each ran 8.1 ms chained and 5.1 ms unchained

    def _chain(self, rows) -> bool:
        return bool(self.pdl) and int(rows) <= self.PDL_MAX_ROWS

    def embed(self, ids, table, out, scale=1.0):
        ops.embed(ids, table, out, scale)

    def embed_norm(self, ids, table, weight, eps, out, scale=1.0):
        ops.embed_norm(ids, table, weight, eps, out, scale)

    def rmsnorm(self, x, weight, eps, out, rows=None):
        ops.rmsnorm(x, weight, eps, out, rows)

    def linear(self, x, weight, out, accumulate=False):
        """out (+)= x @ weight^T; ``x`` may be a :class:`NormedInput`."""
        ops.gemm_nt_plain(as_tensor(x), weight, out, accumulate)

    def pack_gate_up(self, gate, up):
        """Gate and up weights as one matrix, in the layout ``gate_up_swiglu`` wants."""
        return torch.cat([gate, up], dim=0).contiguous(), "halves"

    def gate_up_swiglu(self, x, w_gate_up, layout, out, act=None, row_scale=None):
        """out = silu(x @ gate^T) * (x @ up^T); ``act`` = (kind, limit) names another inner step of the gated unit
        (``ops.gated_activation``); ``row_scale``: one float32 factor per row of ``out``."""
        x = as_tensor(x)
        gate_up = torch.empty((x.shape[0], w_gate_up.shape[0]), dtype=x.dtype, device=x.device)
        self.linear(x, w_gate_up, gate_up)
        kind, limit = act if act else ("silu", 0.0)
        ops.gated_activation(gate_up, out, kind, limit, interleaved=(layout == "interleaved"), row_scale=row_scale,
                             pdl=self._chain(x.shape[0]))

    def rms_add(self, residual, branch, weight, eps, clear=False, next_norm=None, next_out=None):
        """residual += rmsnorm(branch) * weight; with ``next_norm`` (an RMS norm part) its output of the new stream
        into ``next_out`` in the same pass."""
        ops.rms_add(residual, branch, weight, eps, clear, None if next_norm is None else next_norm.weight_f32,
                    0.0 if next_norm is None else next_norm.eps, next_out, pdl=self._chain(residual.shape[0]))

    def project_rope_append(self, x, w_qkv, qkv, position, kv, batch, n_q, n_kv, head_dim, page_shift) -> bool:
        """The q/k/v projection with position encoding and cache append in one kernel: rotated q
        into ``qkv``'s first columns, k and v into the cache.  False: not taken, nothing was done."""
        return False

    def rope_append(self, qkv, cos, sin, batch, page_table, k_cache, v_cache, n_q, n_kv, head_dim,
                    rotary_dim, page_shift, write_cache=True, interleaved=False):
        ops.rope_append(qkv, cos, sin, batch.pos, batch.slot_of_token, page_table, k_cache, v_cache,
                        n_q, n_kv, head_dim, rotary_dim, page_shift, write_cache, interleaved)

    def rope_attention(self, qkv, position, kv, batch, out, n_q, n_kv, head_dim, page_shift, window,
                       scale) -> bool:
        """Position encoding, cache append and attention in one launch, if this set can do it
        for this case; False means the caller runs the two steps separately."""
        return False

    def attention(self, q, k_cache, v_cache, batch, page_table, out, n_q, n_kv, head_dim, page_shift,
                  window: Optional[int], scale: float):
        ops.attention_plain(q, k_cache, v_cache, batch.pos, batch.slot_of_token, page_table, out,
                            n_q, n_kv, head_dim, page_shift, window, scale)

    def swiglu(self, gate_up, out):
        ops.swiglu(gate_up, out)

    # ---- latent attention ------------------------------------------------------------
    def head_linear(self, x, w, out):
        """out[t, h] = w[h] @ x[t, h]: a matrix per head (``x`` [T, H, K] and ``out`` [T, H, N] may be views
        into wider rows, ``w`` [H, N, K])."""
        ops.head_linear_plain(x, w, out)

    def latent_prepare(self, proj, c_off, q_abs, norm_w, eps, position, batch, page_table, cache, n_heads, dim,
                       rot_dim, kv_rank, page_shift, write_cache=True):
        """Rotated query parts into ``q_abs``; the token's cache row [normed latent | rotated key part]."""
        cos, sin, rot_dims = position.rotary_tables()
        ops.latent_prepare(proj, c_off, q_abs, norm_w, eps, cos, sin, batch.pos, batch.slot_of_token, page_table,
                           cache, n_heads, dim, rot_dim, rot_dims, kv_rank, page_shift, write_cache,
                           getattr(position, "interleaved", False))

    def latent_attention(self, q_abs, cache, batch, page_table, out, n_heads, kv_rank, rot_dim, page_shift,
                         window, scale, sinks):
        """Attention of every head over the one cached row per token: keys are the whole rows
        (kv_rank + rot_dim), values their first kv_rank elements; ``sinks`` as in ``ops.attention_plain``.
        ``out`` [T, heads x kv_rank]."""
        ops.attention_plain(q_abs, cache, None, batch.pos, batch.slot_of_token, page_table, out, n_heads, 1,
                            kv_rank + rot_dim, page_shift, window, scale, value_dim=kv_rank, sinks=sinks)

    # ---- linear recurrence -----------------------------------------------------------
    def gated_linear_scan(self, proj, q_off, k_off, v_off, z, z_bias, tau, q_scale, state, batch, out, n_heads,
                          dim, vdim):
        chunk, n_sums, n_decays = ops.scan_chunking(batch.n_seqs, batch.max_new, n_heads, dim, vdim)
        sums = decays = None
        if chunk:                             # a long prompt: its chunks in parallel
            sums = torch.empty(n_sums, dtype=torch.float32, device=out.device)
            decays = torch.empty(n_decays, dtype=torch.float32, device=out.device)
        ops.gated_linear_scan(proj, q_off, k_off, v_off, z, z_bias, tau, q_scale, state, batch.cu_new,
                              batch.seq_slot, out, n_heads, dim, vdim, chunk=chunk, max_new=batch.max_new,
                              sums=sums, decays=decays)

    def head_norm_gate(self, o, weight, eps, gate, out, n_heads, vdim, gate_kind="silu"):
        ops.head_norm_gate(o, weight, eps, gate, out, n_heads, vdim, pdl=self._chain(o.shape[0]), gate_kind=gate_kind)

    def state_scan_prepare(self, z, z_bias, decay_kind, decay_scale, n_heads, dim, proj=None, k_off=0, a_off=0,
                           a_bias=None, unit_eps=0.0, unit=None, log_decay=False):
        """The float32 inputs of a matrix-state recurrence: decays in place of ``z`` (their logarithms for the
        float32 path's scan); unit keys and removal vectors into ``unit`` (see ``ops.state_scan_prepare``)."""
        ops.state_scan_prepare(z, z_bias, decay_kind, decay_scale, n_heads, dim, proj, k_off, a_off, a_bias, unit_eps,
                               unit, log_decay=log_decay, pdl=self._chain(z.shape[0]))

    def matrix_state_scan(self, proj, r_off, k_off, v_off, decay, kind, state, batch, out, n_heads, dim, vdim,
                          unit=None, bonus=None):
        """``kind`` ``"delta"`` (decay, removal along the unit key, then the new pair) or ``"bonus"`` (decay, with
        the token at hand read through a bonus), over every sequence's new tokens from and into its state."""
        ops.matrix_state_scan(proj, r_off, k_off, v_off, decay, kind, state, batch.cu_new, batch.seq_slot, out,
                              n_heads, dim, vdim, unit=unit, bonus=bonus, pdl=self._chain(batch.n_tokens))

    def _scan_scratch(self, n, device):
        return torch.empty(n, dtype=torch.float32, device=device)

    def matrix_state_step(self, proj, r_off, k_off, v_off, g_off, a_off, z, z_bias, decay_kind, decay_scale, a_bias,
                          unit_eps, kind, bonus, state, batch, norm_w, eps, gate_kind, y, n_heads, dim, vdim) -> bool:
        """Decays, the walk and the head norm with its gate of a decode step in one launch, if this set can do it for
        this case; False means the caller runs the three operations."""
        return False

    def gated_unit_scan(self, gates, bias_r, bias_i, rate, u, y, y_bias, state, batch, out, block):
        scratch = None
        if u.dtype == torch.bfloat16 and batch.max_new >= ops.GATED_UNIT_SPLIT_MIN_NEW:       # a long run: chunks in parallel
            scratch = self._scan_scratch(ops.gated_unit_scan_scratch(batch.n_seqs, batch.max_new, state.shape[1]), out.device)
        ops.gated_unit_scan(gates, bias_r, bias_i, rate, u, y, y_bias, state, batch.cu_new, batch.seq_slot, out, block,
                            max_new=batch.max_new, scratch=scratch, pdl=self._chain(batch.n_tokens))

    # ---- along a sequence --------------------------------------------------------------
    def pair_embed(self, ids, table, pair, prev, batch, out, buckets, mul_prev, mul_cur):
        ops.pair_embed(ids, table, pair, prev, batch.cu_new, batch.seq_slot, out, batch.max_new, buckets, mul_prev,
                       mul_cur, pdl=self._chain(batch.n_tokens))

    def dynamic_tanh(self, x, alpha, weight, bias, out, rows=None):
        ops.dynamic_tanh(x, alpha, weight, bias, out, rows, pdl=self._chain(out.shape[0]))

    def shift_mix(self, h, mu, last, batch, out):
        """out[s] = h + (h shifted by one token - h) * mu[s]; ``last`` carries a sequence's last row across steps."""
        ops.shift_mix(h, mu, last, batch.cu_new, batch.seq_slot, out, batch.max_new, pdl=self._chain(batch.n_tokens))

    def tanh_norm_shift(self, x, norm1, norm2, mu, last, batch, mixed, second):
        """A layer's entry in one pass: the first tanh norm with the token shift behind it, and the second tanh norm."""
        ops.tanh_norm_shift(x, norm1, norm2, mu, last, batch.cu_new, batch.seq_slot, mixed, second, batch.max_new,
                            pdl=self._chain(batch.n_tokens))

    def causal_conv(self, x, x_bias, weight, bias, tail, batch, out, pass_cols=0):
        ops.causal_conv(x, x_bias, weight, bias, tail, batch.cu_new, batch.seq_slot, out, batch.max_new,
                        pdl=self._chain(batch.n_tokens), pass_cols=pass_cols)

    def concat_cast(self, x, x0, act, bias, out):
        ops.concat_cast(x, x0, act, bias, out, pdl=self._chain(x.shape[0]))

    def rms_pair_add(self, residual, a, wa, b, wb, eps, scale):
        ops.rms_pair_add(residual, a, wa, b, wb, eps, scale, pdl=self._chain(residual.shape[0]))

    def tanh_(self, x):
        ops.tanh_(x, pdl=self._chain(x.shape[0]))

    # ---- attention with sigmoid weights --------------------------------------------------
    def qk_norm_rope_append(self, qkv, q_weight, k_weight, eps, position, kv, batch, n_q, n_kv, dim, vdim, page_shift,
                            write_cache=True):
        """Per-head RMS norm of q and k, rotation of their first coordinates, k and v into the cache."""
        cos = sin = None
        rot_dims = 0
        if position is not None:
            position.check_range(batch)
            cos, sin, rot_dims = position.rotary_tables()
        k_cache, v_cache, table, _ = kv
        ops.qk_norm_rope_append(qkv, q_weight, k_weight, eps, cos, sin, batch.pos, batch.slot_of_token, table, k_cache,
                                v_cache, n_q, n_kv, dim, vdim, rot_dims, page_shift, write_cache, pdl=self._chain(batch.n_tokens))

    def sigmoid_attention(self, q, k_cache, v_cache, batch, page_table, bias, out, n_q, n_kv, dim, vdim, page_shift,
                          chunk, window, scale):
        ops.sigmoid_attention_plain(q, k_cache, v_cache, batch.pos, batch.slot_of_token, page_table, bias, out, n_q,
                                    n_kv, dim, vdim, page_shift, chunk, window, scale, pdl=self._chain(batch.n_tokens))

    # ---- softmax attention over a window, kept first tokens and pooled runs ---------------------
    def activation(self, u, out, kind, scale=1.0):
        """out = act(u) * scale (``relu_squared``, ``gelu_tanh``, ``silu``)."""
        ops.activation(u, out, kind, scale, pdl=self._chain(u.shape[0]))

    def linear_activation(self, x, weight, out, kind, scale=1.0):
        """out = act(x @ weight^T) * scale."""
        x = as_tensor(x)
        u = torch.empty((x.shape[0], weight.shape[0]), dtype=x.dtype, device=x.device)
        self.linear(x, weight, u)
        self.activation(u, out, kind, scale)

    def qkv_prepare(self, qkv, q_weight, k_weight, norm, eps, position, value_position, kv, batch, n_q, n_kv, dim, vdim,
                    page_shift, write_cache=True, pooled_kv=None, pool=0, v_off=None, q_temp=None, n_v=None) -> bool:
        """Norm of q and k (``norm`` ``"head"``, ``"row"`` or None), rotation of their first coordinates by
        ``position``, of the values over their whole width by ``value_position`` (either may be None), k and v into
        the cache.  With a pooled store and a step of one token a sequence, the tokens that end a run of ``pool``
        tokens write the run's pooled row too; True says so (else the caller runs ``pool_rows``)."""
        pools = bool(pool) and pooled_kv is not None and write_cache and batch.is_decode
        cos = sin = vcos = vsin = None
        rot_dims, inter, v_inter = 0, False, False
        if position is not None:
            position.check_range(batch)
            cos, sin, rot_dims = position.rotary_tables()
            inter = bool(getattr(position, "interleaved", False))
        if value_position is not None:
            value_position.check_range(batch)
            vcos, vsin, _ = value_position.rotary_tables()
            v_inter = bool(getattr(value_position, "interleaved", False))
        k_cache, v_cache, table, _ = kv
        ops.qkv_prepare(qkv, q_weight, k_weight, norm, eps, cos, sin, rot_dims, inter, vcos, vsin, v_inter, batch.pos,
                        batch.slot_of_token, table, k_cache, v_cache, n_q, n_kv, dim, vdim, page_shift, write_cache,
                        pdl=self._chain(batch.n_tokens), pooled=pooled_kv[:3] if pools else None, pool=pool if pools else 0,
                        v_off=v_off, q_temp=q_temp, n_v=n_v)
        return pools

    def pool_rows(self, kv, pooled_kv, batch, n_kv, dim, vdim, page_shift, pool):
        """The mean key and value row of every run of ``pool`` tokens that the step's tokens finish."""
        k_cache, v_cache, table, _ = kv
        pk, pv, ptable, _ = pooled_kv
        ops.pool_rows(k_cache, v_cache, table, pk, pv, ptable, batch.cu_new, batch.seq_start, batch.seq_slot,
                      batch.max_new, n_kv, dim, vdim, page_shift, pool, pdl=self._chain(batch.n_tokens))

    def window_attention(self, q, kv, pooled_kv, batch, out, n_q, n_kv, dim, vdim, page_shift, window, keep_first, pool,
                         scale, softcap, sinks, value_position, out_scale=1.0, v_share=1, gate=None):
        vcos = vsin = None
        v_inter = False
        if value_position is not None:
            vcos, vsin, _ = value_position.rotary_tables()
            v_inter = bool(getattr(value_position, "interleaved", False))
        k_cache, v_cache, table, _ = kv
        pooled = None if pooled_kv is None else pooled_kv[:3]
        ops.window_attention_plain(q, k_cache, v_cache, table, pooled, batch.pos, batch.slot_of_token, out, n_q, n_kv,
                                   dim, vdim, page_shift, window, keep_first, pool, scale, softcap, sinks, vcos, vsin,
                                   v_inter, out_scale, pdl=self._chain(batch.n_tokens), v_share=v_share, gate=gate)

    def map_difference(self, maps, out, n_heads, n_kv, vdim, lam, eps, mult):
        ops.map_difference(maps, out, n_heads, n_kv, vdim, lam, eps, mult, pdl=self._chain(maps.shape[0]))

    def mingru_scan(self, proj, z_bias, x_bias, state, batch, out, width, out_scale=1.0):
        scratch = None
        if batch.max_new >= ops.MINGRU_CHUNKED_MIN_NEW:      # a prompt: every 64 tokens in a block of their own
            scratch = self._scan_scratch(ops.mingru_scan_scratch(batch.n_seqs, batch.max_new, width), out.device)
        ops.mingru_scan(proj, z_bias, x_bias, state, batch.cu_new, batch.seq_slot, out, width, out_scale,
                        tiled=batch.max_new >= ops.MINGRU_TILED_MIN_NEW, pdl=self._chain(batch.n_tokens),
                        max_new=batch.max_new, scratch=scratch)

    # ---- experts ---------------------------------------------------------------------
    expert_tile_rows = 64

    def route_table(self, token_ids, table, n_experts, expert_of, pair_weight):
        ops.route_table(token_ids, table, n_experts, expert_of, pair_weight)

    def route_sigmoid_groups(self, logits, n_experts, correction, n_groups, keep, scale, expert_of, pair_weight,
                             extra_col=None, extra_out=None):
        ops.route_sigmoid_groups(logits, n_experts, correction, n_groups, keep, scale, expert_of, pair_weight, extra_col,
                                 extra_out, pdl=self._chain(logits.shape[0]))

    def group_by_expert(self, expert_of, n_experts, groups):
        """``groups``: the dict of int32 tensors a grouped product reads (offsets, order, tile_expert,
        tile_row0, meta) plus ``max_tiles``."""
        ops.group_by_expert(expert_of, n_experts, groups["tile_rows"], groups["offsets"], groups["order"],
                            groups["tile_expert"], groups["tile_row0"], groups["meta"])

    def grouped_linear(self, a, gather, top, w, out, scatter, groups):
        """Per expert group: out[rows] = a[rows] @ w[e]^T.  ``gather``: a's rows are tokens, looked up through
        the sorted order (pair // top); ``scatter``: out's rows are pairs, written through the order."""
        ops.grouped_gemm_plain(a, groups["order"] if gather else None, top if gather else 1, w, out,
                               groups["order"] if scatter else None, groups["offsets"], groups["tile_expert"],
                               groups["tile_row0"], groups["meta"], groups["max_tiles"])

    def expert_gate_up(self, x, top, w_gate_up, out, groups, act=None):
        """out[sorted row] = silu(x gate_e^T) * (x up_e^T) for the row's expert e; ``w_gate_up`` [E, 2 * inter,
        hidden] holds gate rows, then up rows; ``x``'s rows are tokens (gathered through the order).  ``act`` =
        (kind, limit): another inner step of the gated unit."""
        gate_up = torch.empty((out.shape[0], w_gate_up.shape[1]), dtype=x.dtype, device=x.device)
        self.grouped_linear(x, True, top, w_gate_up, gate_up, False, groups)
        kind, limit = act if act else ("silu", 0.0)
        ops.gated_activation(gate_up, out, kind, limit, pdl=self._chain(out.shape[0]))

    def expert_combine(self, residual, y, pair_weight, top):
        ops.expert_combine(residual, y, pair_weight, top)

    # ---- streams ---------------------------------------------------------------------
    def scale_(self, x, s):
        ops.scale_(x, s)

    def stream_mix(self, streams, weights, n_terms, out):
        ops.stream_mix(streams, weights, n_terms, out)

    def add_into(self, out, x):
        ops.add_into(out, x)

    def argmax(self, logits, out):
        ops.argmax(logits, out)

    def target_nll(self, logits, targets, out):
        ops.target_nll(logits, targets, out)

    def sample(self, logits, temperature, top_k, top_p, slots, rng_state, out, drawn_u=None):
        ops.sample(logits, temperature, top_k, top_p, slots, rng_state, out, drawn_u)


def kernel_set_for(dtype: torch.dtype, prefer: Optional[str] = None, deterministic: bool = False):
    """float32 always runs the plain set (which has no atomics on data); bfloat16 runs the fast set
    unless ``prefer='plain'``, with or without float atomics in its split projections."""
    if dtype == torch.float32 or prefer == "plain":
        return PlainKernels()
    from .fast_sets import FastKernels
    return FastKernels(deterministic=deterministic)
