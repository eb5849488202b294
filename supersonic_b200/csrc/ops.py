"""Python faces of the plain CUDA kernels: tensors in, a launch on the current stream out.

Every wrapper checks what the kernel assumes (device, dtype, contiguity, sizes)
and raises; a non-zero status from the library raises :class:`KernelError`.
There is no CPU path: without a CUDA device, or without the compiled library,
these functions fail.  One wrapper per op, like the reference's
``prefill_ffi`` (crates/kernel-ffi/src/prefill_ffi.rs:1104-3292) with its dtype
codes (crates/gpu-hal/src/scalar_type.rs:25-32).
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from .build import load_library

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}
_ERRORS = {2001: "unsupported dtype", 2002: "unsupported size", 2003: "unsupported configuration",
           2004: "a bounded wait ran out"}


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _CODES[dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16, not {dtype}") from None


def _check(status: int, what: str) -> None:
    global LAUNCHES
    LAUNCHES += 1
    if status:
        reason = _ERRORS.get(status) or f"CUDA error {status}"
        raise KernelError(f"{what}: {reason}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> c_void_p:
    """The current stream's handle (the raw query is several times cheaper than building a
    ``torch.cuda.Stream`` object, and this runs for every launch)."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _need(t: torch.Tensor, name: str, dtype=None, dims: Optional[int] = None, rows_contiguous=True):
    if not t.is_cuda:
        raise KernelError(f"{name} must live on a CUDA device (there is no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, is {t.dtype}")
    if dims is not None and t.dim() != dims:
        raise KernelError(f"{name} must have {dims} dims, has shape {tuple(t.shape)}")
    if rows_contiguous and t.dim() >= 1 and t.numel() and t.stride(-1) != 1:
        raise KernelError(f"{name} must be contiguous in its last dim")
    if t.dim() > 2 and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


_lib_cache = {}
LAUNCHES = 0          # kernels launched through this module (graph replays are counted by their owner)


def _fn(lib: str, name: str):
    key = (lib, name)
    if key not in _lib_cache:
        f = getattr(load_library(lib), name)
        f.restype = c_int
        _lib_cache[key] = f
    return _lib_cache[key]


# ---- plain ops -------------------------------------------------------------------------
def embed(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """out[t] = table[ids[t]] * scale into the float32 residual stream (the product is float32)."""
    _need(ids, "ids", torch.int32, 1); _need(table, "table", None, 2); _need(out, "out", torch.float32, 2)
    if not (table.is_contiguous() and out.is_contiguous()):
        raise KernelError("embed: table and out must be contiguous")
    if out.shape[0] != ids.shape[0] or out.shape[1] != table.shape[1]:
        raise KernelError(f"embed: out {tuple(out.shape)} does not fit {ids.shape[0]} ids of width {table.shape[1]}")
    _check(_fn("plain_ops", "ssb_embed_scaled")(
        _ptr(ids), _ptr(table), c_int(dtype_code(table.dtype)), _ptr(out), c_int(ids.shape[0]),
        c_int(table.shape[1]), c_int(table.shape[0]), c_float(scale), _stream()), "embed")


def embed_norm(ids: torch.Tensor, table: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
               scale: float = 1.0) -> None:
    """out[t] = e / sqrt(mean(e^2) + eps) * weight with e = table[ids[t]] * scale, float32 (``weight`` float32)."""
    _need(ids, "ids", torch.int32, 1); _need(table, "table", None, 2); _need(out, "out", torch.float32, 2)
    _need(weight, "weight", torch.float32, 1)
    if not (table.is_contiguous() and out.is_contiguous()) or out.shape[0] != ids.shape[0] \
            or out.shape[1] != table.shape[1] or weight.shape[0] != table.shape[1]:
        raise KernelError(f"embed_norm: out {tuple(out.shape)} does not fit {ids.shape[0]} ids of width {table.shape[1]}")
    _check(_fn("plain_ops", "ssb_embed_norm")(
        _ptr(ids), _ptr(table), c_int(dtype_code(table.dtype)), _ptr(weight), c_float(eps), _ptr(out), c_int(ids.shape[0]),
        c_int(table.shape[1]), c_int(table.shape[0]), c_float(scale), _stream()), "embed_norm")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None, pdl: bool = False) -> None:
    """out[r] = x[rows[r] or r] * rsqrt(mean(x^2) + eps) * weight, x float32."""
    _need(x, "x", torch.float32, 2); _need(weight, "weight", None, 1); _need(out, "out", None, 2)
    if not (x.is_contiguous() and out.is_contiguous()):
        raise KernelError("rmsnorm: x and out must be contiguous")
    n = out.shape[0]
    if rows is not None:
        _need(rows, "rows", torch.int32, 1)
        if rows.shape[0] != n:
            raise KernelError("rmsnorm: one output row per gathered row")
    elif x.shape[0] != n:
        raise KernelError("rmsnorm: x and out differ in rows")
    if x.shape[1] != out.shape[1] or weight.shape[0] != x.shape[1]:
        raise KernelError("rmsnorm: widths differ")
    _check(_fn("plain_ops", "ssb_rmsnorm")(
        _ptr(x), _ptr(rows), _ptr(weight), c_int(dtype_code(weight.dtype)), c_float(eps), _ptr(out),
        c_int(dtype_code(out.dtype)), c_int(n), c_int(x.shape[1]), c_int(1 if pdl else 0), _stream()), "rmsnorm")


def gemm_nt_plain(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    """out[m, n] (+)= sum_k a[m, k] w[n, k]; float32 accumulation in k order."""
    _need(a, "a", None, 2); _need(w, "w", None, 2); _need(out, "out", None, 2)
    if a.dtype != w.dtype:
        raise KernelError(f"gemm: a is {a.dtype} but w is {w.dtype}")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (M, N):
        raise KernelError(f"gemm: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    _check(_fn("plain_ops", "ssb_gemm_nt_plain")(
        _ptr(a), c_int(a.stride(0)), _ptr(w), c_int(w.stride(0)), c_int(dtype_code(a.dtype)), _ptr(out),
        c_int(out.stride(0)), c_int(dtype_code(out.dtype)), c_int(M), c_int(N), c_int(K),
        c_int(1 if accumulate else 0), _stream()), "gemm_nt_plain")


def rope_append(qkv: torch.Tensor, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                pos: torch.Tensor, slot: torch.Tensor, page_table: torch.Tensor,
                k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], n_q: int, n_kv: int,
                head_dim: int, rotary_dim: int, page_shift: int, write_cache: bool = True,
                interleaved: bool = False) -> None:
    """Rotate q (and k) of every token in place; write k and v into the paged cache entry.  Pairs are
    (i, i + rotary_dim/2), or with ``interleaved`` (2i, 2i + 1)."""
    _need(qkv, "qkv", None, 2); _need(pos, "pos", torch.int32, 1); _need(slot, "slot", torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2)
    T = qkv.shape[0]
    if qkv.shape[1] < (n_q + 2 * n_kv) * head_dim and write_cache:
        raise KernelError("rope_append: qkv rows are too narrow")
    if pos.shape[0] != T or slot.shape[0] != T:
        raise KernelError("rope_append: one position and one slot per token")
    table_positions = 0
    if cos is not None:
        _need(cos, "cos", torch.float32, 2); _need(sin, "sin", torch.float32, 2)
        if cos.shape != sin.shape or cos.shape[1] != rotary_dim // 2 or not cos.is_contiguous() \
                or not sin.is_contiguous():
            raise KernelError("rope_append: cos/sin must be [positions, rotary_dim/2], contiguous")
        table_positions = cos.shape[0]
    if write_cache:
        for c in (k_cache, v_cache):
            _need(c, "cache", qkv.dtype)
            if not c.is_contiguous():
                raise KernelError("rope_append: cache entry must be contiguous")
    _check(_fn("plain_ops", "ssb_rope_append")(
        _ptr(qkv), c_int(qkv.stride(0)), c_int(dtype_code(qkv.dtype)), _ptr(cos), _ptr(sin),
        c_int(table_positions), _ptr(pos), _ptr(slot), _ptr(page_table), c_int(page_table.shape[1]),
        _ptr(k_cache), _ptr(v_cache), c_int(T), c_int(n_q), c_int(n_kv), c_int(head_dim),
        c_int(rotary_dim), c_int(page_shift), c_int(1 if write_cache else 0), c_int(1 if interleaved else 0),
        _stream()), "rope_append")


def attention_plain(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, pos: torch.Tensor,
                    slot: torch.Tensor, page_table: torch.Tensor, out: torch.Tensor, n_q: int, n_kv: int,
                    head_dim: int, page_shift: int, window: Optional[int], scale: float,
                    value_dim: Optional[int] = None, sinks: Optional[torch.Tensor] = None) -> None:
    """Each token attends over keys [max(0, pos-window+1), pos] of its slot in the paged cache.
    ``value_dim``: width of a value and of a head's output when it differs from ``head_dim``;
    ``v_cache`` None: a token's value is the first ``value_dim`` elements of its key row.
    ``sinks`` (float32, one per query head): exp(sink) is added to the softmax's denominator and
    nothing to its numerator."""
    v_dim = head_dim if value_dim is None else int(value_dim)
    v_row = v_dim
    if v_cache is None:
        v_cache, v_row = k_cache, head_dim
    if sinks is not None:
        _need(sinks, "sinks", torch.float32, 1)
        if sinks.shape[0] != n_q:
            raise KernelError("attention: one sink per query head")
    _need(q, "q", None, 2); _need(out, "out", q.dtype, 2)
    _need(k_cache, "k_cache", q.dtype); _need(v_cache, "v_cache", q.dtype)
    _need(pos, "pos", torch.int32, 1); _need(slot, "slot", torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2)
    T = q.shape[0]
    if out.shape[0] != T or out.shape[1] < n_q * v_dim or q.shape[1] < n_q * head_dim:
        raise KernelError("attention: q/out shapes")
    if head_dim > 1024 or v_dim > 1024 or v_dim > v_row or n_q % n_kv:
        raise KernelError(f"attention_plain: head_dim {head_dim}, value_dim {v_dim} (max 1024), heads {n_q}/{n_kv} "
                          "not supported")
    _check(_fn("plain_ops", "ssb_attention_plain")(
        _ptr(q), c_int(q.stride(0)), c_int(dtype_code(q.dtype)), _ptr(k_cache), _ptr(v_cache), _ptr(pos),
        _ptr(slot), _ptr(page_table), c_int(page_table.shape[1]), _ptr(out), c_int(out.stride(0)),
        c_int(T), c_int(n_q), c_int(n_kv), c_int(head_dim), c_int(page_shift),
        c_int(int(window) if window else 0), c_float(scale), c_int(v_dim), c_int(v_row), _ptr(sinks),
        _stream()), "attention_plain")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> None:
    """out[t, c] = silu(gate[t, c]) * up[t, c]; gate and up are the halves of a row of
    ``gate_up``, or (interleaved) alternate as [8 gate | 8 up] per 16 columns."""
    _need(gate_up, "gate_up", None, 2); _need(out, "out", gate_up.dtype, 2)
    T, inter = out.shape
    if gate_up.shape[0] != T or gate_up.shape[1] != 2 * inter:
        raise KernelError("swiglu: gate_up must be [T, 2*I] for out [T, I]")
    _check(_fn("plain_ops", "ssb_swiglu")(
        _ptr(gate_up), c_int(gate_up.stride(0)), _ptr(out), c_int(out.stride(0)),
        c_int(dtype_code(out.dtype)), c_int(T), c_int(inter), c_int(1 if interleaved else 0),
        _stream()), "swiglu")


GATE_KINDS_FF = {"silu": 0, "clamped_swish": 1}


def gated_activation(gate_up: torch.Tensor, out: torch.Tensor, kind: str = "silu", limit: float = 0.0,
                     interleaved: bool = False, row_scale: Optional[torch.Tensor] = None, pdl: bool = False) -> None:
    """out[t, c] = f(gate[t, c], up[t, c]) * row_scale[t] in float32 arithmetic.  ``kind`` ``"silu"``: silu(g) u;
    ``"clamped_swish"``: with g' = min(g, limit), u' = clamp(u, -limit, limit): g' sigmoid(1.702 g') (u' + 1).  Gate and up
    are the halves of a row of ``gate_up``, or (interleaved) alternate as [8 gate | 8 up] per 16 columns."""
    _need(gate_up, "gate_up", None, 2); _need(out, "out", gate_up.dtype, 2)
    if kind not in GATE_KINDS_FF:
        raise KernelError(f"gated_activation: kind {kind!r} is not known (known: {sorted(GATE_KINDS_FF)})")
    T, inter = out.shape
    if gate_up.shape[0] != T or gate_up.shape[1] != 2 * inter:
        raise KernelError("gated_activation: gate_up must be [T, 2*I] for out [T, I]")
    if row_scale is not None:
        _need(row_scale, "row_scale", torch.float32, 1)
        if row_scale.shape[0] != T:
            raise KernelError("gated_activation: one factor per row")
    _check(_fn("plain_ops", "ssb_gated_activation")(
        _ptr(gate_up), c_int(gate_up.stride(0)), _ptr(out), c_int(out.stride(0)), c_int(dtype_code(out.dtype)), c_int(T),
        c_int(inter), c_int(1 if interleaved else 0), c_int(GATE_KINDS_FF[kind]), c_float(limit), _ptr(row_scale),
        c_int(1 if pdl else 0), _stream()), "gated_activation")


def rms_add(residual: torch.Tensor, branch: torch.Tensor, weight: torch.Tensor, eps: float, clear: bool = False,
            next_weight: Optional[torch.Tensor] = None, next_eps: float = 0.0, next_out: Optional[torch.Tensor] = None,
            pdl: bool = False) -> None:
    """residual[t] += branch[t] / sqrt(mean(branch[t]^2) + eps) * weight (both float32; ``weight`` is the multiplier
    itself).  ``clear``: the branch is zeroed behind the read.  With ``next_out``: next_out[t] = the new residual[t]
    / sqrt(mean(.^2) + next_eps) * next_weight, the norm the next sublayer reads."""
    _need(residual, "residual", torch.float32, 2); _need(branch, "branch", torch.float32, 2)
    _need(weight, "weight", torch.float32, 1)
    T, W = residual.shape
    if tuple(branch.shape) != (T, W) or weight.shape[0] != W or not (residual.is_contiguous() and branch.is_contiguous()):
        raise KernelError("rms_add: residual and branch [tokens, width] contiguous, one weight per column")
    if next_out is not None:
        _need(next_out, "next_out", None, 2); _need(next_weight, "next_weight", torch.float32, 1)
        if tuple(next_out.shape) != (T, W) or next_weight.shape[0] != W or not next_out.is_contiguous():
            raise KernelError("rms_add: next_out [tokens, width] contiguous, one weight per column")
    _check(_fn("plain_ops", "ssb_rms_add")(
        _ptr(residual), _ptr(branch), _ptr(weight), c_float(eps), c_int(T), c_int(W), c_int(1 if clear else 0),
        _ptr(next_weight if next_out is not None else None), c_float(next_eps), _ptr(next_out),
        c_int(dtype_code(next_out.dtype) if next_out is not None else F32), c_int(1 if pdl else 0), _stream()), "rms_add")


def add_into(out: torch.Tensor, x: torch.Tensor) -> None:
    """out (float32) += x."""
    _need(out, "out", torch.float32); _need(x, "x")
    if not (out.is_contiguous() and x.is_contiguous()) or out.numel() != x.numel():
        raise KernelError("add_into: contiguous tensors of equal size")
    _check(_fn("plain_ops", "ssb_add_into")(
        _ptr(out), _ptr(x), c_int(dtype_code(x.dtype)), c_longlong(out.numel()), _stream()), "add_into")


def scale_(x: torch.Tensor, s: float) -> None:
    """x (float32, contiguous) *= s."""
    _need(x, "x", torch.float32)
    if not x.is_contiguous():
        raise KernelError("scale_: a contiguous tensor")
    _check(_fn("plain_ops", "ssb_scale")(_ptr(x), c_float(s), c_longlong(x.numel()), _stream()), "scale")


def stream_mix(streams: torch.Tensor, weights: torch.Tensor, n_terms: int, out: torch.Tensor,
               pdl: bool = False) -> None:
    """out = sum_{j < n_terms} weights[j] * streams[j]: ``streams`` [n, ...] float32 contiguous, ``out`` one
    of its planes or a tensor of a plane's size; the terms are added in the order of j."""
    _need(streams, "streams", torch.float32); _need(weights, "weights", torch.float32, 1); _need(out, "out", torch.float32)
    if not (streams.is_contiguous() and out.is_contiguous()) or streams.dim() < 2:
        raise KernelError("stream_mix: contiguous tensors, streams [n, ...]")
    plane = streams[0].numel()
    if out.numel() != plane or not 0 < n_terms <= min(streams.shape[0], weights.shape[0]):
        raise KernelError(f"stream_mix: {n_terms} terms of {tuple(streams.shape)} into {tuple(out.shape)}")
    _check(_fn("plain_ops", "ssb_stream_mix")(
        _ptr(streams), c_longlong(plane), _ptr(weights), c_int(n_terms), _ptr(out), c_longlong(plane),
        c_int(1 if pdl else 0), _stream()), "stream_mix")


def head_linear_plain(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, h, :] = w[h] @ x[t, h, :]: one matrix per head.  ``x`` [T, H, K] and ``out`` [T, H, N] may be
    views into wider rows (any row and head strides, last dim contiguous); ``w`` [H, N, K] contiguous."""
    _need(w, "w", x.dtype, 3)
    if not (x.is_cuda and out.is_cuda) or x.dim() != 3 or out.dim() != 3:
        raise KernelError("head_linear: x and out must be CUDA tensors [T, H, width]")
    T, H, K = x.shape
    N = w.shape[1]
    if tuple(w.shape) != (H, N, K) or tuple(out.shape) != (T, H, N) or not w.is_contiguous():
        raise KernelError(f"head_linear: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    if x.stride(2) != 1 or out.stride(2) != 1:
        raise KernelError("head_linear: x and out must be contiguous in their last dim")
    _check(_fn("plain_ops", "ssb_gemm_nt_plain_batched")(
        _ptr(x), c_int(x.stride(0)), c_longlong(x.stride(1)), _ptr(w), c_int(K), c_longlong(N * K),
        c_int(dtype_code(x.dtype)), _ptr(out), c_int(out.stride(0)), c_longlong(out.stride(1)),
        c_int(dtype_code(out.dtype)), c_int(H), c_int(T), c_int(N), c_int(K), _stream()), "head_linear")


# ---- latent attention ------------------------------------------------------------------
def latent_prepare(proj: torch.Tensor, c_off: int, q_abs: torch.Tensor, norm_w: torch.Tensor, eps: float,
                   cos: torch.Tensor, sin: torch.Tensor, pos: torch.Tensor, slot: torch.Tensor,
                   page_table: torch.Tensor, cache: Optional[torch.Tensor], n_heads: int, dim: int, rot_dim: int,
                   rot_dims: int, kv_rank: int, page_shift: int, write_cache: bool = True,
                   interleaved: bool = True, pdl: bool = False) -> None:
    """From a token's projected row ``proj`` ([queries: heads x (dim + rot_dim) | from ``c_off``: kv_rank latent,
    rot_dim key part]): the rotated query parts into ``q_abs`` ([heads x (kv_rank + rot_dim)], behind each
    head's first kv_rank columns), and the token's cache row [RMS-normed latent * norm_w | rotated key part]
    at its position.  The first ``rot_dims`` coordinates of a rotated part turn, the rest pass."""
    _need(proj, "proj", None, 2); _need(q_abs, "q_abs", proj.dtype, 2); _need(norm_w, "norm_w", None, 1)
    _need(cos, "cos", torch.float32, 2); _need(sin, "sin", torch.float32, 2)
    _need(pos, "pos", torch.int32, 1); _need(slot, "slot", torch.int32, 1); _need(page_table, "page_table", torch.int32, 2)
    T = proj.shape[0]
    if proj.shape[1] < max(n_heads * (dim + rot_dim), c_off + kv_rank + rot_dim) or \
            q_abs.shape[0] != T or q_abs.shape[1] < n_heads * (kv_rank + rot_dim):
        raise KernelError("latent_prepare: rows are too narrow")
    if cos.shape != sin.shape or cos.shape[1] * 2 != rot_dims or not (cos.is_contiguous() and sin.is_contiguous()):
        raise KernelError("latent_prepare: cos/sin must be [positions, rot_dims/2], contiguous")
    if norm_w.shape[0] != kv_rank or pos.shape[0] != T or slot.shape[0] != T:
        raise KernelError("latent_prepare: sizes")
    if write_cache:
        _need(cache, "cache", proj.dtype)
        if not cache.is_contiguous() or cache.shape[-1] != kv_rank + rot_dim:
            raise KernelError("latent_prepare: the cache entry must be contiguous with rows of kv_rank + rot_dim")
    _check(_fn("latent_ops", "ssb_latent_prepare")(
        _ptr(proj), c_int(proj.stride(0)), c_int(c_off), _ptr(q_abs), c_int(q_abs.stride(0)),
        c_int(dtype_code(proj.dtype)), _ptr(norm_w), c_int(dtype_code(norm_w.dtype)), c_float(eps), _ptr(cos),
        _ptr(sin), c_int(cos.shape[0]), _ptr(pos), _ptr(slot), _ptr(page_table), c_int(page_table.shape[1]),
        _ptr(cache), c_int(T), c_int(n_heads), c_int(dim), c_int(rot_dim), c_int(rot_dims), c_int(kv_rank),
        c_int(page_shift), c_int(1 if write_cache else 0), c_int(1 if interleaved else 0), c_int(1 if pdl else 0),
        _stream()), "latent_prepare")


def latent_attention_mma_ok(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, n_heads: int, dk: int, dv: int,
                            page_shift: int) -> bool:
    """Whether the tensor-core latent attention takes these operands (else the plain kernel does)."""
    return (q.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
            and page_shift == 6 and dk % 16 == 0 and dv % 16 == 0 and 0 < dv <= min(dk, 512) and dk <= 656
            and q.is_contiguous() and out.is_contiguous() and cache.is_contiguous()
            and q.shape[1] == n_heads * dk and out.shape[1] == n_heads * dv
            and q.data_ptr() % 16 == 0 and cache.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0)


def latent_attention_mma(q: torch.Tensor, cache: torch.Tensor, cu_new: torch.Tensor, seq_start: torch.Tensor,
                         seq_slot: torch.Tensor, slot_of_token: torch.Tensor, page_table: torch.Tensor,
                         out: torch.Tensor, sinks: Optional[torch.Tensor], max_new: int, n_heads: int, dk: int,
                         dv: int, page_shift: int, window: Optional[int], scale: float, n_splits: int = 1,
                         partial: Optional[torch.Tensor] = None, pdl: bool = False, form: int = 0) -> None:
    """Every head of every new token over its sequence's cached rows [dv values | dk - dv more key elements]
    (``cache`` [pages, 1, 64, dk]); ``q`` [tokens, heads x dk], ``out`` [tokens, heads x dv], both contiguous
    bfloat16.  ``n_splits`` > 1 cuts a sequence's pages into that many parts whose results a second launch
    merges through ``partial`` (float32, tokens x heads x n_splits x (dv + 2)).  ``form``: 0 lets the kernel
    choose how a block's warps are laid out (one group of 16 rows when a sequence brings no more, else two);
    1, 2, 3 ask for 1 x 8, 2 x 4, 2 x 8 (row groups x slices)."""
    if not latent_attention_mma_ok(q, cache, out, n_heads, dk, dv, page_shift):
        raise KernelError("latent_attention_mma: operands it does not take")
    _need(cu_new, "cu_new", torch.int32, 1); _need(seq_start, "seq_start", torch.int32, 1)
    _need(seq_slot, "seq_slot", torch.int32, 1); _need(slot_of_token, "slot_of_token", torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2)
    T, B = q.shape[0], seq_slot.shape[0]
    if out.shape[0] != T or cu_new.shape[0] != B + 1 or seq_start.shape[0] != B or slot_of_token.shape[0] != T:
        raise KernelError("latent_attention_mma: sizes")
    if sinks is not None:
        _need(sinks, "sinks", torch.float32, 1)
        if sinks.shape[0] != n_heads:
            raise KernelError("latent_attention_mma: one sink per head")
    if n_splits > 1:
        _need(partial, "partial", torch.float32)
        if partial.numel() < T * n_heads * n_splits * (dv + 2):
            raise KernelError("latent_attention_mma: the scratch for partial results is too small")
    _check(_fn("latent_attention", "ssb_latent_attention")(
        _ptr(q), _ptr(cache), _ptr(cu_new), _ptr(seq_start), _ptr(seq_slot), _ptr(slot_of_token), _ptr(page_table),
        c_int(page_table.shape[1]), _ptr(out), _ptr(partial), _ptr(sinks), c_int(B), c_int(max_new), c_int(T),
        c_int(n_heads), c_int(dk), c_int(dv), c_int(page_shift), c_int(int(window) if window else 0), c_float(scale),
        c_int(n_splits), c_int(form), c_int(1 if pdl else 0), _stream()), "latent_attention_mma")


# ---- many small matrix products on the tensor cores -------------------------------------------
def head_gemm_mma_ok(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and out.dtype in (torch.bfloat16, torch.float32)
            and x.dim() == 3 and w.dim() == 3 and w.is_contiguous() and x.stride(2) == 1 and out.stride(2) == 1
            and x.shape[2] % 8 == 0 and x.stride(0) % 8 == 0 and x.stride(1) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def head_gemm_mma(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, pdl: bool = False) -> None:
    """``head_linear_plain`` on mma.sync: out[t, h] = w[h] @ x[t, h] for bfloat16 operands."""
    T, H, K = x.shape
    N = w.shape[1]
    if not head_gemm_mma_ok(x, w, out) or tuple(w.shape) != (H, N, K) or tuple(out.shape) != (T, H, N):
        raise KernelError(f"head_gemm_mma: x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    _check(_fn("batched_gemm", "ssb_head_gemm_mma")(
        _ptr(x), c_int(x.stride(0)), c_longlong(x.stride(1)), _ptr(w), c_int(K), c_longlong(N * K), _ptr(out),
        c_int(out.stride(0)), c_longlong(out.stride(1)), c_int(dtype_code(out.dtype)), c_int(H), c_int(T), c_int(N),
        c_int(K), c_int(1 if pdl else 0), _stream()), "head_gemm_mma")


GG_STORE, GG_SWIGLU = 0, 1


def order_rows(a, a_index, out, c_index) -> int:
    """Rows of all groups together, from whichever operand is in sorted order."""
    return int(out.shape[0] if c_index is None else a.shape[0] if a_index is None else a_index.shape[0])


def grouped_gemm_mma_ok(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int) -> bool:
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous() and a.shape[1] % 8 == 0
            and a.stride(0) % 8 == 0 and a.stride(1) == 1 and out.stride(1) == 1 and a.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0 and (w.shape[1] * w.shape[2]) % 8 == 0
            and (out.dtype == torch.bfloat16 or (mode == GG_STORE and out.dtype == torch.float32)))


def grouped_gemm_mma(a: torch.Tensor, a_index: Optional[torch.Tensor], a_div: int, w: torch.Tensor,
                     out: torch.Tensor, c_index: Optional[torch.Tensor], offsets: torch.Tensor,
                     tile_expert: torch.Tensor, tile_row0: torch.Tensor, meta: torch.Tensor, max_tiles: int,
                     mode: int = GG_STORE, pdl: bool = False, act=None) -> None:
    """``grouped_gemm_plain`` on mma.sync (tiles of 64 rows).  mode GG_SWIGLU: ``w`` [E, 2N, K] holds gate rows then
    up rows and ``out`` [rows, N] gets silu(a gate^T) * (a up^T), or with ``act`` = (kind, limit) that inner step of
    the gated unit (``gated_activation``)."""
    kind, limit = act if act else ("silu", 0.0)
    if kind not in GATE_KINDS_FF:
        raise KernelError(f"grouped_gemm_mma: gate {kind!r} is not known (known: {sorted(GATE_KINDS_FF)})")
    E, n_w, K = w.shape
    N = n_w // 2 if mode == GG_SWIGLU else n_w
    if not grouped_gemm_mma_ok(a, w, out, mode) or a.shape[1] != K or out.shape[1] != N:
        raise KernelError(f"grouped_gemm_mma: a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    _check(_fn("batched_gemm", "ssb_grouped_gemm_mma")(
        _ptr(a), c_int(a.stride(0)), _ptr(a_index), c_int(a_div), _ptr(w), c_int(K), c_longlong(n_w * K), _ptr(out),
        c_int(out.stride(0)), _ptr(c_index), c_int(dtype_code(out.dtype)), _ptr(offsets), _ptr(tile_expert),
        _ptr(tile_row0), _ptr(meta), c_int(max_tiles), c_int(order_rows(a, a_index, out, c_index)), c_int(N), c_int(K),
        c_int(mode), c_int(GATE_KINDS_FF[kind]), c_float(limit), c_int(1 if pdl else 0), _stream()), "grouped_gemm_mma")


# ---- linear recurrences ----------------------------------------------------------------
SCAN_MAX_DIM = 256


def gated_linear_scan(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, z: torch.Tensor,
                      z_bias: torch.Tensor, tau: float, q_scale: float, state: torch.Tensor,
                      cu_new: torch.Tensor, seq_slot: torch.Tensor, out: torch.Tensor, n_heads: int, dim: int,
                      vdim: int, pdl: bool = False, chunk: int = 0, max_new: int = 0,
                      sums: Optional[torch.Tensor] = None, decays: Optional[torch.Tensor] = None) -> None:
    """Per sequence and head, over the sequence's new tokens in order:
    S = diag(sigmoid(z + z_bias)^(1/tau)) S + k v^T;  out = S^T (q * q_scale), with S [dim, vdim] float32 read
    from and left in ``state[slot]``.  q, k (heads x dim) and v (heads x vdim) are columns of ``proj``; ``z`` is
    overwritten with the decays.
    ``chunk`` > 0: every sequence's tokens are cut into chunks of that many that run in parallel (each chunk's
    own sum from zero, the state carried across the chunks in order, then the outputs of every chunk from the
    state at its start), through the float32 scratch ``sums`` (sequences x chunks x heads x dim x vdim) and
    ``decays`` (sequences x chunks x heads x dim), chunks = ceil(``max_new`` / chunk)."""
    _need(proj, "proj", None, 2); _need(z, "z", torch.float32, 2); _need(z_bias, "z_bias", torch.float32, 1)
    _need(state, "state", torch.float32, 2); _need(out, "out", torch.float32, 2)
    _need(cu_new, "cu_new", torch.int32, 1); _need(seq_slot, "seq_slot", torch.int32, 1)
    T, B = proj.shape[0], seq_slot.shape[0]
    if z.shape[0] != T or out.shape[0] != T or z.shape[1] < n_heads * dim or out.shape[1] < n_heads * vdim \
            or z_bias.shape[0] != n_heads * dim or cu_new.shape[0] != B + 1:
        raise KernelError("gated_linear_scan: sizes")
    if max(q_off, k_off) + n_heads * dim > proj.shape[1] or v_off + n_heads * vdim > proj.shape[1]:
        raise KernelError("gated_linear_scan: proj rows are too narrow")
    if state.shape[1] != n_heads * dim * vdim or not state.is_contiguous() or dim > SCAN_MAX_DIM:
        raise KernelError(f"gated_linear_scan: state rows of heads x dim x vdim, dim up to {SCAN_MAX_DIM}")
    max_chunks = 0
    if chunk > 0:
        max_chunks = -(-max_new // chunk)
        _need(sums, "sums", torch.float32); _need(decays, "decays", torch.float32)
        if max_chunks < 1 or sums.numel() < B * max_chunks * n_heads * dim * vdim \
                or decays.numel() < B * max_chunks * n_heads * dim:
            raise KernelError("gated_linear_scan: the scratch of the chunked run is too small")
    _check(_fn("recurrence_ops", "ssb_gated_linear_scan")(
        _ptr(proj), c_int(proj.stride(0)), c_int(dtype_code(proj.dtype)), c_int(q_off), c_int(k_off), c_int(v_off),
        _ptr(z), c_int(z.stride(0)), _ptr(z_bias), c_float(tau), c_float(q_scale), _ptr(state), _ptr(cu_new),
        _ptr(seq_slot), _ptr(out), c_int(out.stride(0)), c_int(B), c_int(T), c_int(n_heads), c_int(dim), c_int(vdim),
        c_int(chunk), c_int(max_chunks), _ptr(sums), _ptr(decays), c_int(1 if pdl else 0), _stream()),
        "gated_linear_scan")


SCAN_CHUNK = 128                 # tokens of a chunk when a long prompt's recurrence runs chunk-parallel (2,048 tokens of
                                 # 4 heads x 256 x 512: 1.18 ms in chunks of 64, 1.00 ms in chunks of 128, 4.4 ms in one go)
SCAN_CHUNK_MIN_NEW = 256         # shorter runs of new tokens are walked in one go
SCAN_SCRATCH_BYTES = 1 << 30     # the most the chunk sums of a step may take


def scan_chunking(n_seqs: int, max_new: int, n_heads: int, dim: int, vdim: int):
    """(chunk, floats of sums, floats of decays) for a step's recurrence; chunk 0: walk every sequence in one
    go.  The chunk grows beyond SCAN_CHUNK where the sums of all chunks would not fit the scratch bound."""
    if max_new < SCAN_CHUNK_MIN_NEW:
        return 0, 0, 0
    per = n_heads * dim * vdim
    most = SCAN_SCRATCH_BYTES // (4 * per * n_seqs)
    if most < 2:
        return 0, 0, 0
    chunk = max(SCAN_CHUNK, -(-max_new // most))
    n = -(-max_new // chunk)
    return chunk, n_seqs * n * per, n_seqs * n * n_heads * dim


def head_norm_gate(o: torch.Tensor, weight: torch.Tensor, eps: float, gate: torch.Tensor, out: torch.Tensor,
                   n_heads: int, vdim: int, pdl: bool = False, gate_kind: str = "silu") -> None:
    """out[t, h] = o[t, h] / sqrt(mean(o[t, h]^2) + eps) * weight * act(gate[t, h]): every head's ``vdim``
    outputs normalised on their own, weighted (``weight`` [vdim]: one vector for all heads; [heads x vdim]: one
    per head), then gated; ``gate_kind``: ``"silu"``, ``"sigmoid"`` or ``"none"`` (the gate as given).  ``o`` float32."""
    _need(o, "o", torch.float32, 2); _need(weight, "weight", None, 1); _need(gate, "gate", None, 2)
    _need(out, "out", gate.dtype, 2)
    T = o.shape[0]
    if gate.shape[0] != T or out.shape[0] != T or min(o.shape[1], gate.shape[1], out.shape[1]) < n_heads * vdim \
            or weight.shape[0] not in (vdim, n_heads * vdim) or not weight.is_contiguous():
        raise KernelError("head_norm_gate: sizes")
    w_stride = vdim if weight.shape[0] == n_heads * vdim and n_heads > 1 else 0
    _check(_fn("recurrence_ops", "ssb_head_norm_gate")(
        _ptr(o), c_int(o.stride(0)), _ptr(weight), c_int(dtype_code(weight.dtype)), c_int(w_stride), c_float(eps),
        _ptr(gate), c_int(gate.stride(0)), c_int(GATE_KINDS[gate_kind]), _ptr(out), c_int(out.stride(0)),
        c_int(dtype_code(out.dtype)), c_int(T), c_int(n_heads), c_int(vdim), c_int(1 if pdl else 0), _stream()),
        "head_norm_gate")


GATE_KINDS = {"silu": 0, "sigmoid": 1, "none": 2}
DECAY_KINDS = {"double_exp": 0, "exp_sigmoid": 1}
STATE_SCAN_KINDS = {"delta": 0, "bonus": 1}


def state_scan_prepare(z: torch.Tensor, z_bias: torch.Tensor, decay_kind: str, decay_scale: float, n_heads: int,
                       dim: int, proj: Optional[torch.Tensor] = None, k_off: int = 0, a_off: int = 0,
                       a_bias: Optional[torch.Tensor] = None, unit_eps: float = 0.0,
                       unit: Optional[torch.Tensor] = None, log_decay: bool = False, pdl: bool = False) -> None:
    """What a matrix-state recurrence reads besides its projections, in float32.  ``z`` [T, heads x dim] is
    overwritten with the decays: ``"double_exp"``: exp(-exp(z + z_bias)); ``"exp_sigmoid"``:
    exp(-decay_scale * sigmoid(z + z_bias)); with ``log_decay`` their logarithms instead, which is what
    ``matrix_state_scan`` wants beside float32 projections.  With ``unit`` [T, 2 x heads x dim]: its first half gets the unit keys
    u = k / sqrt(sum_head(k^2) + unit_eps), its second half a * u with a = sigmoid(proj[a_off ..] + a_bias);
    k and the removal's pre-activation are columns of ``proj``."""
    _need(z, "z", torch.float32, 2); _need(z_bias, "z_bias", torch.float32, 1)
    T, HD = z.shape[0], n_heads * dim
    if z.shape[1] < HD or z_bias.shape[0] != HD:
        raise KernelError("state_scan_prepare: sizes")
    ld = ldu = 0
    dt = F32
    if unit is not None:
        _need(unit, "unit", torch.float32, 2); _need(proj, "proj", None, 2); _need(a_bias, "a_bias", torch.float32, 1)
        if unit.shape[0] != T or unit.shape[1] < 2 * HD or proj.shape[0] != T or max(k_off, a_off) + HD > proj.shape[1] \
                or a_bias.shape[0] != HD:
            raise KernelError("state_scan_prepare: sizes of the unit keys")
        ld, ldu, dt = proj.stride(0), unit.stride(0), dtype_code(proj.dtype)
    _check(_fn("recurrence_ops", "ssb_state_scan_prepare")(
        _ptr(z), c_int(z.stride(0)), _ptr(z_bias), c_int(DECAY_KINDS[decay_kind]), c_int(1 if log_decay else 0),
        c_float(decay_scale),
        _ptr(proj if unit is not None else None), c_int(ld), c_int(dt), c_int(k_off), c_int(a_off),
        _ptr(a_bias if unit is not None else None), c_float(unit_eps), _ptr(unit), c_int(ldu), c_int(T), c_int(n_heads),
        c_int(dim), c_int(1 if pdl else 0), _stream()), "state_scan_prepare")


def matrix_state_scan(proj: torch.Tensor, r_off: int, k_off: int, v_off: int, decay: torch.Tensor, kind: str,
                      state: torch.Tensor, cu_new: torch.Tensor, seq_slot: torch.Tensor, out: torch.Tensor,
                      n_heads: int, dim: int, vdim: int, unit: Optional[torch.Tensor] = None,
                      bonus: Optional[torch.Tensor] = None, pdl: bool = False) -> None:
    """Per sequence and head over the sequence's new tokens in order, S [dim, vdim] float32 read from and left in
    ``state[slot]`` (kept there as [heads, vdim, dim]: a value column's rows together).  ``"delta"``: S = diag(w) S - (a u)(u^T S) + k v^T, out = S^T r, with ``unit`` = [u | a u] as
    ``state_scan_prepare`` leaves it; ``"bonus"``: out = (S + diag(bonus) k v^T)^T r, then S = diag(w) S + k v^T.
    ``decay`` [T, heads x dim] float32 holds w, or log w if ``proj`` is float32 (that path takes the exponential in
    double and carries the state of a step's tokens in double); r, k (heads x dim) and v (heads x vdim) are columns of ``proj``."""
    _need(proj, "proj", None, 2); _need(decay, "decay", torch.float32, 2); _need(state, "state", torch.float32, 2)
    _need(out, "out", torch.float32, 2); _need(cu_new, "cu_new", torch.int32, 1); _need(seq_slot, "seq_slot", torch.int32, 1)
    T, B, HD = proj.shape[0], seq_slot.shape[0], n_heads * dim
    if decay.shape[0] != T or out.shape[0] != T or decay.shape[1] < HD or out.shape[1] < n_heads * vdim \
            or cu_new.shape[0] != B + 1 or max(r_off, k_off) + HD > proj.shape[1] or v_off + n_heads * vdim > proj.shape[1]:
        raise KernelError("matrix_state_scan: sizes")
    if state.shape[1] != HD * vdim or not state.is_contiguous() or dim > SCAN_MAX_DIM:
        raise KernelError(f"matrix_state_scan: state rows of heads x dim x vdim, dim up to {SCAN_MAX_DIM}")
    if kind == "delta":
        _need(unit, "unit", torch.float32, 2)
        if unit.shape[0] != T or unit.shape[1] < 2 * HD:
            raise KernelError("matrix_state_scan: unit keys")
    if bonus is not None:
        _need(bonus, "bonus", torch.float32)
        if bonus.numel() != HD or not bonus.is_contiguous():
            raise KernelError("matrix_state_scan: one bonus per head and key channel")
    _check(_fn("recurrence_ops", "ssb_matrix_state_scan")(
        _ptr(proj), c_int(proj.stride(0)), c_int(dtype_code(proj.dtype)), c_int(r_off), c_int(k_off), c_int(v_off),
        _ptr(decay), c_int(decay.stride(0)), c_int(STATE_SCAN_KINDS[kind]), _ptr(unit),
        c_int(unit.stride(0) if unit is not None else 0), _ptr(bonus), _ptr(state), _ptr(cu_new), _ptr(seq_slot),
        _ptr(out), c_int(out.stride(0)), c_int(B), c_int(n_heads), c_int(dim), c_int(vdim), c_int(1 if pdl else 0),
        _stream()), "matrix_state_scan")


GATED_UNIT_SPLIT_MIN_NEW = 64    # runs of new tokens from which the vector-state recurrence takes its chunked form
GATED_UNIT_CHUNK = 128


def matrix_state_step(proj: torch.Tensor, r_off: int, k_off: int, v_off: int, g_off: int, a_off: int, z: torch.Tensor,
                      z_bias: torch.Tensor, decay_kind: str, decay_scale: float, a_bias: Optional[torch.Tensor],
                      unit_eps: float, kind: str, bonus: Optional[torch.Tensor], state: torch.Tensor, cu_new: torch.Tensor,
                      seq_slot: torch.Tensor, norm_w: torch.Tensor, eps: float, gate_kind: str, y: torch.Tensor,
                      n_heads: int, dim: int, vdim: int, pdl: bool = False) -> None:
    """A decode step of a matrix-state recurrence in one launch, for bfloat16 projections and one new token a sequence:
    ``state_scan_prepare`` (``z`` is read, not overwritten), ``matrix_state_scan`` and ``head_norm_gate`` of every
    sequence's token; ``y`` gets the normed and gated head outputs."""
    _need(proj, "proj", torch.bfloat16, 2); _need(z, "z", torch.float32, 2); _need(z_bias, "z_bias", torch.float32, 1)
    _need(state, "state", torch.float32, 2); _need(y, "y", torch.bfloat16, 2); _need(norm_w, "norm_w", torch.bfloat16, 1)
    _need(cu_new, "cu_new", torch.int32, 1); _need(seq_slot, "seq_slot", torch.int32, 1)
    T, B, HD = proj.shape[0], seq_slot.shape[0], n_heads * dim
    if z.shape[0] != T or y.shape[0] != T or z.shape[1] < HD or y.shape[1] < n_heads * vdim or z_bias.shape[0] != HD \
            or cu_new.shape[0] != B + 1 or max(r_off, k_off) + HD > proj.shape[1] \
            or max(v_off, g_off) + n_heads * vdim > proj.shape[1] or norm_w.shape[0] not in (vdim, n_heads * vdim):
        raise KernelError("matrix_state_step: sizes")
    if state.shape[1] != HD * vdim or not state.is_contiguous() or dim > SCAN_MAX_DIM:
        raise KernelError(f"matrix_state_step: state rows of heads x dim x vdim, dim up to {SCAN_MAX_DIM}")
    if kind == "delta":
        _need(a_bias, "a_bias", torch.float32, 1)
        if a_bias.shape[0] != HD or a_off + HD > proj.shape[1]:
            raise KernelError("matrix_state_step: the removal's pre-activation and bias")
    if bonus is not None:
        _need(bonus, "bonus", torch.float32)
        if bonus.numel() != HD or not bonus.is_contiguous():
            raise KernelError("matrix_state_step: one bonus per head and key channel")
    w_stride = vdim if norm_w.shape[0] == n_heads * vdim and n_heads > 1 else 0
    _check(_fn("recurrence_ops", "ssb_matrix_state_step")(
        _ptr(proj), c_int(proj.stride(0)), c_int(r_off), c_int(k_off), c_int(v_off), c_int(g_off), c_int(a_off), _ptr(z),
        c_int(z.stride(0)), _ptr(z_bias), c_int(DECAY_KINDS[decay_kind]), c_float(decay_scale), _ptr(a_bias),
        c_float(unit_eps), c_int(STATE_SCAN_KINDS[kind]), _ptr(bonus), _ptr(state), _ptr(cu_new), _ptr(seq_slot),
        _ptr(norm_w), c_int(w_stride), c_float(eps), c_int(GATE_KINDS[gate_kind]), _ptr(y), c_int(y.stride(0)), c_int(B),
        c_int(n_heads), c_int(dim), c_int(vdim), c_int(1 if pdl else 0), _stream()), "matrix_state_step")


def gated_unit_scan_scratch(n_seqs: int, max_new: int, channels: int) -> int:
    """float32 elements of scratch the chunked walk needs: (A, B) per sequence, chunk and channel."""
    return 2 * n_seqs * (-(-max_new // GATED_UNIT_CHUNK)) * channels


def gated_unit_scan(gates: torch.Tensor, bias_r: torch.Tensor, bias_i: torch.Tensor, rate: torch.Tensor,
                    u: torch.Tensor, y: torch.Tensor, y_bias: Optional[torch.Tensor], state: torch.Tensor,
                    cu_new: torch.Tensor, seq_slot: torch.Tensor, out: torch.Tensor, block: int,
                    max_new: int = 1, scratch: Optional[torch.Tensor] = None, pdl: bool = False) -> None:
    """Per sequence and channel over the new tokens: r = sigmoid(g_r + bias_r), i = sigmoid(g_i + bias_i),
    a = exp(rate * r), S = a S + sqrt(1 - a^2) i u, out = S * gelu_tanh(y + y_bias).  ``gates`` [T, 2 x channels]
    float32 holds [g_r | g_i] per block of ``block`` channels; S float32 lives in ``state[slot]``.  Runs of
    ``GATED_UNIT_SPLIT_MIN_NEW`` and more new tokens in bfloat16, given ``scratch`` (float32,
    ``gated_unit_scan_scratch`` elements), take several launches: what does not depend on the state for all tokens at
    once (written over ``gates``, and the activation of ``y`` over ``y``), then the walk over chunks of 128 tokens in
    parallel (each chunk from zero, the chunks' ends in order, each chunk from its true start)."""
    _need(gates, "gates", torch.float32, 2); _need(u, "u", None, 2); _need(y, "y", u.dtype, 2); _need(out, "out", u.dtype, 2)
    _need(state, "state", torch.float32, 2)
    C = state.shape[1]
    for name, v in (("bias_r", bias_r), ("bias_i", bias_i), ("rate", rate)) + ((("y_bias", y_bias),) if y_bias is not None else ()):
        _need(v, name, torch.float32, 1)
        if v.shape[0] != C:
            raise KernelError(f"gated_unit_scan: {name} must have one value per channel")
    T, B = u.shape[0], seq_slot.shape[0]
    if gates.shape[0] != T or gates.shape[1] < 2 * C or min(u.shape[1], y.shape[1], out.shape[1]) < C or y.shape[0] != T \
            or out.shape[0] != T or cu_new.shape[0] != B + 1 or C % block or not state.is_contiguous():
        raise KernelError("gated_unit_scan: sizes")
    if u.dtype == torch.bfloat16 and max_new >= GATED_UNIT_SPLIT_MIN_NEW and scratch is not None:
        _need(scratch, "scratch", torch.float32)
        if scratch.numel() < gated_unit_scan_scratch(B, max_new, C):
            raise KernelError("gated_unit_scan: the scratch of the chunked walk is too small")
        _check(_fn("recurrence_ops", "ssb_gated_unit_scan_split")(
            _ptr(gates), c_int(gates.stride(0)), _ptr(bias_r), _ptr(bias_i), _ptr(rate), _ptr(u), c_int(u.stride(0)),
            _ptr(y), c_int(y.stride(0)), _ptr(y_bias), _ptr(state), _ptr(cu_new), _ptr(seq_slot), _ptr(out),
            c_int(out.stride(0)), c_int(B), c_int(T), c_int(max_new), c_int(C), c_int(block), _ptr(scratch),
            c_int(1 if pdl else 0), _stream()), "gated_unit_scan_split")
        return
    _check(_fn("recurrence_ops", "ssb_gated_unit_scan")(
        _ptr(gates), c_int(gates.stride(0)), _ptr(bias_r), _ptr(bias_i), _ptr(rate), _ptr(u), c_int(u.stride(0)),
        _ptr(y), c_int(y.stride(0)), _ptr(y_bias), _ptr(state), _ptr(cu_new), _ptr(seq_slot), _ptr(out),
        c_int(out.stride(0)), c_int(dtype_code(u.dtype)), c_int(B), c_int(C), c_int(block), c_int(1 if pdl else 0),
        _stream()), "gated_unit_scan")


# ---- operations along a sequence -----------------------------------------------------------
def pair_embed(ids: torch.Tensor, table: torch.Tensor, pair: torch.Tensor, prev: torch.Tensor, cu_new: torch.Tensor,
               seq_slot: torch.Tensor, out: torch.Tensor, max_new: int, buckets: int, mul_prev: int, mul_cur: int,
               pdl: bool = False) -> None:
    """out[t] = table[id_t] + pair[(id_(t-1) * mul_prev + id_t * mul_cur) mod buckets], row ``buckets`` of ``pair`` for
    a sequence's first token; ``prev`` [slots, 1] int32 keeps a sequence's last token id + 1 (0: none yet)."""
    _need(ids, "ids", torch.int32, 1); _need(table, "table", None, 2); _need(pair, "pair", table.dtype, 2)
    _need(prev, "prev", torch.int32, 2); _need(out, "out", torch.float32, 2)
    if not (table.is_contiguous() and pair.is_contiguous() and out.is_contiguous() and prev.is_contiguous()) \
            or prev.shape[1] != 1 or pair.shape[0] != buckets + 1 or pair.shape[1] != table.shape[1] \
            or tuple(out.shape) != (ids.shape[0], table.shape[1]) or cu_new.shape[0] != seq_slot.shape[0] + 1:
        raise KernelError("pair_embed: shapes")
    _check(_fn("sequence_ops", "ssb_pair_embed")(
        _ptr(ids), _ptr(table), _ptr(pair), c_int(dtype_code(table.dtype)), _ptr(prev), _ptr(cu_new), _ptr(seq_slot),
        _ptr(out), c_int(seq_slot.shape[0]), c_int(max_new), c_int(table.shape[1]), c_int(table.shape[0]),
        c_int(buckets), c_longlong(mul_prev), c_longlong(mul_cur), c_int(1 if pdl else 0), _stream()), "pair_embed")


def dynamic_tanh(x: torch.Tensor, alpha: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, out: torch.Tensor,
                 rows: Optional[torch.Tensor] = None, pdl: bool = False) -> None:
    """out[r] = tanh(alpha * x[rows[r] or r]) * weight + bias; x, alpha [1], weight and bias float32."""
    _need(x, "x", torch.float32, 2); _need(alpha, "alpha", torch.float32, 1); _need(weight, "weight", torch.float32, 1)
    _need(bias, "bias", torch.float32, 1); _need(out, "out", None, 2)
    n, width = out.shape[0], x.shape[1]
    if not (x.is_contiguous() and out.is_contiguous()) or out.shape[1] != width or weight.shape[0] != width \
            or bias.shape[0] != width or alpha.numel() != 1 or (rows is None and x.shape[0] != n):
        raise KernelError("dynamic_tanh: shapes")
    if rows is not None:
        _need(rows, "rows", torch.int32, 1)
        if rows.shape[0] != n:
            raise KernelError("dynamic_tanh: one output row per gathered row")
    _check(_fn("sequence_ops", "ssb_dynamic_tanh")(
        _ptr(x), _ptr(rows), _ptr(alpha), _ptr(weight), _ptr(bias), _ptr(out), c_int(dtype_code(out.dtype)), c_int(n),
        c_int(width), c_int(1 if pdl else 0), _stream()), "dynamic_tanh")


def shift_mix(h: torch.Tensor, mu: torch.Tensor, last: torch.Tensor, cu_new: torch.Tensor, seq_slot: torch.Tensor,
              out: torch.Tensor, max_new: int, pdl: bool = False) -> None:
    """out[s, t] = h[t] + (h[t-1] - h[t]) * mu[s] for every mix s; the row before a step's first token is
    ``last[slot]`` (float32; zeros at a sequence's start), which afterwards holds the step's last h."""
    _need(h, "h", None, 2); _need(mu, "mu", torch.float32, 2); _need(last, "last", torch.float32, 2)
    _need(out, "out", h.dtype, 3)
    T, W = h.shape
    if tuple(out.shape) != (mu.shape[0], T, W) or mu.shape[1] != W or last.shape[1] != W or not mu.is_contiguous() \
            or not last.is_contiguous() or cu_new.shape[0] != seq_slot.shape[0] + 1:
        raise KernelError("shift_mix: shapes")
    _check(_fn("sequence_ops", "ssb_shift_mix")(
        _ptr(h), c_int(h.stride(0)), c_int(dtype_code(h.dtype)), _ptr(mu), c_int(mu.shape[0]), _ptr(last), _ptr(cu_new),
        _ptr(seq_slot), _ptr(out), c_longlong(T * W), c_int(W), c_int(seq_slot.shape[0]), c_int(max_new), c_int(W),
        c_int(1 if pdl else 0), _stream()), "shift_mix")


def tanh_norm_shift(x: torch.Tensor, norm1, norm2, mu: torch.Tensor, last: torch.Tensor, cu_new: torch.Tensor,
                    seq_slot: torch.Tensor, mixed: torch.Tensor, second: Optional[torch.Tensor], max_new: int,
                    pdl: bool = False) -> None:
    """``dynamic_tanh`` with ``norm1 = (alpha, weight, bias)`` followed by ``shift_mix`` with the one mix ``mu`` into
    ``mixed``, and ``dynamic_tanh`` with ``norm2`` of the same rows into ``second`` (None: no second norm), in one
    pass over ``x``."""
    _need(x, "x", torch.float32, 2); _need(mu, "mu", torch.float32); _need(last, "last", torch.float32, 2)
    _need(mixed, "mixed", None, 2)
    T, W = x.shape
    vecs = list(norm1) + (list(norm2) if second is not None else [])
    for v in vecs:
        _need(v, "norm tensor", torch.float32, 1)
    if not x.is_contiguous() or tuple(mixed.shape) != (T, W) or not mixed.is_contiguous() or mu.numel() != W \
            or last.shape[1] != W or not last.is_contiguous() or cu_new.shape[0] != seq_slot.shape[0] + 1 \
            or any(v.numel() != (1 if i % 3 == 0 else W) for i, v in enumerate(vecs)):
        raise KernelError("tanh_norm_shift: shapes")
    if second is not None:
        _need(second, "second", mixed.dtype, 2)
        if tuple(second.shape) != (T, W) or not second.is_contiguous():
            raise KernelError("tanh_norm_shift: shapes of the second norm's output")
    a2, w2, b2 = norm2 if second is not None else (None, None, None)
    _check(_fn("sequence_ops", "ssb_tanh_norm_shift")(
        _ptr(x), _ptr(norm1[0]), _ptr(norm1[1]), _ptr(norm1[2]), _ptr(a2), _ptr(w2), _ptr(b2), _ptr(mu), _ptr(last),
        _ptr(cu_new), _ptr(seq_slot), _ptr(mixed), _ptr(second), c_int(dtype_code(mixed.dtype)), c_int(seq_slot.shape[0]),
        c_int(max_new), c_int(W), c_int(1 if pdl else 0), _stream()), "tanh_norm_shift")


CONV_MAX_TAPS = 16


def causal_conv(x: torch.Tensor, x_bias: Optional[torch.Tensor], weight: torch.Tensor, bias: Optional[torch.Tensor],
                tail: torch.Tensor, cu_new: torch.Tensor, seq_slot: torch.Tensor, out: torch.Tensor, max_new: int,
                pdl: bool = False, pass_cols: int = 0) -> None:
    """out[t, c] = bias[c] + sum_j weight[c, j] * in[t - (taps - 1 - j), c] with in = x + x_bias; inputs from before
    the step are ``tail[slot]`` ([taps - 1, channels] float32, oldest first), which is brought up to date.  The
    ``pass_cols`` columns behind the channels are copied to ``out`` as they are."""
    _need(x, "x", None, 2); _need(weight, "weight", torch.float32, 2); _need(tail, "tail", torch.float32, 2)
    _need(out, "out", x.dtype, 2)
    C, taps = weight.shape
    if taps > CONV_MAX_TAPS or x.shape[1] < C + pass_cols or out.shape[1] < C + pass_cols or out.shape[0] != x.shape[0] \
            or tail.shape[1] != (taps - 1) * C or not weight.is_contiguous() \
            or not tail.is_contiguous() or cu_new.shape[0] != seq_slot.shape[0] + 1:
        raise KernelError(f"causal_conv: shapes (up to {CONV_MAX_TAPS} taps)")
    for v in (x_bias, bias):
        if v is not None:
            _need(v, "bias", torch.float32, 1)
            if v.shape[0] != C:
                raise KernelError("causal_conv: one bias per channel")
    _check(_fn("sequence_ops", "ssb_causal_conv")(
        _ptr(x), c_int(x.stride(0)), c_int(dtype_code(x.dtype)), _ptr(x_bias), _ptr(weight), _ptr(bias), _ptr(tail),
        _ptr(cu_new), _ptr(seq_slot), _ptr(out), c_int(out.stride(0)), c_int(seq_slot.shape[0]), c_int(max_new),
        c_int(C), c_int(taps), c_int(pass_cols), c_int(1 if pdl else 0), _stream()), "causal_conv")


def concat_cast(x: torch.Tensor, x0: torch.Tensor, act: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                pdl: bool = False) -> None:
    """act[t] = [x[t] | x0[t]] in ``act``'s type; out[t] = bias (zeros without one)."""
    _need(x, "x", torch.float32, 2); _need(x0, "x0", torch.float32, 2); _need(act, "act", None, 2)
    _need(out, "out", torch.float32, 2)
    T, W = x.shape
    if tuple(x0.shape) != (T, W) or tuple(act.shape) != (T, 2 * W) or tuple(out.shape) != (T, W) \
            or not (x.is_contiguous() and x0.is_contiguous() and act.is_contiguous() and out.is_contiguous()):
        raise KernelError("concat_cast: shapes")
    if bias is not None:
        _need(bias, "bias", torch.float32, 1)
        if bias.shape[0] != W:
            raise KernelError("concat_cast: bias")
    _check(_fn("sequence_ops", "ssb_concat_cast")(
        _ptr(x), _ptr(x0), _ptr(act), c_int(dtype_code(act.dtype)), _ptr(bias), _ptr(out), c_int(T), c_int(W),
        c_int(1 if pdl else 0), _stream()), "concat_cast")


def rms_pair_add(residual: torch.Tensor, a: torch.Tensor, wa: torch.Tensor, b: torch.Tensor, wb: torch.Tensor,
                 eps: float, scale: float, pdl: bool = False) -> None:
    """residual[t] += scale * (a[t] / rms(a[t]) * wa + b[t] / rms(b[t]) * wb), all float32."""
    for name, v in (("residual", residual), ("a", a), ("b", b)):
        _need(v, name, torch.float32, 2)
        if v.shape != residual.shape or not v.is_contiguous():
            raise KernelError("rms_pair_add: shapes")
    _need(wa, "wa", torch.float32, 1); _need(wb, "wb", torch.float32, 1)
    if wa.shape[0] != residual.shape[1] or wb.shape[0] != residual.shape[1]:
        raise KernelError("rms_pair_add: weights")
    _check(_fn("sequence_ops", "ssb_rms_pair_add")(
        _ptr(residual), _ptr(a), _ptr(wa), _ptr(b), _ptr(wb), c_float(eps), c_float(scale), c_int(residual.shape[0]),
        c_int(residual.shape[1]), c_int(1 if pdl else 0), _stream()), "rms_pair_add")


def tanh_(x: torch.Tensor, pdl: bool = False) -> None:
    """x <- tanh(x) in place; ``x`` [rows, n] may be a view into wider rows."""
    _need(x, "x", None, 2)
    _check(_fn("sequence_ops", "ssb_tanh")(_ptr(x), c_int(x.stride(0)), c_int(dtype_code(x.dtype)), c_int(x.shape[0]),
                                           c_int(x.shape[1]), c_int(1 if pdl else 0), _stream()), "tanh")


# ---- attention with sigmoid weights ----------------------------------------------------------
def qk_norm_rope_append(qkv: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
                        eps: float, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], pos: torch.Tensor,
                        slot: torch.Tensor, page_table: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                        n_q: int, n_kv: int, dim: int, vdim: int, rot_dims: int, page_shift: int,
                        write_cache: bool = True, pdl: bool = False) -> None:
    """Rows [q (n_q x dim) | k (n_kv x dim) | v (n_kv x vdim)]: every q and k head is divided by its root mean
    square (eps inside the root) and multiplied by the weight vector of its kind, its first ``rot_dims``
    coordinates are rotated by the token's position (i with i + rot_dims/2); q is written back in place, k and
    v go to the token's place in the paged cache."""
    _need(qkv, "qkv", None, 2); _need(pos, "pos", torch.int32, 1); _need(slot, "slot", torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2)
    T = qkv.shape[0]
    if qkv.shape[1] < n_q * dim + (n_kv * (dim + vdim) if write_cache else 0) or pos.shape[0] != T or slot.shape[0] != T:
        raise KernelError("qk_norm_rope_append: rows are too narrow, or not one position and slot per token")
    for w in (q_weight, k_weight):
        if w is not None:
            _need(w, "norm weight", torch.float32, 1)
            if w.shape[0] != dim:
                raise KernelError("qk_norm_rope_append: a norm weight per coordinate of a head")
    positions = 0
    if cos is not None and rot_dims:
        _need(cos, "cos", torch.float32, 2); _need(sin, "sin", torch.float32, 2)
        if cos.shape != sin.shape or cos.shape[1] * 2 != rot_dims or not (cos.is_contiguous() and sin.is_contiguous()):
            raise KernelError("qk_norm_rope_append: cos/sin must be [positions, rot_dims/2], contiguous")
        positions = cos.shape[0]
    else:
        cos = sin = None
    if write_cache:
        _need(k_cache, "k_cache", qkv.dtype); _need(v_cache, "v_cache", qkv.dtype)
        if not (k_cache.is_contiguous() and v_cache.is_contiguous()) or k_cache.shape[-1] != dim or v_cache.shape[-1] != vdim:
            raise KernelError("qk_norm_rope_append: cache rows of dim and vdim, contiguous")
    _check(_fn("gated_attention", "ssb_qk_norm_rope_append")(
        _ptr(qkv), c_int(qkv.stride(0)), c_int(dtype_code(qkv.dtype)), _ptr(q_weight), _ptr(k_weight), c_float(eps),
        _ptr(cos), _ptr(sin), c_int(positions), _ptr(pos), _ptr(slot), _ptr(page_table), c_int(page_table.shape[1]),
        _ptr(k_cache), _ptr(v_cache), c_int(T), c_int(n_q), c_int(n_kv), c_int(dim), c_int(vdim), c_int(rot_dims),
        c_int(page_shift), c_int(1 if write_cache else 0), c_int(1 if pdl else 0), _stream()), "qk_norm_rope_append")


SIGMOID_MMA_DIMS = {(64, 64), (64, 128), (96, 64), (96, 96), (128, 64), (128, 128)}


def sigmoid_attention_mma_ok(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor, dim: int,
                             vdim: int, page_shift: int) -> bool:
    return (q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and v_cache.dtype == torch.bfloat16
            and out.dtype == torch.bfloat16 and (dim, vdim) in SIGMOID_MMA_DIMS and page_shift == 6
            and q.stride(0) % 2 == 0 and out.stride(0) % 2 == 0 and q.data_ptr() % 4 == 0 and out.data_ptr() % 4 == 0
            and k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.data_ptr() % 16 == 0
            and v_cache.data_ptr() % 16 == 0)


def sigmoid_attention_mma(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, cu_new: torch.Tensor,
                          seq_start: torch.Tensor, seq_slot: torch.Tensor, page_table: torch.Tensor,
                          bias: Optional[torch.Tensor], out: torch.Tensor, max_new: int, n_q: int, n_kv: int, dim: int,
                          vdim: int, page_shift: int, chunk: Optional[int], window: Optional[int], scale: float,
                          split: Optional[bool] = None, pdl: bool = False) -> None:
    """``sigmoid_attention_plain`` on mma.sync for bfloat16: a block streams a sequence's pages once for a tile of
    (token, head of one kv group) rows; weights float32, entering the second product as hi + lo bfloat16.
    ``split`` (default: steps of one token a sequence): 16 rows a block, the warps share a page's keys."""
    if not sigmoid_attention_mma_ok(q, k_cache, v_cache, out, dim, vdim, page_shift) or n_q % n_kv:
        raise KernelError(f"sigmoid_attention_mma: dim {dim}, vdim {vdim}, heads {n_q}/{n_kv} or operands not supported")
    _need(cu_new, "cu_new", torch.int32, 1); _need(seq_start, "seq_start", torch.int32, 1); _need(seq_slot, "seq_slot", torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2)
    B = seq_slot.shape[0]
    if cu_new.shape[0] != B + 1 or seq_start.shape[0] != B or out.shape[0] != q.shape[0] or out.shape[1] < n_q * vdim \
            or q.shape[1] < n_q * dim:
        raise KernelError("sigmoid_attention_mma: shapes")
    if bias is not None:
        _need(bias, "bias", torch.float32, 1)
        if bias.shape[0] != n_q:
            raise KernelError("sigmoid_attention_mma: one bias per query head")
    if split is None:
        split = max_new * (n_q // n_kv) <= 16
    _check(_fn("gated_attention", "ssb_sigmoid_attention_mma")(
        _ptr(q), c_int(q.stride(0)), _ptr(k_cache), _ptr(v_cache), _ptr(cu_new), _ptr(seq_start), _ptr(seq_slot),
        _ptr(page_table), c_int(page_table.shape[1]), _ptr(bias), _ptr(out), c_int(out.stride(0)), c_int(B),
        c_int(max_new), c_int(n_q), c_int(n_kv), c_int(dim), c_int(vdim), c_int(page_shift),
        c_int(int(chunk) if chunk else 0), c_int(int(window) if window else 0), c_float(scale), c_int(1 if split else 0),
        c_int(1 if pdl else 0), _stream()), "sigmoid_attention_mma")


def sigmoid_attention_plain(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, pos: torch.Tensor,
                            slot: torch.Tensor, page_table: torch.Tensor, bias: Optional[torch.Tensor],
                            out: torch.Tensor, n_q: int, n_kv: int, dim: int, vdim: int, page_shift: int,
                            chunk: Optional[int], window: Optional[int], scale: float, pdl: bool = False) -> None:
    """out[t, h] = sum_j sigmoid((q . k_j) * scale + bias[h]) v_j over the keys j <= pos of the token's slot that lie
    in the same chunk of ``chunk`` positions (counted from position 0) and within ``window``."""
    _need(q, "q", None, 2); _need(out, "out", q.dtype, 2); _need(k_cache, "k_cache", q.dtype); _need(v_cache, "v_cache", q.dtype)
    _need(pos, "pos", torch.int32, 1); _need(slot, "slot", torch.int32, 1); _need(page_table, "page_table", torch.int32, 2)
    T = q.shape[0]
    if out.shape[0] != T or out.shape[1] < n_q * vdim or q.shape[1] < n_q * dim or n_q % n_kv:
        raise KernelError("sigmoid_attention: q/out shapes")
    if bias is not None:
        _need(bias, "bias", torch.float32, 1)
        if bias.shape[0] != n_q:
            raise KernelError("sigmoid_attention: one bias per query head")
    _check(_fn("gated_attention", "ssb_sigmoid_attention_plain")(
        _ptr(q), c_int(q.stride(0)), c_int(dtype_code(q.dtype)), _ptr(k_cache), _ptr(v_cache), _ptr(pos), _ptr(slot),
        _ptr(page_table), c_int(page_table.shape[1]), _ptr(bias), _ptr(out), c_int(out.stride(0)), c_int(T), c_int(n_q),
        c_int(n_kv), c_int(dim), c_int(vdim), c_int(page_shift), c_int(int(chunk) if chunk else 0),
        c_int(int(window) if window else 0), c_float(scale), c_int(1 if pdl else 0), _stream()), "sigmoid_attention_plain")


# ---- softmax attention over a window, kept first tokens and pooled runs ---------------------------
ACTIVATIONS = {"relu_squared": 0, "gelu_tanh": 1, "silu": 2}


def activation(u: torch.Tensor, out: torch.Tensor, kind: str, scale: float = 1.0, pdl: bool = False) -> None:
    """out[t, c] = act(u[t, c]) * scale in float32 arithmetic; ``kind``: ``relu_squared`` (relu(u)^2),
    ``gelu_tanh`` (0.5 u (1 + tanh(sqrt(2/pi) (u + 0.044715 u^3)))) or ``silu``."""
    _need(u, "u", None, 2); _need(out, "out", u.dtype, 2)
    if kind not in ACTIVATIONS:
        raise KernelError(f"activation {kind!r} is not known (known: {sorted(ACTIVATIONS)})")
    if tuple(out.shape) != tuple(u.shape):
        raise KernelError("activation: out must have u's shape")
    _check(_fn("plain_ops", "ssb_activation")(
        _ptr(u), c_int(u.stride(0)), _ptr(out), c_int(out.stride(0)), c_int(dtype_code(u.dtype)), c_int(u.shape[0]),
        c_int(u.shape[1]), c_int(ACTIVATIONS[kind]), c_float(scale), c_int(1 if pdl else 0), _stream()), "activation")


QK_NORM_MODES = {None: 0, "none": 0, "head": 1, "row": 2}


def _rotation_tables(cos, sin, dims: int, what: str) -> int:
    _need(cos, what + " cos", torch.float32, 2); _need(sin, what + " sin", torch.float32, 2)
    if cos.shape != sin.shape or cos.shape[1] * 2 != dims or not (cos.is_contiguous() and sin.is_contiguous()):
        raise KernelError(f"{what}: cos/sin must be [positions, {dims}/2], contiguous")
    return cos.shape[0]


def qkv_prepare(qkv: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], norm: Optional[str],
                eps: float, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rot_dims: int, interleaved: bool,
                v_cos: Optional[torch.Tensor], v_sin: Optional[torch.Tensor], v_interleaved: bool, pos: torch.Tensor,
                slot: torch.Tensor, page_table: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, n_q: int,
                n_kv: int, dim: int, vdim: int, page_shift: int, write_cache: bool = True, pdl: bool = False,
                pooled=None, pool: int = 0, v_off: Optional[int] = None, q_temp=None, n_v: Optional[int] = None) -> None:
    """Rows [q (n_q x dim) | k (n_kv x dim) | v (n_kv x vdim)].  ``norm`` ``"head"``: every q and k head is divided
    by its root mean square (eps inside the root) and multiplied by a weight vector [dim] shared by the heads;
    ``"row"``: all heads of q (of k) together are divided by one root mean square, weights [heads x dim]; None:
    no norm.  Then the first ``rot_dims`` coordinates of every q and k head are turned by the token's position, and
    with ``v_cos``/``v_sin`` [positions, vdim / 2] every value head over its whole width.  q is written back in
    place; k and v go to the token's place in the paged cache.  ``pooled`` = (keys, values, page table) of a store
    with a row per run of ``pool`` tokens, only for steps that bring one token a sequence: the token that ends a
    run writes the run's pooled row as ``pool_rows`` would.  ``v_off``: the column where the values start (default:
    behind the keys; the keys' own column for values that are the keys as projected, before their norm).  ``q_temp`` =
    (coef, every): the queries at position p are multiplied by 1 + coef ln(floor((p + 1) / every) + 1).  ``n_v``:
    value heads, if fewer than key heads (several score maps over the same values)."""
    _need(qkv, "qkv", None, 2); _need(pos, "pos", torch.int32, 1); _need(slot, "slot", torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2)
    if norm not in QK_NORM_MODES:
        raise KernelError(f"qkv_prepare: norm {norm!r} is not known ('head', 'row' or None)")
    mode = QK_NORM_MODES[norm]
    T = qkv.shape[0]
    v_off = (n_q + n_kv) * dim if v_off is None else int(v_off)
    n_v = n_kv if n_v is None else int(n_v)
    need = max(n_q * dim + n_kv * dim, v_off + n_v * vdim) if write_cache else n_q * dim
    if qkv.shape[1] < need or v_off < 0 or pos.shape[0] != T or slot.shape[0] != T:
        raise KernelError("qkv_prepare: rows are too narrow, or not one position and slot per token")
    coef, every = (float(q_temp[0]), int(q_temp[1])) if q_temp else (0.0, 0)
    if q_temp and every < 1:
        raise KernelError("qkv_prepare: the query temperature's period must be at least one token")
    if mode:
        for w, heads in ((q_weight, n_q), (k_weight, n_kv)):
            _need(w, "norm weight", torch.float32, 1)
            if w.shape[0] != (dim if mode == 1 else heads * dim):
                raise KernelError("qkv_prepare: a norm weight per coordinate of a head ('head') or of the row ('row')")
    else:
        q_weight = k_weight = None
    positions = 0
    if cos is not None and rot_dims:
        positions = _rotation_tables(cos, sin, rot_dims, "qkv_prepare")
    else:
        cos = sin = None
        rot_dims = 0
    if v_cos is not None:
        v_positions = _rotation_tables(v_cos, v_sin, vdim, "qkv_prepare values")
        positions = v_positions if cos is None else min(positions, v_positions)
    if write_cache:
        _need(k_cache, "k_cache", qkv.dtype); _need(v_cache, "v_cache", qkv.dtype)
        if not (k_cache.is_contiguous() and v_cache.is_contiguous()) or k_cache.shape[-1] != dim or v_cache.shape[-1] != vdim:
            raise KernelError("qkv_prepare: cache rows of dim and vdim, contiguous")
    pk = pv = ptable = None
    if pool:
        if not write_cache or pooled is None:
            raise KernelError("qkv_prepare: pooling needs the cache written and the pooled store")
        pk, pv, ptable = pooled[:3]
        _need(pk, "pooled keys", qkv.dtype); _need(pv, "pooled values", qkv.dtype); _need(ptable, "pooled page table", torch.int32, 2)
        if pk.shape[-1] != dim or pv.shape[-1] != vdim or not (pk.is_contiguous() and pv.is_contiguous()):
            raise KernelError("qkv_prepare: pooled rows of dim and vdim, contiguous")
    _check(_fn("window_attention", "ssb_qkv_prepare")(
        _ptr(qkv), c_int(qkv.stride(0)), c_int(dtype_code(qkv.dtype)), _ptr(q_weight), _ptr(k_weight), c_int(mode),
        c_float(eps), _ptr(cos), _ptr(sin), c_int(rot_dims), c_int(1 if interleaved else 0), _ptr(v_cos), _ptr(v_sin),
        c_int(1 if v_interleaved else 0), c_int(positions), _ptr(pos), _ptr(slot), _ptr(page_table),
        c_int(page_table.shape[1]), _ptr(k_cache), _ptr(v_cache), c_int(T), c_int(n_q), c_int(n_kv), c_int(dim), c_int(vdim),
        c_int(page_shift), c_int(1 if write_cache else 0), _ptr(pk), _ptr(pv), _ptr(ptable),
        c_int(ptable.shape[1] if ptable is not None else 0), c_int(int(pool) if pool else 0), c_int(v_off), c_int(n_v),
        c_float(coef), c_int(every), c_int(1 if pdl else 0), _stream()), "qkv_prepare")


def pool_rows(k_cache: torch.Tensor, v_cache: torch.Tensor, page_table: torch.Tensor, pk_cache: torch.Tensor,
              pv_cache: torch.Tensor, pool_table: torch.Tensor, cu_new: torch.Tensor, seq_start: torch.Tensor,
              seq_slot: torch.Tensor, max_new: int, n_kv: int, dim: int, vdim: int, page_shift: int, pool: int,
              pdl: bool = False) -> None:
    """For every run of ``pool`` tokens that a sequence's new tokens finish: the mean of the run's cached key rows
    (and value rows), summed in rising order in float32, into row ``run`` of the pooled store."""
    for t, n in ((k_cache, "k_cache"), (v_cache, "v_cache"), (pk_cache, "pk_cache"), (pv_cache, "pv_cache")):
        _need(t, n, k_cache.dtype)
        if not t.is_contiguous():
            raise KernelError(f"pool_rows: {n} must be contiguous")
    _need(cu_new, "cu_new", torch.int32, 1); _need(seq_start, "seq_start", torch.int32, 1); _need(seq_slot, "seq_slot", torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2); _need(pool_table, "pool_table", torch.int32, 2)
    B = seq_slot.shape[0]
    if cu_new.shape[0] != B + 1 or seq_start.shape[0] != B or k_cache.shape[-1] != dim or pk_cache.shape[-1] != dim \
            or v_cache.shape[-1] != vdim or pv_cache.shape[-1] != vdim or pool < 1:
        raise KernelError("pool_rows: shapes")
    _check(_fn("window_attention", "ssb_pool_rows")(
        _ptr(k_cache), _ptr(v_cache), _ptr(page_table), c_int(page_table.shape[1]), _ptr(pk_cache), _ptr(pv_cache),
        _ptr(pool_table), c_int(pool_table.shape[1]), c_int(dtype_code(k_cache.dtype)), _ptr(cu_new), _ptr(seq_start),
        _ptr(seq_slot), c_int(B), c_int(max_new), c_int(n_kv), c_int(dim), c_int(vdim), c_int(page_shift), c_int(pool),
        c_int(1 if pdl else 0), _stream()), "pool_rows")


def _window_attention_args(q, k_cache, v_cache, page_table, pooled, out, n_q, n_kv, dim, vdim, window, keep_first, pool,
                           sinks, v_cos, v_sin, what, v_share=1, gate=None):
    _need(q, "q", None, 2); _need(out, "out", q.dtype, 2); _need(k_cache, "k_cache", q.dtype); _need(v_cache, "v_cache", q.dtype)
    _need(page_table, "page_table", torch.int32, 2)
    T = q.shape[0]
    if out.shape[0] != T or out.shape[1] < n_q * vdim or q.shape[1] < n_q * dim or n_q % n_kv \
            or k_cache.shape[-1] != dim or v_cache.shape[-1] != vdim:
        raise KernelError(f"{what}: q/out/cache shapes")
    if v_share < 1 or n_kv % v_share or (pool and v_share > 1):
        raise KernelError(f"{what}: {n_kv} key heads do not share values {v_share} at a time (and not with pooled runs)")
    if gate is not None:
        _need(gate, "gate", q.dtype, 2)
        if gate.shape[0] != T or gate.shape[1] < n_q:
            raise KernelError(f"{what}: one gate per token and head")
    pk = pv = ptable = None
    if pool:
        if not window:
            raise KernelError(f"{what}: pooled runs stand for what has left a window: a window is needed")
        pk, pv, ptable = pooled
        _need(pk, "pooled keys", q.dtype); _need(pv, "pooled values", q.dtype); _need(ptable, "pooled page table", torch.int32, 2)
        if pk.shape[-1] != dim or pv.shape[-1] != vdim:
            raise KernelError(f"{what}: pooled rows of dim and vdim")
    if sinks is not None and not isinstance(sinks, bool):
        _need(sinks, "sinks", torch.float32, 1)
        if sinks.shape[0] != n_q:
            raise KernelError(f"{what}: one sink per query head")
    positions = 0
    if v_cos is not None:
        positions = _rotation_tables(v_cos, v_sin, vdim, what + " values")
    return pk, pv, ptable, positions


def window_attention_plain(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, page_table: torch.Tensor,
                           pooled, pos: torch.Tensor, slot: torch.Tensor, out: torch.Tensor, n_q: int, n_kv: int, dim: int,
                           vdim: int, page_shift: int, window: Optional[int], keep_first: int, pool: int, scale: float,
                           softcap: Optional[float], sinks, v_cos: Optional[torch.Tensor], v_sin: Optional[torch.Tensor],
                           v_interleaved: bool, out_scale: float = 1.0, pdl: bool = False, v_share: int = 1,
                           gate: Optional[torch.Tensor] = None) -> None:
    """Softmax attention of every token over its slot's cache: the keys j with pos - window < j <= pos, the first
    ``keep_first`` tokens, and (``pool`` > 0, ``pooled`` = (keys, values, page table) of the pooled store) the
    pooled row of every run of ``pool`` tokens that ends at or before pos - window.  Scores times ``scale``, then
    ``softcap * tanh(s / softcap)`` if a cap is given.  ``sinks``: None, True (a sink of score 0 in the
    denominator) or one float per query head.  With ``v_cos``/``v_sin`` the head's sum is turned back by the
    token's position.  ``out`` is multiplied by ``out_scale``.  ``v_share``: that many key heads in a row read one
    value head (the value store has n_kv / v_share heads).  ``gate`` [tokens, >= n_q]: head h of token t is
    multiplied by sigmoid(gate[t, h])."""
    pk, pv, ptable, positions = _window_attention_args(q, k_cache, v_cache, page_table, pooled, out, n_q, n_kv, dim, vdim,
                                                       window, keep_first, pool, sinks, v_cos, v_sin, "window_attention",
                                                       v_share, gate)
    _need(pos, "pos", torch.int32, 1); _need(slot, "slot", torch.int32, 1)
    zero_sink = sinks is True
    _check(_fn("window_attention", "ssb_window_attention_plain")(
        _ptr(q), c_int(q.stride(0)), c_int(dtype_code(q.dtype)), _ptr(k_cache), _ptr(v_cache), _ptr(page_table),
        c_int(page_table.shape[1]), _ptr(pk), _ptr(pv), _ptr(ptable), c_int(ptable.shape[1] if ptable is not None else 0),
        _ptr(pos), _ptr(slot), _ptr(out), c_int(out.stride(0)), c_int(q.shape[0]), c_int(n_q), c_int(n_kv), c_int(dim),
        c_int(vdim), c_int(page_shift), c_int(int(window) if window else 0), c_int(int(keep_first or 0)),
        c_int(int(pool or 0)), c_float(scale), c_float(float(softcap) if softcap else 0.0),
        _ptr(None if (sinks is None or isinstance(sinks, bool)) else sinks), c_int(1 if zero_sink else 0), _ptr(v_cos),
        _ptr(v_sin), c_int(1 if v_interleaved else 0), c_int(positions), c_float(out_scale), c_int(v_share), _ptr(gate),
        c_int(gate.stride(0) if gate is not None else 0), c_int(1 if pdl else 0), _stream()), "window_attention_plain")


def window_attention_mma_ok(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, pooled, out: torch.Tensor,
                            dim: int, vdim: int, page_shift: int) -> bool:
    ok = (q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and v_cache.dtype == torch.bfloat16
          and out.dtype == torch.bfloat16 and dim % 8 == 0 and vdim % 8 == 0 and 0 < dim <= 128 and 0 < vdim <= 128
          and page_shift == 6 and q.stride(0) % 2 == 0 and out.stride(0) % 2 == 0 and q.data_ptr() % 4 == 0
          and out.data_ptr() % 4 == 0 and k_cache.is_contiguous() and v_cache.is_contiguous()
          and k_cache.data_ptr() % 16 == 0 and v_cache.data_ptr() % 16 == 0)
    if ok and pooled is not None:
        ok = all(t.dtype == torch.bfloat16 and t.is_contiguous() and t.data_ptr() % 16 == 0 for t in pooled[:2])
    return ok


def window_attention_mma(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, page_table: torch.Tensor, pooled,
                         cu_new: torch.Tensor, seq_start: torch.Tensor, seq_slot: torch.Tensor, out: torch.Tensor,
                         max_new: int, n_q: int, n_kv: int, dim: int, vdim: int, page_shift: int, window: Optional[int],
                         keep_first: int, pool: int, scale: float, softcap: Optional[float], sinks,
                         v_cos: Optional[torch.Tensor], v_sin: Optional[torch.Tensor], v_interleaved: bool,
                         out_scale: float = 1.0, split: Optional[bool] = None, pdl: bool = False, v_share: int = 1,
                         gate: Optional[torch.Tensor] = None) -> None:
    """``window_attention_plain`` on mma.sync for bfloat16: a block streams what a tile of (token, head of one kv
    group) rows can see once (pooled rows, kept first tokens, the window's pages); scores, weights and sums
    float32, the weights entering the second product as hi + lo bfloat16.  ``split`` (default: steps of one
    token a sequence): 16 rows a block, the warps share a page's keys."""
    if not window_attention_mma_ok(q, k_cache, v_cache, pooled if pool else None, out, dim, vdim, page_shift):
        raise KernelError(f"window_attention_mma: dim {dim}, vdim {vdim} or operands not supported")
    pk, pv, ptable, positions = _window_attention_args(q, k_cache, v_cache, page_table, pooled, out, n_q, n_kv, dim, vdim,
                                                       window, keep_first, pool, sinks, v_cos, v_sin, "window_attention_mma",
                                                       v_share, gate)
    _need(cu_new, "cu_new", torch.int32, 1); _need(seq_start, "seq_start", torch.int32, 1); _need(seq_slot, "seq_slot", torch.int32, 1)
    B = seq_slot.shape[0]
    if cu_new.shape[0] != B + 1 or seq_start.shape[0] != B:
        raise KernelError("window_attention_mma: one start and slot per sequence, and one more row offset")
    if split is None:
        split = max_new * (n_q // n_kv) <= 16
    _check(_fn("window_attention_mma", "ssb_window_attention_mma")(
        _ptr(q), c_int(q.stride(0)), _ptr(k_cache), _ptr(v_cache), _ptr(page_table), c_int(page_table.shape[1]), _ptr(pk),
        _ptr(pv), _ptr(ptable), c_int(ptable.shape[1] if ptable is not None else 0), _ptr(cu_new), _ptr(seq_start),
        _ptr(seq_slot), _ptr(out), c_int(out.stride(0)), c_int(B), c_int(max_new), c_int(n_q), c_int(n_kv), c_int(dim),
        c_int(vdim), c_int(page_shift), c_int(int(window) if window else 0), c_int(int(keep_first or 0)),
        c_int(int(pool or 0)), c_float(scale), c_float(float(softcap) if softcap else 0.0),
        _ptr(None if (sinks is None or isinstance(sinks, bool)) else sinks), c_int(1 if sinks is True else 0), _ptr(v_cos),
        _ptr(v_sin), c_int(1 if v_interleaved else 0), c_int(positions), c_float(out_scale), c_int(v_share), _ptr(gate),
        c_int(gate.stride(0) if gate is not None else 0), c_int(1 if split else 0), c_int(1 if pdl else 0), _stream()),
        "window_attention_mma")


def map_difference(maps: torch.Tensor, out: torch.Tensor, n_heads: int, n_kv: int, vdim: int, lam: float, eps: float,
                   mult: float, pdl: bool = False) -> None:
    """Two score maps per head over the same values, the second taken off the first: with a1, a2 the maps' results of
    head h, o = a1 - lam a2 and out[t, h] = o / sqrt(mean(o^2) + eps) * mult.  ``maps`` [tokens, 2 n_heads vdim] in
    the order [kv head][map][head of the group][vdim]; ``out`` [tokens, n_heads vdim], heads in their own order."""
    _need(maps, "maps", None, 2); _need(out, "out", maps.dtype, 2)
    T = maps.shape[0]
    if out.shape[0] != T or maps.shape[1] < 2 * n_heads * vdim or out.shape[1] < n_heads * vdim or n_heads % n_kv:
        raise KernelError("map_difference: shapes")
    _check(_fn("window_attention", "ssb_map_difference")(
        _ptr(maps), c_int(maps.stride(0)), _ptr(out), c_int(out.stride(0)), c_int(dtype_code(maps.dtype)), c_int(T),
        c_int(n_heads), c_int(n_kv), c_int(vdim), c_float(lam), c_float(eps), c_float(mult), c_int(1 if pdl else 0),
        _stream()), "map_difference")


# ---- minGRU --------------------------------------------------------------------------------
MINGRU_TILED_MIN_NEW = 64
MINGRU_CHUNKED_MIN_NEW = 256
MINGRU_CHUNK = 64           # tokens a block of the chunked scan takes


def mingru_scan_scratch(n_seqs: int, max_new: int, width: int) -> int:
    """float32 elements of scratch the chunked scan needs for runs of up to ``max_new`` tokens."""
    return n_seqs * (2 * (-(-max_new // MINGRU_CHUNK)) + 1) * width


def mingru_scan(proj: torch.Tensor, z_bias: Optional[torch.Tensor], x_bias: Optional[torch.Tensor], state: torch.Tensor,
                cu_new: torch.Tensor, seq_slot: torch.Tensor, out: torch.Tensor, width: int, out_scale: float = 1.0,
                tiled: bool = False, pdl: bool = False, max_new: int = 0, scratch: Optional[torch.Tensor] = None) -> None:
    """Rows of ``proj`` are [zp | up | gp], ``width`` columns each.  Per channel, over every sequence's new tokens
    from and into its row of ``state`` [slots, width] (float32): z = sigmoid(zp + bz), cand = up + bu + 1/2 where
    up + bu >= 0 and sigmoid(up + bu) below, S <- (1 - z) S + z cand, out = out_scale * S * silu(gp).  ``tiled``:
    the form that spreads a run of tokens over the warps of a block (even width and strides); with ``scratch``
    (``mingru_scan_scratch`` floats) and ``max_new``, every 64 tokens of a run get a block of their own."""
    _need(proj, "proj", None, 2); _need(out, "out", None, 2); _need(state, "state", torch.float32, 2)
    _need(cu_new, "cu_new", torch.int32, 1); _need(seq_slot, "seq_slot", torch.int32, 1)
    B = seq_slot.shape[0]
    if proj.shape[1] < 3 * width or out.shape[1] < width or out.shape[0] != proj.shape[0] or state.shape[1] != width \
            or cu_new.shape[0] != B + 1 or not state.is_contiguous():
        raise KernelError("mingru_scan: shapes")
    for b in (z_bias, x_bias):
        if b is not None:
            _need(b, "bias", torch.float32, 1)
            if b.shape[0] != width:
                raise KernelError("mingru_scan: a bias per channel")
    if tiled and (width % 2 or proj.stride(0) % 2 or out.stride(0) % 2 or proj.data_ptr() % 8 or out.data_ptr() % 8):
        tiled = False
    form = 1 if tiled else 0
    if tiled and scratch is not None and max_new > 0:
        _need(scratch, "scratch", torch.float32, 1)
        if scratch.numel() < mingru_scan_scratch(B, max_new, width) or scratch.data_ptr() % 8:
            raise KernelError("mingru_scan: scratch is too small")
        form = 2
    _check(_fn("mingru_ops", "ssb_mingru_scan")(
        _ptr(proj), c_int(proj.stride(0)), c_int(dtype_code(proj.dtype)), _ptr(z_bias), _ptr(x_bias), _ptr(state),
        _ptr(cu_new), _ptr(seq_slot), _ptr(out), c_int(out.stride(0)), c_int(dtype_code(out.dtype)), c_int(B), c_int(width),
        c_float(out_scale), c_int(form), _ptr(scratch if form == 2 else None), c_int(max_new), c_int(1 if pdl else 0),
        _stream()), "mingru_scan")


# ---- experts -----------------------------------------------------------------------------
def route_table(token_ids: torch.Tensor, table: torch.Tensor, n_experts: int, expert_of: torch.Tensor,
                pair_weight: torch.Tensor, pdl: bool = False) -> None:
    """expert_of[t, k] = table[token_ids[t], k], pair_weight[t, k] = 1 / top."""
    _need(token_ids, "token_ids", torch.int32, 1); _need(table, "table", torch.int32, 2)
    _need(expert_of, "expert_of", torch.int32, 2); _need(pair_weight, "pair_weight", torch.float32, 2)
    T, top = token_ids.shape[0], table.shape[1]
    if tuple(expert_of.shape) != (T, top) or tuple(pair_weight.shape) != (T, top) or not (
            table.is_contiguous() and expert_of.is_contiguous() and pair_weight.is_contiguous()):
        raise KernelError("route_table: expert_of and pair_weight must be [tokens, top], contiguous")
    _check(_fn("expert_ops", "ssb_route_table")(
        _ptr(token_ids), _ptr(table), c_int(table.shape[0]), c_int(top), c_int(n_experts), _ptr(expert_of),
        _ptr(pair_weight), c_int(T), c_int(1 if pdl else 0), _stream()), "route_table")


def route_sigmoid_groups(logits: torch.Tensor, n_experts: int, correction: Optional[torch.Tensor], n_groups: int, keep: int,
                         scale: float, expert_of: torch.Tensor, pair_weight: torch.Tensor, extra_col: Optional[int] = None,
                         extra_out: Optional[torch.Tensor] = None, pdl: bool = False) -> None:
    """Per token, from float32 router logits [tokens, >= n_experts]: s = sigmoid(z); the ``top`` experts with the
    largest s + correction among the experts of the ``keep`` best of ``n_groups`` equal groups of neighbours (a
    group's score: the sum of its two largest s + correction); pair_weight = s * scale of the chosen.  ``extra_col``:
    a further column whose sigmoid per token goes to ``extra_out``."""
    _need(logits, "logits", torch.float32, 2)
    _need(expert_of, "expert_of", torch.int32, 2); _need(pair_weight, "pair_weight", torch.float32, 2)
    T, top = logits.shape[0], expert_of.shape[1]
    if logits.shape[1] < n_experts or tuple(expert_of.shape) != (T, top) or tuple(pair_weight.shape) != (T, top) \
            or not (expert_of.is_contiguous() and pair_weight.is_contiguous()):
        raise KernelError("route_sigmoid_groups: logits [tokens, >= experts]; expert_of and pair_weight [tokens, top], contiguous")
    if correction is not None:
        _need(correction, "correction", torch.float32, 1)
        if correction.shape[0] != n_experts:
            raise KernelError("route_sigmoid_groups: one correction per expert")
    if extra_col is not None:
        _need(extra_out, "extra_out", torch.float32, 1)
        if not 0 <= extra_col < logits.shape[1] or extra_out.shape[0] != T:
            raise KernelError("route_sigmoid_groups: the extra column lies in the logits' rows, its result is one number per token")
    _check(_fn("expert_ops", "ssb_route_sigmoid_groups")(
        _ptr(logits), c_int(logits.stride(0)), _ptr(correction), c_int(T), c_int(n_experts), c_int(n_groups), c_int(keep),
        c_int(top), c_float(scale), c_int(-1 if extra_col is None else extra_col), _ptr(expert_of), _ptr(pair_weight),
        _ptr(extra_out if extra_col is not None else None), c_int(1 if pdl else 0), _stream()), "route_sigmoid_groups")


def expert_tiles_bound(n_pairs: int, n_experts: int, tile_rows: int) -> int:
    """The most row tiles ``n_pairs`` pairs spread over ``n_experts`` groups can make."""
    return n_pairs // tile_rows + min(n_experts, n_pairs)


def group_by_expert(expert_of: torch.Tensor, n_experts: int, tile_rows: int, offsets: torch.Tensor,
                    order: torch.Tensor, tile_expert: torch.Tensor, tile_row0: torch.Tensor, meta: torch.Tensor,
                    pdl: bool = False) -> None:
    """Sort the (token, choice) pairs by expert: ``order[r]`` is the pair at sorted row r, ``offsets[e]`` the
    first row of expert e, and (tile_expert, tile_row0)[i < meta[0]] the row tiles of ``tile_rows`` rows."""
    for t, n in ((expert_of, "expert_of"), (offsets, "offsets"), (order, "order"), (tile_expert, "tile_expert"),
                 (tile_row0, "tile_row0"), (meta, "meta")):
        _need(t, n, torch.int32)
        if not t.is_contiguous():
            raise KernelError(f"group_by_expert: {n} must be contiguous")
    P = expert_of.numel()
    bound = expert_tiles_bound(P, n_experts, tile_rows)
    if offsets.numel() < n_experts + 1 or order.numel() < P or tile_expert.numel() < bound or tile_row0.numel() < bound:
        raise KernelError("group_by_expert: outputs are too small")
    _check(_fn("expert_ops", "ssb_group_by_expert")(
        _ptr(expert_of), c_int(P), c_int(n_experts), c_int(tile_rows), _ptr(offsets), _ptr(order),
        _ptr(tile_expert), _ptr(tile_row0), _ptr(meta), c_int(1 if pdl else 0), _stream()), "group_by_expert")


def grouped_gemm_plain(a: torch.Tensor, a_index: Optional[torch.Tensor], a_div: int, w: torch.Tensor,
                       out: torch.Tensor, c_index: Optional[torch.Tensor], offsets: torch.Tensor,
                       tile_expert: torch.Tensor, tile_row0: torch.Tensor, meta: torch.Tensor, max_tiles: int) -> None:
    """For sorted row r of expert e: out[c_index[r] or r] = w[e] @ a[a_index[r] // a_div or r]; ``w`` [E, N, K].
    Tiles of 64 rows (``group_by_expert`` with tile_rows = 64)."""
    _need(a, "a", None, 2); _need(w, "w", a.dtype, 3); _need(out, "out", None, 2)
    E, N, K = w.shape
    if a.shape[1] != K or out.shape[1] != N or not w.is_contiguous():
        raise KernelError(f"grouped_gemm: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    _check(_fn("expert_ops", "ssb_grouped_gemm_plain")(
        _ptr(a), c_int(a.stride(0)), _ptr(a_index), c_int(a_div), _ptr(w), c_int(K), c_longlong(N * K),
        c_int(dtype_code(a.dtype)), _ptr(out), c_int(out.stride(0)), _ptr(c_index), c_int(dtype_code(out.dtype)),
        _ptr(offsets), _ptr(tile_expert), _ptr(tile_row0), _ptr(meta), c_int(max_tiles), c_int(N), c_int(K),
        _stream()), "grouped_gemm_plain")


def expert_combine(residual: torch.Tensor, y: torch.Tensor, pair_weight: torch.Tensor, top: int,
                   pdl: bool = False) -> None:
    """residual[t] += sum_k pair_weight[t, k] * y[t * top + k], in the order of k."""
    _need(residual, "residual", torch.float32, 2); _need(y, "y", None, 2); _need(pair_weight, "pair_weight", torch.float32, 2)
    T, width = residual.shape
    if tuple(y.shape) != (T * top, width) or tuple(pair_weight.shape) != (T, top) or not pair_weight.is_contiguous():
        raise KernelError("expert_combine: y [tokens * top, width], pair_weight [tokens, top]")
    _check(_fn("expert_ops", "ssb_expert_combine")(
        _ptr(residual), c_int(residual.stride(0)), _ptr(y), c_int(y.stride(0)), c_int(dtype_code(y.dtype)),
        _ptr(pair_weight), c_int(top), c_int(T), c_int(width), c_int(1 if pdl else 0), _stream()), "expert_combine")


# ---- sampling --------------------------------------------------------------------------
def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    _need(logits, "logits", torch.float32, 2); _need(out, "out", torch.int32, 1)
    if out.shape[0] != logits.shape[0]:
        raise KernelError("argmax: one output per row")
    _check(_fn("sampling", "ssb_argmax")(
        _ptr(logits), c_longlong(logits.stride(0)), c_int(logits.shape[0]), c_int(logits.shape[1]),
        _ptr(out), _stream()), "argmax")


def target_nll(logits: torch.Tensor, targets: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = -log softmax(logits[r])[targets[r]] (float32; NaN for a target outside the vocabulary)."""
    _need(logits, "logits", torch.float32, 2); _need(targets, "targets", torch.int32, 1)
    _need(out, "out", torch.float32, 1)
    if targets.shape[0] != logits.shape[0] or out.shape[0] != logits.shape[0]:
        raise KernelError("target_nll: one target and one output per row")
    _check(_fn("sampling", "ssb_target_nll")(
        _ptr(logits), c_longlong(logits.stride(0)), c_int(logits.shape[0]), c_int(logits.shape[1]),
        _ptr(targets), _ptr(out), _stream()), "target_nll")


def sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float,
           slots: Optional[torch.Tensor], rng_state: torch.Tensor, out: torch.Tensor,
           drawn_u: Optional[torch.Tensor] = None) -> None:
    _need(logits, "logits", torch.float32, 2); _need(out, "out", torch.int32, 1)
    _need(rng_state, "rng_state", torch.int64, 1)
    n = logits.shape[0]
    if slots is not None:
        _need(slots, "slots", torch.int32, 1)
        if slots.shape[0] != n:
            raise KernelError("sample: one slot per row")
    elif rng_state.shape[0] < n:
        raise KernelError("sample: one generator state per row")
    if drawn_u is not None:
        _need(drawn_u, "drawn_u", torch.float32, 1)
    if out.shape[0] != n:
        raise KernelError("sample: one output per row")
    _check(_fn("sampling", "ssb_sample")(
        _ptr(logits), c_longlong(logits.stride(0)), c_int(n), c_int(logits.shape[1]),
        c_float(temperature), c_int(int(top_k)), c_float(top_p), _ptr(slots), _ptr(rng_state), _ptr(out),
        _ptr(drawn_u), _stream()), "sample")


# ---- decode kernels --------------------------------------------------------------------
SG_STORE, SG_ACCUMULATE, SG_SWIGLU = 0, 1, 2


def skinny_gemm_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the skinny GEMM takes these operands (else the plain kernels do)."""
    return (w.dtype == torch.bfloat16 and x.dtype == torch.bfloat16 and x.shape[0] <= 64 and w.shape[1] % 8 == 0
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0)


def skinny_gemm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int = SG_STORE,
                pdl: bool = False) -> None:
    """out = x @ w^T for up to 64 rows on mma.sync (the decode projection for shapes the tcgen05
    kernels refuse).  ``pdl``: launch as a programmatic dependent of the kernel before it on the
    stream (its weights are prefetched while that kernel ends).  mode: store, add into float32
    ``out``, or SwiGLU over rows of ``w`` that come as [8 gate | 8 up] per 16 (``out`` is [rows, N/2])."""
    _need(x, "x", torch.bfloat16, 2); _need(w, "w", torch.bfloat16, 2); _need(out, "out", None, 2)
    B, K = x.shape
    N = w.shape[0]
    n_out = N // 2 if mode == SG_SWIGLU else N
    if w.shape[1] != K or tuple(out.shape) != (B, n_out):
        raise KernelError(f"skinny_gemm: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    _check(_fn("decode_ops", "ssb_skinny_gemm")(
        _ptr(x), c_int(x.stride(0)), _ptr(w), c_int(w.stride(0)), _ptr(out), c_int(out.stride(0)),
        c_int(dtype_code(out.dtype)), c_int(B), c_int(N), c_int(K), c_int(mode), c_int(1 if pdl else 0),
        _stream()), "skinny_gemm")


def attention_decode_scratch(n_seqs: int, n_q: int, n_kv: int, head_dim: int, n_splits: int):
    """(float32 elements of scratch, int32 counters) one launch needs; counters start at zero."""
    lib = load_library("decode_ops")
    lib.ssb_attention_decode_scratch_floats.restype = c_longlong
    return (int(lib.ssb_attention_decode_scratch_floats(c_int(n_seqs), c_int(n_q), c_int(head_dim),
                                                        c_int(n_splits))),
            int(lib.ssb_attention_decode_counters(c_int(n_seqs), c_int(n_q), c_int(n_kv))))


def _attention_decode_checks(q, k_cache, v_cache, pos, slot, page_table, out, n_q, n_kv, head_dim, cos, sin, what):
    _need(q, "q", torch.bfloat16, 2); _need(out, "out", torch.bfloat16, 2)
    _need(k_cache, "k_cache", torch.bfloat16); _need(v_cache, "v_cache", torch.bfloat16)
    _need(pos, "pos", torch.int32, 1); _need(slot, "slot", torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2)
    B = q.shape[0]
    if pos.shape[0] != B or slot.shape[0] != B or out.shape[0] != B:
        raise KernelError(f"{what}: one position, slot and output row per sequence")
    if cos is not None:
        _need(cos, "cos", torch.float32, 2); _need(sin, "sin", torch.float32, 2)
        if cos.shape != sin.shape or cos.shape[1] * 2 != head_dim or not (cos.is_contiguous() and sin.is_contiguous()):
            raise KernelError(f"{what}: cos/sin must be [positions, head_dim/2], contiguous")
        if head_dim not in (32, 64, 128, 256) or q.shape[1] < (n_q + 2 * n_kv) * head_dim:
            raise KernelError(f"{what}: fused rotation needs head_dim 32/64/128/256 and [q|k|v] rows")
    return B


def attention_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, pos: torch.Tensor,
                     slot: torch.Tensor, page_table: torch.Tensor, out: torch.Tensor, n_q: int, n_kv: int,
                     head_dim: int, page_shift: int, window: Optional[int], scale: float, n_splits: int,
                     scratch: Optional[torch.Tensor], counters: Optional[torch.Tensor],
                     pdl: bool = False, cos: Optional[torch.Tensor] = None,
                     sin: Optional[torch.Tensor] = None) -> None:
    """One query token per sequence (row) over its cached keys, the keys split ``n_splits`` ways, on
    CUDA cores (any head size up to 256).  With ``cos``/``sin`` ([positions, head_dim/2] float32) the
    rows of ``q`` are the raw fused projection [q | k | v]: queries and the token's key are rotated
    inside the kernel, and key and value are appended to the cache (no separate rope/append launch)."""
    B = _attention_decode_checks(q, k_cache, v_cache, pos, slot, page_table, out, n_q, n_kv, head_dim, cos, sin,
                                 "attention_decode")
    if n_splits > 64:
        raise KernelError("attention_decode: at most 64 splits")
    if n_splits > 1:
        need_f, need_c = attention_decode_scratch(B, n_q, n_kv, head_dim, n_splits)
        _need(scratch, "scratch", torch.float32); _need(counters, "counters", torch.int32)
        if scratch.numel() < need_f or counters.numel() < need_c:
            raise KernelError(f"attention_decode: scratch of {need_f} floats and {need_c} counters needed")
    _check(_fn("decode_ops", "ssb_attention_decode")(
        _ptr(q), c_int(q.stride(0)), _ptr(k_cache), _ptr(v_cache), _ptr(pos), _ptr(slot), _ptr(page_table),
        c_int(page_table.shape[1]), _ptr(out), c_int(out.stride(0)), c_int(B), c_int(n_q), c_int(n_kv),
        c_int(head_dim), c_int(page_shift), c_int(int(window) if window else 0), c_float(scale),
        c_int(n_splits), _ptr(scratch), _ptr(counters), c_int(1 if pdl else 0), _ptr(cos), _ptr(sin),
        _stream()), "attention_decode")


def attention_decode_chunked_ok(n_seqs: int, n_q: int, n_kv: int, head_dim: int, ldq: int, page_shift: int) -> bool:
    """Whether the tensor-core decode attention takes this case (head sizes 64 and 128, at most 16
    query heads per kv head, 64-token pages, at most 1,024 sequences)."""
    return bool(_fn("decode_ops", "ssb_attention_decode_chunked_ok")(
        c_int(n_seqs), c_int(n_q), c_int(n_kv), c_int(head_dim), c_int(ldq), c_int(page_shift)))


_chunked_blocks = {}


def attention_decode_chunked_blocks(n_seqs: int, n_q: int, n_kv: int, head_dim: int, fused: bool) -> int:
    """Blocks of the tensor-core decode attention that the current device holds at once for this case
    (the size of its persistent grid)."""
    key = (torch.cuda.current_device(), min(n_seqs, 1024) > 64, min(n_seqs, 1024) > 256, n_seqs > 512, n_q, n_kv,
           head_dim, bool(fused))
    if key not in _chunked_blocks:
        lib = load_library("decode_ops")
        lib.ssb_attention_decode_chunked_blocks.restype = c_longlong
        _chunked_blocks[key] = int(lib.ssb_attention_decode_chunked_blocks(
            c_int(n_seqs), c_int(n_q), c_int(n_kv), c_int(head_dim), c_int(1 if fused else 0)))
    return _chunked_blocks[key]


_chunked_clusters = {}


def attention_decode_chunked_clusters(n_q: int, n_kv: int, head_dim: int, fused: bool, cluster: int) -> int:
    """Thread-block clusters of ``cluster`` (2, 4 or 8) blocks of the tensor-core decode attention that the
    current device holds at once (0: it cannot place one)."""
    key = (torch.cuda.current_device(), n_q, n_kv, head_dim, bool(fused), cluster)
    if key not in _chunked_clusters:
        _chunked_clusters[key] = int(_fn("decode_ops", "ssb_attention_decode_chunked_clusters")(
            c_int(n_q), c_int(n_kv), c_int(head_dim), c_int(1 if fused else 0), c_int(cluster)))
    return _chunked_clusters[key]


def attention_decode_chunked_scratch(n_seqs: int, n_q: int, n_kv: int, head_dim: int, max_chunks: int):
    """(float32 elements of scratch, int32 counters) a launch needs; counters start at zero."""
    lib = load_library("decode_ops")
    lib.ssb_attention_decode_chunked_scratch_floats.restype = c_longlong
    return (int(lib.ssb_attention_decode_chunked_scratch_floats(c_int(n_seqs), c_int(n_q), c_int(head_dim),
                                                                c_int(max_chunks))), n_seqs * n_kv)


def attention_decode_chunked(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, pos: torch.Tensor,
                             slot: torch.Tensor, page_table: torch.Tensor, out: torch.Tensor, n_q: int, n_kv: int,
                             head_dim: int, page_shift: int, window: Optional[int], scale: float,
                             chunk_pages: int, max_chunks: int, scratch: Optional[torch.Tensor],
                             counters: Optional[torch.Tensor], pdl: bool = False,
                             cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None,
                             cluster: int = 0) -> None:
    """``attention_decode`` on the tensor cores with a persistent grid: every sequence's pages are cut
    into chunks of about ``chunk_pages`` pages (a cut that depends on the sequence alone), a work item
    is (sequence, chunk, kv head), and as many blocks as the device holds at once walk the items.
    ``chunk_pages`` 0: the kernel sizes the chunks itself so that the items about fill those blocks.
    ``max_chunks`` bounds the chunks of one sequence and sizes the scratch
    (:func:`attention_decode_chunked_scratch`); a longer sequence gets ``max_chunks`` larger chunks.
    Pages come in through the TMA unit with bounded waits (:func:`check_device_errors`).
    ``cluster`` 2, 4 or 8: every sequence is cut into that many chunks, the chunks of a (sequence, kv
    head) are the blocks of a thread-block cluster and merge through its shared memory (no scratch);
    for small batches whose blocks all fit the device at once."""
    global _tc_unchecked
    B = _attention_decode_checks(q, k_cache, v_cache, pos, slot, page_table, out, n_q, n_kv, head_dim, cos, sin,
                                 "attention_decode_chunked")
    if chunk_pages < 0 or max_chunks < 1:
        raise KernelError("attention_decode_chunked: chunk_pages must not be negative, max_chunks at least 1")
    if cluster not in (0, 2, 4, 8):
        raise KernelError("attention_decode_chunked: a cluster holds 2, 4 or 8 chunks")
    if max_chunks > 1 and not cluster:
        need_f, need_c = attention_decode_chunked_scratch(B, n_q, n_kv, head_dim, max_chunks)
        _need(scratch, "scratch", torch.float32); _need(counters, "counters", torch.int32)
        if scratch.numel() < need_f or counters.numel() < need_c:
            raise KernelError(f"attention_decode_chunked: scratch of {need_f} floats and {need_c} counters needed")
    _check(_fn("decode_ops", "ssb_attention_decode_chunked")(
        _ptr(q), c_int(q.stride(0)), _ptr(k_cache), _ptr(v_cache), _ptr(pos), _ptr(slot), _ptr(page_table),
        c_int(page_table.shape[1]), _ptr(out), c_int(out.stride(0)), c_int(B), c_int(n_q), c_int(n_kv),
        c_int(head_dim), c_int(page_shift), c_int(int(window) if window else 0), c_float(scale),
        c_int(chunk_pages), c_int(max_chunks), _ptr(scratch), _ptr(counters), c_int(1 if pdl else 0), _ptr(cos),
        _ptr(sin), c_longlong(k_cache.numel() // head_dim), _ptr(tc_error_word(q.device)), c_int(cluster),
        _stream()), "attention_decode_chunked")
    _tc_unchecked += 1


# ---- prefill GEMM on tcgen05 ---------------------------------------------------------------
TC_STORE, TC_ACCUMULATE, TC_SWIGLU = 0, 1, 2
TC_TILE_PAIR = 512        # ``tile_n`` that asks for 256 x 256 tiles on SM pairs (tcgen05 cta_group::2)
_TC_ERRORS = {1: "the TMA producer", 2: "the MMA issuer", 3: "the epilogue"}
_tc_error_words = {}
_tc_unchecked = 0      # tcgen05 launches since the error words were last read


_after_error = []       # weak references to callables that put scratch back in order after a failed launch


def after_device_error(method) -> None:
    """Register a bound method to be called when a bounded wait is found to have run out, before the
    error is raised: a launch that gave up may have left arrival counters and zero-between-uses
    scratch in a state that later launches would trip over.  Held weakly."""
    import weakref
    _after_error.append(weakref.WeakMethod(method))


def _raise_wait_ran_out(code: int):
    for ref in list(_after_error):
        fn = ref()
        if fn is None:
            _after_error.remove(ref)
        else:
            fn()
    raise KernelError(f"tcgen05 kernel: a bounded wait ran out in {_TC_ERRORS.get(code, code)}; "
                      "the result of that launch is invalid")


def bounded_wait_launches() -> int:
    """Launches since the last look at the error words of kernels whose waits are bounded."""
    return _tc_unchecked


def note_bounded_wait_launches(n: int) -> None:
    """A captured graph that holds ``n`` such launches was replayed: they ran without passing
    through this module, so the error word counts as unread."""
    global _tc_unchecked
    _tc_unchecked += int(n)


def tc_error_word(device) -> torch.Tensor:
    """The device word in which tcgen05 kernels record a wait that ran out (zero = all well)."""
    key = torch.device(device)
    if key not in _tc_error_words:
        _tc_error_words[key] = torch.zeros(1, dtype=torch.int32, device=key)
    return _tc_error_words[key]


def check_device_errors(device=None) -> None:
    """Raise if a kernel recorded a bounded wait that ran out.  Reads one word per device, and
    only if a kernel that could have set it was launched since the last look."""
    global _tc_unchecked
    if not _tc_unchecked:
        return
    _tc_unchecked = 0
    for dev, word in list(_tc_error_words.items()):
        if device is not None and torch.device(device) != dev:
            continue
        code = int(word.item())
        if code:
            word.zero_()
            _raise_wait_ran_out(code)


_fetch_buffers = {}


def fetch_with_errors(values: torch.Tensor) -> list:
    """The int32 values of a device tensor as a host list, read in the same wait as the device's
    error word: one synchronisation a step instead of two.  Raises like ``check_device_errors``."""
    global _tc_unchecked
    dev = values.device
    n = values.numel()
    word = _tc_error_words.get(dev) if _tc_unchecked else None
    buf = _fetch_buffers.get(dev)
    if buf is None or buf.numel() < n + 1:
        buf = _fetch_buffers[dev] = torch.empty(max(n + 1, 4097), dtype=torch.int32, pin_memory=True)
    buf[:n].copy_(values.view(-1), non_blocking=True)
    if word is not None:
        buf[n:n + 1].copy_(word, non_blocking=True)
    torch.cuda.current_stream(dev).synchronize()
    out = buf[:n].tolist()
    if word is not None:
        _tc_unchecked = 0
        code = int(buf[n])
        if code:
            word.zero_()
            _raise_wait_ran_out(code)
    return out


class Fetch:
    """An int32 device tensor on its way to the host (:func:`start_fetch`)."""

    __slots__ = ("buf", "n", "event", "with_word", "device")


_fetch_ring = {}


def start_fetch(values: torch.Tensor) -> Fetch:
    """Begin copying the int32 ``values`` (and the device's error word, if a kernel that could set it
    ran since the last look) to pinned host memory on the current stream; nothing waits.  The ring
    holds four copies in flight per device."""
    global _tc_unchecked
    dev = values.device
    n = values.numel()
    ring = _fetch_ring.setdefault(dev, {"bufs": [None] * 4, "turn": 0})
    i = ring["turn"]
    ring["turn"] = (i + 1) % 4
    buf = ring["bufs"][i]
    if buf is None or buf.numel() < n + 1:
        buf = ring["bufs"][i] = torch.empty(max(n + 1, 4097), dtype=torch.int32, pin_memory=True)
    f = Fetch()
    f.buf, f.n, f.device = buf, n, dev
    f.with_word = bool(_tc_unchecked) and dev in _tc_error_words
    buf[:n].copy_(values.view(-1), non_blocking=True)
    if f.with_word:
        buf[n:n + 1].copy_(_tc_error_words[dev], non_blocking=True)
        _tc_unchecked = 0
    f.event = torch.cuda.Event()
    f.event.record()
    return f


def finish_fetch(f: Fetch) -> list:
    """Wait for the copy and return the values; raises like ``check_device_errors``."""
    f.event.synchronize()
    out = f.buf[:f.n].tolist()
    if f.with_word:
        code = int(f.buf[f.n])
        if code:
            _tc_error_words[f.device].zero_()
            _raise_wait_ran_out(code)
    return out


def tc_wait_probe(device="cuda:0") -> None:
    """Launch a block whose only wait can never be satisfied: after about a second it gives up and
    records that in the device's error word, which ``check_device_errors`` then reports."""
    global _tc_unchecked
    _tc_unchecked += 1
    _check(_fn("gemm_tc", "ssb_tc_wait_probe")(_ptr(tc_error_word(device)), _stream()), "tc_wait_probe")


def gemm_tc_ok(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    """Whether the tcgen05 GEMM takes these operands (else the plain kernel does)."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[1] % 8 == 0
            and w.shape[0] % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0
            and out.stride(0) % (4 if out.dtype == torch.float32 else 8) == 0)


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int = TC_STORE,
            tile_n: Optional[int] = None, splits: int = 1) -> None:
    """out = a @ w^T on the tensor cores (tcgen05, TMA-fed).  mode: store, add into float32
    ``out``, or SwiGLU over rows of ``w`` that come as [8 gate | 8 up] per 16.  ``splits`` > 1
    (mode accumulate): every tile's K range is cut into that many parts, which add with float atomics."""
    _need(a, "a", torch.bfloat16, 2); _need(w, "w", torch.bfloat16, 2); _need(out, "out", None, 2)
    M, K = a.shape
    N = w.shape[0]
    n_out = N // 2 if mode == TC_SWIGLU else N
    if w.shape[1] != K or tuple(out.shape) != (M, n_out):
        raise KernelError(f"gemm_tc: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    if tile_n is None:
        tile_n = 256 if N > 128 else 128
    if tile_n == TC_TILE_PAIR and splits != 1:
        raise KernelError("gemm_tc: tiles on SM pairs do not split K")
    global _tc_unchecked
    _tc_unchecked += 1
    _check(_fn("gemm_tc", "ssb_gemm_tc")(
        _ptr(a), c_int(a.stride(0)), _ptr(w), c_int(w.stride(0)), _ptr(out), c_int(out.stride(0)),
        c_int(dtype_code(out.dtype)), c_int(M), c_int(N), c_int(K), c_int(mode), c_int(tile_n), c_int(splits),
        _ptr(tc_error_word(a.device)), _stream()), "gemm_tc")


def _gate_args(act, row_scale, rows: int, what: str):
    kind, limit = act if act else ("silu", 0.0)
    if kind not in GATE_KINDS_FF:
        raise KernelError(f"{what}: gate {kind!r} is not known (known: {sorted(GATE_KINDS_FF)})")
    if row_scale is not None:
        _need(row_scale, "row_scale", torch.float32, 1)
        if row_scale.shape[0] != rows:
            raise KernelError(f"{what}: one factor per row")
    return GATE_KINDS_FF[kind], float(limit)


def gemm_tc_gate(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, act=None, row_scale: Optional[torch.Tensor] = None,
                 tile_n: Optional[int] = None) -> None:
    """out = f(a @ gate^T, a @ up^T) * row_scale on the tensor cores, the inner step on the float32 sums; ``w``'s rows
    come as [8 gate | 8 up] per 16; ``act`` = (kind, limit) as in :func:`gated_activation`, None for silu(g) u."""
    _need(a, "a", torch.bfloat16, 2); _need(w, "w", torch.bfloat16, 2); _need(out, "out", torch.bfloat16, 2)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (M, N // 2):
        raise KernelError(f"gemm_tc_gate: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    kind, limit = _gate_args(act, row_scale, M, "gemm_tc_gate")
    if tile_n is None:
        tile_n = 256 if N > 128 else 128
    global _tc_unchecked
    _tc_unchecked += 1
    _check(_fn("gemm_tc", "ssb_gemm_tc_gate")(
        _ptr(a), c_int(a.stride(0)), _ptr(w), c_int(w.stride(0)), _ptr(out), c_int(out.stride(0)), c_int(M), c_int(N),
        c_int(K), c_int(kind), c_float(limit), _ptr(row_scale), c_int(tile_n), _ptr(tc_error_word(a.device)), _stream()),
        "gemm_tc_gate")


def gemm_tc_act(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, kind: str, scale: float = 1.0,
                tile_n: Optional[int] = None) -> None:
    """out (bfloat16) = act(a @ w^T) * scale on the tensor cores: the activation (a kind of ``ACTIVATIONS``) is taken
    on the float32 sums where the product finishes them, before their one rounding."""
    _need(a, "a", torch.bfloat16, 2); _need(w, "w", torch.bfloat16, 2); _need(out, "out", torch.bfloat16, 2)
    M, K = a.shape
    N = w.shape[0]
    if kind not in ACTIVATIONS:
        raise KernelError(f"activation {kind!r} is not known (known: {sorted(ACTIVATIONS)})")
    if w.shape[1] != K or tuple(out.shape) != (M, N):
        raise KernelError(f"gemm_tc_act: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    if tile_n is None:
        tile_n = 256 if N > 128 else 128
    global _tc_unchecked
    _tc_unchecked += 1
    _check(_fn("gemm_tc", "ssb_gemm_tc_act")(
        _ptr(a), c_int(a.stride(0)), _ptr(w), c_int(w.stride(0)), _ptr(out), c_int(out.stride(0)), c_int(M), c_int(N),
        c_int(K), c_int(ACTIVATIONS[kind]), c_float(scale), c_int(tile_n), _ptr(tc_error_word(a.device)), _stream()),
        "gemm_tc_act")


def gemm_tc_rope_append(a: torch.Tensor, w: torch.Tensor, q_out: torch.Tensor, cos: torch.Tensor,
                        sin: torch.Tensor, pos: torch.Tensor, slot: torch.Tensor, page_table: torch.Tensor,
                        k_cache: torch.Tensor, v_cache: torch.Tensor, n_q: int, n_kv: int, head_dim: int,
                        page_shift: int, tile_n: int = 256) -> None:
    """The fused query/key/value projection of packed tokens (``w`` = [q; k; v] rows) on tcgen05
    whose epilogue rotates q and k from the float32 sums, writes q (bfloat16) into ``q_out`` and
    k and v into the paged cache entry; nothing else is written.  head_dim 64 or 128, full-width
    rotation, tables [positions, head_dim/2] float32.  Rows with a negative slot are skipped."""
    _need(a, "a", torch.bfloat16, 2); _need(w, "w", torch.bfloat16, 2); _need(q_out, "q_out", torch.bfloat16, 2)
    _need(pos, "pos", torch.int32, 1); _need(slot, "slot", torch.int32, 1); _need(page_table, "page_table", torch.int32, 2)
    _need(cos, "cos", torch.float32, 2); _need(sin, "sin", torch.float32, 2)
    _need(k_cache, "k_cache", torch.bfloat16); _need(v_cache, "v_cache", torch.bfloat16)
    M, K = a.shape
    if head_dim not in (64, 128):
        raise KernelError(f"gemm_tc_rope_append: head_dim {head_dim} (64 or 128)")
    if tuple(w.shape) != ((n_q + 2 * n_kv) * head_dim, K) or q_out.shape[0] != M or q_out.shape[1] < n_q * head_dim:
        raise KernelError(f"gemm_tc_rope_append: shapes a{tuple(a.shape)} w{tuple(w.shape)} q_out{tuple(q_out.shape)}")
    if pos.shape[0] != M or slot.shape[0] != M:
        raise KernelError("gemm_tc_rope_append: one position and one slot per row")
    if cos.shape != sin.shape or cos.shape[1] * 2 != head_dim or not (cos.is_contiguous() and sin.is_contiguous()):
        raise KernelError("gemm_tc_rope_append: cos/sin must be [positions, head_dim/2], contiguous")
    if not k_cache.is_contiguous() or not v_cache.is_contiguous() or k_cache.shape != v_cache.shape \
            or tuple(k_cache.shape[1:]) != (n_kv, 1 << page_shift, head_dim):
        raise KernelError(f"gemm_tc_rope_append: cache shape {tuple(k_cache.shape)}")
    if not gemm_tc_ok(a, w, q_out):
        raise KernelError("gemm_tc_rope_append: operands must be 16-byte aligned with strides in multiples of 8")
    global _tc_unchecked
    _tc_unchecked += 1
    _check(_fn("gemm_tc", "ssb_gemm_tc_rope_append")(
        _ptr(a), c_int(a.stride(0)), _ptr(w), c_int(w.stride(0)), _ptr(q_out), c_int(q_out.stride(0)), c_int(M),
        c_int(K), _ptr(pos), _ptr(slot), _ptr(page_table), c_int(page_table.shape[1]), _ptr(k_cache), _ptr(v_cache),
        _ptr(cos), _ptr(sin), c_int(n_q), c_int(n_kv), c_int(head_dim), c_int(page_shift), c_int(tile_n),
        _ptr(tc_error_word(a.device)), _stream()), "gemm_tc_rope_append")


# ---- prefill attention -------------------------------------------------------------------------
def attention_prefill_ok(q: torch.Tensor, head_dim: int) -> bool:
    return q.dtype == torch.bfloat16 and head_dim in (64, 128) and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0


def attention_prefill(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, cu_new: torch.Tensor,
                      seq_start: torch.Tensor, seq_slot: torch.Tensor, page_table: torch.Tensor,
                      out: torch.Tensor, max_new: int, n_q: int, n_kv: int, head_dim: int, page_shift: int,
                      window: Optional[int], scale: float) -> None:
    """Causal attention of each sequence's new tokens (packed rows of ``q``) over its cached keys,
    which already include the new ones."""
    _need(q, "q", torch.bfloat16, 2); _need(out, "out", torch.bfloat16, 2)
    _need(k_cache, "k_cache", torch.bfloat16); _need(v_cache, "v_cache", torch.bfloat16)
    for name, t in (("cu_new", cu_new), ("seq_start", seq_start), ("seq_slot", seq_slot)):
        _need(t, name, torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2)
    n_seqs = seq_slot.shape[0]
    if cu_new.shape[0] != n_seqs + 1 or seq_start.shape[0] != n_seqs:
        raise KernelError("attention_prefill: cu_new has one more entry than there are sequences")
    if out.shape[0] != q.shape[0] or out.shape[1] < n_q * head_dim or q.shape[1] < n_q * head_dim:
        raise KernelError("attention_prefill: q/out shapes")
    _check(_fn("prefill_attention", "ssb_attention_prefill")(
        _ptr(q), c_int(q.stride(0)), _ptr(k_cache), _ptr(v_cache), _ptr(cu_new), _ptr(seq_start),
        _ptr(seq_slot), _ptr(page_table), c_int(page_table.shape[1]), _ptr(out), c_int(out.stride(0)),
        c_int(n_seqs), c_int(max_new), c_int(n_q), c_int(n_kv), c_int(head_dim), c_int(page_shift),
        c_int(int(window) if window else 0), c_float(scale), _stream()), "attention_prefill")


def attention_prefill_tc_ok(q: torch.Tensor, out: torch.Tensor, head_dim: int, page_shift: int) -> bool:
    return (q.dtype == torch.bfloat16 and head_dim in (64, 128) and page_shift == 6 and q.stride(0) % 8 == 0
            and out.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0)


def attention_prefill_tc(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, cu_new: torch.Tensor,
                         seq_start: torch.Tensor, seq_slot: torch.Tensor, page_table: torch.Tensor,
                         out: torch.Tensor, max_new: int, n_q: int, n_kv: int, head_dim: int, page_shift: int,
                         window: Optional[int], scale: float) -> None:
    """``attention_prefill`` on tcgen05: scores and probabilities in tensor memory, pages by TMA.
    head_dim 64 or 128 and 64-token pages only.  A wait that runs out sets the device's error word
    (``check_device_errors``)."""
    _need(q, "q", torch.bfloat16, 2); _need(out, "out", torch.bfloat16, 2)
    _need(k_cache, "k_cache", torch.bfloat16); _need(v_cache, "v_cache", torch.bfloat16)
    for name, t in (("cu_new", cu_new), ("seq_start", seq_start), ("seq_slot", seq_slot)):
        _need(t, name, torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2)
    n_seqs = seq_slot.shape[0]
    if cu_new.shape[0] != n_seqs + 1 or seq_start.shape[0] != n_seqs:
        raise KernelError("attention_prefill_tc: cu_new has one more entry than there are sequences")
    if out.shape[0] != q.shape[0] or out.shape[1] < n_q * head_dim or q.shape[1] < n_q * head_dim:
        raise KernelError("attention_prefill_tc: q/out shapes")
    if not k_cache.is_contiguous() or not v_cache.is_contiguous() or k_cache.shape != v_cache.shape \
            or tuple(k_cache.shape[1:]) != (n_kv, 1 << page_shift, head_dim):
        raise KernelError(f"attention_prefill_tc: cache shape {tuple(k_cache.shape)}")
    global _tc_unchecked
    _tc_unchecked += 1
    _check(_fn("prefill_attention_tc", "ssb_attention_prefill_tc")(
        _ptr(q), c_int(q.stride(0)), c_int(q.shape[0]), _ptr(k_cache), _ptr(v_cache), c_int(k_cache.shape[0]),
        _ptr(cu_new), _ptr(seq_start), _ptr(seq_slot), _ptr(page_table), c_int(page_table.shape[1]),
        _ptr(out), c_int(out.stride(0)), c_int(n_seqs), c_int(max_new), c_int(n_q), c_int(n_kv),
        c_int(head_dim), c_int(page_shift), c_int(int(window) if window else 0), c_float(scale),
        _ptr(tc_error_word(q.device)), _stream()), "attention_prefill_tc")


# ---- decode projections on tcgen05, weights on the M side ------------------------------------------
_sm_counts = {}


def sm_count() -> int:
    """Streaming multiprocessors of the current device (asked once per device)."""
    dev = torch.cuda.current_device()
    if dev not in _sm_counts:
        _sm_counts[dev] = torch.cuda.get_device_properties(dev).multi_processor_count
    return _sm_counts[dev]


GEMV_TC_MAX_ROWS = 128     # rows of x that gemv_tc takes (the N side of its MMA: 16, 32, 64 or 128)


def gemv_tc_splits(n: int, k: int) -> int:
    """Blocks that share the K range of one 128-row tile of W: up to two blocks per SM in all
    (every SM must pull for the memory system to be busy), at least 4 k-blocks (256 columns) each and
    at most 16 (measured on decode steps of 1B, 3B and 8B sizes: with 8 and 8 the small projections
    of a narrow model filled a third of the SMs, and its steps took 5 to 7 % longer)."""
    tiles = (n + 127) // 128
    return max(1, min(2 * sm_count() // tiles, (k // 64) // 4, 16))


def gemv_tc_scratch(rows: int, n: int, splits: int):
    lib = load_library("gemv_tc")
    lib.ssb_gemv_tc_scratch_floats.restype = c_longlong
    return (int(lib.ssb_gemv_tc_scratch_floats(c_int(rows), c_int(n), c_int(splits))),
            int(lib.ssb_gemv_tc_counters(c_int(n))))


def gemv_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int = TC_STORE, splits: int = 1,
            partials: Optional[torch.Tensor] = None, counters: Optional[torch.Tensor] = None,
            pdl: bool = False) -> None:
    """out = x @ w^T for up to 128 rows with the weights as the M side of tcgen05.mma (they stream
    once, 16 KB a stage).  ``splits`` > 1 shares the K range of a row tile among blocks: store
    and SwiGLU outputs then need ``partials``/``counters`` sized by :func:`gemv_tc_scratch`
    (counters zeroed once) and are summed in a fixed order; mode accumulate adds with float
    atomics instead (no scratch; the last bits may differ between runs)."""
    _need(x, "x", torch.bfloat16, 2); _need(w, "w", torch.bfloat16, 2); _need(out, "out", None, 2)
    B, K = x.shape
    N = w.shape[0]
    n_out = N // 2 if mode == TC_SWIGLU else N
    if w.shape[1] != K or tuple(out.shape) != (B, n_out) or B > GEMV_TC_MAX_ROWS:
        raise KernelError(f"gemv_tc: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    if splits > 1 and (mode != TC_ACCUMULATE or partials is not None):
        nf, nc = gemv_tc_scratch(B, N, splits)
        _need(partials, "partials", torch.float32); _need(counters, "counters", torch.int32)
        if partials.numel() < nf or counters.numel() < nc:
            raise KernelError(f"gemv_tc: scratch of {nf} floats and {nc} counters needed")
    global _tc_unchecked
    _tc_unchecked += 1
    _check(_fn("gemv_tc", "ssb_gemv_tc")(
        _ptr(x), c_int(x.stride(0)), _ptr(w), c_int(w.stride(0)), _ptr(out), c_int(out.stride(0)),
        c_int(dtype_code(out.dtype)), c_int(B), c_int(N), c_int(K), c_int(mode), c_int(splits),
        _ptr(partials), _ptr(counters), _ptr(tc_error_word(x.device)), c_int(1 if pdl else 0), _stream()),
        "gemv_tc")


def gemv_tc_gate(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, act=None, row_scale: Optional[torch.Tensor] = None,
                 pdl: bool = False) -> None:
    """:func:`gemm_tc_gate` for up to 128 rows, the weights on the M side of the MMA."""
    _need(x, "x", torch.bfloat16, 2); _need(w, "w", torch.bfloat16, 2); _need(out, "out", torch.bfloat16, 2)
    B, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (B, N // 2) or B > GEMV_TC_MAX_ROWS:
        raise KernelError(f"gemv_tc_gate: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    kind, limit = _gate_args(act, row_scale, B, "gemv_tc_gate")
    global _tc_unchecked
    _tc_unchecked += 1
    _check(_fn("gemv_tc", "ssb_gemv_tc_gate")(
        _ptr(x), c_int(x.stride(0)), _ptr(w), c_int(w.stride(0)), _ptr(out), c_int(out.stride(0)), c_int(B), c_int(N),
        c_int(K), c_int(kind), c_float(limit), _ptr(row_scale), _ptr(tc_error_word(x.device)), c_int(1 if pdl else 0),
        _stream()), "gemv_tc_gate")


# ---- vector element-wise kernels ------------------------------------------------------------------
def rmsnorm_vec_ok(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> bool:
    return (out.dtype == torch.bfloat16 and x.dtype == torch.float32 and x.shape[1] % 4 == 0
            and x.shape[1] <= 8192 and x.is_contiguous() and out.is_contiguous()
            and x.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0 and weight.dtype in _CODES)


def rmsnorm_vec(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
                rows: Optional[torch.Tensor] = None, pdl: bool = False) -> None:
    """As :func:`rmsnorm` with bfloat16 output, 16-byte loads and the row kept in registers."""
    _need(x, "x", torch.float32, 2); _need(weight, "weight", None, 1); _need(out, "out", torch.bfloat16, 2)
    n = out.shape[0]
    if rows is not None:
        _need(rows, "rows", torch.int32, 1)
        if rows.shape[0] != n:
            raise KernelError("rmsnorm_vec: one output row per gathered row")
    elif x.shape[0] != n:
        raise KernelError("rmsnorm_vec: x and out differ in rows")
    if x.shape[1] != out.shape[1] or weight.shape[0] != x.shape[1]:
        raise KernelError("rmsnorm_vec: widths differ")
    _check(_fn("elementwise_ops", "ssb_rmsnorm_vec")(
        _ptr(x), _ptr(rows), _ptr(weight), c_int(dtype_code(weight.dtype)), c_float(eps), _ptr(out), c_int(n),
        c_int(x.shape[1]), c_int(1 if pdl else 0), _stream()), "rmsnorm_vec")


def round_and_clear(sums: torch.Tensor, out: torch.Tensor, pdl: bool = False, act: Optional[str] = None,
                    scale: float = 1.0) -> None:
    """out (bfloat16) = sums (float32, contiguous, same shape) rounded; sums is left zero.  With ``act`` (a kind of
    ``ACTIVATIONS``): out = act(sums) * scale, taken in float32 before the rounding."""
    _need(sums, "sums", torch.float32, 2); _need(out, "out", torch.bfloat16, 2)
    if sums.shape != out.shape or not sums.is_contiguous() or sums.shape[1] % 8:
        raise KernelError(f"round_and_clear: shapes sums{tuple(sums.shape)} out{tuple(out.shape)}")
    if act is not None and act not in ACTIVATIONS:
        raise KernelError(f"activation {act!r} is not known (known: {sorted(ACTIVATIONS)})")
    _check(_fn("elementwise_ops", "ssb_round_act_clear")(
        _ptr(sums), _ptr(out), c_int(out.stride(0)), c_int(sums.shape[0]), c_int(sums.shape[1]),
        c_int(-1 if act is None else ACTIVATIONS[act]), c_float(scale), c_int(1 if pdl else 0), _stream()), "round_and_clear")


def rope_append_vec_ok(qkv: torch.Tensor, cos, head_dim: int, rotary_dim: int, write_cache: bool) -> bool:
    return (qkv.dtype == torch.bfloat16 and cos is not None and write_cache and rotary_dim == head_dim
            and head_dim % 8 == 0 and qkv.stride(0) % 8 == 0 and qkv.data_ptr() % 16 == 0)


def rope_append_vec(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, pos: torch.Tensor,
                    slot: torch.Tensor, page_table: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    n_q: int, n_kv: int, head_dim: int, page_shift: int) -> None:
    """As :func:`rope_append` for bfloat16, full-width rotation, with vector loads and stores."""
    _need(qkv, "qkv", torch.bfloat16, 2); _need(pos, "pos", torch.int32, 1); _need(slot, "slot", torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2); _need(cos, "cos", torch.float32, 2); _need(sin, "sin", torch.float32, 2)
    _need(k_cache, "k_cache", torch.bfloat16); _need(v_cache, "v_cache", torch.bfloat16)
    T = qkv.shape[0]
    if qkv.shape[1] < (n_q + 2 * n_kv) * head_dim or pos.shape[0] != T or slot.shape[0] != T:
        raise KernelError("rope_append_vec: qkv rows too narrow, or not one position and slot per token")
    if cos.shape != sin.shape or cos.shape[1] * 2 != head_dim or not (cos.is_contiguous() and sin.is_contiguous()):
        raise KernelError("rope_append_vec: cos/sin must be [positions, head_dim/2], contiguous")
    _check(_fn("elementwise_ops", "ssb_rope_append_vec")(
        _ptr(qkv), c_int(qkv.stride(0)), _ptr(cos), _ptr(sin), c_int(cos.shape[0]), _ptr(pos), _ptr(slot),
        _ptr(page_table), c_int(page_table.shape[1]), _ptr(k_cache), _ptr(v_cache), c_int(T), c_int(n_q),
        c_int(n_kv), c_int(head_dim), c_int(page_shift), _stream()), "rope_append_vec")
