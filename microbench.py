"""Times single kernels at given sizes with CUDA events (inputs larger than L2 are rotated
so that weights come from DRAM), and reports bytes or FLOPs per second.

    python microbench.py attention_decode --batch 64 --context 520
    python microbench.py linear --rows 8 --n 6144 --k 4096 [--kernel skinny|tc64|tc128|tc256]
    python microbench.py attention_prefill --tokens 2048 --seqs 1 [--kernel tc]
    python microbench.py gemm --rows 2048 --n 28672 --k 4096 --tile 256
    python microbench.py sampling --rows 64 --vocab 128256 --temperature 0.7 --top-k 40 --top-p 0.9
    python microbench.py latent_attention --tokens 2048 --heads 16 --k 576 --n 512
    python microbench.py latent_attention --tokens 1 --batch 64 --context 520 --splits 2 --heads 16 --k 576 --n 512
    python microbench.py grouped_gemm --tokens 2048 --experts 64 --top 6 --n 1408 --k 2048 --kernel swiglu
    python microbench.py gated_linear_scan --tokens 2048 --heads 4 --k 256 --n 512 --chunk 128

One JSON line per run.  It is also the small, self-ending workload that profiler captures
are taken on.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from supersonic_b200.csrc import ops  # noqa: E402

DEV = "cuda:0"


def _time(fn, iters, warmup=3):
    """Microseconds per launch: ``iters`` launches captured in one CUDA graph (so that host
    time per launch does not count) and replayed between two events."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for i in range(iters):
                fn(i)
    torch.cuda.current_stream().wait_stream(side)
    graph.replay()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    graph.replay()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / iters * 1e3


def attention_decode(args):
    n_q, n_kv, hd, B, ctx = args.heads, args.kv_heads, args.head_dim, args.batch, args.context
    pages_per = (ctx + 63) // 64 + 1
    n_pages = B * pages_per
    k = torch.randn(n_pages, n_kv, 64, hd, device=DEV).bfloat16()
    v = torch.randn(n_pages, n_kv, 64, hd, device=DEV).bfloat16()
    table = torch.randperm(n_pages).to(torch.int32).view(B, pages_per).to(DEV)
    pos = torch.full((B,), ctx - 1, dtype=torch.int32, device=DEV)
    if args.ragged:
        pos = torch.randint(0, ctx, (B,), generator=torch.Generator().manual_seed(0)).to(torch.int32).to(DEV)
    slot = torch.arange(B, dtype=torch.int32, device=DEV)
    q = torch.randn(B, (n_q + 2 * n_kv) * hd, device=DEV).bfloat16()
    out = torch.empty(B, n_q * hd, dtype=torch.bfloat16, device=DEV)
    splits = args.splits
    pages = (ctx + 63) // 64
    chunk = 0 if args.chunk_pages < 0 else (args.chunk_pages or -(-pages // splits))     # negative: the kernel decides
    max_chunks = -(-pages // chunk) if chunk else min(-(-pages // 2), 296 // n_kv + 1)
    if args.kind == 2:
        nf, nc = ops.attention_decode_chunked_scratch(B, n_q, n_kv, hd, max_chunks)
    else:
        nf, nc = ops.attention_decode_scratch(B, n_q, n_kv, hd, splits)
    scratch = torch.empty(max(nf, 1), device=DEV)
    counters = torch.zeros(max(nc, 1), dtype=torch.int32, device=DEV)
    cos = sin = None
    if args.fused:                                   # rotation and append inside, as a decode step runs it
        ang = torch.arange(ctx, device=DEV, dtype=torch.float64)[:, None] * \
            (1.0 / 10000 ** (torch.arange(hd // 2, device=DEV, dtype=torch.float64) * 2 / hd))[None, :]
        cos, sin = ang.cos().float().contiguous(), ang.sin().float().contiguous()
    if args.kind == 2:                               # the tensor-core kernel on its persistent grid
        fn = lambda i: ops.attention_decode_chunked(q, k, v, pos, slot, table, out, n_q, n_kv, hd, 6, None,
                                                    1 / math.sqrt(hd), chunk, max_chunks, scratch, counters,
                                                    cos=cos, sin=sin, pdl=args.pdl, cluster=args.cluster)
    else:
        fn = lambda i: ops.attention_decode(q, k, v, pos, slot, table, out, n_q, n_kv, hd, 6, None,
                                            1 / math.sqrt(hd), splits, scratch, counters, cos=cos, sin=sin, pdl=args.pdl)
    us = _time(fn, args.iters)
    nbytes = int((pos.long() + 1).sum()) * n_kv * hd * 2 * 2
    return {"kernel": "attention_decode", "kind": args.kind, "fused": bool(args.fused), "batch": B, "context": ctx, "splits": splits, "us": round(us, 2),
            "GB/s": round(nbytes / us / 1e3, 1)}


def linear(args):
    B, N, K = args.rows, args.n, args.k
    copies = max(2, int(400e6 // (N * K * 2)) + 1)
    ws = [(torch.randn(N, K, device=DEV) * 0.02).bfloat16() for _ in range(copies)]
    x = torch.randn(B, K, device=DEV).bfloat16()
    out = torch.empty(B, N, dtype=torch.bfloat16, device=DEV)
    if args.kernel == "skinny":                             # the mma.sync skinny GEMM, one block per row tile
        fn = lambda i: ops.skinny_gemm(x, ws[i % copies], out, pdl=args.pdl)
    elif args.kernel.startswith("gv"):                      # gv = automatic splits, gv4 = 4 splits
        splits = int(args.kernel[2:]) if len(args.kernel) > 2 else ops.gemv_tc_splits(N, K)
        nf, nc = ops.gemv_tc_scratch(B, N, splits)
        partials = torch.empty(max(nf, 4), device=DEV)
        counters = torch.zeros(max(nc, 1), dtype=torch.int32, device=DEV)
        if args.accumulate:
            acc = torch.zeros(B, N, device=DEV)
            fn = lambda i: ops.gemv_tc(x, ws[i % copies], acc, mode=ops.TC_ACCUMULATE, splits=splits, pdl=args.pdl)
        else:
            fn = lambda i: ops.gemv_tc(x, ws[i % copies], out, splits=splits, partials=partials, counters=counters,
                                       pdl=args.pdl)
    else:
        tile = int(args.kernel[2:])
        fn = lambda i: ops.gemm_tc(x, ws[i % copies], out, tile_n=tile)
    us = _time(fn, args.iters)
    ops.check_device_errors()
    return {"kernel": args.kernel, "rows": B, "n": N, "k": K, "pdl": bool(args.pdl), "us": round(us, 2),
            "GB/s": round(N * K * 2 / us / 1e3, 1)}


def gemm(args):
    M, N, K = args.rows, args.n, args.k
    copies = max(2, int(300e6 // (N * K * 2)) + 1)
    ws = [(torch.randn(N, K, device=DEV) * 0.02).bfloat16() for _ in range(copies)]
    a = torch.randn(M, K, device=DEV).bfloat16()
    if args.accumulate:                               # add into a float32 output, as the o and down projections do
        out = torch.zeros(M, N, device=DEV)
        us = _time(lambda i: ops.gemm_tc(a, ws[i % copies], out, mode=ops.TC_ACCUMULATE, tile_n=args.tile,
                                         splits=args.k_parts), args.iters)
    else:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
        us = _time(lambda i: ops.gemm_tc(a, ws[i % copies], out, tile_n=args.tile), args.iters)
    ops.check_device_errors()
    return {"kernel": f"gemm_tc{args.tile}", "accumulate": bool(args.accumulate), "k_parts": args.k_parts, "m": M, "n": N, "k": K, "us": round(us, 2),
            "TFLOP/s": round(2.0 * M * N * K / us / 1e6, 1)}


def attention_prefill(args):
    n_q, n_kv, hd, S, T = args.heads, args.kv_heads, args.head_dim, args.seqs, args.tokens
    pages_per = (T + 63) // 64
    k = torch.randn(S * pages_per, n_kv, 64, hd, device=DEV).bfloat16()
    v = torch.randn(S * pages_per, n_kv, 64, hd, device=DEV).bfloat16()
    table = torch.randperm(S * pages_per).to(torch.int32).view(S, pages_per).to(DEV)
    q = torch.randn(S * T, (n_q + 2 * n_kv) * hd, device=DEV).bfloat16()
    out = torch.empty(S * T, n_q * hd, dtype=torch.bfloat16, device=DEV)
    cu = torch.arange(S + 1, dtype=torch.int32, device=DEV) * T
    start = torch.zeros(S, dtype=torch.int32, device=DEV)
    slot = torch.arange(S, dtype=torch.int32, device=DEV)
    kernel = ops.attention_prefill_tc if args.kernel == "tc" else ops.attention_prefill   # --kernel tc: tcgen05
    us = _time(lambda i: kernel(q, k, v, cu, start, slot, table, out, T, n_q, n_kv, hd, 6, None,
                                1 / math.sqrt(hd)), args.iters)
    ops.check_device_errors()
    flops = S * 4.0 * n_q * hd * T * (T + 1) / 2
    return {"kernel": "attention_prefill_tc" if args.kernel == "tc" else "attention_prefill", "seqs": S, "tokens": T,
            "us": round(us, 2),
            "TFLOP/s": round(flops / us / 1e6, 1)}


def latent_attention(args):
    """One prompt of --tokens tokens (or --batch decode rows over --context cached tokens with --splits) of
    latent attention: --heads heads over one cached row of --k elements per token whose first --n are the values."""
    H, dk, dv = args.heads, args.k, args.n
    decode = args.tokens <= 1
    S, new, total = (args.batch, 1, args.context) if decode else (args.seqs, args.tokens, args.tokens)
    pages_per = (total + 63) // 64
    cache = (torch.randn(S * pages_per, 1, 64, dk, device=DEV) * 0.5).bfloat16()
    table = torch.randperm(S * pages_per).to(torch.int32).view(S, pages_per).to(DEV)
    q = (torch.randn(S * new, H * dk, device=DEV) * 0.5).bfloat16()
    out = torch.empty(S * new, H * dv, dtype=torch.bfloat16, device=DEV)
    cu = torch.arange(S + 1, dtype=torch.int32, device=DEV) * new
    start = torch.full((S,), total - new, dtype=torch.int32, device=DEV)
    slot = torch.arange(S, dtype=torch.int32, device=DEV)
    slot_tok = slot.repeat_interleave(new)
    sinks = torch.zeros(H, device=DEV)
    splits = args.splits if decode else 1
    partial = torch.empty(S * new * H * splits * (dv + 2), device=DEV) if splits > 1 else None
    us = _time(lambda i: ops.latent_attention_mma(q, cache, cu, start, slot, slot_tok, table, out, sinks, new, H, dk, dv, 6,
                                                  None, dk ** -0.5, splits, partial, form=args.form), args.iters)
    keys = S * (total if decode else new * (new + 1) / 2)
    return {"kernel": "latent_attention_mma", "seqs": S, "new": new, "context": total, "heads": H, "dk": dk, "dv": dv,
            "splits": splits, "form": args.form, "us": round(us, 2), "TFLOP/s": round(2.0 * keys * H * (dk + dv) / us / 1e6, 1),
            "GB/s": round(S * total * dk * 2 / us / 1e3, 1)}


def grouped_gemm(args):
    """The experts' gate/up product with SwiGLU (--kernel swiglu) or a plain one: --tokens tokens, --top of
    --experts experts each, matrices of --n x --k."""
    T, top, E, K, N = args.tokens, args.top, args.experts, args.k, args.n
    expert_of = torch.rand(T, E, device=DEV).argsort(1)[:, :top].int().contiguous()
    P = T * top
    mt = ops.expert_tiles_bound(P, E, 64)
    offsets, order, te, tr, meta = [torch.zeros(n, dtype=torch.int32, device=DEV) for n in (E + 1, P, mt, mt, 1)]
    ops.group_by_expert(expert_of, E, 64, offsets, order, te, tr, meta)
    swiglu = args.kernel == "swiglu"
    x = torch.randn(T, K, device=DEV).bfloat16()
    w = (torch.randn(E, (2 if swiglu else 1) * N, K, device=DEV) * 0.05).bfloat16()
    out = torch.empty(P, N, dtype=torch.bfloat16, device=DEV)
    us = _time(lambda i: ops.grouped_gemm_mma(x, order, top, w, out, None, offsets, te, tr, meta, mt,
                                              ops.GG_SWIGLU if swiglu else ops.GG_STORE), args.iters)
    used = E * (1.0 - (1.0 - top / E) ** T)
    return {"kernel": "grouped_gemm_mma", "swiglu": swiglu, "tokens": T, "top": top, "experts": E, "n": N, "k": K,
            "us": round(us, 2), "TFLOP/s": round(2.0 * P * w.shape[1] * K / us / 1e6, 1),
            "GB/s": round(used * w.shape[1] * K * 2 / us / 1e3, 1)}


def gated_linear_scan(args):
    """The recurrence of gated linear attention over one prompt of --tokens tokens: --heads heads with a state of
    --k x --n, in chunks of --chunk tokens (0: in one go)."""
    H, d, dv, T = args.heads, args.k, args.n, args.tokens
    proj = (torch.randn(T, 2 * H * d + H * dv, device=DEV) * 0.5).bfloat16()
    z, bias = torch.randn(T, H * d, device=DEV), torch.randn(H * d, device=DEV)
    state = torch.zeros(2, H * d * dv, device=DEV)
    cu = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    slots = torch.tensor([1], dtype=torch.int32, device=DEV)
    out = torch.zeros(T, H * dv, device=DEV)
    n = -(-T // args.chunk) if args.chunk else 0
    sums = torch.empty(n * H * d * dv, device=DEV) if n else None
    decays = torch.empty(n * H * d, device=DEV) if n else None
    us = _time(lambda i: ops.gated_linear_scan(proj, 0, H * d, 2 * H * d, z, bias, 16.0, d ** -0.5, state, cu, slots, out, H,
                                               d, dv, chunk=args.chunk, max_new=T, sums=sums, decays=decays), args.iters)
    return {"kernel": "gated_linear_scan", "tokens": T, "heads": H, "dim": d, "vdim": dv, "chunk": args.chunk,
            "us": round(us, 2), "float32 GFLOP/s": round(4.0 * T * H * d * dv / us / 1e3, 1)}


def matrix_state_scan(args):
    """The delta-rule (--kernel delta) or bonus (--kernel bonus) recurrence over --seqs prompts of --tokens tokens:
    --heads heads with a state of --k x --k."""
    H, d, T, B = args.heads, args.k, args.tokens, args.seqs
    kind = "bonus" if args.kernel == "bonus" else "delta"
    proj = (torch.randn(B * T, 3 * H * d, device=DEV) * 0.5).bfloat16()
    decay = torch.rand(B * T, H * d, device=DEV) * 0.1 + 0.9
    unit = torch.randn(B * T, 2 * H * d, device=DEV) * d ** -0.5
    bonus = torch.randn(H * d, device=DEV) * 0.3
    state = torch.zeros(B + 1, H * d * d, device=DEV)
    cu = torch.arange(0, (B + 1) * T, T, dtype=torch.int32, device=DEV)
    slots = torch.arange(1, B + 1, dtype=torch.int32, device=DEV)
    out = torch.zeros(B * T, H * d, device=DEV)
    us = _time(lambda i: ops.matrix_state_scan(proj, 0, H * d, 2 * H * d, decay, kind, state, cu, slots, out, H, d, d,
                                               unit=unit if kind == "delta" else None,
                                               bonus=bonus if kind == "bonus" else None), args.iters)
    fma = 4 if kind == "delta" else 3
    return {"kernel": "matrix_state_scan", "kind": kind, "seqs": B, "tokens": T, "heads": H, "dim": d, "us": round(us, 2),
            "float32 GFLOP/s": round(2.0 * fma * B * T * H * d * d / us / 1e3, 1)}


def gated_unit_scan(args):
    """The vector-state recurrence over --seqs prompts of --tokens tokens and --n channels in blocks of --k."""
    C, T, B, bs = args.n, args.tokens, args.seqs, args.k
    gates = torch.randn(B * T, 2 * C, device=DEV)
    u, y = (torch.randn(B * T, C, device=DEV).bfloat16() for _ in range(2))
    br, bi, yb = (torch.randn(C, device=DEV) for _ in range(3))
    rate = -8.0 * torch.rand(C, device=DEV)
    state = torch.zeros(B + 1, C, device=DEV)
    cu = torch.arange(0, (B + 1) * T, T, dtype=torch.int32, device=DEV)
    slots = torch.arange(1, B + 1, dtype=torch.int32, device=DEV)
    out = torch.empty(B * T, C, device=DEV, dtype=torch.bfloat16)
    scratch = torch.empty(ops.gated_unit_scan_scratch(B, T, C), device=DEV)
    us = _time(lambda i: ops.gated_unit_scan(gates, br, bi, rate, u, y, yb, state, cu, slots, out, bs, max_new=T,
                                             scratch=scratch), args.iters)
    return {"kernel": "gated_unit_scan", "seqs": B, "tokens": T, "channels": C, "us": round(us, 2),
            "GB/s": round(B * T * C * 14 / us / 1e3, 1)}


def sigmoid_attention(args):
    """Attention with sigmoid weights in chunks of --chunk positions: --seqs prompts of --tokens tokens (or, with
    --tokens 1, decode steps at --context), --heads over --kv-heads heads of --head-dim."""
    H, G, d, B, T, ps = args.heads, args.kv_heads, args.head_dim, args.seqs, args.tokens, 6
    ctx = args.context if T == 1 else T
    pages = -(-ctx // 64)
    kc = (torch.randn(B * pages + 1, G, 64, d, device=DEV) * 0.5).bfloat16()
    vc = (torch.randn(B * pages + 1, G, 64, d, device=DEV) * 0.5).bfloat16()
    table = (torch.arange(B * pages, dtype=torch.int32, device=DEV) + 1).view(B, pages).contiguous()
    q = (torch.randn(B * T, H * d + 8 * ((H + 7) // 8), device=DEV) * 0.5).bfloat16()
    gate = q[:, H * d:] if args.gate else None
    start = ctx - T
    pos = (torch.arange(T, dtype=torch.int32, device=DEV) + start).repeat(B)
    slot = torch.arange(B, dtype=torch.int32, device=DEV).repeat_interleave(T)
    cu = torch.arange(0, (B + 1) * T, T, dtype=torch.int32, device=DEV)
    seq_start = torch.full((B,), start, dtype=torch.int32, device=DEV)
    seq_slot = torch.arange(B, dtype=torch.int32, device=DEV)
    bias = torch.randn(H, device=DEV)
    out = torch.empty(B * T, H * d, device=DEV, dtype=torch.bfloat16)
    c = args.chunk
    if args.kernel == "plain":
        fn = lambda i: ops.sigmoid_attention_plain(q, kc, vc, pos, slot, table, bias, out, H, G, d, d, ps, c, None, d ** -0.5)
    else:
        fn = lambda i: ops.sigmoid_attention_mma(q, kc, vc, cu, seq_start, seq_slot, table, bias, out, T, H, G, d, d, ps, c,
                                                 None, d ** -0.5)
    us = _time(fn, args.iters)
    pairs = sum(min(p % c, p - start) + 1 if c else p + 1 for p in range(start, ctx)) * B
    return {"kernel": "sigmoid_attention_" + ("plain" if args.kernel == "plain" else "mma"), "seqs": B, "tokens": T,
            "context": ctx, "chunk": c, "us": round(us, 2), "TFLOP/s": round(4.0 * pairs * H * d / us / 1e6, 2)}


def window_attention(args):
    """Softmax attention over a window of --window tokens with --keep kept first tokens or pooled runs of --pool
    tokens, scores capped at --cap, values turned (--turn): --seqs prompts of --tokens tokens (or, with --tokens 1,
    decode steps at --context), --heads over --kv-heads heads of --head-dim.  --maps 2: two score maps a head over
    the same values of --vdim (twice the query and key heads, two key heads a value head); --gate: a sigmoid gate per
    head and token.  --window 0: every earlier token."""
    M = args.maps
    H, G, d, B, T, ps = args.heads * M, args.kv_heads * M, args.head_dim, args.seqs, args.tokens, 6
    dv = args.vdim or d
    W, P, F = args.window, args.pool, args.keep
    ctx = args.context if T == 1 else T
    pages = -(-ctx // 64)
    kc = (torch.randn(B * pages + 1, G, 64, d, device=DEV) * 0.5).bfloat16()
    vc = (torch.randn(B * pages + 1, G // M, 64, dv, device=DEV) * 0.5).bfloat16()
    table = (torch.arange(B * pages, dtype=torch.int32, device=DEV) + 1).view(B, pages).contiguous()
    pooled = None
    if P:
        pp = -(-(ctx // P) // 64) or 1
        pooled = ((torch.randn(B * pp + 1, G, 64, d, device=DEV) * 0.5).bfloat16(),
                  (torch.randn(B * pp + 1, G, 64, d, device=DEV) * 0.5).bfloat16(),
                  (torch.arange(B * pp, dtype=torch.int32, device=DEV) + 1).view(B, pp).contiguous())
    q = (torch.randn(B * T, H * d + 8 * ((H + 7) // 8), device=DEV) * 0.5).bfloat16()
    gate = q[:, H * d:] if args.gate else None
    start = ctx - T
    pos = (torch.arange(T, dtype=torch.int32, device=DEV) + start).repeat(B)
    slot = torch.arange(B, dtype=torch.int32, device=DEV).repeat_interleave(T)
    cu = torch.arange(0, (B + 1) * T, T, dtype=torch.int32, device=DEV)
    seq_start = torch.full((B,), start, dtype=torch.int32, device=DEV)
    seq_slot = torch.arange(B, dtype=torch.int32, device=DEV)
    vcos = vsin = None
    if args.turn:
        angle = torch.arange(ctx, device=DEV).float()[:, None] * (10000.0 ** (-torch.arange(d // 2, device=DEV).float() * 2 / d))
        vcos, vsin = angle.cos().contiguous(), angle.sin().contiguous()
    out = torch.empty(B * T, H * dv, device=DEV, dtype=torch.bfloat16)
    cap, sink = (args.cap or None), (True if F else None)
    if args.kernel == "plain":
        fn = lambda i: ops.window_attention_plain(q, kc, vc, table, pooled, pos, slot, out, H, G, d, dv, ps, W, F, P, d ** -0.5,
                                                  cap, sink, vcos, vsin, False, v_share=M, gate=gate)
    else:
        fn = lambda i: ops.window_attention_mma(q, kc, vc, table, pooled, cu, seq_start, seq_slot, out, T, H, G, d, dv, ps, W, F,
                                                P, d ** -0.5, cap, sink, vcos, vsin, False, v_share=M, gate=gate)
    us = _time(fn, args.iters)
    lo = lambda p: max(0, p - W + 1) if W else 0
    pairs = sum(p - lo(p) + 1 + (lo(p) // P if P else min(F, lo(p))) for p in range(start, ctx)) * B
    return {"kernel": "window_attention_" + ("plain" if args.kernel == "plain" else "mma"), "seqs": B, "tokens": T,
            "context": ctx, "window": W, "pool": P, "keep": F, "maps": M, "us": round(us, 2),
            "TFLOP/s": round(2.0 * pairs * H * (d + dv) / us / 1e6, 2)}


def norm_add(args):
    """A sublayer's float32 result normed, added to the stream and zeroed behind the read, with (--kernel next) or
    without the next sublayer's normed rows written in the same pass: --rows tokens of width --n."""
    T, Wd = args.rows, args.n
    res = [torch.randn(T, Wd, device=DEV) for _ in range(4)]          # four sets in turn: larger than L2 at real sizes
    br = [torch.randn(T, Wd, device=DEV) for _ in range(4)]
    w1, w2 = torch.randn(Wd, device=DEV), torch.randn(Wd, device=DEV)
    nxt = torch.empty(T, Wd, device=DEV, dtype=torch.bfloat16) if args.kernel == "next" else None
    us = _time(lambda i: ops.rms_add(res[i % 4], br[i % 4], w1, 1e-6, clear=True, next_weight=w2 if nxt is not None else None,
                                     next_eps=1e-6, next_out=nxt), args.iters)
    nbytes = T * Wd * (16 + (2 if nxt is not None else 0))
    return {"kernel": "rms_add" + ("_next" if nxt is not None else ""), "rows": T, "width": Wd, "us": round(us, 2),
            "GB/s": round(nbytes / us / 1e3, 1)}


def mingru_scan(args):
    """minGRU over --seqs prompts of --tokens tokens and --n channels: --kernel walk, tiled or chunked."""
    C, T, B = args.n, args.tokens, args.seqs
    proj = torch.randn(B * T, 3 * C, device=DEV).bfloat16()
    bz, bu = (torch.randn(C, device=DEV) for _ in range(2))
    state = torch.zeros(B + 1, C, device=DEV)
    cu = torch.arange(0, (B + 1) * T, T, dtype=torch.int32, device=DEV)
    slots = torch.arange(1, B + 1, dtype=torch.int32, device=DEV)
    out = torch.empty(B * T, C, device=DEV, dtype=torch.bfloat16)
    scratch = torch.empty(ops.mingru_scan_scratch(B, T, C), device=DEV) if args.kernel == "chunked" else None
    us = _time(lambda i: ops.mingru_scan(proj, bz, bu, state, cu, slots, out, C, 1.0, tiled=args.kernel != "walk", max_new=T,
                                         scratch=scratch), args.iters)
    return {"kernel": "mingru_scan_" + args.kernel, "seqs": B, "tokens": T, "channels": C, "us": round(us, 2),
            "GB/s": round(B * T * C * 8 / us / 1e3, 1)}


def sampling(args):
    """The pick of a step: argmax at temperature 0, else a draw under the given cuts.  Eight sets of
    logits in turn (64 rows of 128,256 are 33 MB each)."""
    rows, V = args.rows, args.vocab
    g = torch.Generator(device=DEV).manual_seed(3)
    logits = [3 * torch.randn(rows, V, device=DEV, generator=g) for _ in range(8)]
    slots = torch.arange(rows, dtype=torch.int32, device=DEV)
    state = (torch.arange(1, rows + 1, dtype=torch.int64, device=DEV) * 0x9E3779B97F4A7C15) & ((1 << 62) - 1)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    if args.temperature <= 0:
        us = _time(lambda i: ops.argmax(logits[i % 8], out), args.iters)
    else:
        us = _time(lambda i: ops.sample(logits[i % 8], args.temperature, args.top_k, args.top_p, slots, state, out), args.iters)
    return {"kernel": "argmax" if args.temperature <= 0 else "sample", "rows": rows, "vocab": V,
            "temperature": args.temperature, "top_k": args.top_k, "top_p": args.top_p, "us": round(us, 2),
            "GB/s": round(rows * V * 4 / us / 1e3, 1)}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="what", required=True)
    for name in ("attention_decode", "linear", "gemm", "attention_prefill", "sampling", "latent_attention", "grouped_gemm",
                 "gated_linear_scan", "matrix_state_scan", "gated_unit_scan", "sigmoid_attention", "window_attention",
                 "mingru_scan", "norm_add"):
        p = sub.add_parser(name)
        p.add_argument("--iters", type=int, default=20)
        p.add_argument("--heads", type=int, default=32)
        p.add_argument("--kv-heads", type=int, default=8)
        p.add_argument("--head-dim", type=int, default=128)
        p.add_argument("--batch", type=int, default=8)
        p.add_argument("--context", type=int, default=520)
        p.add_argument("--splits", type=int, default=8)
        p.add_argument("--rows", type=int, default=8)
        p.add_argument("--n", type=int, default=6144)
        p.add_argument("--k", type=int, default=4096)
        p.add_argument("--kernel", default="skinny")
        p.add_argument("--tile", type=int, default=256)
        p.add_argument("--k-parts", type=int, default=1, help="gemm --accumulate: parts a tile's K range is cut into")
        p.add_argument("--kind", type=int, default=2, help="attention_decode: 1 CUDA cores, 2 tensor cores (persistent grid)")
        p.add_argument("--chunk-pages", type=int, default=0, help="attention_decode --kind 2: pages per chunk (default: pages / --splits)")
        p.add_argument("--cluster", type=int, default=0,
                       help="attention_decode --kind 2: chunks a sequence as a thread-block cluster (2, 4, 8; 0: the persistent grid)")
        p.add_argument("--ragged", action="store_true", help="attention_decode: lengths uniform in [1, --context]")
        p.add_argument("--accumulate", action="store_true", help="linear gv*, gemm: add into a float32 output")
        p.add_argument("--pdl", action="store_true", help="launch as programmatic dependents")
        p.add_argument("--fused", action="store_true", help="attention_decode: rotate and append inside")
        p.add_argument("--seqs", type=int, default=1)
        p.add_argument("--tokens", type=int, default=2048)
        p.add_argument("--vocab", type=int, default=128256)
        p.add_argument("--temperature", type=float, default=0.0, help="sampling: 0 is the greedy pick")
        p.add_argument("--top-k", type=int, default=0)
        p.add_argument("--top-p", type=float, default=1.0)
        p.add_argument("--form", type=int, default=0, help="latent_attention: warps of a block as 1 x 8, 2 x 4, 2 x 8 (1, 2, 3)")
        p.add_argument("--experts", type=int, default=64)
        p.add_argument("--top", type=int, default=6)
        p.add_argument("--chunk", type=int, default=128, help="gated_linear_scan: tokens a chunk (0: in one go); sigmoid_attention: positions a chunk")
        p.add_argument("--window", type=int, default=512, help="window_attention: tokens a query sees behind it")
        p.add_argument("--pool", type=int, default=0, help="window_attention: tokens a pooled run (0: none)")
        p.add_argument("--keep", type=int, default=0, help="window_attention: kept first tokens (with a sink)")
        p.add_argument("--cap", type=float, default=0.0, help="window_attention: score cap (0: none)")
        p.add_argument("--turn", action="store_true", help="window_attention: values stored turned by their position")
        p.add_argument("--maps", type=int, default=1, help="window_attention: score maps a head (2: over the same values)")
        p.add_argument("--vdim", type=int, default=0, help="window_attention: width of a value row (0: the head size)")
        p.add_argument("--gate", action="store_true", help="window_attention: a sigmoid gate per head and token")
    args = ap.parse_args(argv)
    print(json.dumps(globals()[args.what](args)))


if __name__ == "__main__":
    main()
