"""The Ronelorn design in the engine against the plain statement of it (``plain_ronelorn``): every mixer alone
through a cache of its own, the kernels against one another, then whole models through the step function in
every way of cutting and batching, and generation through the entry point."""
import copy

import numpy as np
import pytest
import torch

import plain_ronelorn as pr
import tiny_ronelorn as tr

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def make_model(cfg, store, dtype, max_tokens=2048, **kw):
    from supersonic_b200.engine import Model
    return Model.from_config(cfg, store, dtype=dtype, device=DEV, max_tokens=max_tokens, **kw)


def run_in_portions(model, tokens, cuts):
    """Logits of every position [T, vocab] with the sequence fed in portions of the given sizes."""
    from supersonic_b200.engine import StepEntry
    slot, at, rows = model.open_sequence(), 0, []
    for n in cuts:
        rows.append(model.step([StepEntry(slot, tokens[at:at + n], list(range(n)))]).cpu())
        at += n
    assert at == len(tokens)
    model.close_sequence(slot)
    model.check_errors()
    return torch.cat(rows).double()


def position_errors(got, ref):
    return (got - ref).pow(2).mean(-1).sqrt() / ref.std(-1).clamp_min(1e-6)


def close(got, ref, dtype, what=""):
    """float32: a few units of float32 rounding of the logits' size.  bfloat16: the error's root mean square per
    position against the spread of that position's logits: the typical position, how many are far off, and the
    worst one.  The float32 runs of the same tests are the sharp ones."""
    assert torch.isfinite(got).all(), what
    if dtype == torch.float32:
        assert float((got - ref).abs().max()) < 2e-4 * max(1.0, float(ref.abs().max())), what
    else:
        rel = position_errors(got, ref)
        assert float(rel.median()) < 0.05 and float((rel > 0.08).double().mean()) <= 0.1 and float(rel.max()) < 0.4, \
            (what, rel.median(), (rel > 0.08).double().mean(), rel.max())


def tokens_of(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg.vocab, n).tolist()


def reference(cfg, plain, tokens):
    return pr.forward(tokens, plain, cfg.to_dict())[0]


# ---- the parts alone ---------------------------------------------------------------------------------
def part_context(dtype, store, max_positions=600):
    from supersonic_b200.csrc.kernel_sets import kernel_set_for
    from supersonic_b200.parts import BuildContext, WeightAccess
    return BuildContext(torch.device(DEV), dtype, kernel_set_for(dtype), WeightAccess(store, DEV), max_positions)


def step_context(build, cache, entries):
    from supersonic_b200.engine import StepContext, pack_step
    starts = [cache.length(e.slot) for e in entries]
    batch = pack_step(entries, starts, DEV)
    for e in entries:
        cache.reserve(e.slot, len(e.tokens))
    cache.sync()
    return StepContext(batch, cache, build.kernels, build.dtype)


def mixer_alone(spec, position, store, dtype, x, pieces):
    """What the mixer adds into a zeroed stream for one sequence whose rows ``x`` arrive in pieces, through a cache
    of its own that holds the mixer's need under id 0."""
    from supersonic_b200.cache import SequenceCache
    from supersonic_b200.engine import StepEntry
    from supersonic_b200.parts import MIXERS, POSITION_ENCODINGS
    build = part_context(dtype, store)
    mixer = MIXERS[spec.kind](spec.params, spec.weights, build)
    pos = None if position is None else POSITION_ENCODINGS[position.kind](position.params, {}, build)
    cache = SequenceCache({0: mixer.cache_need()}, 1024, 1024, dtype, DEV)
    slot, at, out = cache.acquire(), 0, []
    for n in pieces:
        ctx = step_context(build, cache, [StepEntry(slot, [0] * n)])
        res = torch.zeros(n, x.shape[1], device=DEV)
        mixer.forward(ctx, x[at:at + n].to(DEV, dtype), res, 0, True, pos)
        cache.advance(slot, n)
        out.append(res.cpu())
        at += n
    cache.check()
    return torch.cat(out).double()


PIECES = [70, 2, 2, 59] + [1] * 17 + [90, 1, 1, 1, 2]      # crosses page borders; portions of two; token by token
T_ALONE = sum(PIECES)


def rows_for(cfg, seed, dtype):
    return torch.randn(T_ALONE, cfg.width, generator=torch.Generator().manual_seed(seed)).to(dtype)


def tolerance(dtype, ref, loose=0.04):
    return (1e-4 if dtype == torch.float32 else loose) * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,layer", [("A", 0), ("B", 1), ("C", 0), ("C", 3), ("D", 0), ("D", 3)])
def test_window_attention_with_pooled_runs_alone(dtype, name, layer):
    """Windows of 5 to 100 tokens and runs of 3 to 16 against pages of 64: a prompt that crosses window, run and
    page borders, then portions of two and single tokens; values turned and turned back; capped and uncapped."""
    cfg, store, plain = tr.build(name)
    block = cfg.build_spec().blocks[layer]
    x = rows_for(cfg, layer, dtype)
    ref = cfg.residual_mult * pr.attention(x.double(), plain, f"l{layer}.mix", cfg.layers[layer]["mixer"], cfg.norm_eps)
    got = mixer_alone(block.mixer, block.position, store, dtype, x, PIECES)
    assert float((got - ref).abs().max()) < tolerance(dtype, ref)


@pytest.mark.parametrize("dim,vdim,heads,kv_heads,window,keep,pool,cap,sink,turn", [
    (64, 64, 8, 2, 45, 0, 4, 20.0, None, "halves"), (128, 128, 4, 1, 70, 0, 3, None, None, "interleaved"),
    (32, 48, 6, 6, 20, 5, 0, None, True, None), (80, 128, 16, 1, 64, 70, 0, 8.0, "each", None),
    (128, 64, 3, 3, 129, 2, 7, None, True, "halves"), (24, 8, 40, 2, 33, 0, 0, None, None, None),
    (64, 64, 4, 2, None, 0, 0, 15.0, True, "interleaved")])
def test_window_attention_kernels_agree(dim, vdim, heads, kv_heads, window, keep, pool, cap, sink, turn):
    """The tensor-core kernel against the plain one in bfloat16, for head sizes that fill its tiles and for ones
    that it pads: three sequences of unequal lengths as prompts that continue a cache, and as decode steps, with
    pages in a shuffled order and a pooled store of its own; the two differ by the rounding of the output alone."""
    from supersonic_b200.csrc import ops
    g = torch.Generator(device=DEV).manual_seed(dim + vdim)
    lens, new = [330, 64, 131], [170, 64, 1]
    pages_per, B = 6, 3
    kc = (torch.randn(B * pages_per + 1, kv_heads, 64, dim, device=DEV, generator=g) * 0.6).bfloat16()
    vc = (torch.randn(B * pages_per + 1, kv_heads, 64, vdim, device=DEV, generator=g) * 0.6).bfloat16()
    table = (torch.randperm(B * pages_per, device=DEV, generator=g).int() + 1).view(B, pages_per).contiguous()
    pooled = None
    if pool:
        pk = (torch.randn(B * 2 + 1, kv_heads, 64, dim, device=DEV, generator=g) * 0.6).bfloat16()
        pv = (torch.randn(B * 2 + 1, kv_heads, 64, vdim, device=DEV, generator=g) * 0.6).bfloat16()
        pooled = (pk, pv, (torch.randperm(B * 2, device=DEV, generator=g).int() + 1).view(B, 2).contiguous())
    sinks = (torch.randn(heads, device=DEV, generator=g) + 1.0) if sink == "each" else sink
    vcos = vsin = None
    if turn:
        angle = torch.arange(400, device=DEV).float()[:, None] * (50.0 ** (-torch.arange(vdim // 2, device=DEV).float() * 2 / vdim))
        vcos, vsin = angle.cos().contiguous(), angle.sin().contiguous()
    for counts in (new, [1, 1, 1]):
        T = sum(counts)
        q = (torch.randn(T, heads * dim + 8, device=DEV, generator=g) * 0.6).bfloat16()[:, :heads * dim]
        pos = torch.cat([torch.arange(n - c, n) for n, c in zip(lens, counts)]).int().to(DEV)
        slot = torch.cat([torch.full((c,), i) for i, c in enumerate(counts)]).int().to(DEV)
        cu = torch.tensor([0] + list(np.cumsum(counts)), dtype=torch.int32, device=DEV)
        start = torch.tensor([n - c for n, c in zip(lens, counts)], dtype=torch.int32, device=DEV)
        seq_slot = torch.arange(B, dtype=torch.int32, device=DEV)
        want = torch.empty(T, heads * vdim, device=DEV, dtype=torch.bfloat16)
        ops.window_attention_plain(q, kc, vc, table, pooled, pos, slot, want, heads, kv_heads, dim, vdim, 6, window, keep, pool,
                                   dim ** -0.5, cap, sinks, vcos, vsin, turn == "interleaved", 0.5)
        for split in (None, True, False):
            got = torch.zeros_like(want)
            ops.window_attention_mma(q, kc, vc, table, pooled, cu, start, seq_slot, got, max(counts), heads, kv_heads, dim, vdim,
                                     6, window, keep, pool, dim ** -0.5, cap, sinks, vcos, vsin, turn == "interleaved", 0.5,
                                     split=split)
            err = float((got.float() - want.float()).abs().max())
            assert err < 0.01 * max(1.0, float(want.float().abs().max())), (counts, split, err)


def test_window_attention_decode_step_of_many_sequences():
    """A decode step with more blocks than the device has SMs takes the shallow ring of the decode form: 90
    sequences of unequal lengths (their page tables point into the same few pages, which are only read) against
    the plain kernel."""
    from supersonic_b200.csrc import ops
    g = torch.Generator(device=DEV).manual_seed(11)
    heads, kv_heads, dim, vdim, B, pages_per = 8, 2, 64, 64, 90, 5
    kc = (torch.randn(12, kv_heads, 64, dim, device=DEV, generator=g) * 0.6).bfloat16()
    vc = (torch.randn(12, kv_heads, 64, vdim, device=DEV, generator=g) * 0.6).bfloat16()
    pk = (torch.randn(7, kv_heads, 64, dim, device=DEV, generator=g) * 0.6).bfloat16()
    pv = (torch.randn(7, kv_heads, 64, vdim, device=DEV, generator=g) * 0.6).bfloat16()
    table = torch.randint(0, 12, (B, pages_per), device=DEV, generator=g).int()
    pooled = (pk, pv, torch.randint(0, 7, (B, 1), device=DEV, generator=g).int())
    lens = torch.randint(1, 64 * pages_per, (B,), generator=torch.Generator().manual_seed(3))
    q = (torch.randn(B, heads * dim, device=DEV, generator=g) * 0.6).bfloat16()
    pos = (lens - 1).int().to(DEV)
    slot = torch.arange(B, dtype=torch.int32, device=DEV)
    cu = torch.arange(B + 1, dtype=torch.int32, device=DEV)
    want, got = (torch.zeros(B, heads * vdim, device=DEV, dtype=torch.bfloat16) for _ in range(2))
    ops.window_attention_plain(q, kc, vc, table, pooled, pos, slot, want, heads, kv_heads, dim, vdim, 6, 100, 0, 8, dim ** -0.5,
                               25.0, None, None, None, False)
    ops.window_attention_mma(q, kc, vc, table, pooled, cu, pos, slot, got, 1, heads, kv_heads, dim, vdim, 6, 100, 0, 8,
                             dim ** -0.5, 25.0, None, None, None, False)
    err = float((got.float() - want.float()).abs().max())
    assert err < 0.01 * max(1.0, float(want.float().abs().max())), err


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,layer", [("A", 2), ("B", 0), ("C", 1), ("D", 1), ("D", 4)])
def test_window_attention_with_kept_tokens_and_sink_alone(dtype, name, layer):
    """One to seventy kept tokens, windows of one to 130 tokens; the norm over the whole projection."""
    cfg, store, plain = tr.build(name)
    block = cfg.build_spec().blocks[layer]
    x = rows_for(cfg, 10 + layer, dtype)
    ref = cfg.residual_mult * pr.attention_2(x.double(), plain, f"l{layer}.mix", cfg.layers[layer]["mixer"], cfg.norm_eps)
    got = mixer_alone(block.mixer, block.position, store, dtype, x, PIECES)
    assert float((got - ref).abs().max()) < tolerance(dtype, ref)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,layer", [("A", 1), ("A", 4), ("B", 2), ("C", 2), ("D", 2)])
def test_min_gru_alone(dtype, name, layer):
    cfg, store, plain = tr.build(name)
    block = cfg.build_spec().blocks[layer if name != "A" or layer < 3 else 3]     # A's entry 3 has no block of its own
    x = rows_for(cfg, 20 + layer, dtype)
    ref = cfg.residual_mult * pr.min_gru(x.double(), plain, f"l{layer}.mix", cfg.layers[layer]["mixer"])
    got = mixer_alone(block.mixer, None, store, dtype, x, PIECES)
    assert float((got - ref).abs().max()) < tolerance(dtype, ref)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [64, 130, 322])
def test_min_gru_scan_forms_agree(dtype, width):
    """The walk, the tiled scan and the scan with a block per 64 tokens on the same rows: three sequences of
    unequal lengths (one of a single token, one that ends inside a tile, one of several tiles and a rest) that
    continue a state, twice in a row, against the recurrence written out in float64."""
    from supersonic_b200.csrc import ops
    g = torch.Generator(device=DEV).manual_seed(width)
    counts = [300, 1, 77]
    T, B = sum(counts), len(counts)
    cu = torch.tensor([0] + list(np.cumsum(counts)), dtype=torch.int32, device=DEV)
    slots = torch.tensor([2, 0, 1], dtype=torch.int32, device=DEV)
    bz, bu = torch.randn(width, device=DEV, generator=g), torch.randn(width, device=DEV, generator=g)
    states = [torch.zeros(3, width, device=DEV) for _ in range(3)]
    ref_state = torch.zeros(3, width, dtype=torch.float64)
    for _ in range(2):
        proj = (torch.randn(T, 3 * width + 8, device=DEV, generator=g) * 2.0).to(dtype)[:, :3 * width]
        outs = [torch.zeros(T, width, device=DEV, dtype=dtype) for _ in range(3)]
        scratch = torch.empty(ops.mingru_scan_scratch(B, max(counts), width), device=DEV)
        ops.mingru_scan(proj, bz, bu, states[0], cu, slots, outs[0], width, 0.7)
        ops.mingru_scan(proj, bz, bu, states[1], cu, slots, outs[1], width, 0.7, tiled=True)
        ops.mingru_scan(proj, bz, bu, states[2], cu, slots, outs[2], width, 0.7, tiled=True, max_new=max(counts), scratch=scratch)
        p64 = proj.double().cpu()
        z = torch.sigmoid(p64[:, :width] + bz.double().cpu())
        u = p64[:, width:2 * width] + bu.double().cpu()
        cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
        gate = torch.nn.functional.silu(p64[:, 2 * width:])
        ref = torch.zeros(T, width, dtype=torch.float64)
        for b, n in enumerate(counts):
            S = ref_state[int(slots[b])]
            for t in range(int(cu[b]), int(cu[b]) + n):
                S = (1 - z[t]) * S + z[t] * cand[t]
                ref[t] = 0.7 * S * gate[t]
            ref_state[int(slots[b])] = S
        tol = (2e-5 if dtype == torch.float32 else 0.01) * max(1.0, float(ref.abs().max()))
        for form, (o, st) in enumerate(zip(outs, states)):
            assert float((o.double().cpu() - ref).abs().max()) < tol, form
            assert float((st.double().cpu() - ref_state).abs().max()) < 2e-5 * max(1.0, float(ref_state.abs().max())), form


@pytest.mark.parametrize("kind", ["relu_squared", "gelu_tanh", "silu"])
@pytest.mark.parametrize("rows,n,k", [(5, 256, 128), (70, 264, 192), (200, 512, 256), (1500, 1024, 512), (3, 100, 60)])
def test_product_with_the_activation_where_it_finishes(kind, rows, n, k):
    """The serving set's product with its activation in one (the tensor-core product's last step, or the pass that
    rounds the sums of a product whose K is split) against the float64 statement, for row counts that take each
    of its ways and for sizes that none of them takes."""
    from supersonic_b200.csrc.kernel_sets import kernel_set_for
    g = torch.Generator(device=DEV).manual_seed(rows + n)
    x = torch.randn(rows, k, device=DEV, generator=g).bfloat16()
    w = (torch.randn(n, k, device=DEV, generator=g) * k ** -0.5).bfloat16()
    u = x.double() @ w.double().T
    ref = {"relu_squared": lambda v: torch.relu(v) ** 2, "silu": torch.nn.functional.silu,
           "gelu_tanh": lambda v: torch.nn.functional.gelu(v, approximate="tanh")}[kind](u) * 0.3
    for deterministic in (False, True):
        ks = kernel_set_for(torch.bfloat16, deterministic=deterministic)
        for _ in range(2):                                  # the scratch of a split product is left clean for the next
            out = torch.zeros(rows, n, device=DEV, dtype=torch.bfloat16)
            ks.linear_activation(x, w, out, kind, 0.3)
            assert float((out.double() - ref).abs().max()) < 0.01 * max(1.0, float(ref.abs().max())), deterministic


@pytest.mark.parametrize("dtype", DTYPES)
def test_dense_feed_forward_norm_and_embedding_alone(dtype):
    from supersonic_b200.parts import EMBEDDINGS, FEED_FORWARDS, NORMS
    from supersonic_b200.engine import StepEntry
    from supersonic_b200.cache import SequenceCache, StateNeed
    cfg, store, plain = tr.build("A")
    spec = cfg.build_spec()
    build = part_context(dtype, store)
    cache = SequenceCache({0: StateNeed(1)}, 256, 256, dtype, DEV)
    tokens = tokens_of(cfg, 37, 1)
    ctx = step_context(build, cache, [StepEntry(cache.acquire(), tokens)])
    emb = EMBEDDINGS[spec.embedding.kind](spec.embedding.params, spec.embedding.weights, build)
    x = emb(ctx, ctx.batch.token_ids)
    want = plain["embed"].double()[torch.tensor(tokens)] * cfg.embedding_scale
    assert x.dtype == torch.float32 and float((x.cpu().double() - want).abs().max()) < 1e-5 * float(want.abs().max())
    block = spec.blocks[0]
    norm = NORMS[block.feed_forward_norm.kind](block.feed_forward_norm.params, block.feed_forward_norm.weights, build)
    ff = FEED_FORWARDS[block.feed_forward.kind](block.feed_forward.params, block.feed_forward.weights, build)
    rows = torch.randn(37, cfg.width, generator=torch.Generator().manual_seed(5)) * 3.0
    normed = norm(ctx, rows.to(DEV))
    assert normed.dtype == dtype
    ref_n = pr.block_norm(rows.double(), plain, "l0.norm2", cfg.norm_eps)
    assert float((normed.cpu().double() - ref_n).abs().max()) < tolerance(dtype, ref_n, 0.01)
    res = torch.zeros(37, cfg.width, device=DEV)
    ff.forward(ctx, normed, res)
    ref = cfg.residual_mult * pr.dense(normed.cpu().double(), plain, "l0.mlp")
    assert float((res.cpu().double() - ref).abs().max()) < tolerance(dtype, ref, 0.02)


# ---- whole models through the step function --------------------------------------------------------
def test_stream_after_every_layer():
    """float32: the stream after every layer (one that runs with another's tensors counts as a layer of its own),
    and the logits, against the plain statement."""
    from supersonic_b200.engine import StepEntry
    for name in ("A", "B", "C", "D", "E"):
        cfg, store, plain = tr.build(name)
        model = make_model(cfg, store, torch.float32)
        tokens = tokens_of(cfg, 90, 3)
        ref, streams = pr.forward(tokens, plain, cfg.to_dict())
        seen = []
        model.layer_probe = lambda stop, x: seen.append(x.cpu().double())
        slot = model.open_sequence()
        got = model.step([StepEntry(slot, tokens, list(range(len(tokens))))]).cpu().double()
        assert len(seen) == len(streams) == len(cfg.layers)
        for i, s in enumerate(seen):
            assert float((s - streams[i]).abs().max()) < 1e-4 * max(1.0, float(streams[i].abs().max())), (name, i)
        close(got, ref, torch.float32, name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "E"])
def test_portions_of_every_size_and_token_by_token(dtype, name):
    cfg, store, plain = tr.build(name)
    model = make_model(cfg, store, dtype)
    T = 150
    tokens = tokens_of(cfg, T, 5)
    ref = reference(cfg, plain, tokens)
    for cuts in ([T], [64, 64, 22], [63, 2, 2, 61, 3, 7, 2, 10], [1] * 6 + [2] * 3 + [138], [100] + [1] * 50, [1] * T):
        close(run_in_portions(model, tokens, cuts), ref, dtype, (name, cuts))
    assert model.cache.slots.n_held == 0
    model.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["C", "D"])
def test_sizes_that_no_fast_kernel_takes_and_sizes_that_all_take(dtype, name):
    """Odd widths and head sizes (every operation on its plain kernel, also in bfloat16) and round ones: a prompt
    in portions, then decoding, in a batch of two."""
    from supersonic_b200.engine import StepEntry
    cfg, store, plain = tr.build(name)
    model = make_model(cfg, store, dtype)
    seqs = [tokens_of(cfg, 230, 31), tokens_of(cfg, 150, 32)]
    refs = [reference(cfg, plain, q) for q in seqs]
    slots = [model.open_sequence() for _ in seqs]
    got = [[], []]
    plan = [((0, 180), (0, 146)), ((180, 210), (146, 148))] + \
           [((210 + i, 211 + i), (148 + i, 149 + i) if i < 2 else None) for i in range(20)]
    for step in plan:
        entries = [StepEntry(slots[i], seqs[i][lo_hi[0]:lo_hi[1]], list(range(lo_hi[1] - lo_hi[0])))
                   for i, lo_hi in enumerate(step) if lo_hi]
        rows = model.step(entries).cpu().double()
        at = 0
        for i, lo_hi in enumerate(step):
            if lo_hi:
                got[i].append(rows[at:at + lo_hi[1] - lo_hi[0]])
                at += lo_hi[1] - lo_hi[0]
    close(torch.cat(got[0]), refs[0], dtype, name)
    close(torch.cat(got[1]), refs[1], dtype, name)
    model.check_errors()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "D", "E"])
def test_unequal_batches_against_each_alone_and_reused_slots(dtype, name):
    """Requests of 1 to 260 tokens start together and decode together, the short ones ending first; then other
    requests run in the slots, pages, pooled rows and state rows those gave back."""
    from supersonic_b200.engine import StepEntry
    cfg, store, plain = tr.build(name)
    model = make_model(cfg, store, dtype, max_tokens=1024)
    for round_, lens in enumerate(([1, 5, 64, 65, 131], [131, 2, 66], [260, 3, 195, 64], [7, 129, 64, 3])):
        decode = [3, 9, 14, 6, 11][: len(lens)]
        seqs = [tokens_of(cfg, n + d, 100 * round_ + i) for i, (n, d) in enumerate(zip(lens, decode))]
        refs = [reference(cfg, plain, s) for s in seqs]
        slots = [model.open_sequence() for _ in seqs]
        got = [[] for _ in seqs]
        rows = model.step([StepEntry(s, q[:n], list(range(n))) for s, q, n in zip(slots, seqs, lens)]).cpu().double()
        at = 0
        for i, n in enumerate(lens):
            got[i].append(rows[at:at + n])
            at += n
        for step in range(max(decode)):
            live = [i for i in range(len(seqs)) if step < decode[i]]
            rows = model.step([StepEntry(slots[i], [seqs[i][lens[i] + step]], [0]) for i in live]).cpu().double()
            for r, i in enumerate(live):
                got[i].append(rows[r:r + 1])
            for i in live:
                if step == decode[i] - 1:
                    model.close_sequence(slots[i])          # its slot, pages and state go back while the others go on
        for i in range(len(seqs)):
            close(torch.cat(got[i]), refs[i], dtype, (round_, i))
        model.check_errors()
        assert model.cache.slots.n_held == 0
        model.cache.check()


def sharpened(name="A", gate=-5.5, sharp=5.0, sharp_kept=10.0, loud_kept=3.0):
    """The configuration's weights changed so that faults show.  The weights of the norms of q are scaled up, so
    that a query's output stands on the few keys whose scores are high: a key, a kept token or a pooled run more
    or less then moves the logits by far more than any tolerance.  The recurrent layers' update gates are pushed
    down, so that what the state took in hundreds of tokens back still counts."""
    cfg, store, plain = tr.build(name)
    changes = {}
    for i, l in enumerate(cfg.layers):
        if l.get("weights_of") is not None:
            continue
        if l["type"] == "mingru":
            changes[f"l{i}.mix.z.b"] = plain[f"l{i}.mix.z.b"].float() + gate
        elif l["type"] == "attention_2":           # its sink takes weight from every key: sharper still, and louder
            changes[f"l{i}.mix.q.norm"] = plain[f"l{i}.mix.q.norm"].float() * sharp_kept
            changes[f"l{i}.mix.o"] = plain[f"l{i}.mix.o"].float() * loud_kept
        else:
            changes[f"l{i}.mix.q.norm"] = plain[f"l{i}.mix.q.norm"].float() * sharp
    store, plain = tr.changed(plain, **{k.replace(".", "__"): v for k, v in changes.items()})
    return cfg, store, plain


def _variant(cfg, layer, **mask):
    d = copy.deepcopy(cfg.to_dict())
    for l in d["layers"]:
        if l is d["layers"][layer] or l.get("weights_of") == layer:
            l["mixer"]["mask"].update(mask)
    return d


@pytest.mark.parametrize("dtype", DTYPES)
def test_window_edges_kept_tokens_pooled_runs_far_tokens_and_page_borders_show(dtype):
    cfg, store, plain = sharpened("A")
    T = 330
    tokens = tokens_of(cfg, T, 9)
    ref = reference(cfg, plain, tokens)
    # the test is sharp: a window one token longer, a kept token more, runs of another length (which are seen
    # earlier or later) each give other logits at most positions behind the first window ...
    # (one key of a window of 17 beside a sink seldom carries a query, so the second layer's share is smaller)
    for layer, mask, share in ((0, {"size": 21}, 0.5), (2, {"size": 18}, 0.3), (2, {"keep_first": 4}, 0.2),
                               (0, {"pool": 5}, 0.5), (0, {"pool": 0}, 0.5)):
        other = position_errors(pr.forward(tokens, plain, _variant(cfg, layer, **mask))[0], ref)
        assert float((other[40:] > 0.08).double().mean()) > share and float(other[40:].median()) > 0.03, (layer, mask)
    # ... and a sequence that has lost what came 200 and more positions before gives other logits at its end
    tail = position_errors(pr.forward(tokens[200:], plain, cfg.to_dict())[0], ref[200:])
    assert float(tail[-30:].min()) > 0.2
    model = make_model(cfg, store, dtype)
    # cuts at window edges (17, 20), run ends (4, 8, ...), one before and one behind them, at page borders (64, 128),
    # the first tokens one by one, and decoding across all of these
    for cuts in ([T], [1, 1, 1, 1, 12, 1, 1, 1, 1, 1, 1, 1, 18, 1, 1, 19, 1, 63, 1, 1, 202],
                 [16, 2, 2, 2, 19, 2, 21, 64] + [1] * 202, [256] + [1] * 74, [2] * 165):
        close(run_in_portions(model, tokens, cuts), ref, dtype, cuts)


def test_long_decoding_keeps_every_state():
    """400 tokens decoded one by one after a prompt of two, in float32 and with slow gates: the recurrent state, the
    kept tokens' pages and the pooled rows are carried over hundreds of steps and several pages."""
    cfg, store, plain = sharpened("B")
    model = make_model(cfg, store, torch.float32)
    tokens = tokens_of(cfg, 402, 21)
    close(run_in_portions(model, tokens, [2] + [1] * 400), reference(cfg, plain, tokens), torch.float32)


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_point(dtype):
    """Prompts of unequal lengths in batches of three through ``Engine.generate`` (its scheduler, cache and
    sampler): the tokens are those the plain statement picks greedily, and in bfloat16 every picked token
    is the plain statement's first or close second choice."""
    from supersonic_b200.api import Engine
    cfg, store, plain = tr.build("A")
    model = make_model(cfg, store, dtype, max_tokens=1024, max_seq_tokens=128)
    prompts = [tokens_of(cfg, n, 40 + n) for n in (1, 9, 64, 17, 70)]
    out = Engine(model).generate(prompts, max_new_tokens=30, temperature=0.0, ignore_eos=True, batch_size=3)
    assert [len(o) for o in out] == [30] * len(prompts)
    for prompt, new in zip(prompts, out):
        seq = list(prompt)
        for tok in new:
            logits = reference(cfg, plain, seq)[-1]
            if dtype == torch.float32:
                assert tok == int(logits.argmax())
            else:
                assert float(logits.max() - logits[tok]) < 0.05 * float(logits.std())
            seq.append(tok)
    assert model.cache.slots.n_held == 0


def test_trace_replay_of_a_model_folder(tmp_path):
    """``bin/trace_run`` on a written folder: a batch of two prompts, decode steps, and a third request in a freed
    slot, logits against the plain statement."""
    import json, os, subprocess, sys
    from supersonic_b200.weights import WeightStore, write_model_folder
    cfg, _, _ = tr.build("A")
    folder = write_model_folder(cfg, 3, str(tmp_path / "m"), std=0.3)
    st = WeightStore.from_dir(folder)
    plain = {n: st.get(n) for n in st.names()}
    a, b, c = tokens_of(cfg, 70, 1), tokens_of(cfg, 5, 2), tokens_of(cfg, 9, 3)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:66], "want": [0, 65]}, {"id": "b", "tokens": b[:3], "want": [2]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[66:67], "want": [0]}, {"id": "b", "tokens": b[3:4], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[67:68], "want": [0]}, {"id": "b", "tokens": b[4:5], "want": [0]}], "end": ["b"]},
             {"step": 3, "entries": [{"id": "a", "tokens": a[68:70], "want": [1]}], "end": ["a"]},
             {"step": 4, "entries": [{"id": "c", "tokens": c, "want": [8]}], "end": ["c"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                        "--out", str(out), "--max-tokens", "256"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(5)]
    ra, rb, rc = (reference(cfg, plain, s) for s in (a, b, c))
    want = {0: torch.cat([ra[[0, 65]], rb[[2]]]), 1: ra[[66]], 2: torch.cat([ra[[67]], rb[[4]]]), 3: ra[[69]], 4: rc[[8]]}
    for i, ref in want.items():
        got = torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, cfg.vocab)).double()
        close(got, ref, torch.float32, i)
