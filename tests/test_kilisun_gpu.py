"""The Kilisun design in the engine against the plain statement of it (``plain_kilisun``): every mechanism alone,
the kernels against one another, then whole models through the step function in every way of cutting and batching,
and generation through the entry point."""
import copy

import numpy as np
import pytest
import torch

import plain_kilisun as pk
import tiny_kilisun as tk

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
    position against the spread of that position's logits: the typical position, and how many are far off.  A token
    whose best experts are nearly level may get another one in bfloat16, which moves that position by its whole
    size and, through the keys it leaves, the positions behind it a little: such positions are bounded in number,
    not in size.  The float32 runs of the same tests are the sharp ones."""
    assert torch.isfinite(got).all(), what
    if dtype == torch.float32:
        assert float((got - ref).abs().max()) < 2e-4 * max(1.0, float(ref.abs().max())), what
    else:
        rel = position_errors(got, ref)
        far = int((rel > 0.15).sum())
        assert float(rel.median()) < 0.05 and far <= max(1, 0.1 * rel.numel()) and float(rel.max()) < 2.0, \
            (what, rel.median(), far, rel.numel(), rel.max())


def build_for(name, dtype):
    """The configuration's weights; for bfloat16 with decisive routers (``tiny_kilisun.decisive``), so that a token's
    experts do not hang on the rounding of a score.  float32 runs keep the routers as drawn."""
    cfg, store, plain = tk.build(name)
    if dtype != torch.float32:
        store, plain = tk.decisive(plain)
    return cfg, store, plain


def tokens_of(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg.vocab, n).tolist()


def reference(cfg, plain, tokens):
    return pk.forward(cfg.to_dict(), plain, tokens)[0]


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


def mixers_alone(specs, store, dtype, xs, pieces):
    """What mixers add into zeroed streams for one sequence whose rows arrive in pieces.  ``specs``: (mixer spec,
    position spec) each; the first writes cache entry 0, the others read it with rows ``xs[i]`` of their own."""
    from supersonic_b200.cache import SequenceCache
    from supersonic_b200.engine import StepEntry
    from supersonic_b200.parts import MIXERS, POSITION_ENCODINGS
    build = part_context(dtype, store)
    mixers = [MIXERS[m.kind](m.params, m.weights, build) for m, _ in specs]
    poss = [None if p is None else POSITION_ENCODINGS[p.kind](p.params, {}, build) for _, p in specs]
    cache = SequenceCache({0: mixers[0].cache_need()}, 1024, 1024, dtype, DEV)
    for m in mixers[1:]:
        assert m.cache_need() == mixers[0].cache_need()
    slot, at, outs = cache.acquire(), 0, [[] for _ in specs]
    for n in pieces:
        ctx = step_context(build, cache, [StepEntry(slot, [0] * n)])
        for i, (mixer, pos) in enumerate(zip(mixers, poss)):
            res = torch.zeros(n, xs[i].shape[1], device=DEV)
            mixer.forward(ctx, xs[i][at:at + n].to(DEV, dtype), res, 0, i == 0, pos)
            outs[i].append(res.cpu())
        cache.advance(slot, n)
        at += n
    cache.check()
    return [torch.cat(o).double() for o in outs]


PIECES = [70, 2, 2, 59] + [1] * 17 + [90, 1, 1, 1, 2]      # crosses page borders; portions of two; token by token
T_ALONE = sum(PIECES)


def rows_for(width, seed, dtype):
    return torch.randn(T_ALONE, width, generator=torch.Generator().manual_seed(seed)).to(dtype)


def tolerance(dtype, ref, loose=0.04):
    return (1e-4 if dtype == torch.float32 else loose) * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,layer", [("A", 1), ("A", 4), ("B", 0), ("B", 4), ("C", 1), ("C", 3), ("D", 2)])
def test_attention_over_convolved_keys_alone(dtype, name, layer):
    """Convolutions of 1 to 16 taps whose state crosses portions of one and two tokens, values that are the keys, a
    temperature that steps every 1 to 40 tokens, a gate per head; one to eight heads over one to five kv heads."""
    cfg, store, plain = tk.build(name)
    block = cfg.build_spec().blocks[layer]
    x = rows_for(cfg.width, layer, dtype)
    ref = pk.conv_attention(x.double(), plain, f"l{layer}.mix", cfg.layers[layer]["mixer"], cfg.norm_eps)
    got, = mixers_alone([(block.mixer, block.position)], store, dtype, [x], PIECES)
    assert float((got - ref).abs().max()) < tolerance(dtype, ref)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,layer", [("A", 0), ("A", 2), ("B", 1), ("B", 2), ("C", 0), ("C", 2), ("D", 0)])
def test_differential_attention_alone(dtype, name, layer):
    """Two maps over the same values inside windows of 1 to 150 tokens against pages of 64; rotation of all, some and
    none of a map's coordinates; capped and uncapped; value rows narrower and wider than a map."""
    cfg, store, plain = tk.build(name)
    block = cfg.build_spec().blocks[layer]
    x = rows_for(cfg.width, layer, dtype)
    ref = pk.diff_attention(x.double(), plain, f"l{layer}.mix", cfg.layers[layer]["mixer"], cfg.norm_eps)
    got, = mixers_alone([(block.mixer, block.position)], store, dtype, [x], PIECES)
    assert float((got - ref).abs().max()) < tolerance(dtype, ref)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,writer,readers", [("A", 0, [3]), ("B", 1, [3, 5]), ("D", 0, [1, 3])])
def test_layers_that_read_another_layers_keys(dtype, name, writer, readers):
    """Readers with longer and shorter windows and other query heads than the layer whose entry they read, fed rows of
    their own: the entry keeps tokens for the longest window, and every reader masks by its own."""
    cfg, store, plain = tk.build(name)
    spec = cfg.build_spec()
    layers = [writer] + readers
    xs = [rows_for(cfg.width, 10 + i, dtype) for i in layers]
    kv = pk.diff_keys_values(xs[0].double(), plain, f"l{writer}.mix", cfg.layers[writer]["mixer"], cfg.norm_eps)
    got = mixers_alone([(spec.blocks[i].mixer, spec.blocks[i].position) for i in layers], store, dtype, xs, PIECES)
    for i, x, g in zip(layers, xs, got):
        ref = pk.diff_attention(x.double(), plain, f"l{i}.mix", cfg.layers[i]["mixer"], cfg.norm_eps, kv=kv)
        assert float((g - ref).abs().max()) < tolerance(dtype, ref), i


@pytest.mark.parametrize("heads,kv_heads,dim,vdim,window,cap,share,gated", [
    (8, 4, 64, 128, 100, 30.0, 2, False), (4, 2, 128, 64, 70, None, 2, False), (12, 4, 40, 80, 150, 25.0, 2, False),
    (4, 2, 64, 64, None, None, 1, True), (8, 1, 128, 128, None, None, 1, True), (6, 3, 96, 96, 33, 9.0, 1, True)])
def test_window_attention_kernels_agree_with_shared_values_and_gates(heads, kv_heads, dim, vdim, window, cap, share, gated):
    """The tensor-core kernel against the plain one in bfloat16 with key heads that share value heads (two score
    maps) and with a gate per head: three sequences of unequal lengths as prompts that continue a cache, and as
    decode steps, with pages in a shuffled order; the two differ by the rounding of the output alone."""
    from supersonic_b200.csrc import ops
    g = torch.Generator(device=DEV).manual_seed(dim + vdim)
    lens, new = [330, 64, 131], [170, 64, 1]
    pages_per, B = 6, 3
    kc = (torch.randn(B * pages_per + 1, kv_heads, 64, dim, device=DEV, generator=g) * 0.6).bfloat16()
    vc = (torch.randn(B * pages_per + 1, kv_heads // share, 64, vdim, device=DEV, generator=g) * 0.6).bfloat16()
    table = (torch.randperm(B * pages_per, device=DEV, generator=g).int() + 1).view(B, pages_per).contiguous()
    for decode in (False, True):
        n_new = [1] * B if decode else new
        T = sum(n_new)
        q = (torch.randn(T, heads * dim + 8, device=DEV, generator=g) * 0.7).bfloat16()
        gate = q[:, heads * dim:] if gated else None
        cu = torch.tensor([0] + list(np.cumsum(n_new)), dtype=torch.int32, device=DEV)
        start = torch.tensor([l - n for l, n in zip(lens, n_new)], dtype=torch.int32, device=DEV)
        slots = torch.arange(B, dtype=torch.int32, device=DEV)
        pos = torch.cat([torch.arange(l - n, l, dtype=torch.int32) for l, n in zip(lens, n_new)]).to(DEV)
        slot_of = torch.cat([torch.full((n,), i, dtype=torch.int32) for i, n in enumerate(n_new)]).to(DEV)
        a, b = (torch.zeros(T, heads * vdim, dtype=torch.bfloat16, device=DEV) for _ in range(2))
        ops.window_attention_plain(q, kc, vc, table, None, pos, slot_of, a, heads, kv_heads, dim, vdim, 6, window, 0, 0,
                                   dim ** -0.5, cap, None, None, None, False, 0.5, v_share=share, gate=gate)
        ops.window_attention_mma(q, kc, vc, table, None, cu, start, slots, b, max(n_new), heads, kv_heads, dim, vdim, 6,
                                 window, 0, 0, dim ** -0.5, cap, None, None, None, False, 0.5, v_share=share, gate=gate)
        torch.cuda.synchronize()
        assert float((a.float() - b.float()).abs().max()) < 0.02 * max(1.0, float(a.float().abs().max())), decode


@pytest.mark.parametrize("dtype", DTYPES)
def test_map_difference_and_norm_and_add(dtype):
    from supersonic_b200.csrc import ops
    g = torch.Generator().manual_seed(2)
    T, H, G, V = 19, 6, 2, 20
    maps = torch.randn(T, G, 2, H // G, V, generator=g).to(dtype)
    out = torch.empty(T, H * V, dtype=dtype, device=DEV)
    ops.map_difference(maps.reshape(T, -1).to(DEV), out, H, G, V, 0.37, 1e-5, 0.6)
    m = maps.double()
    o = (m[:, :, 0] - 0.37 * m[:, :, 1]).reshape(T, H, V)
    ref = (pk.unit_rms(o, 1e-5) * 0.6).reshape(T, -1)
    assert float((out.cpu().double() - ref).abs().max()) < tolerance(dtype, ref, 0.01)
    # the norm behind a sublayer, with the next sublayer's entry norm in the same pass; the branch is zero afterwards
    W = 50
    res, br = torch.randn(T, W, generator=g), torch.randn(T, W, generator=g) * 4
    w1, w2 = torch.randn(W, generator=g), torch.randn(W, generator=g)
    r, b = res.to(DEV), br.to(DEV)
    nxt = torch.empty(T, W, dtype=dtype, device=DEV)
    ops.rms_add(r, b, w1.to(DEV), 1e-4, clear=True, next_weight=w2.to(DEV), next_eps=1e-3, next_out=nxt)
    ref_r = res.double() + pk.unit_rms(br.double(), 1e-4) * w1.double()
    assert float((r.cpu().double() - ref_r).abs().max()) < 1e-5 and float(b.abs().max()) == 0.0
    ref_n = pk.unit_rms(ref_r, 1e-3) * w2.double()
    assert float((nxt.cpu().double() - ref_n).abs().max()) < tolerance(dtype, ref_n, 0.01)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,layer", [("A", 0), ("A", 1), ("A", 3), ("B", 2), ("B", 5), ("C", 1), ("D", 1)])
def test_feed_forwards_alone(dtype, name, layer):
    """The clamped gated unit (inputs beyond the limits on both sides), and experts: 2 to 16 in 1 to 4 groups of which
    1 to 3 are kept, 1 to 4 a token, with and without a gated shared expert."""
    from supersonic_b200.engine import StepEntry
    from supersonic_b200.parts import FEED_FORWARDS
    cfg, store, plain = tk.build(name)
    spec = cfg.build_spec().blocks[layer].feed_forward
    build = part_context(dtype, store)
    ff = FEED_FORWARDS[spec.kind](spec.params, spec.weights, build)
    x = (torch.randn(83, cfg.width, generator=torch.Generator().manual_seed(layer)) * 2.0).to(dtype)
    ref = pk.feed_forward(x.double(), plain, f"l{layer}.mlp", cfg.layers[layer]["mlp"])
    from supersonic_b200.cache import SequenceCache, StateNeed
    cache = SequenceCache({0: StateNeed(1)}, 256, 256, dtype, DEV)
    ctx = step_context(build, cache, [StepEntry(cache.acquire(), [0] * 83)])
    res = torch.zeros(83, cfg.width, device=DEV)
    ff.forward(ctx, x.to(DEV), res)
    assert float((res.cpu().double() - ref).abs().max()) < tolerance(dtype, ref, 0.03)


@pytest.mark.parametrize("rows", [1, 40, 128, 200, 1500])
def test_gated_unit_inside_the_products(rows):
    """The serving set's products that end in the gated unit's inner step (rows streamed against the weights, tiles
    on the tensor cores, groups of rows per expert) against product, then activation, of the plain set: both inner
    steps, with and without a factor per row, inputs beyond the clamp on both sides."""
    from supersonic_b200.csrc.fast_sets import FastKernels
    from supersonic_b200.csrc.kernel_sets import PlainKernels
    from supersonic_b200.csrc import ops
    g = torch.Generator().manual_seed(rows)
    fast, plain = FastKernels(), PlainKernels()
    K, I = 192, 160
    x = (torch.randn(rows, K, generator=g) * 1.5).bfloat16().to(DEV)
    gate, up = ((torch.randn(I, K, generator=g) * 0.15).bfloat16().to(DEV) for _ in range(2))
    scale = torch.rand(rows, generator=g).to(DEV)
    for act in (None, ("clamped_swish", 1.25)):
        for rs in (None, scale):
            outs = []
            for ks in (fast, plain):
                w, layout = ks.pack_gate_up(gate, up)
                out = torch.empty(rows, I, dtype=torch.bfloat16, device=DEV)
                ks.gate_up_swiglu(x, w, layout, out, act=act, row_scale=rs)
                outs.append(out.float())
            ops.check_device_errors()
            assert float((outs[0] - outs[1]).abs().max()) < 0.02 * max(1.0, float(outs[1].abs().max())), (act, rs is None)
    # experts: pairs sorted by expert, rows gathered through the order
    E, top = 6, 2
    expert_of = torch.randint(0, E, (rows, top), generator=g).int().to(DEV)
    w = (torch.randn(E, 2 * I, K, generator=g) * 0.15).bfloat16().to(DEV)
    P = rows * top
    max_tiles = P // 64 + min(E, P)
    ints = torch.empty(E + 1 + P + 2 * max_tiles + 1, dtype=torch.int32, device=DEV)
    groups = {"tile_rows": 64, "max_tiles": max_tiles, "offsets": ints[: E + 1], "order": ints[E + 1: E + 1 + P],
              "tile_expert": ints[E + 1 + P: E + 1 + P + max_tiles],
              "tile_row0": ints[E + 1 + P + max_tiles: E + 1 + P + 2 * max_tiles], "meta": ints[-1:]}
    fast.group_by_expert(expert_of, E, groups)
    for act in (None, ("clamped_swish", 0.75)):
        a, b = (torch.zeros(P, I, dtype=torch.bfloat16, device=DEV) for _ in range(2))
        fast.expert_gate_up(x, top, w, a, groups, act=act)
        plain.expert_gate_up(x, top, w, b, groups, act=act)
        assert float((a.float() - b.float()).abs().max()) < 0.02 * max(1.0, float(b.float().abs().max())), act


def test_router_alone():
    """Choice by score plus correction inside the best groups only, weights from the score alone: corrections large
    enough to change the choice, and negative choice scores in the groups that lose."""
    from supersonic_b200.csrc import ops
    g = torch.Generator().manual_seed(4)
    T, W, E, top, groups, keep = 64, 24, 12, 3, 4, 2
    x, w = torch.randn(T, W, generator=g), torch.randn(E, W, generator=g) * 0.5
    corr, extra = torch.randn(E, generator=g) * 0.8 - 0.9, torch.randn(1, W, generator=g)
    chosen, weight = pk.route(x.double(), {"r.router": w, "r.correction": corr}, "r",
                              {"experts": E, "top": top, "scale": 1.7, "groups": {"count": groups, "keep": keep}})
    eo = torch.empty(T, top, dtype=torch.int32, device=DEV)
    pw, xo = torch.empty(T, top, device=DEV), torch.empty(T, device=DEV)
    logits = torch.cat([x @ w.T, x @ extra.T, torch.zeros(T, 3)], dim=1).to(DEV)
    ops.route_sigmoid_groups(logits, E, corr.to(DEV), groups, keep, 1.7, eo, pw, extra_col=E, extra_out=xo)
    assert eo.cpu().tolist() == chosen
    assert float((pw.cpu().double() - torch.tensor(weight)).abs().max()) < 1e-5
    assert float((xo.cpu().double() - pk.sigmoid(x.double() @ extra.double().T)[:, 0]).abs().max()) < 1e-5


# ---- whole models through the step function --------------------------------------------------------
def test_stream_after_every_layer():
    """float32: the stream after every layer, and the logits, against the plain statement."""
    from supersonic_b200.engine import StepEntry
    for name in ("A", "B", "C", "D"):
        cfg, store, plain = tk.build(name)
        model = make_model(cfg, store, torch.float32)
        tokens = tokens_of(cfg, 90, 3)
        ref, streams = pk.forward(cfg.to_dict(), plain, tokens)
        seen = []
        model.layer_probe = lambda stop, x: seen.append(x.cpu().double())
        slot = model.open_sequence()
        got = model.step([StepEntry(slot, tokens, list(range(len(tokens))))]).cpu().double()
        assert len(seen) == len(streams) == len(cfg.layers)
        for i, s in enumerate(seen):
            assert float((s - streams[i]).abs().max()) < 1e-4 * max(1.0, float(streams[i].abs().max())), (name, i)
        close(got, ref, torch.float32, name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_portions_of_every_size_and_token_by_token(dtype, name):
    cfg, store, plain = build_for(name, dtype)
    model = make_model(cfg, store, dtype)
    T = 150
    tokens = tokens_of(cfg, T, 5)
    ref = reference(cfg, plain, tokens)
    for cuts in ([T], [64, 64, 22], [63, 2, 2, 61, 3, 7, 2, 10], [1] * 6 + [2] * 3 + [138], [100] + [1] * 50, [1] * T):
        close(run_in_portions(model, tokens, cuts), ref, dtype, (name, cuts))
    assert model.cache.slots.n_held == 0
    model.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_unequal_batches_against_each_alone_and_reused_slots(dtype, name):
    """Requests of 1 to 260 tokens start together and decode together, the short ones ending first; then other
    requests run in the slots, pages and convolution rows those gave back."""
    from supersonic_b200.engine import StepEntry
    cfg, store, plain = build_for(name, dtype)
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


def sharpened(name="A", sharp=6.0, dtype=torch.float32):
    """The configuration's weights changed so that faults show: the weights of the norms of q are scaled up, so that
    a query's output stands on the few keys whose scores are high: a key more or less then moves the logits by far
    more than any tolerance."""
    cfg, store, plain = build_for(name, dtype)
    changes = {f"l{i}.mix.q.norm": plain[f"l{i}.mix.q.norm"].float() * sharp for i in range(len(cfg.layers))}
    store, plain = tk.changed(plain, **{k.replace(".", "__"): v for k, v in changes.items()})
    return cfg, store, plain


def _variant(cfg, layer, path, value):
    d = copy.deepcopy(cfg.to_dict())
    at = d["layers"][layer]
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    return d


@pytest.mark.parametrize("dtype", DTYPES)
def test_window_edges_far_tokens_groups_and_page_borders_show(dtype):
    # bfloat16 takes the edges with milder weights: a softmax that stands on one key turns the rounding of a score
    # into another key, which says nothing about the masks
    cfg, store, plain = sharpened("A", 6.0 if dtype == torch.float32 else 2.0, dtype)
    T = 330
    tokens = tokens_of(cfg, T, 9)
    ref = reference(cfg, plain, tokens)
    # the test is sharp: a window one token longer or shorter (the writer's, the reader's), no query temperature (where it steps
    # is pinned by the mixer alone in float32), a group more kept, another offset of the maps' factor, each give other logits at most positions behind the first window ...
    for layer, path, value, share in () if dtype != torch.float32 else (
                                     (0, ("mixer", "mask", "size"), 10, 0.4), (0, ("mixer", "mask", "size"), 8, 0.4),
                                      (3, ("mixer", "mask", "size"), 31, 0.3), (3, ("mixer", "mask", "size"), 29, 0.3),
                                      (2, ("mixer", "mask", "size"), 22, 0.3), (1, ("mixer", "q_temp", "coef"), 0.0, 0.3),
                                      (0, ("mlp", "router", "groups", "keep"), 3, 0.2), (0, ("mixer", "diff"), 0.4, 0.5)):
        other = position_errors(pk.forward(_variant(cfg, layer, path, value), plain, tokens)[0], ref)
        assert float((other[40:] > 0.08).double().mean()) > share and float(other[40:].median()) > 0.02, (layer, path)
    # ... and a sequence that has lost what came 200 and more positions before gives other logits at its end: the
    # layers that see every earlier token read keys far back
    tail = position_errors(pk.forward(cfg.to_dict(), plain, tokens[200:])[0], ref[200:])
    assert float(tail[-30:].min()) > (0.1 if dtype == torch.float32 else 0.02)
    model = make_model(cfg, store, dtype)
    # cuts at window edges (9, 21, 30), one before and one behind them, at page borders (64, 128), the first tokens
    # one by one, and decoding across all of these
    for cuts in ([T], [1, 1, 1, 1, 4, 1, 1, 1, 10, 1, 1, 1, 6, 1, 1, 1, 32, 1, 1, 62, 1, 1, 199],
                 [8, 2, 2, 8, 2, 8, 2, 32, 64] + [1] * 202, [256] + [1] * 74, [2] * 165):
        close(run_in_portions(model, tokens, cuts), ref, dtype, cuts)


def test_long_decoding_keeps_every_state():
    """400 tokens decoded one by one after a prompt of two, in float32: the convolutions' rows and the windows'
    pages are carried over hundreds of steps and several pages, windows pass over decoded tokens only."""
    cfg, store, plain = sharpened("D")
    model = make_model(cfg, store, torch.float32)
    tokens = tokens_of(cfg, 402, 21)
    close(run_in_portions(model, tokens, [2] + [1] * 400), reference(cfg, plain, tokens), torch.float32)


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_point(dtype):
    """Prompts of unequal lengths in batches of three through ``Engine.generate`` (its scheduler, cache and
    sampler): the tokens are those the plain statement picks greedily, and in bfloat16 every picked token
    is the plain statement's first or close second choice."""
    from supersonic_b200.api import Engine
    cfg, store, plain = build_for("B", dtype)
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
    cfg, _, _ = tk.build("A")
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
