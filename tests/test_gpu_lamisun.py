"""Lamisun on the GPU against the plain implementation: each new mechanism alone (the pair
table, the input convolutions, the streams' average, xielu, attention over latent rows,
differential attention within chunks), then the engine over whole requests, decoded tails,
portions down to two tokens, mixed batches with pages and slots used again, keys far away and at
the edges of chunks, long decoding, replayed graphs and greedy generation."""

import math

import pytest
import torch

import plain_lamisun as plain
from lamisun_models import (CONFIGS, PlainModel, assert_rows_close as assert_close, dense,
                            differential, latent, make_model_dir)
from tiny_models import cut, mixed_schedule, prompts, replay

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]
DEVICE = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from mlx_one_b200.kernels import default_ops
    return default_ops(DEVICE)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("lamisun")
    return {name: make_model_dir(name, root) for name in CONFIGS}


@pytest.fixture(scope="module")
def models(folders):
    return {name: PlainModel(folder) for name, folder in folders.items()}


def engine(folder, dtype, page_size, capacity, max_requests=4):
    from mlx_one_b200.cache import CacheManager
    from mlx_one_b200.engine.loading import load_model
    from mlx_one_b200.engine.runner import Runner

    loaded = load_model(folder, dtype, DEVICE)
    cache = CacheManager(loaded.model.cache_needs, page_size=page_size, capacity_tokens=capacity,
                         max_requests=max_requests, dtype=dtype, device=DEVICE)
    return Runner(loaded.model, cache), cache


def runtime(dtype):
    from mlx_one_b200.kernels import default_ops
    from mlx_one_b200.parts import Runtime
    return Runtime(dtype, torch.device(DEVICE), default_ops(DEVICE))


def ints(values):
    return torch.tensor(values, dtype=torch.int32, device=DEVICE)


def context(portions, histories, token_ids=None):
    """A StepContext for requests that bring ``portions`` tokens after ``histories`` tokens."""
    from mlx_one_b200.parts import StepContext

    positions, owner, starts = [], [], [0]
    for r, (n, before) in enumerate(zip(portions, histories)):
        positions += list(range(before, before + n))
        owner += [r] * n
        starts.append(starts[-1] + n)
    ids = [0] * len(positions) if token_ids is None else token_ids
    return StepContext(tokens=len(positions), requests=len(portions), token_ids=ints(ids),
                       positions=ints(positions), token_request=ints(owner),
                       request_start=ints(starts), history=ints(histories),
                       max_portion=max(portions),
                       max_context=max(p + h for p, h in zip(portions, histories)))


def on(tensor):
    return tensor.to(DEVICE)


def schedule_of(lengths, sizes):
    """Steps of a ragged batch: request r brings its tokens in portions of ``sizes[r]`` (cycled);
    a request that has none left drops out. Yields per step [(request, first, count)]."""
    at = [0] * len(lengths)
    turn = 0
    while any(a < n for a, n in zip(at, lengths)):
        step = []
        for r, n in enumerate(lengths):
            if at[r] < n:
                count = min(sizes[r][turn % len(sizes[r])], n - at[r])
                step.append((r, at[r], count))
                at[r] += count
        turn += 1
        yield step


# ------------------------------------------------------------------ the stream's mechanisms


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("vocab, hidden, buckets, mul_prev, mul_cur, scale", [
    (300, 64, 97, 13, 5, 2.0), (70, 40, 1, 7, 11, 1.0), (1000, 136, 4093, 1000003, 0, 0.5),
    (50, 8, 2, 0, 1, 3.0)])
def test_pair_table_in_portions(ops, dtype, vocab, hidden, buckets, mul_prev, mul_cur, scale):
    """Three requests of unequal length in portions (some of one token): the token before a
    portion comes from the request's slot; a slot that is used again starts a sequence anew."""
    from mlx_one_b200.parts import FixedState, StateView

    generator = torch.Generator().manual_seed(vocab)
    table = torch.randn(vocab, hidden, generator=generator).to(dtype)
    pairs = torch.randn(buckets + 1, hidden, generator=generator).to(dtype)
    lengths = (23, 1, 9)
    rule = {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}
    state = torch.zeros(5, 1, dtype=torch.int32, device=DEVICE)
    slots = (3, 0, 4)
    for again in range(2):
        sequences = [torch.randint(0, vocab, (n,), generator=generator).tolist() for n in lengths]
        want = [plain.embed(s, table.double(), scale, pairs.double(), rule) for s in sequences]
        for r in slots:
            state[r] = 0                                  # what the cache does for a new request
        for step in schedule_of(lengths, ((5, 1, 2), (1,), (4, 3))):
            rows = [r for r, _, _ in step]
            ids = [t for r, first, count in step for t in sequences[r][first:first + count]]
            ctx = context([count for _, _, count in step], [first for _, first, _ in step], ids)
            view = StateView(state, ints([slots[r] for r in rows]), FixedState((1,), "int32"))
            got = ops.embedding_pairs(ctx.token_ids, on(table), scale, on(pairs),
                                      rule=(buckets, mul_prev, mul_cur), ctx=ctx, view=view)
            expect = torch.cat([want[r][first:first + count] for r, first, count in step])
            assert (got.cpu().double() - expect).abs().max() < 1e-5, f"pass {again}"
    bare = ops.embedding_pairs(ints([1, 2]), on(table), scale, None, rule=None,
                               ctx=context([2], [0], [1, 2]), view=None)
    assert (bare.cpu().double() - table[[1, 2]].double() * scale).abs().max() < 1e-6
    ops.check_errors()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps, hidden", [(1, 72), (2, 64), (3, 40), (4, 192), (5, 130), (7, 8)])
def test_input_convolution_in_portions(ops, dtype, taps, hidden):
    """x + conv(x) for both sublayers of a layer, requests side by side in portions shorter and
    longer than the taps; the rows before a portion come from the slot (32-bit, unrounded)."""
    from mlx_one_b200.parts import FixedState, StateView

    generator = torch.Generator().manual_seed(taps)
    lengths = (31, 2, 12, 1)
    kernels = [0.5 * torch.randn(hidden, taps, generator=generator) for _ in range(2)]
    streams = [[torch.randn(n, hidden, generator=generator) for n in lengths] for _ in range(2)]
    want = [[plain.input_convolution(x.double(), w.double()) for x in xs]
            for xs, w in zip(streams, kernels)]
    state = torch.full((6, 2, max(taps - 1, 1), hidden), 7.0, device=DEVICE)
    slots = (5, 1, 2, 0)
    for r in slots:
        state[r] = 0
    need = FixedState((2, taps - 1, hidden), "float32")
    tolerance = 1e-5 if dtype == torch.float32 else 0.04
    for step in schedule_of(lengths, ((1, 2, 9, 1), (2,), (3, 1), (1,))):
        ctx = context([count for _, _, count in step], [first for _, first, _ in step])
        view = StateView(state[:, :, :taps - 1], ints([slots[r] for r, _, _ in step]), need) \
            if taps > 1 else None
        for sublayer in range(2):
            x = torch.cat([streams[sublayer][r][first:first + count] for r, first, count in step])
            got = ops.stream_conv(on(x), on(kernels[sublayer]), taps=taps, ctx=ctx, view=view,
                                  sublayer=sublayer, write=True, dtype=dtype)
            expect = torch.cat([want[sublayer][r][first:first + count] for r, first, count in step])
            assert got.dtype == dtype
            assert (got.cpu().double() - expect).abs().max() < tolerance, f"sublayer {sublayer}"
    rounded = ops.stream_conv(on(streams[0][0]), None, taps=0, ctx=context([31], [0]), view=None,
                              sublayer=0, write=True, dtype=dtype)
    assert torch.equal(rounded.cpu(), streams[0][0].to(dtype))


@pytest.mark.parametrize("count, tokens, hidden", [(2, 1, 72), (3, 5, 64), (9, 300, 192), (33, 7, 40)])
def test_streams_average(ops, count, tokens, hidden):
    generator = torch.Generator().manual_seed(count)
    kept = torch.randn(count + 1, tokens, hidden, generator=generator)
    weights = torch.randn(count, generator=generator)
    want = (kept[:count].double() * weights.double()[:, None, None]).sum(0)
    device = on(kept)
    got = ops.stream_average(device, on(weights), count, device[count])
    assert got.data_ptr() == device[count].data_ptr()
    assert (got.cpu().double() - want).abs().max() < 1e-5
    assert torch.equal(device[:count].cpu(), kept[:count])
    copy = ops.stream_average(device, None, 1, device[1])
    assert torch.equal(copy.cpu(), kept[0])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("p, q", [(0.3, -0.2), (-2.0, 1.5), (0.0, 0.0), (4.0, -6.0)])
def test_xielu(ops, dtype, p, q):
    """Both branches, zero itself, and values far enough below zero that e^z vanishes."""
    z = torch.cat([torch.linspace(-30, 30, 4001), torch.tensor([0.0, -0.0, 1e-4, -1e-4])]).to(dtype)
    want = plain.xielu(z.double(), p, q)
    params = (plain.softplus(p), 0.5 + plain.softplus(q))
    got = ops.activation(on(z), "xielu", params).cpu().double()
    error = (got - want).abs() / (1 + want.abs())
    assert error.max() < (1e-5 if dtype == torch.float32 else 6e-3)
    generator = torch.Generator().manual_seed(3)
    for rows in (3, 200):
        x = torch.randn(rows, 96, generator=generator).to(dtype)
        w = (torch.randn(160, 96, generator=generator) / 96 ** 0.5).to(dtype)
        got = ops.linear_act(on(x), on(w), "xielu", params).cpu().double()
        want = plain.xielu(x.double() @ w.double().T, p, q)
        error = (got - want).abs() / (1 + want.abs())
        assert error.max() < (1e-4 if dtype == torch.float32 else 0.03)


# ------------------------------------------------------------------ the two mixers alone


def page_tables(lengths, page, generator, spare=3):
    """Distinct pages in a random order for requests of the given lengths: (table [requests,
    width] int32 on the host, pages in the pool)."""
    blocks = [-(-n // page) for n in lengths]
    pool = sum(blocks) + spare
    order = torch.randperm(pool, generator=generator).tolist()
    table = torch.full((len(lengths), max(blocks)), -1, dtype=torch.int32)
    for r, count in enumerate(blocks):
        table[r, :count] = torch.tensor([order.pop() for _ in range(count)], dtype=torch.int32)
    return table, pool


def run_mixer(part, need, kv, table, page, inputs, sizes, dtype):
    """A mixer over requests side by side, each in portions of ``sizes[r]``; returns its outputs
    per request. Requests that have ended drop out, so rows of the table move between steps."""
    from mlx_one_b200.parts import PagedView

    lengths = [x.shape[0] for x in inputs]
    outputs = [[] for _ in inputs]
    for step in schedule_of(lengths, sizes):
        rows = [r for r, _, _ in step]
        ctx = context([count for _, _, count in step], [first for _, first, _ in step])
        view = PagedView(kv, on(table[rows].contiguous()), page, need)
        x = torch.cat([inputs[r][first:first + count] for r, first, count in step]).to(dtype)
        got = part.forward(on(x), ctx, view, True).float().cpu()
        at = 0
        for r, _, count in step:
            outputs[r].append(got[at:at + count])
            at += count
    part.ops.check_errors()
    return [torch.cat(parts) for parts in outputs]


LATENT_SIZES = [
    # heads, dim, rot_dim, vdim, kv_rank, hidden, page
    (4, 24, 16, 32, 48, 64, 16),
    (3, 4, 6, 20, 40, 96, 8),           # a row of 46 values
    (1, 8, 2, 12, 16, 32, 4),
    (6, 32, 32, 16, 96, 128, 16),
    (2, 10, 4, 24, 18, 72, 2),
    (16, 64, 32, 64, 128, 256, 32),
    (5, 48, 64, 40, 192, 80, 16),       # a row of 256 values
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, dim, rot_dim, vdim, kv_rank, hidden, page", LATENT_SIZES)
def test_latent_attention_part(dtype, heads, dim, rot_dim, vdim, kv_rank, hidden, page):
    """Whole sequences, then the same in portions and single tokens beside each other, against
    the plain mixer that builds every head's keys and values from the latents."""
    from mlx_one_b200.parts import MIXERS, PartSpec

    generator = torch.Generator().manual_seed(heads * 100 + dim)
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
         "scale": 1.7 / math.sqrt(dim + rot_dim), "rot": {"base": 300.0, "dims": rot_dim}}
    shapes = {"q": (heads * (dim + rot_dim), hidden), "dkv": (kv_rank + rot_dim, hidden),
              "uk": (heads * dim, kv_rank), "uv": (heads * vdim, kv_rank),
              "g": (heads * vdim, hidden), "o": (hidden, heads * vdim)}
    w = {name: (1.5 * torch.randn(shape, generator=generator) / shape[1] ** 0.5).to(dtype)
         for name, shape in shapes.items()}
    w["dkv.norm"] = (1 + 0.2 * torch.randn(kv_rank, generator=generator)).to(dtype)
    spec = PartSpec("latent_attention", {
        "hidden": hidden, "heads": heads, "head_dim": dim, "rot_dim": rot_dim, "value_dim": vdim,
        "latent": kv_rank, "eps": 1e-5, "scale": m["scale"], "gate": True,
        "position": PartSpec("rope_long", {"theta": 300.0, "rotary_dim": rot_dim,
                                           "layout": "neighbours", "factor": None})})
    roles = {"q": "q", "down": "dkv", "down_norm": "dkv.norm", "up_k": "uk", "up_v": "uv",
             "gate": "g", "out": "o"}
    part = MIXERS.get("latent_attention")(spec, {role: on(w[name]) for role, name in roles.items()},
                                          runtime(dtype))
    need = MIXERS.get("latent_attention").cache_need(spec)
    assert need.planes == 1 and need.kv_heads == 1 and need.head_dim == kv_rank + rot_dim
    lengths = (75, 33, 6)
    inputs = [torch.randn(n, hidden, generator=generator).to(dtype).float() for n in lengths]
    wide = {name: t.double() for name, t in w.items()}
    want = [plain.latent_attention(x.double(), wide, m, 1e-5, "") for x in inputs]
    table, pool = page_tables(lengths, page, generator)
    tolerance = 2e-4 if dtype == torch.float32 else 0.08
    for sizes in (((1000,),) * 3, ((7, 1, 1, 20, 2), (1,), (2, 3))):
        kv = torch.full((1, pool, 1, page, kv_rank + rot_dim), 50.0, dtype=dtype, device=DEVICE)
        got = run_mixer(part, need, kv, table, page, inputs, sizes, dtype)
        for r, (a, b) in enumerate(zip(got, want)):
            spread = b.pow(2).mean().sqrt()
            assert (a.double() - b).abs().max() < tolerance * max(float(spread), 1.0), \
                f"request {r}, portions {sizes[r]}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, latent_size, rot_dim", [(8, 64, 16), (3, 40, 6), (16, 128, 32),
                                                        (20, 200, 24), (16, 512, 64), (5, 72, 8)])
def test_latent_rows_far_away(ops, dtype, heads, latent_size, rot_dim):
    """One row near the start of 900 matches the last queries by far: their outputs are that
    row's latent, in a prompt's portion and for single tokens of requests side by side."""
    from mlx_one_b200.parts import PagedKeyValues, PagedView

    generator = torch.Generator().manual_seed(heads)
    T, page, row = 900, 16, latent_size + rot_dim
    rows = 0.3 * torch.randn(T, row, generator=generator)
    q = 0.3 * torch.randn(T, heads, row, generator=generator)
    rows[3, 5] = 6.0
    rows[3, 6:latent_size] = 1.5
    q[-40:, :, 5] = 8.0
    scale = 0.2
    rows, q = rows.to(dtype), q.to(dtype)
    scores = torch.einsum("thd,sd->hts", q.double(), rows.double()) * scale
    weights = plain.softmax_rows(scores, plain.visible(T))
    want = torch.einsum("hts,sd->thd", weights, rows.double()[:, :latent_size])
    assert want[-1, :, 6].min() > 0.5                    # the far row is what the output is
    table, pool = page_tables((T,), page, generator)
    kv = torch.full((1, pool, 1, page, row), 100.0).to(dtype)
    for t in range(T):
        kv[0, table[0, t // page], 0, t % page] = rows[t]
    need = PagedKeyValues(1, row, planes=1)
    tolerance = 1e-4 if dtype == torch.float32 else 0.04
    for portions, histories in (([40], [T - 40]), ([T], [0]), ([1] * 3, [T - 1, T - 2, T - 3]),
                                ([333, 1, 70], [T - 333, 63, 58]),
                                ([1] * 30, [T - 1 - i for i in range(30)]), ([2, 1], [T - 2, 4])):
        ctx = context(portions, histories)
        positions = ctx.positions.tolist()
        view = PagedView(on(kv), on(table.repeat(len(portions), 1).contiguous()), page, need)
        got = ops.latent_attention(on(q[positions]).contiguous(), heads=heads, latent=latent_size,
                                   scale=scale, ctx=ctx, view=view).cpu().double()
        assert (got[:, :, :latent_size] - want[positions]).abs().max() < tolerance, str(portions)
    ops.check_errors()


DIFFERENTIAL_SIZES = [
    # heads, kv_heads, dim, vdim, chunk, hidden, page, diff
    (4, 2, 16, 32, 24, 64, 16, 0.5),
    (3, 3, 24, 8, 5, 96, 8, 0.3),
    (1, 1, 16, 16, None, 32, 4, 0.8),
    (4, 1, 64, 64, 100, 128, 16, 0.6),
    (2, 2, 8, 40, 1, 72, 2, 0.2),
    (6, 2, 8, 24, 1000, 72, 16, 0.4),
    (8, 4, 128, 128, 37, 192, 32, 0.7),
    (4, 4, 32, 64, 16, 64, 16, 0.0),    # chunks that are pages
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, dim, vdim, chunk, hidden, page, diff", DIFFERENTIAL_SIZES)
def test_differential_attention_part(dtype, heads, kv_heads, dim, vdim, chunk, hidden, page, diff):
    from mlx_one_b200.parts import MIXERS, PartSpec

    generator = torch.Generator().manual_seed(heads * 100 + dim)
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff,
         "scale": 2.0 / math.sqrt(dim)}
    if chunk is not None:
        m["mask"] = {"size": chunk}
    shapes = {"q": (heads * 2 * dim, hidden), "k": (kv_heads * 2 * dim, hidden),
              "v": (kv_heads * vdim, hidden), "o": (hidden, heads * vdim)}
    w = {name: (1.5 * torch.randn(shape, generator=generator) / shape[1] ** 0.5).to(dtype)
         for name, shape in shapes.items()}
    for name in ("q.norm", "k.norm"):
        w[name] = (1 + 0.2 * torch.randn(dim, generator=generator)).to(dtype)
    for name in ("lq1", "lk1", "lq2", "lk2"):
        w[name] = (0.7 * torch.randn(dim, generator=generator) / dim ** 0.5).to(dtype)
    spec = PartSpec("differential_attention", {
        "hidden": hidden, "heads": heads, "kv_heads": kv_heads, "head_dim": dim, "value_dim": vdim,
        "eps": 1e-5, "scale": m["scale"], "diff": diff, "chunk": chunk})
    roles = {"q": "q", "k": "k", "v": "v", "q_norm": "q.norm", "k_norm": "k.norm", "out": "o",
             "lq1": "lq1", "lk1": "lk1", "lq2": "lq2", "lk2": "lk2"}
    kind = MIXERS.get("differential_attention")
    part = kind(spec, {role: on(w[name]) for role, name in roles.items()}, runtime(dtype))
    need = kind.cache_need(spec)
    assert need.kv_heads == 2 * kv_heads and need.chunk == chunk
    lengths = (75, 33, 6)
    inputs = [torch.randn(n, hidden, generator=generator).to(dtype).float() for n in lengths]
    wide = {name: t.double() for name, t in w.items()}
    want = [plain.differential_attention(x.double(), wide, m, 1e-5, "") for x in inputs]
    table, pool = page_tables(lengths, page, generator)
    tolerance = 3e-4 if dtype == torch.float32 else 0.1
    for sizes in (((1000,),) * 3, ((7, 1, 1, 20, 2), (1,), (2, 3))):
        kv = torch.full((2, pool, need.kv_heads, page, need.head_dim), 50.0, dtype=dtype,
                        device=DEVICE)
        got = run_mixer(part, need, kv, table, page, inputs, sizes, dtype)
        for r, (a, b) in enumerate(zip(got, want)):
            spread = b.pow(2).mean().sqrt()
            assert (a.double() - b).abs().max() < tolerance * max(float(spread), 1.0), \
                f"request {r}, portions {sizes[r]}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("value_dim, row_dim, mix", [(8, 24, -0.7), (64, 64, 1.3), (40, 40, 0.0),
                                                     (16, 32, 2.5)])
def test_two_maps_combined(ops, dtype, value_dim, row_dim, mix):
    generator = torch.Generator().manual_seed(value_dim)
    heads, tokens = 3, 37
    maps = torch.randn(tokens, 2, heads, row_dim, generator=generator).to(dtype)
    first, second = maps.double()[:, 0, :, :value_dim], maps.double()[:, 1, :, :value_dim]
    o = first - float(torch.tensor(mix, dtype=torch.float32)) * second
    want = (o / plain.rms(o, 1e-6) * 0.4).reshape(tokens, heads * value_dim)
    got = ops.differential_combine(on(maps).view(tokens, -1), heads=heads, row_dim=row_dim,
                                   value_dim=value_dim, mix=mix, eps=1e-6, factor=0.4)
    assert (got.cpu().double() - want).abs().max() < (1e-5 if dtype == torch.float32 else 0.02)


def chunk_edges(T, heads, kv_heads, dim, chunk, generator):
    """Queries, keys and values of one sequence in which, for every third query beyond the
    first chunk, the last key of the chunk before (just outside) matches head 0 best by far and
    the first key of the query's own chunk (just inside) matches head 1 of the same key head:
    chunks that are one position off show as wholly different outputs."""
    q = 0.3 * torch.randn(T, heads, dim, generator=generator)
    k = 0.3 * torch.randn(T, kv_heads, dim, generator=generator)
    v = 0.1 * torch.randn(T, kv_heads, dim, generator=generator)
    second = 1 if heads // kv_heads > 1 else None
    for start in range(chunk, T, chunk):
        k[start - 1, 0] = 0.05 * torch.randn(dim, generator=generator)
        k[start - 1, 0, 0] = 6.0
        v[start - 1, 0] = 3.0
        if second is not None and chunk > 1:
            k[start, 0, 1] = 6.0
            v[start, 0] = -2.0
    for i in range(chunk, T):
        if i % 3 == 0 or i % chunk in (0, chunk - 1):
            q[i, 0, 0] = 8.0
            if second is not None:
                q[i, second, 1] = 8.0
    return q, k, v


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, dim, chunk, page, T", [
    (4, 2, 32, 24, 16, 200), (2, 2, 64, 5, 8, 90), (8, 2, 16, 100, 16, 420), (4, 1, 128, 16, 16, 130),
    (3, 3, 40, 33, 4, 150), (2, 1, 32, 1, 16, 70), (4, 2, 64, 120, 16, 700)])
def test_chunk_edges_in_prompts_and_decoding(ops, dtype, heads, kv_heads, dim, chunk, page, T):
    """Keys just inside and just outside a chunk's start, read by a prompt in one piece, by
    portions that cut chunks and pages, and by single tokens of requests side by side."""
    from mlx_one_b200.parts import PagedKeyValues, PagedView

    generator = torch.Generator().manual_seed(T)
    q, k, v = (x.to(dtype) for x in chunk_edges(T, heads, kv_heads, dim, chunk, generator))
    mask = plain.visible(T, chunk)
    want = torch.zeros(T, heads, dim, dtype=torch.float64)
    for head in range(heads):
        group = head // (heads // kv_heads)
        scores = (q[:, head].double() @ k[:, group].double().T) * 0.25
        want[:, head] = plain.softmax_rows(scores, mask) @ v[:, group].double()
    inside_differs = (want[chunk:, 0] - want[chunk:, min(1, heads - 1)]).abs().max()
    assert heads // kv_heads < 2 or chunk < 2 or inside_differs > 1.0
    table, pool = page_tables((T,), page, generator)
    kv = torch.full((2, pool, kv_heads, page, dim), 100.0).to(dtype)
    for t in range(T):
        kv[0, table[0, t // page], :, t % page] = k[t]
        kv[1, table[0, t // page], :, t % page] = v[t]
    need = PagedKeyValues(kv_heads, dim, chunk=chunk)
    tolerance = 1e-4 if dtype == torch.float32 else 0.05
    first_of_last = (T - 1) // chunk * chunk
    cases = [([T], [0]), ([T - 50, 9], [50, 3]), ([1] * 4, [T - 1, first_of_last, first_of_last - 1, chunk]),
             ([1] * 40, [T - 1 - i for i in range(40)]), ([2, 1, 7], [first_of_last - 1, 0, max(chunk - 3, 0)])]
    for portions, histories in cases:
        ctx = context(portions, histories)
        positions = ctx.positions.tolist()
        view = PagedView(on(kv), on(table.repeat(len(portions), 1).contiguous()), page, need)
        got = ops.paged_attention(on(q[positions]).contiguous(), heads=heads, kv_heads=kv_heads,
                                  head_dim=dim, scale=0.25, window=None, chunk=chunk, ctx=ctx,
                                  view=view).cpu().double().view(-1, heads, dim)
        assert (got - want[positions]).abs().max() < tolerance, f"{portions} after {histories}"
    ops.check_errors()


# ------------------------------------------------------------------ the engine


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_requests_and_first_tokens(folders, models, name, dtype):
    config, _, page = CONFIGS[name]
    runner, cache = engine(folders[name], dtype, page, 256)
    for tokens in prompts(config["vocab"], (150, 1, 2, 5), seed=3):
        got = replay(runner, cache, [([("w", tokens)], ["w"])])["w"]
        assert_close(got, models[name].logits(tokens), dtype, f"{name} whole {len(tokens)}")


def test_the_stream_after_every_layer(folders, models):
    for name in ("L1", "L4"):
        config, _, page = CONFIGS[name]
        runner, cache = engine(folders[name], torch.float32, page, 64)
        (tokens,) = prompts(config["vocab"], (19,), seed=2)
        seen = []
        runner.model.observer = lambda place, residual, delta: seen.append(residual.clone())
        replay(runner, cache, [([("r", tokens)], ["r"])])
        runner.model.observer = None
        states = []
        models[name].logits(tokens, states)
        assert len(seen) == len(states) == len(config["layers"]) + 1
        for place, (got, want) in enumerate(zip(seen, states)):
            # (a step's rows may be padded to a shape that is replayed)
            got = got[:len(tokens)].cpu().double()
            assert (got - want).abs().max() < 2e-4, f"{name} after call {place - 1}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_prefill_against_token_by_token(folders, models, name, dtype):
    config, _, page = CONFIGS[name]
    runner, cache = engine(folders[name], dtype, page, 128)
    (tokens,) = prompts(config["vocab"], (70,), seed=4)
    want = models[name].logits(tokens)
    whole = replay(runner, cache, [([("w", tokens)], ["w"])])["w"]
    steps = [([("d", [token])], []) for token in tokens]
    steps[-1] = (steps[-1][0], ["d"])
    single = replay(runner, cache, steps)["d"]
    assert_close(whole, want, dtype, f"{name} whole")
    assert_close(single, want, dtype, f"{name} token by token")
    if dtype == torch.float32:
        assert (whole - single).abs().max() < 2e-4


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_portions_of_changing_size(folders, models, name, dtype):
    config, _, page = CONFIGS[name]
    runner, cache = engine(folders[name], dtype, page, 192)
    (tokens,) = prompts(config["vocab"], (170,), seed=5)
    want = models[name].logits(tokens)
    for sizes in ((7, 2, 40, 3, 1, 1), (2,), (64, 1), (33, 31)):
        steps = [([("p", part)], []) for part in cut(tokens, sizes)]
        steps[-1] = (steps[-1][0], ["p"])
        assert_close(replay(runner, cache, steps)["p"], want, dtype, f"{name} portions {sizes}")
    assert not cache.requests()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_mixed_batches_with_pages_and_slots_used_again(folders, models, name, dtype):
    config, _, page = CONFIGS[name]
    lengths = (150, 64, 23, 50, 17, 9, 2, 1, 40)
    requests = dict(enumerate(prompts(config["vocab"], lengths, seed=6)))
    runner, cache = engine(folders[name], dtype, page, 4 * 192, max_requests=4)
    got = replay(runner, cache, mixed_schedule(requests))
    for key, tokens in requests.items():
        assert_close(got[key], models[name].logits(tokens), dtype, f"{name} mixed request {key}")
        alone = replay(runner, cache, [([("alone", tokens)], ["alone"])])["alone"]
        if dtype == torch.float32:
            assert (alone - got[key]).abs().max() < 2e-4, f"{name} request {key} beside others"
    assert not cache.requests()
    cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["L1", "L2"])
def test_steps_of_a_repeated_shape_are_replayed(folders, models, name, dtype):
    """Single tokens of three requests step after step: the runner captures the step's shape and
    replays it with other tokens, positions and tables; the logits stay the plain model's."""
    config, _, page = CONFIGS[name]
    runner, cache = engine(folders[name], dtype, page, 512, max_requests=3)
    requests = dict(zip("abc", prompts(config["vocab"], (60, 41, 52), seed=7)))
    steps = [([(key, tokens[:20]) for key, tokens in requests.items()], [])]
    for i in range(20, 60):
        live = [(key, [tokens[i]]) for key, tokens in requests.items() if i < len(tokens)]
        steps.append((live, [key for key, tokens in requests.items() if i == len(tokens) - 1]))
    got = replay(runner, cache, steps)
    for key, tokens in requests.items():
        assert_close(got[key], models[name].logits(tokens), dtype, f"{name} request {key}")
    assert not cache.requests()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_over_chunks_and_far_rows(tmp_path, dtype):
    """A prompt in portions that cut pages and chunks, then 260 tokens decoded one by one, so
    that several chunks start and end among decoded tokens; the third token still moves the last
    logits through the latent layers (the plain model says by how much)."""
    config = {"architecture": "Lamisun", "vocab": 200, "width": 64, "norm": {"eps": 1e-5},
              "canon": {"taps": 4},
              "embedding": {"scale": 1.5, "bigram": {"buckets": 211, "mul_prev": 17, "mul_cur": 3}},
              "layers": [latent(4, 16, 8, 16, 32, 0.2, 10000.0, dense(128)),
                         differential(4, 2, 16, 16, 0.25, 0.55, 70, dense(128)),
                         latent(2, 24, 16, 40, 56, 0.16, 50000.0, None),
                         differential(2, 1, 32, 24, 0.18, 0.35, 48, dense(96))]}
    folder = make_model_dir("L1", tmp_path, config)
    model = PlainModel(folder)
    (tokens,) = prompts(config["vocab"], (640,), seed=21)
    want = model.logits(tokens)
    changed = list(tokens)
    changed[2] = (changed[2] + 1) % config["vocab"]
    moved = (model.logits(changed)[-1] - want[-1]).abs().max()
    runner, cache = engine(folder, dtype, 16, 640, max_requests=2)
    sizes = [209, 129, 2, 3, 37] + [1] * 260
    assert sum(sizes) == len(tokens)
    steps, at = [], 0
    for size in sizes:
        steps.append(([("long", tokens[at:at + size])], []))
        at += size
    steps[-1] = (steps[-1][0], ["long"])
    got = replay(runner, cache, steps)["long"]
    assert_close(got, want, dtype, "long decoding")
    if dtype == torch.float32:
        assert moved > 1e-3 and moved > 20 * (got[-1].cpu() - want[-1]).abs().max(), \
            "the first tokens no longer show at the end"


def test_greedy_generation_through_the_entry_point(folders, models):
    from mlx_one_b200 import BatchingConfig, CacheConfig, Engine, TextGenerationOptions

    for name, dtype in (("L1", "float32"), ("L4", "float32"), ("L2", "bfloat16")):
        config, _, page = CONFIGS[name]
        engine_ = Engine(folders[name], execution_dtype=dtype,
                         cache_config=CacheConfig(block_size_tokens=page, capacity_tokens=512),
                         batching_config=BatchingConfig(max_sequences=3, prefill_chunk_size=16))
        batch = prompts(config["vocab"], (7, 30, 3, 19, 12), seed=8)
        results = engine_.generate_batch_ids(batch, TextGenerationOptions(max_tokens=12, ignore_eos=True))
        if dtype == "float32":
            for prompt, result in zip(batch, results):
                assert list(result.token_ids) == models[name].greedy(prompt, 12)
        else:
            assert all(len(result.token_ids) == 12 for result in results)
        engine_.close()


def test_command_line_and_trace_replay(folders, models, tmp_path):
    """`mlx-one generate` with token ids (greedy against the plain model) and `trace_run` as a
    process: steps on standard input, logits files out, requests ended and their slots used
    again."""
    import json
    import subprocess
    import sys
    from pathlib import Path

    import numpy as np

    root = Path(__file__).resolve().parent.parent
    folder = folders["L1"]
    greedy = subprocess.run([sys.executable, str(root / "bin" / "mlx-one"), "generate", str(folder),
                             "5 17 3 200", "--token-ids", "--max-tokens", "6", "--dtype", "float32"],
                            capture_output=True, text=True, timeout=600)
    assert greedy.returncode == 0, greedy.stderr
    assert [int(t) for t in greedy.stdout.split()] == models["L1"].greedy([5, 17, 3, 200], 6)

    vocab = CONFIGS["L1"][0]["vocab"]
    a, b, c = prompts(vocab, (21, 9, 30), seed=17)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:8], "want": [0, 7]},
                                     {"id": "b", "tokens": b, "want": [8]}], "end": ["b"]},
             {"step": 1, "entries": [{"id": "a", "tokens": a[8:20], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[20:], "want": [0]},
                                     {"id": "c", "tokens": c[:2], "want": [1]}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "c", "tokens": c[2:], "want": [27]}], "end": ["c"]}]
    out = tmp_path / "logits"
    done = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(folder),
                           "--dtype", "float32", "--out", str(out), "--max-tokens", "128",
                           "--max-requests", "2"],
                          input="".join(json.dumps(step) + "\n" for step in steps),
                          capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr
    assert [line for line in done.stdout.split("\n") if line.startswith("done")] == \
        [f"done {i}" for i in range(4)]
    read = lambda step, rows: torch.from_numpy(np.fromfile(out / f"{step}.f32", dtype="<f4")).view(rows, vocab)
    assert not (out / "1.f32").exists()
    wa, wb, wc = (models["L1"].logits(t) for t in (a, b, c))
    close = lambda got, want: (got - want).abs().max() < 2e-4
    assert close(read(0, 3), torch.stack([wa[0], wa[7], wb[8]]))
    assert close(read(2, 2), torch.stack([wa[20], wc[1]]))
    assert close(read(3, 1), wc[29:30])
