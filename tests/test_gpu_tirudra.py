"""Tirudra on the GPU against the plain implementation: each new mechanism alone, then the
engine over whole requests, decoded tails, portions down to two tokens, mixed batches with
pages and slots used again, keys at the edges of windows, among the kept first tokens and far
away, long decoding, replayed graphs, and greedy generation through the entry point."""

import math

import pytest
import torch

from plain_tirudra import (PlainModel, conv_over_time, masked_attention, routing,
                           selective_state_space, silu, softplus, unit_rms)
from tiny_models import cut, mixed_schedule, prompts, replay
from tirudra_models import (CONFIGS, T5, assert_rows_close as assert_close, conv_attention,
                            make_model_dir, routed, shared_attention, sliced, state_space, turns,
                            write_model)

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]
DEVICE = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from mlx_one_b200.kernels import default_ops
    return default_ops(DEVICE)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("tirudra")
    return {name: make_model_dir(name, root) for name in CONFIGS}


@pytest.fixture(scope="module")
def plain(folders):
    return {name: PlainModel(folder) for name, folder in folders.items()}


def engine(folder, dtype, page_size, capacity, max_requests=4):
    from mlx_one_b200.cache import CacheManager
    from mlx_one_b200.engine.loading import load_model
    from mlx_one_b200.engine.runner import Runner

    loaded = load_model(folder, dtype, DEVICE)
    cache = CacheManager(loaded.model.cache_needs, page_size=page_size, capacity_tokens=capacity,
                         max_requests=max_requests, dtype=dtype, device=DEVICE)
    return Runner(loaded.model, cache), cache


def context(portions, histories, leading_single=0):
    """A StepContext for requests that bring ``portions`` tokens after ``histories`` tokens."""
    from mlx_one_b200.parts import StepContext

    ints = lambda values: torch.tensor(values, dtype=torch.int32, device=DEVICE)
    positions, owner, starts = [], [], [0]
    for r, (n, before) in enumerate(zip(portions, histories)):
        positions += list(range(before, before + n))
        owner += [r] * n
        starts.append(starts[-1] + n)
    return StepContext(tokens=len(positions), requests=len(portions), token_ids=ints([0] * len(positions)),
                       positions=ints(positions), token_request=ints(owner),
                       request_start=ints(starts), history=ints(histories),
                       max_portion=max(portions), max_context=max(p + h for p, h in zip(portions, histories)),
                       leading_single=leading_single)


def on(tensor):
    return tensor.to(DEVICE)


def slots_view(shape, dtype, slots, count=6):
    """A state group's view with ``count`` slots full of NaN but for the given ones (zero, as
    the cache manager hands them out)."""
    from mlx_one_b200.parts import FixedState, StateView

    state = torch.full((count, *shape), float("nan"), dtype=dtype, device=DEVICE)
    state[slots] = 0
    return StateView(state, torch.tensor(slots, dtype=torch.int32, device=DEVICE),
                     FixedState(tuple(shape)))


# ------------------------------------------------------------------ mechanisms alone


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("channels, taps, activation, bias", [
    (40, 3, None, False), (204, 2, "silu", True), (96, 4, "silu", True), (7, 1, None, True),
    (130, 5, None, False)])
def test_convolution_over_time(ops, dtype, channels, taps, activation, bias):
    """Two requests of 37 and 50 tokens in one step, in portions of 1 to 20 tokens, and token by
    token, the inputs a slice of wider rows: the state carries the last taps - 1 rows."""
    generator = torch.Generator().manual_seed(channels + taps)
    lengths = (37, 50)
    rows = [torch.randn(n, channels + 24, generator=generator).to(dtype) for n in lengths]
    kernel = torch.randn(channels, taps, generator=generator)
    b = torch.randn(channels, generator=generator) if bias else None
    act = silu if activation else (lambda z: z)
    want = [act(conv_over_time(r[:, 8:8 + channels].double(), kernel.double(),
                               None if b is None else b.double())) for r in rows]
    tolerance = 1e-5 if dtype == torch.float32 else 0.03
    for sizes in ((37,), (5, 1, 2, 20, 1, 1, 3), (1,)):
        view = slots_view((max(taps - 1, 1), channels), dtype, [4, 1]) if taps > 1 else None
        done = [0, 0]
        got = [[], []]
        for index in range(64):
            size = sizes[index % len(sizes)]
            portions = [min(size, n - d) for n, d in zip(lengths, done)]
            live = [r for r in range(2) if portions[r] > 0]
            if not live:
                break
            step = torch.cat([rows[r][done[r]:done[r] + portions[r]] for r in live])
            ctx = context([portions[r] for r in live], [done[r] for r in live])
            if view is not None:
                view.slots = torch.tensor([[4, 1][r] for r in live], dtype=torch.int32, device=DEVICE)
            out = ops.channel_conv(on(step)[:, 8:8 + channels], on(kernel), None if b is None else on(b),
                                   taps=taps, activation=activation, ctx=ctx, view=view, write=True)
            at = 0
            for r in live:
                got[r].append(out[at:at + portions[r]].cpu())
                at += portions[r]
                done[r] += portions[r]
        for r in range(2):
            error = (torch.cat(got[r]).double() - want[r]).abs().max()
            assert error < tolerance * max(1.0, float(want[r].abs().max())), (sizes, r, float(error))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, value_dim, state_dim, groups", [
    (4, 16, 16, 2), (3, 20, 24, 3), (4, 64, 128, 1), (1, 8, 4, 1), (2, 40, 200, 2), (6, 32, 64, 3)])
def test_state_space_recurrence(ops, dtype, heads, value_dim, state_dim, groups):
    """Two requests in one step (one long enough for segments that run side by side), in
    portions of 1 to 300 tokens and token by token, with a state that forgets slowly; the other
    slots are full of NaN."""
    generator = torch.Generator().manual_seed(heads * 100 + state_dim)
    lengths = (330, 75)
    inner, wide = heads * value_dim, groups * state_dim
    a_log = -2.5 + 0.8 * torch.randn(heads, generator=generator)
    dt_bias = -1.0 + 0.5 * torch.randn(heads, generator=generator)
    skip = torch.randn(heads, generator=generator)
    mixed = [(0.5 * torch.randn(n, inner + 2 * wide, generator=generator)).to(dtype) for n in lengths]
    steps = [torch.randn(n, heads + 5, generator=generator).to(dtype) for n in lengths]
    want = []
    for m, s in zip(mixed, steps):
        m, n = m.double(), m.shape[0]
        dt = softplus(s[:, 3:3 + heads].double() + dt_bias.double())
        want.append(selective_state_space(
            m[:, :inner].view(n, heads, value_dim), m[:, inner:inner + wide].view(n, groups, state_dim),
            m[:, inner + wide:].view(n, groups, state_dim), dt, torch.exp(a_log.double()),
            skip.double()).reshape(n, inner))
    for sizes in ((330,), (7, 1, 300, 2, 1, 1), (1,), (140, 3)):
        view = slots_view((heads * state_dim * value_dim,), torch.float32, [2, 5])
        done = [0, 0]
        got = [[], []]
        for index in range(400):
            size = sizes[index % len(sizes)]
            portions = [min(size, n - d) for n, d in zip(lengths, done)]
            live = [r for r in range(2) if portions[r] > 0]
            if not live:
                break
            ctx = context([portions[r] for r in live], [done[r] for r in live])
            view.slots = torch.tensor([[2, 5][r] for r in live], dtype=torch.int32, device=DEVICE)
            m = torch.cat([mixed[r][done[r]:done[r] + portions[r]] for r in live])
            s = torch.cat([steps[r][done[r]:done[r] + portions[r]] for r in live])
            y = ops.state_space_scan(on(m), on(s)[:, 3:3 + heads], a_log=on(a_log), dt_bias=on(dt_bias),
                                     skip=on(skip), ctx=ctx, view=view, write=True, heads=heads,
                                     value_dim=value_dim, state_dim=state_dim, groups=groups)
            at = 0
            for r in live:
                got[r].append(y[at:at + portions[r]].cpu())
                at += portions[r]
                done[r] += portions[r]
        for r in range(2):
            error = (torch.cat(got[r]).double() - want[r]).abs().max()
            assert error < 2e-4 * max(1.0, float(want[r].abs().max())), (sizes, r, float(error))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("inner, groups", [(64, 2), (60, 1), (256, 4), (8, 8), (1536, 3)])
def test_gate_and_norm_in_parts(ops, dtype, inner, groups):
    generator = torch.Generator().manual_seed(inner)
    y = torch.randn(19, inner, generator=generator)
    gate = torch.randn(19, inner + 16, generator=generator).to(dtype)
    weight = 1 + 0.2 * torch.randn(inner, generator=generator)
    v = (y.double() * silu(gate[:, 16:].double())).view(19, groups, -1)
    want = (unit_rms(v, 1e-5).reshape(19, inner) * weight.double())
    got = ops.gated_group_norm(on(y), on(gate)[:, 16:], on(weight), groups=groups, eps=1e-5, dtype=dtype)
    assert (got.cpu().double() - want).abs().max() < (1e-5 if dtype == torch.float32 else 0.03)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, row_dim, value_dim, per_head", [
    (4, 32, 32, False), (3, 40, 24, False), (6, 48, 48, True), (2, 40, 24, True)])
def test_gates_on_the_heads_outputs(ops, dtype, heads, row_dim, value_dim, per_head):
    generator = torch.Generator().manual_seed(heads + row_dim)
    mixed = torch.randn(11, heads * row_dim, generator=generator).to(dtype)
    width = heads * (1 if per_head else value_dim)
    gate = torch.randn(11, width + 8, generator=generator).to(dtype)
    g = torch.sigmoid(gate[:, 8:].double())
    g = g.view(11, heads, 1) if per_head else g.view(11, heads, value_dim)
    want = (mixed.double().view(11, heads, row_dim)[:, :, :value_dim] * g).reshape(11, -1)
    got = ops.gate_heads(on(mixed), on(gate)[:, 8:], heads=heads, row_dim=row_dim,
                         value_dim=value_dim, per_head=per_head)
    assert (got.cpu().double() - want).abs().max() < (1e-6 if dtype == torch.float32 else 0.03)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("experts, identity, top, shared", [
    (6, 2, 3, True), (5, 0, 1, False), (2, 1, 3, False), (16, 3, 5, True), (3, 1, 2, True)])
def test_routing_with_a_correction_and_identity_outputs(ops, dtype, experts, identity, top, shared):
    """The choice goes by score + correction, the weights are the scores; identity outputs' weights
    are summed; the shared expert's gate is a sigmoid. Corrections are large enough to move the
    choice away from the best scores."""
    generator = torch.Generator().manual_seed(experts * 10 + top)
    hidden, tokens, outputs = 72, 50, experts + identity
    x = torch.randn(tokens, hidden + 8, generator=generator).to(dtype)
    router = torch.randn(outputs + (1 if shared else 0), hidden, generator=generator) / hidden ** 0.5
    correction = 0.3 * torch.randn(outputs, generator=generator)
    h = x[:, 8:].double()
    want = routing(h, router[:outputs].double(), correction.double(), top)
    plain_choice = routing(h, router[:outputs].double(), torch.zeros(outputs, dtype=torch.float64), top)
    assert top == outputs or ((want > 0) != (plain_choice > 0)).any()
    weights, others = ops.route_general(on(x)[:, 8:], on(router), on(correction), experts=experts,
                                        identity=identity, top=top, scores="softmax",
                                        normalize=False, shared_gate=shared)
    assert (weights.cpu().double() - want[:, :experts]).abs().max() < 1e-5
    assert (others[0].cpu().double() - want[:, experts:].sum(-1)).abs().max() < 1e-5
    if shared:
        gate = torch.sigmoid(h @ router[outputs].double())
        assert (others[1].cpu().double() - gate).abs().max() < 1e-5
    out = torch.randn(tokens, hidden, generator=generator).to(dtype)
    summed = out.double() + h * others[0].cpu().double()[:, None]
    moved = on(out).clone()
    ops.add_scaled_rows(moved, on(x)[:, 8:], others[0])
    assert (moved.cpu().double() - summed).abs().max() < (1e-5 if dtype == torch.float32 else 0.05)


def paged(keys, values, page, dtype, generator, missing=()):
    """One request's keys and values [T, G, D] in pages handed out in a random order; what no
    token has written holds large numbers (a key or value read from there would show), and the
    blocks in ``missing`` have no page at all, as if they had been given back."""
    T, G, D = keys.shape
    blocks = -(-T // page)
    pages = blocks + 3
    order = torch.randperm(pages - 1, generator=generator)[:blocks]
    kv = torch.full((2, pages, G, page, D), 100.0).to(dtype)
    for t in range(T):
        kv[0, order[t // page], :, t % page] = keys[t].to(dtype)
        kv[1, order[t // page], :, t % page] = values[t].to(dtype)
    table = order.to(torch.int32)
    for block in missing:
        kv[:, table[block]] = float("nan")
        table[block] = -1
    return kv, table[None, :].contiguous()


def edge_case(T, heads, kv_heads, dim, window, keep, generator):
    """Queries, keys and values of one sequence in which, for every third query behind the
    window's first reach, the key just outside the window matches head 0 best by far (unless it
    is one of the kept first tokens, it must not be seen), the last kept token matches the last
    head (it must be seen from everywhere) and the first token that is not kept matches nothing
    but is large: a window or a kept run that is one token off shows as another output."""
    q = 0.3 * torch.randn(T, heads, dim, generator=generator)
    k = 0.3 * torch.randn(T, kv_heads, dim, generator=generator)
    v = 0.1 * torch.randn(T, kv_heads, dim, generator=generator)
    if keep:
        k[keep - 1, -1] = 0.05 * torch.randn(dim, generator=generator)
        k[keep - 1, -1, 2] = 6.0
        v[keep - 1, -1] = 2.0
    if keep < T:
        k[keep, -1, 2] = 5.0            # the first token behind the kept ones: seen only in a window
        v[keep, -1] = -4.0
    for i in range(max(window, 1), T):
        if i % 3:
            continue
        outside = i - window
        if outside > keep:
            k[outside, 0] = 0.05 * torch.randn(dim, generator=generator)
            k[outside, 0, 0] = 6.0
            v[outside, 0] = 3.0
        q[i, 0, 0] = 8.0
        q[i, heads - 1, 2] = 7.0
    return q, k, v


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, dim, window, keep, page, T", [
    (4, 2, 32, 24, 3, 4, 90), (6, 2, 96, 33, 16, 16, 150), (3, 3, 40, 7, 9, 8, 60),
    (8, 1, 64, 100, 4, 16, 330), (2, 1, 16, 1, 1, 2, 12), (4, 4, 128, 64, 70, 8, 300),
    (10, 1, 48, 200, 33, 16, 700), (2, 2, 64, 40, 0, 16, 130)])
def test_window_edges_and_kept_first_tokens(ops, dtype, heads, kv_heads, dim, window, keep, page, T):
    """softmax over the window and the kept first tokens: whole prompts, a prompt's second
    portion, single tokens (several key splits where the window is long), against the plain
    function. The pages between the kept tokens and the window are gone for the late queries."""
    from mlx_one_b200.parts import PagedKeyValues, PagedView

    generator = torch.Generator().manual_seed(heads * 1000 + dim + window)
    q, k, v = edge_case(T, heads, kv_heads, dim, window, keep, generator)
    scale = 0.7 / math.sqrt(dim)
    round_trip = lambda x: x.to(dtype).double()
    want = masked_attention(round_trip(q), round_trip(k), round_trip(v), scale, window,
                            keep).reshape(T, -1)
    need = PagedKeyValues(kv_heads, dim, window, keep_first=keep)
    kv, table = paged(k, v, page, dtype, generator)
    view = PagedView(on(kv), on(table), page, need)
    call = lambda queries, ctx, view: ops.paged_attention(
        on(queries.to(dtype)).contiguous(), heads=heads, kv_heads=kv_heads, head_dim=dim,
        scale=scale, window=window, keep_first=keep, ctx=ctx, view=view).cpu().double()
    tolerance = 1e-4 if dtype == torch.float32 else 0.05
    got = call(q, context([T], [0]), view)
    assert (got - want).abs().max() < tolerance, "whole prompt"
    half = T // 2 + 1
    got = call(q[half:], context([T - half], [half]), view)
    assert (got - want[half:]).abs().max() < tolerance, "second portion"
    # the last tokens alone, with every page gone that no query from there on can see
    tail = max(T - 12, 1)
    first_needed = max(tail - window + 1, 0) // page
    gone = [b for b in range(-(-keep // page), first_needed)]
    kv, table = paged(k, v, page, dtype, generator, missing=gone)
    view = PagedView(on(kv), on(table), page, need)
    for t in range(tail, T):
        got = call(q[t:t + 1], context([1], [t]), view)
        assert (got - want[t:t + 1]).abs().max() < tolerance, f"token {t} alone"
    got = call(q[tail:], context([T - tail], [tail]), view)
    assert (got - want[tail:]).abs().max() < tolerance, "the tail as a portion"
    # four requests' single tokens in one step (the same sequence at four positions)
    spots = [T - 1, T - 2, T - 5, T - 9] if T > 12 else [T - 1] * 4
    view = PagedView(on(kv), on(table.repeat(4, 1)), page, need)
    ctx = context([1] * 4, spots)
    got = call(q[spots], ctx, view)
    assert (got - want[spots]).abs().max() < tolerance, "single tokens side by side"


# ------------------------------------------------------------------ the engine


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_requests_decoded_tails_and_portions(folders, plain, dtype, name):
    config, _, page = CONFIGS[name]
    runner, cache = engine(folders[name], dtype, page, 512)
    (tokens,) = prompts(config["vocab"], (140,), seed=11)
    want = plain[name].logits(tokens)
    got = replay(runner, cache, [([("w", tokens)], ["w"])])["w"]
    assert_close(got, want, dtype, f"{name} whole")
    steps = [([("d", tokens[:60])], [])] + [([("d", [t])], []) for t in tokens[60:]]
    steps[-1] = (steps[-1][0], ["d"])
    assert_close(replay(runner, cache, steps)["d"], want, dtype, f"{name} decoded tail")
    steps = [([("s", [t])], []) for t in tokens[:50]]
    steps[-1] = (steps[-1][0], ["s"])
    assert_close(replay(runner, cache, steps)["s"], sliced(want, 50), dtype, f"{name} token by token")
    for sizes in ((7, 2, 40, 3, 1), (2,), (33, 1, 1)):
        steps = [([("p", part)], []) for part in cut(tokens, sizes)]
        steps[-1] = (steps[-1][0], ["p"])
        assert_close(replay(runner, cache, steps)["p"], want, dtype, f"{name} portions {sizes}")
    cache.check()
    assert not cache.requests()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["T1", "T2", "T3", "T5"])
def test_mixed_batches_with_pages_and_slots_used_again(folders, plain, dtype, name):
    """Ten unequal requests through four slots and a pool of 256 tokens, twice (the second
    time the steps come from CUDA graphs where their shapes repeat)."""
    config, _, page = CONFIGS[name]
    lengths = (40, 64, 23, 50, 17, 9, 2, 1, 33, 70)
    requests = dict(enumerate(prompts(config["vocab"], lengths, seed=12)))
    want = {key: plain[name].logits(tokens) for key, tokens in requests.items()}
    runner, cache = engine(folders[name], dtype, page, 256, max_requests=4)
    for turn in range(2):
        got = replay(runner, cache, mixed_schedule(requests))
        for key in requests:
            assert_close(got[key], want[key], dtype, f"{name} turn {turn} request {key}")
        cache.check()
        assert not cache.requests()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_past_windows_and_pages(folders, plain, dtype):
    """A prompt of 50 tokens and 400 decoded ones: the windows pass over decoded tokens, pages
    behind them come back while the first tokens' stay, the state space carries on."""
    config, _, page = CONFIGS["T5"]
    runner, cache = engine(folders["T5"], dtype, page, 512, max_requests=2)
    (tokens,) = prompts(config["vocab"], (450,), seed=13)
    want = plain["T5"].logits(tokens)
    steps = [([("d", tokens[:50])], [])] + [([("d", [t])], []) for t in tokens[50:]]
    steps[-1] = (steps[-1][0], ["d"])
    assert_close(replay(runner, cache, steps)["d"], want, dtype, "long decoding")


def test_the_state_space_remembers_the_first_tokens(tmp_path):
    """A model of state spaces alone that forget slowly: the plain model says how much the
    third token still moves the logits 300 tokens later, and the engine (prompt in portions,
    then single tokens) follows it."""
    config = {"architecture": "Tirudra", "vocab": 90, "width": 48, "norm": {"eps": 1e-5},
              "logit_scale": 1.0,
              "layers": [state_space(2, 24, 16, 1, 2, 1, None), state_space(3, 16, 8, 3, 3, 1, None)]}
    folder = write_model(tmp_path, config, 77)
    from plain_tirudra import read_tensors
    from mlx_one_b200.weights.safetensors_io import write_safetensors
    tensors = read_tensors(folder / "model.safetensors")
    for name in tensors:
        if name.endswith("A_log"):
            tensors[name] = torch.full_like(tensors[name], -6.0)
    write_safetensors(folder / "model.safetensors", tensors, {"format": "pt"})
    plain = PlainModel(folder)
    (tokens,) = prompts(90, (320,), seed=14)
    other = list(tokens)
    other[2] = (other[2] + 1) % 90
    want, moved = plain.logits(tokens), plain.logits(other)
    assert (want[-1] - moved[-1]).abs().max() > 0.02        # the third token still counts
    runner, cache = engine(folder, torch.float32, 16, 512)
    steps = [([("r", part)], []) for part in cut(tokens[:200], (64, 3, 130))]
    steps += [([("r", [t])], []) for t in tokens[200:]]
    steps[-1] = (steps[-1][0], ["r"])
    assert_close(replay(runner, cache, steps)["r"], want, torch.float32, "a slow state")


def test_greedy_generation_through_the_entry_point(folders, plain):
    """The engine's own entry point and scheduler: prompts in portions of eight tokens, three
    requests at a time, greedy tokens against the plain model's."""
    from mlx_one_b200 import BatchingConfig, CacheConfig, Engine, TextGenerationOptions

    config, _, page = CONFIGS["T5"]
    batch = prompts(config["vocab"], (7, 30, 3, 19, 45), seed=15)
    for dtype in ("float32", "bfloat16"):
        engine_ = Engine(folders["T5"], execution_dtype=dtype, device=DEVICE,
                         cache_config=CacheConfig(block_size_tokens=page, capacity_tokens=512),
                         batching_config=BatchingConfig(max_sequences=3, prefill_chunk_size=8))
        results = engine_.generate_batch_ids(batch, TextGenerationOptions(max_tokens=12, ignore_eos=True))
        for prompt, result in zip(batch, results):
            want = plain["T5"].greedy(prompt, 12)
            got = list(result.token_ids)
            if dtype == "float32":
                assert got == want
            else:
                assert got[:3] == want[:3]          # (a later near-tie may fall the other way)
        engine_.close()
