"""Lamisun without a GPU: configuration, the weight names, what the cache keeps, and the
engine's bookkeeping (the token before a step, the inputs before a step's convolutions, the
streams of all layers, pages of chunks, single-plane pages) run with the plain kernel set
against the plain model."""

import copy
import json

import pytest
import torch

from lamisun_models import CONFIGS, L1, L2, L3, L4, PlainModel, assert_rows_close, make_model_dir
from plain_ops import PlainOps
from tiny_models import cut, mixed_schedule, prompts, replay


def engine(folder, page_size, capacity, max_requests=4):
    from mlx_one_b200.cache import CacheManager
    from mlx_one_b200.engine.loading import load_model
    from mlx_one_b200.engine.runner import Runner

    loaded = load_model(folder, "float32", "cpu", PlainOps())
    cache = CacheManager(loaded.model.cache_needs, page_size=page_size, capacity_tokens=capacity,
                         max_requests=max_requests, dtype=torch.float32, device="cpu")
    return Runner(loaded.model, cache), cache


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("lamisun_cpu")
    return {name: make_model_dir(name, root) for name in CONFIGS}


# ------------------------------------------------------------------ configuration


def test_config_round_trip_and_registry(tmp_path):
    from mlx_one_b200.config import LamisunConfig, read_config

    for name, (config, _, _) in CONFIGS.items():
        typed = LamisunConfig.from_dict(config)
        assert LamisunConfig.from_dict(typed.to_dict()) == typed, name
    (tmp_path / "config.json").write_text(json.dumps(L1))
    entry, typed = read_config(tmp_path)
    assert entry.name == "lamisun" and typed.width == 64 and typed.taps == 3
    assert typed.bigram.buckets == 97 and typed.bigram.mul_prev == 13 and typed.embedding_scale == 2.0
    assert typed.layers[0].mixer.kv_rank == 48 and typed.layers[0].mixer.rot.dims == 16
    assert typed.layers[1].mixer.chunk == 24 and typed.layers[1].mixer.diff == 0.5
    assert typed.layers[2].mlp is None and typed.layers[1].mlp.ff == 80
    three = LamisunConfig.from_dict(L3)
    assert three.bigram is None and three.taps is None and three.layers[1].mixer.chunk is None


@pytest.mark.parametrize("path, value, text", [
    (("layers", 0, "type"), "lightning", "type"),
    (("layers", 1, "mixer", "kv_heads"), 3, "kv_heads"),
    (("layers", 0, "mixer", "rot", "dims"), 7, "dims"),
    (("layers", 0, "mixer", "rot", "dims"), 64, "dims"),
    (("layers", 1, "mixer", "mask", "size"), 0, "mask.size"),
    (("layers", 0, "mlp", "kind"), "moe", "kind"),
    (("layers", 0, "mixer", "kv_rank"), 0, "kv_rank"),
    (("embedding", "bigram", "buckets"), 0, "buckets"),
    (("embedding", "bigram", "mul_prev"), -1, "mul_prev"),
    (("canon", "taps"), 0, "taps"),
    (("norm", "eps"), -1.0, "eps"),
])
def test_config_rejections(path, value, text):
    from mlx_one_b200.config import ConfigError, LamisunConfig

    config = copy.deepcopy(L1)
    at = config
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(ConfigError, match=text):
        LamisunConfig.from_dict(config)


def test_missing_key_is_named():
    from mlx_one_b200.config import ConfigError, LamisunConfig

    config = copy.deepcopy(L1)
    del config["layers"][0]["mixer"]["rot"]["base"]
    with pytest.raises(ConfigError, match=r"layers\[0\]\.mixer\.rot\.base"):
        LamisunConfig.from_dict(config)
    config = copy.deepcopy(L1)
    del config["layers"][1]["mixer"]["diff"]
    with pytest.raises(ConfigError, match=r"layers\[1\]\.mixer\.diff"):
        LamisunConfig.from_dict(config)


def test_weight_names_and_what_the_cache_keeps():
    from mlx_one_b200.architectures.lamisun import describe
    from mlx_one_b200.config import LamisunConfig
    from mlx_one_b200.parts import FixedState, PagedKeyValues, cache_entries, expected_tensors

    spec = describe(LamisunConfig.from_dict(L1))
    names = expected_tensors(spec)
    assert names["bigram"].shape == (98, 64) and names["embed"].shape == (300, 64)
    assert names["l0.mix.q"].shape == (4 * 40, 64) and names["l0.mix.dkv"].shape == (64, 64)
    assert names["l0.mix.dkv.norm"].shape == (48,) and names["l0.mix.uk"].shape == (96, 48)
    assert names["l0.mix.uv"].shape == (128, 48) and names["l0.mix.g"].shape == (128, 64)
    assert names["l1.mix.q"].shape == (4 * 2 * 16, 64) and names["l1.mix.k"].shape == (64, 64)
    assert names["l1.mix.v"].shape == (64, 64) and names["l1.mix.lq2"].shape == (16,)
    assert names["l1.mix.q.norm"].shape == (16,) and names["l1.mlp.act"].shape == (2,)
    assert names["l0.canon1"].shape == (64, 3) and names["l2.dwa"].shape == (4,)
    assert "l2.canon2" not in names and "l2.norm2" not in names and "l2.mlp.up" not in names
    needs = cache_entries(spec)
    assert needs[0] == PagedKeyValues(1, 64, planes=1)            # one row [latent | shared key]
    assert needs[1] == PagedKeyValues(4, 32, chunk=24)            # both maps' key heads
    assert needs[(0, "block:inputs")] == FixedState((2, 2, 64), "float32")
    assert needs[(2, "block:inputs")] == FixedState((1, 2, 64), "float32")
    assert FixedState((1,), "int32") in needs.values()           # the token before a step
    bare = cache_entries(describe(LamisunConfig.from_dict(L3)))
    assert all(isinstance(need, PagedKeyValues) for need in bare.values()) and len(bare) == 2


def test_a_wrong_tensor_is_one_error(folders, tmp_path):
    from mlx_one_b200.engine.loading import load_model
    from mlx_one_b200.weights import WeightError
    from mlx_one_b200.weights.safetensors_io import write_safetensors
    from plain_lamisun import read_tensors

    tensors = read_tensors(folders["L1"] / "model.safetensors")
    del tensors["l0.mix.dkv.norm"]
    tensors["l1.dwa"] = tensors["l1.dwa"][:2]
    tensors["extra.one"] = torch.zeros(2, dtype=torch.bfloat16)
    write_safetensors(tmp_path / "model.safetensors", tensors, {"format": "pt"})
    (tmp_path / "config.json").write_text(json.dumps(L1))
    with pytest.raises(WeightError) as caught:
        load_model(tmp_path, "float32", "cpu", PlainOps())
    text = str(caught.value)
    assert "l0.mix.dkv.norm" in text and "l1.dwa" in text and "extra.one" in text


# ------------------------------------------------------------------ the engine's bookkeeping


@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_portions_and_single_tokens(folders, name):
    config, _, page = CONFIGS[name]
    plain = PlainModel(folders[name])
    runner, cache = engine(folders[name], page, 256)
    (tokens,) = prompts(config["vocab"], (90,), seed=4)
    want = plain.logits(tokens)
    got = replay(runner, cache, [([("w", tokens)], ["w"])])["w"]
    assert_rows_close(got, want, torch.float32, f"{name} whole")
    for sizes in ((7, 2, 13, 1, 1, 3), (2,)):
        steps = [([("r", part)], []) for part in cut(tokens, sizes)]
        steps[-1] = (steps[-1][0], ["r"])
        assert_rows_close(replay(runner, cache, steps)["r"], want, torch.float32, f"{name} {sizes}")
    assert not cache.requests()


def test_the_stream_after_every_layer(folders):
    runner, cache = engine(folders["L4"], 16, 64)
    (tokens,) = prompts(L4["vocab"], (19,), seed=2)
    seen = []
    runner.model.observer = lambda place, residual, delta: seen.append(residual.clone())
    replay(runner, cache, [([("r", tokens)], ["r"])])
    runner.model.observer = None
    states = []
    PlainModel(folders["L4"]).logits(tokens, states)
    assert len(seen) == len(states) == 5
    for place, (got, want) in enumerate(zip(seen, states)):
        assert (got.double() - want).abs().max() < 1e-4, f"after call {place - 1}"


@pytest.mark.parametrize("name", ["L1", "L2", "L5"])
def test_mixed_batches_with_pages_and_slots_used_again(folders, name):
    config, _, page = CONFIGS[name]
    plain = PlainModel(folders[name])
    lengths = (40, 30, 23, 50, 17, 9, 2, 1)
    requests = dict(enumerate(prompts(config["vocab"], lengths, seed=5)))
    runner, cache = engine(folders[name], page, 4 * 64, max_requests=4)
    got = replay(runner, cache, mixed_schedule(requests))
    for request_id, tokens in requests.items():
        assert_rows_close(got[request_id], plain.logits(tokens), torch.float32,
                          f"{name} mixed request {request_id}")
    assert not cache.requests()
    cache.check()


def test_pages_of_ended_chunks_come_back(folders):
    """A request far longer than the pool of the chunked layers: the pages of chunks that have
    ended are handed out again, and the logits stay those of the plain model. (The layer that
    sees every earlier token keeps all its pages, so it bounds the request; its pool is larger.)"""
    from mlx_one_b200.cache import CacheManager
    from mlx_one_b200.parts import PagedKeyValues

    config, _, page = CONFIGS["L2"]                         # chunks of 5, pages of 8
    runner, cache = engine(folders["L2"], page, 208, max_requests=1)
    chunked = [group for group in cache.paged if group.need.chunk]
    assert len(chunked) == 1 and len(chunked[0].entries) == 2
    (tokens,) = prompts(config["vocab"], (200,), seed=6)
    steps = [([("r", part)], []) for part in cut(tokens, (5, 1, 9, 2))]
    steps[-1] = (steps[-1][0], ["r"])
    got = replay(runner, cache, steps)["r"]
    assert_rows_close(got, PlainModel(folders["L2"]).logits(tokens), torch.float32, "a long request")
    # the bookkeeping alone: a chunked group never holds more than its reach plus a step
    alone = CacheManager({0: PagedKeyValues(2, 8, chunk=5)}, page_size=8, capacity_tokens=32,
                         max_requests=1, dtype=torch.float32, device="cpu", allocate=False)
    alone.open("x")
    most = 0
    for _ in range(100):
        alone.grow("x", 3)
        alone.advance("x", 3)
        most = max(most, sum(page >= 0 for page in alone.get("x").tables[0]))
    assert most <= 2
    alone.close("x")
    alone.check()


def test_greedy_generation_through_the_entry_point(folders):
    """The engine's own entry point and scheduler: prompts in portions of eight tokens, three
    requests at a time, greedy tokens against the plain model's."""
    from mlx_one_b200 import BatchingConfig, CacheConfig, Engine, TextGenerationOptions

    config, _, page = CONFIGS["L1"]
    plain = PlainModel(folders["L1"])
    batch = prompts(config["vocab"], (7, 30, 3, 19), seed=8)
    engine_ = Engine(folders["L1"], execution_dtype="float32", ops=PlainOps(), device="cpu",
                     cache_config=CacheConfig(block_size_tokens=page, capacity_tokens=256),
                     batching_config=BatchingConfig(max_sequences=3, prefill_chunk_size=8))
    results = engine_.generate_batch_ids(batch, TextGenerationOptions(max_tokens=6, ignore_eos=True))
    for prompt, result in zip(batch, results):
        assert list(result.token_ids) == plain.greedy(prompt, 6)
    engine_.close()
