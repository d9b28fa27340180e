"""Tirudra without a GPU: configuration, the weight contract, the plain functions against each
other, and the engine's bookkeeping (pages of windows that keep first tokens, state slots of
convolutions and state spaces) run with the plain kernel set against the plain model."""

import copy
import json

import pytest
import torch

from plain_ops import PlainOps
from plain_tirudra import (PlainModel, conv_over_time, masked_attention, routing,
                           selective_state_space, stretched_frequencies)
from tiny_models import cut, mixed_schedule, prompts, replay
from tirudra_models import CONFIGS, T1, T2, T4, assert_rows_close, make_model_dir


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
    root = tmp_path_factory.mktemp("tirudra_cpu")
    return {name: make_model_dir(name, root) for name in CONFIGS}


# ------------------------------------------------------------------ configuration


def test_config_round_trip_and_registry(tmp_path):
    from mlx_one_b200.config.registry import read_config
    from mlx_one_b200.config.tirudra import TirudraConfig

    for name, (config, _, _) in CONFIGS.items():
        typed = TirudraConfig.from_dict(config)
        assert TirudraConfig.from_dict(typed.to_dict()) == typed, name
    (tmp_path / "config.json").write_text(json.dumps(T1))
    entry, typed = read_config(tmp_path)
    assert entry.name == "tirudra" and typed.width == 64 and typed.logit_scale == 0.5
    first, second, third = typed.layers[0].mixer, typed.layers[1].mixer, typed.layers[2].mixer
    assert (first.state, first.groups, first.conv, first.norm_groups) == (16, 2, 4, 2)
    assert (second.window, second.keep_first, second.conv) == (24, 3, 4)
    assert second.rot.scaling == {"factor": 4.0, "original": 64.0, "fast": 8.0, "slow": 1.0}
    assert third.rot.scaling["high"] == 3.0 and typed.layers[2].mlp is None
    assert typed.layers[0].mlp.identity == 2 and typed.layers[0].mlp.shared_ff == 40
    two = TirudraConfig.from_dict(T2)
    assert two.layers[3].mixer.window is None and two.layers[3].mixer.rot is None
    assert two.layers[0].mlp.identity == 0 and two.layers[0].mlp.shared_ff is None


@pytest.mark.parametrize("path, value, text", [
    (("layers", 0, "type"), "lightning", "type"),
    (("layers", 1, "mixer", "kv_heads"), 3, "kv_heads"),
    (("layers", 1, "mixer", "rot", "dims"), 7, "dims"),
    (("layers", 1, "mixer", "rot", "scaling"), {"factor": 2.0, "original": 8, "low": 1, "high": 2},
     "scaling"),
    (("layers", 1, "mixer", "mask", "keep_first"), -1, "keep_first"),
    (("layers", 2, "mixer", "vdim"), 16, "vdim"),
    (("layers", 0, "mixer", "groups"), 3, "groups"),
    (("layers", 0, "mixer", "norm_groups"), 5, "norm_groups"),
    (("layers", 0, "mlp", "router", "top"), 9, "top"),
    (("layers", 0, "mlp", "kind"), "dense", "kind"),
    (("norm",), {}, "norm.eps"),
])
def test_config_errors_name_the_key(path, value, text):
    from mlx_one_b200.config.base import ConfigError
    from mlx_one_b200.config.tirudra import TirudraConfig

    config = copy.deepcopy(T1)
    at = config
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(ConfigError) as caught:
        TirudraConfig.from_dict(config)
    assert text in str(caught.value)


def test_a_missing_key_is_named():
    from mlx_one_b200.config.base import ConfigError
    from mlx_one_b200.config.tirudra import TirudraConfig

    config = copy.deepcopy(T1)
    del config["layers"][0]["mixer"]["state"]
    with pytest.raises(ConfigError, match=r"layers\[0\]\.mixer\.state"):
        TirudraConfig.from_dict(config)


def test_the_weight_contract():
    from mlx_one_b200.architectures.tirudra import describe
    from mlx_one_b200.config.tirudra import TirudraConfig
    from mlx_one_b200.parts import cache_entries, expected_tensors

    spec = describe(TirudraConfig.from_dict(T2))
    names = {name: tuple(want.shape) for name, want in expected_tensors(spec).items()}
    assert names["l0.mix.q"] == (72, 72) and names["l0.mix.v"] == (40, 72)
    assert names["l0.mix.q.conv"] == (72, 2) and names["l0.mix.v.conv"] == (40, 2)
    assert names["l0.mix.g"] == (120, 72) and names["l0.mix.o"] == (72, 120)
    assert names["l0.mix.q.norm"] == (24,) and names["l0.norm1b"] == (72,)
    assert names["l1.mix.in"] == (60 + 60 + 2 * 72 + 3, 72) and names["l1.mix.conv"] == (204, 2)
    assert names["l1.mix.conv.b"] == (204,) and names["l1.mix.norm"] == (60,)
    assert "l1.norm2" not in names and "l1.norm2b" not in names
    assert names["l2.mix.g"] == (3, 72) and names["l2.mix.q.b"] == (48,) and "l2.mix.v" not in names
    assert names["l3.mlp.router"] == (4, 72) and names["l3.mlp.correction"] == (4,)
    assert names["l3.mlp.shared.sg"] == (1, 72) and "l0.mlp.shared.sg" not in names
    assert "l3.mix.q.norm" in names and names["head"] == (100, 72)
    needs = cache_entries(spec)
    assert needs[(0, "pages")].window == 7 and needs[(0, "pages")].keep_first == 9
    assert needs[(0, "inputs")].shape == (1, 72 + 24 + 40)
    assert needs[(1, "state")].shape == (3 * 24 * 20,) and needs[(1, "state")].dtype == "float32"
    assert needs[2].window is None and needs[(3, "pages")].window is None


def test_a_wrong_tensor_is_one_error(folders, tmp_path):
    from mlx_one_b200.engine.loading import load_model
    from mlx_one_b200.weights import WeightError
    from mlx_one_b200.weights.safetensors_io import write_safetensors
    from plain_tirudra import read_tensors

    tensors = read_tensors(folders["T1"] / "model.safetensors")
    del tensors["l1.mix.k.conv"]
    tensors["l0.mlp.correction"] = tensors["l0.mlp.correction"][:3]
    tensors["l2.mix.v"] = torch.zeros(64, 64, dtype=torch.bfloat16)
    write_safetensors(tmp_path / "model.safetensors", tensors, {"format": "pt"})
    (tmp_path / "config.json").write_text(json.dumps(T1))
    with pytest.raises(WeightError) as caught:
        load_model(tmp_path, "float32", "cpu", PlainOps())
    text = str(caught.value)
    assert "l1.mix.k.conv" in text and "l0.mlp.correction" in text and "l2.mix.v" in text


# ------------------------------------------------------------------ the plain functions


def test_plain_pieces_by_hand():
    u = torch.tensor([[1.0], [2.0], [4.0]], dtype=torch.float64)
    y = conv_over_time(u, torch.tensor([[0.5, 0.25, 2.0]], dtype=torch.float64),
                       torch.tensor([1.0], dtype=torch.float64))
    assert y.flatten().tolist() == [3.0, 5.25, 10.0]
    # a window of two keys that keeps the first token: query 3 sees keys 0, 2 and 3
    q = torch.ones(4, 1, 1, dtype=torch.float64)
    k = torch.zeros(4, 1, 1, dtype=torch.float64)
    v = torch.tensor([1.0, 10.0, 100.0, 1000.0], dtype=torch.float64).view(4, 1, 1)
    out = masked_attention(q, k, v, 1.0, 2, 1).flatten()
    assert torch.allclose(out, torch.tensor([1.0, 5.5, 37.0, 367.0], dtype=torch.float64))
    # a state of one value: S = a S + dt B x, y = S C + D x
    y = selective_state_space(torch.tensor([[[2.0]], [[3.0]]], dtype=torch.float64),
                              torch.tensor([[[1.0]], [[0.5]]], dtype=torch.float64),
                              torch.tensor([[[1.0]], [[2.0]]], dtype=torch.float64),
                              torch.tensor([[0.5], [1.0]], dtype=torch.float64),
                              torch.tensor([0.0], dtype=torch.float64), torch.tensor([10.0], dtype=torch.float64))
    assert torch.allclose(y.flatten(), torch.tensor([21.0, 35.0], dtype=torch.float64))
    # the correction moves the choice, not the weights
    w = routing(torch.eye(3, dtype=torch.float64), torch.eye(3, dtype=torch.float64),
                torch.tensor([0.0, 0.0, 5.0], dtype=torch.float64), 1)
    assert w[0].tolist()[:2] == [0.0, 0.0] and abs(float(w[0, 2]) - 1 / (2 + torch.e)) < 1e-12
    f, amplitude = stretched_frequencies({"base": 100.0, "dims": 4}, torch.float64)
    assert f.tolist() == [1.0, 0.1] and amplitude == 1.0


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


@pytest.mark.parametrize("name", ["T1", "T2", "T4"])
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
    cache.check()
    assert not cache.requests()


def test_pages_behind_a_window_come_back_but_the_first_stay(folders):
    """A request far longer than the windowed layers would need: their pages that have left the
    window are handed out again, the pages of the kept first tokens never, and the logits stay
    those of the plain model."""
    config, _, page = CONFIGS["T2"]                         # a window of 7 that keeps 9, pages of 8
    runner, cache = engine(folders["T2"], page, 256, max_requests=1)
    (tokens,) = prompts(config["vocab"], (200,), seed=6)
    steps = [([("r", part)], []) for part in cut(tokens, (5, 1, 9, 2))]
    last = steps.pop()
    got = replay(runner, cache, steps)
    group = next(i for i, g in enumerate(cache.paged) if g.need.keep_first == 9)
    table = cache.get("r").tables[group]
    assert table[0] >= 0 and table[1] >= 0 and table[2] == -1 and table[-1] >= 0
    assert sum(page >= 0 for page in table) <= 2 + 3
    rest = replay(runner, cache, [(last[0], ["r"])])
    got = torch.cat([got["r"], rest["r"]])
    assert_rows_close(got, PlainModel(folders["T2"]).logits(tokens), torch.float32, "a long request")
    cache.check()


def test_greedy_generation_through_the_entry_point(folders):
    """The engine's own entry point and scheduler: prompts in portions of eight tokens, three
    requests at a time, greedy tokens against the plain model's."""
    from mlx_one_b200 import BatchingConfig, CacheConfig, Engine, TextGenerationOptions

    config, _, page = CONFIGS["T1"]
    plain = PlainModel(folders["T1"])
    batch = prompts(config["vocab"], (7, 30, 3, 19), seed=8)
    engine_ = Engine(folders["T1"], execution_dtype="float32", ops=PlainOps(), device="cpu",
                     cache_config=CacheConfig(block_size_tokens=page, capacity_tokens=256),
                     batching_config=BatchingConfig(max_sequences=3, prefill_chunk_size=8))
    results = engine_.generate_batch_ids(batch, TextGenerationOptions(max_tokens=6, ignore_eos=True))
    for prompt, result in zip(batch, results):
        assert list(result.token_ids) == plain.greedy(prompt, 6)
    engine_.close()
