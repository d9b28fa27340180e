"""Tirudra models whose every size and constant is drawn at random (seeded): the 32-bit engine
against the plain model over whole requests, decoded tails, portions and mixed batches; the
bfloat16 engine over the same, up to each request's first position that is routed by a hair."""

import json
import random

import pytest
import torch

from plain_tirudra import PlainModel
from tiny_models import cut, mixed_schedule, prompts, replay
from tirudra_models import (assert_rows_close, conv_attention, routed, shared_attention,
                            state_space, turns, waves, write_model)

pytestmark = pytest.mark.gpu
DEVICE = "cuda:0"


def random_config(seed: int) -> dict:
    rng = random.Random(seed)
    width = rng.choice([48, 64, 72, 80, 96, 128, 160, 192])

    def feed_forward():
        if rng.random() < 0.2:
            return None
        experts = rng.choice([2, 3, 4, 6, 8, 12, 16])
        identity = rng.choice([None, 0, 1, 2, 3])
        top = rng.randint(1, min(5, experts + (identity or 0)))
        return routed(rng.choice([8, 24, 40, 64, 96]), experts, top, identity,
                      rng.choice([None, 16, 48, 128]))

    def conv_attention_layer():
        dim = rng.choice([8, 16, 24, 32, 40, 48, 64, 80, 96, 128])
        vdim = dim if rng.random() < 0.7 else rng.choice([8, 16, 32, 48, 64, 96])
        kv_heads = rng.choice([1, 2, 3, 4])
        heads = kv_heads * rng.choice([1, 2, 3, 4] if kv_heads > 1 else [1, 2, 4, 8, 10])
        rot = None
        if rng.random() < 0.85:
            dims = rng.choice([2, dim // 2 // 2 * 2 or 2, dim])
            if rng.random() < 0.7:
                slow = rng.choice([0.5, 1.0, 2.0])
                rot = turns(rng.choice([100.0, 10000.0, 500000.0]), dims, rng.choice([2.0, 4.0, 16.0]),
                            rng.choice([16, 64, 256, 4096]), slow * rng.choice([4.0, 16.0, 32.0]), slow)
            else:
                rot = turns(rng.choice([100.0, 10000.0]), dims)
        mask = None
        if rng.random() < 0.85:
            mask = (rng.choice([1, 3, 8, 17, 33, 40, 64, 96, 100, 200]),
                    rng.choice([None, 0, 1, 2, 4, 5, 16, 20, 70]))
        return conv_attention(heads, kv_heads, dim, vdim, rng.uniform(0.05, 0.3),
                              rng.choice([None, 1, 2, 3, 4, 5]), mask, rot, feed_forward())

    def shared_attention_layer():
        dim = rng.choice([8, 16, 24, 32, 40, 48, 64, 96, 128])
        kv_heads = rng.choice([1, 2, 3, 4])
        heads = kv_heads * rng.choice([1, 2, 3, 4])
        rot = None
        if rng.random() < 0.85:
            dims = rng.choice([2, dim // 2 // 2 * 2 or 2, dim, dim])
            if rng.random() < 0.7:
                low = rng.choice([0.5, 1.0, 2.0])
                rot = waves(rng.choice([100.0, 10000.0, 500000.0]), dims, rng.choice([2.0, 8.0, 32.0]),
                            rng.choice([16, 64, 512, 4096]), low, low * rng.choice([2.0, 4.0, 8.0]))
            else:
                rot = waves(rng.choice([100.0, 10000.0]), dims)
        return shared_attention(heads, kv_heads, dim, rng.uniform(0.05, 0.3), rot, feed_forward())

    def state_space_layer():
        groups = rng.choice([1, 1, 2, 3])
        heads = groups * rng.choice([1, 2, 3, 4])
        vdim = rng.choice([4, 8, 16, 24, 32, 48, 64, 100])
        parts = rng.choice([g for g in (1, 2, 3, 4, heads) if (heads * vdim) % g == 0])
        return state_space(heads, vdim, rng.choice([4, 8, 16, 24, 48, 64, 128, 136, 200]), groups,
                           rng.choice([1, 2, 3, 4, 5]), parts, feed_forward())

    makers = {"a": conv_attention_layer, "b": shared_attention_layer, "m": state_space_layer}
    count = rng.randint(2, 6)
    kinds = [rng.choice("abm") for _ in range(count)]
    kinds[rng.randrange(count)] = "a"
    kinds[(kinds.index("a") + 1) % count] = "m"
    return {"architecture": "Tirudra", "vocab": rng.randint(50, 700), "width": width,
            "norm": {"eps": rng.choice([1e-6, 1e-5])},
            "logit_scale": rng.choice([0.125, 0.3, 1.0, 1.7]),
            "layers": [makers[kind]() for kind in kinds]}


def engine(folder, dtype, page_size, capacity, max_requests=4):
    from mlx_one_b200.cache import CacheManager
    from mlx_one_b200.engine.loading import load_model
    from mlx_one_b200.engine.runner import Runner

    loaded = load_model(folder, dtype, DEVICE)
    cache = CacheManager(loaded.model.cache_needs, page_size=page_size, capacity_tokens=capacity,
                         max_requests=max_requests, dtype=dtype, device=DEVICE)
    return Runner(loaded.model, cache), cache


@pytest.mark.parametrize("seed", range(12))
def test_a_model_drawn_at_random(tmp_path, seed):
    config = random_config(seed)
    write_model(tmp_path, config, 100 + seed)
    plain = PlainModel(tmp_path)
    page = (16, 16, 8, 4)[seed % 4]
    lengths = (150, 64, 23, 50, 9, 2, 1)
    requests = dict(enumerate(prompts(config["vocab"], lengths, seed=seed)))
    want = {key: plain.logits(tokens) for key, tokens in requests.items()}
    for dtype in (torch.float32, torch.bfloat16):
        runner, cache = engine(tmp_path, dtype, page, 4 * 192, max_requests=4)
        tokens = requests[0]
        got = replay(runner, cache, [([("w", tokens)], ["w"])])["w"]
        assert_rows_close(got, want[0], dtype, f"seed {seed} whole {json.dumps(config)[:0]}")
        steps = [([("d", tokens[:110])], [])] + [([("d", [t])], []) for t in tokens[110:]]
        steps[-1] = (steps[-1][0], ["d"])
        assert_rows_close(replay(runner, cache, steps)["d"], want[0], dtype, f"seed {seed} decoded tail")
        steps = [([("p", part)], []) for part in cut(tokens, (7, 2, 40, 3, 1))]
        steps[-1] = (steps[-1][0], ["p"])
        assert_rows_close(replay(runner, cache, steps)["p"], want[0], dtype, f"seed {seed} portions")
        got = replay(runner, cache, mixed_schedule(requests))
        for key in requests:
            assert_rows_close(got[key], want[key], dtype, f"seed {seed} mixed request {key}")
        cache.check()
        assert not cache.requests()
