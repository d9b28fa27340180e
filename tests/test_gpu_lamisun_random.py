"""Lamisun models whose every size and constant is drawn at random (seeded): the 32-bit and the
bfloat16 engine against the plain model over whole requests, decoded tails, portions and mixed
batches."""

import json
import random

import pytest
import torch

from lamisun_models import (PlainModel, assert_rows_close, dense, differential, draw_tensors,
                            latent)
from tiny_models import cut, mixed_schedule, prompts, replay

pytestmark = pytest.mark.gpu
DEVICE = "cuda:0"


def random_config(seed: int) -> dict:
    rng = random.Random(seed)
    width = rng.choice([48, 64, 80, 96, 128, 160, 192, 256])

    def feed_forward():
        return None if rng.random() < 0.15 else dense(rng.choice([32, 40, 96, 200, 256, 384]))

    def latent_layer():
        rot_dim = rng.choice([2, 4, 8, 16, 24, 32, 64])
        return latent(rng.choice([1, 2, 3, 4, 6, 8, 12, 16]), rng.choice([4, 8, 16, 24, 32, 48, 64, 96]),
                      rot_dim, rng.choice([8, 16, 20, 32, 64, 96]),
                      rng.choice([8, 16, 24, 40, 64, 96, 128, 160, 192]), rng.uniform(0.05, 0.3),
                      rng.choice([100.0, 10000.0, 1000000.0]), feed_forward())

    def differential_layer():
        dim = rng.choice([8, 16, 24, 32, 40, 48, 64, 96, 128])
        vdim = dim if rng.random() < 0.5 else rng.choice([8, 16, 32, 48, 64, 96, 128])
        kv_heads = rng.choice([1, 2, 3, 4])
        heads = kv_heads * rng.choice([1, 2, 3, 4] if kv_heads > 1 else [1, 2, 4, 8])
        chunk = rng.choice([1, 3, 8, 16, 17, 33, 64, 96, 100, 120, 200, 1000, None])
        return differential(heads, kv_heads, dim, vdim, rng.uniform(0.05, 0.3),
                            rng.choice([0.0, 0.2, 0.5, 0.6, 0.8]), chunk, feed_forward())

    count = rng.randint(2, 7)
    kinds = [rng.choice("ld") for _ in range(count)]
    kinds[rng.randrange(count)] = "l"
    kinds[(kinds.index("l") + 1) % count] = "d"
    config = {"architecture": "Lamisun", "vocab": rng.randint(50, 700), "width": width,
              "norm": {"eps": rng.choice([1e-6, 1e-5])},
              "embedding": {"scale": rng.choice([0.5, 1.0, 2.0, 3.0, 8.0])},
              "layers": [latent_layer() if kind == "l" else differential_layer() for kind in kinds]}
    if rng.random() < 0.85:
        config["embedding"]["bigram"] = {"buckets": rng.choice([1, 7, 97, 1021, 4099]),
                                         "mul_prev": rng.choice([0, 1, 31, 1000003]),
                                         "mul_cur": rng.choice([0, 1, 7, 999983])}
    if rng.random() < 0.85:
        config["canon"] = {"taps": rng.randint(1, 6)}
    return config


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
    from mlx_one_b200.weights.safetensors_io import write_safetensors

    config = random_config(seed)
    write_safetensors(tmp_path / "model.safetensors", draw_tensors(config, 100 + seed), {"format": "pt"})
    (tmp_path / "config.json").write_text(json.dumps(config))
    plain = PlainModel(tmp_path)
    page = (16, 16, 8, 4, 32, 64)[seed % 6]
    lengths = (150, 64, 23, 50, 9, 2, 1)
    requests = dict(enumerate(prompts(config["vocab"], lengths, seed=seed)))
    want = {key: plain.logits(tokens) for key, tokens in requests.items()}
    for dtype in (torch.float32, torch.bfloat16):
        runner, cache = engine(tmp_path, dtype, page, 4 * 192, max_requests=4)
        tokens = requests[0]
        got = replay(runner, cache, [([("w", tokens)], ["w"])])["w"]
        assert_rows_close(got, want[0], dtype, f"seed {seed} whole")
        steps = [([("d", tokens[:110])], [])] + [([("d", [t])], []) for t in tokens[110:]]
        steps[-1] = (steps[-1][0], ["d"])
        assert_rows_close(replay(runner, cache, steps)["d"], want[0], dtype, f"seed {seed} decoded tail")
        steps = [([("p", part)], []) for part in cut(tokens, (7, 2, 40, 3, 1))]
        steps[-1] = (steps[-1][0], ["p"])
        assert_rows_close(replay(runner, cache, steps)["p"], want[0], dtype, f"seed {seed} portions")
        got = replay(runner, cache, mixed_schedule(requests))
        for key in requests:
            assert_rows_close(got[key], want[key], dtype, f"seed {seed} mixed request {key}")
        assert not cache.requests()
