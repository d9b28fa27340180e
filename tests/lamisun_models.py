"""Tiny Lamisun configurations for the tests, with weights drawn large enough that every
mechanism moves the logits.

The configurations differ in every size: width, vocabulary, the pair table's buckets and
factors (also none), the taps of the input convolutions (2 to 5, one, none), latent attention
(one to six heads; unrotated dimensions shorter and longer than the rotated part; latents that
are multiples of 32, of 16, of neither; values longer and shorter than keys), differential
attention (every query head its own key head, all on one, groups; keys equal to, shorter and
longer than the values; chunks shorter than a page, of a few pages, longer than every prompt,
of one position, none), feed-forwards (also none), and the order of the layers.
"""

from __future__ import annotations

import json
import tempfile
from pathlib import Path

import torch


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, base, mlp):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim,
                      "kv_rank": kv_rank, "scale": scale, "rot": {"base": base, "dims": rot_dim}},
            "mlp": mlp}


def differential(heads, kv_heads, dim, vdim, scale, diff, chunk, mlp):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
             "diff": diff}
    if chunk is not None:
        mixer["mask"] = {"size": chunk}
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


# latent rows of 48 + 16 = 64 (a multiple of 32), chunks of a few pages, heads in pairs on a key
# head, keys shorter than values, a layer without a feed-forward
L1 = {"architecture": "Lamisun", "vocab": 300, "width": 64, "norm": {"eps": 1e-5},
      "canon": {"taps": 3},
      "embedding": {"scale": 2.0, "bigram": {"buckets": 97, "mul_prev": 13, "mul_cur": 5}},
      "layers": [
          latent(4, 24, 16, 32, 48, 0.16, 10000.0, dense(96)),
          differential(4, 2, 16, 32, 0.25, 0.5, 24, dense(80)),
          latent(4, 24, 16, 32, 48, 0.16, 10000.0, None)]}

# two differential layers first; every query head its own key head; keys longer than values; a
# chunk shorter than a page; a latent that is a multiple of nothing (40 + 6); two taps; the
# embedding's scale 1; three latent heads whose unrotated part is shorter than the rotated one
L2 = {"architecture": "Lamisun", "vocab": 257, "width": 96, "norm": {"eps": 1e-6},
      "canon": {"taps": 2},
      "embedding": {"scale": 1.0, "bigram": {"buckets": 50, "mul_prev": 3, "mul_cur": 1000003}},
      "layers": [
          differential(3, 3, 24, 8, 0.2, 0.3, 5, dense(64)),
          differential(3, 3, 24, 8, 0.2, 0.3, 5, None),
          latent(3, 4, 6, 20, 40, 0.3, 500.0, dense(100))]}

# no pair table and no input convolution; one latent head; one differential head with keys as
# long as values and no chunks at all; the last layer a differential one
L3 = {"architecture": "Lamisun", "vocab": 64, "width": 32, "norm": {"eps": 1e-5},
      "embedding": {"scale": 4.0},
      "layers": [
          latent(1, 8, 2, 12, 16, 0.4, 100.0, dense(48)),
          differential(1, 1, 16, 16, 0.3, 0.8, None, dense(48))]}

# five taps; six latent heads on a latent of 96 + 32; four differential heads on one key head,
# heads of 64, chunks of 100 on pages of 16; one bucket (every pair takes the same row)
L4 = {"architecture": "Lamisun", "vocab": 512, "width": 128, "norm": {"eps": 2e-6},
      "canon": {"taps": 5},
      "embedding": {"scale": 3.0, "bigram": {"buckets": 1, "mul_prev": 7, "mul_cur": 11}},
      "layers": [
          differential(4, 1, 64, 64, 0.125, 0.6, 100, dense(192)),
          latent(6, 32, 32, 16, 96, 0.12, 1000000.0, dense(192)),
          differential(4, 1, 64, 64, 0.125, 0.6, 100, dense(192)),
          latent(6, 32, 32, 16, 96, 0.12, 1000000.0, dense(192))]}

# a convolution of one tap (no state); chunks of one position (a query sees only itself);
# chunks longer than every prompt; width 72 and a vocabulary of 100
L5 = {"architecture": "Lamisun", "vocab": 100, "width": 72, "norm": {"eps": 3e-6},
      "canon": {"taps": 1},
      "embedding": {"scale": 0.5, "bigram": {"buckets": 1021, "mul_prev": 1, "mul_cur": 1}},
      "layers": [
          differential(2, 2, 8, 40, 0.35, 0.2, 1, dense(60)),
          latent(2, 10, 4, 24, 18, 0.27, 50.0, None),
          differential(6, 2, 8, 24, 0.35, 0.4, 1000, dense(60))]}

CONFIGS = {"L1": (L1, 31, 16), "L2": (L2, 32, 8), "L3": (L3, 33, 4), "L4": (L4, 34, 16),
           "L5": (L5, 35, 2)}   # config, seed, page


def draw_tensors(config: dict, seed: int) -> dict[str, torch.Tensor]:
    """Weights for ``config``, by the names and shapes that the engine expects: matrices
    ~ N(0, 1/in), tables N(0, 1), norm weights around 1, convolution weights ~ N(0, 0.5), the
    streams' weights around 1 / their count, the activation's two numbers and the vectors of
    the maps' factor ~ N(0, 0.3)."""
    from mlx_one_b200.architectures.lamisun import describe
    from mlx_one_b200.config import LamisunConfig
    from mlx_one_b200.parts import expected_tensors

    generator = torch.Generator().manual_seed(seed)
    out = {}
    for name, want in expected_tensors(describe(LamisunConfig.from_dict(config))).items():
        values = torch.randn(want.shape, generator=generator)
        if want.init == "norm":
            values = 1.0 + 0.2 * values
        elif name in ("embed", "bigram"):
            pass
        elif ".canon" in name:
            values = 0.5 * values
        elif name.endswith(".dwa"):
            values = (1.0 + 0.5 * values) / want.shape[0]
        elif len(want.shape) == 2:
            values = values / want.shape[1] ** 0.5
        else:
            values = 0.3 * values
        out[name] = values.to(torch.bfloat16)
    return out


def make_model_dir(name: str, root: Path | None = None, config: dict | None = None,
                   tensors: dict | None = None) -> Path:
    """Writes the tiny model ``name`` into a fresh temporary folder (never into the repo)."""
    from mlx_one_b200.weights.safetensors_io import write_safetensors

    base, seed, _ = CONFIGS[name]
    config = base if config is None else config
    folder = Path(tempfile.mkdtemp(prefix=f"tiny_{name}_", dir=root))
    write_safetensors(folder / "model.safetensors",
                      draw_tensors(config, seed) if tensors is None else tensors, {"format": "pt"})
    (folder / "config.json").write_text(json.dumps(config, indent=1))
    return folder


class PlainModel:
    """The plain implementation on a model folder: logits of whole sequences in 64-bit."""

    def __init__(self, folder):
        import plain_lamisun

        self.plain = plain_lamisun
        self.config, self.weights = plain_lamisun.load(folder)

    def logits(self, tokens, streams=None):
        return self.plain.forward(self.config, self.weights, list(tokens), streams=streams).float()

    def greedy(self, prompt, count):
        tokens, out = list(prompt), []
        for _ in range(count):
            out.append(int(self.logits(tokens)[-1].argmax()))
            tokens.append(out[-1])
        return out


# bfloat16: a row's error is the root mean square over the vocabulary of (engine - plain), its
# mean taken off, relative to the spread of the plain logits. Rounding alone gives a few percent
# on these models; a wrong key, a lost state or a token fed twice gives 15 % and more.
BF16_ROW_ERROR = 0.12


def assert_rows_close(got, want, dtype, what: str = "") -> None:
    """float32: every logit within 2e-4 + 2e-4 |plain|. bfloat16: every row's error (see above)
    within ``BF16_ROW_ERROR``."""
    got, want = got.float().cpu(), want.float().cpu()
    assert got.shape == want.shape, f"{what}: {tuple(got.shape)} against {tuple(want.shape)}"
    if dtype == torch.float32:
        excess = (got - want).abs() - (2e-4 + 2e-4 * want.abs())
        assert excess.max() <= 0, (f"{what}: logits differ by {(got - want).abs().max():.3e}; rows "
                                   f"{torch.nonzero((excess > 0).any(-1)).flatten().tolist()[:8]}")
        return
    difference = got - want
    difference = difference - difference.mean(-1, keepdim=True)
    spread = (want - want.mean(-1, keepdim=True)).pow(2).mean().sqrt()
    rows = difference.pow(2).mean(-1).sqrt() / spread
    bad = rows > BF16_ROW_ERROR
    assert not bad.any(), (f"{what}: row error {rows.max():.3f} of the spread; rows "
                           f"{torch.nonzero(bad).flatten().tolist()[:8]}")
