"""Tiny Tirudra configurations for the tests, with weights drawn large enough that every
mechanism moves the logits.

The configurations differ in every size: width, vocabulary, head counts and groupings, key and
value sizes (equal, value shorter, value longer; multiples of 32, of 16, of neither), the rotated
part of a head (all of it, a part, two dimensions, nothing) with and without stretched
frequencies, windows (shorter than a page, a few pages, one token, none) with first tokens kept
(none, fewer than a page, more than the window), taps of the convolutions (1 to 4, none), state
spaces with states of 4 to 128 values, one group to one per head, norms in one part to one per
head, routed experts (with and without identity outputs and a shared expert, one expert per
token, all outputs chosen, none), and the order of the layers.
"""

from __future__ import annotations

import json
import tempfile
from pathlib import Path

import torch


def conv_attention(heads, kv_heads, dim, vdim, scale, conv, mask, rot, mlp):
    """``mask``: None or (size, keep_first or None)."""
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if conv is not None:
        mixer["conv"] = conv
    if mask is not None:
        mixer["mask"] = {"size": mask[0]}
        if mask[1] is not None:
            mixer["mask"]["keep_first"] = mask[1]
    if rot is not None:
        mixer["rot"] = rot
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def shared_attention(heads, kv_heads, dim, scale, rot, mlp):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if rot is not None:
        mixer["rot"] = rot
    return {"type": "attention_2", "mixer": mixer, "mlp": mlp}


def state_space(heads, vdim, state, groups, conv, norm_groups, mlp):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state,
                                        "groups": groups, "conv": conv, "norm_groups": norm_groups},
            "mlp": mlp}


def routed(ff, experts, top, identity=None, shared=None):
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if identity is not None:
        out["router"]["identity"] = identity
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def turns(base, dims, factor=None, original=None, fast=None, slow=None):
    rot = {"base": base, "dims": dims}
    if factor is not None:
        rot["scaling"] = {"factor": factor, "original": original, "fast": fast, "slow": slow}
    return rot


def waves(base, dims, factor=None, original=None, low=None, high=None):
    rot = {"base": base, "dims": dims}
    if factor is not None:
        rot["scaling"] = {"factor": factor, "original": original, "low": low, "high": high}
    return rot


# heads of 32, a window of a few pages that keeps three tokens, four taps; the second attention
# on the kernel that prepares and attends in one for single tokens; a state space whose heads
# share two groups; identity outputs and a gated shared expert
T1 = {"architecture": "Tirudra", "vocab": 300, "width": 64, "norm": {"eps": 1e-5},
      "logit_scale": 0.5,
      "layers": [
          state_space(4, 16, 16, 2, 4, 2, routed(32, 6, 3, 2, 40)),
          conv_attention(4, 2, 32, 32, 0.2, 4, (24, 3), turns(10000.0, 16, 4.0, 64, 8.0, 1.0),
                         routed(32, 6, 3, 2, 40)),
          shared_attention(4, 2, 32, 0.18, waves(10000.0, 32, 8.0, 64, 1.0, 3.0), None),
          conv_attention(4, 2, 32, 32, 0.2, 4, (24, 3), turns(10000.0, 16, 4.0, 64, 8.0, 1.0),
                         routed(32, 6, 3, 2, 40))]}

# sizes that are multiples of nothing much: width 72, vocabulary 100; values longer than keys,
# two taps, more first tokens kept than the window is long, six rotated dimensions with their
# frequencies as they are; a state space with a group per head, columns that fill no warp, one
# norm over everything; every query head its own key head with a part of the head rotated; one
# expert per token, no identity outputs, no shared expert; a layer without a feed-forward
T2 = {"architecture": "Tirudra", "vocab": 100, "width": 72, "norm": {"eps": 3e-6},
      "logit_scale": 1.0,
      "layers": [
          conv_attention(3, 1, 24, 40, 0.21, 2, (7, 9), turns(5000.0, 6), routed(20, 5, 1)),
          state_space(3, 20, 24, 3, 2, 1, None),
          shared_attention(3, 3, 16, 0.25, waves(1000.0, 8), routed(20, 5, 1)),
          conv_attention(2, 2, 40, 24, 0.15, 3, None, None, routed(48, 3, 2, 1, 24))]}

# heads of 64 on one key head, a window of 100 that keeps four tokens; states of 128 values in
# one group, a norm part per head; eight experts and two identity outputs of which three are used
T3 = {"architecture": "Tirudra", "vocab": 512, "width": 128, "norm": {"eps": 2e-6},
      "logit_scale": 0.25,
      "layers": [
          conv_attention(8, 1, 64, 64, 0.11, 3, (100, 4), turns(300.0, 64, 2.0, 40, 6.0, 0.5),
                         routed(48, 8, 3, 2, 64)),
          state_space(4, 64, 128, 1, 4, 4, routed(48, 8, 3, 2, 64)),
          shared_attention(4, 2, 64, 0.125, waves(8000.0, 64, 4.0, 32, 2.0, 5.0),
                           routed(48, 8, 3, 2, 64))]}

# one head everywhere, a window of one token that keeps one, a single tap, two rotated
# dimensions, states of four values; nothing rotated in the second attention; every output of
# the router is chosen (two experts and an identity output)
T4 = {"architecture": "Tirudra", "vocab": 64, "width": 32, "norm": {"eps": 1e-5},
      "logit_scale": 2.0,
      "layers": [conv_attention(1, 1, 8, 8, 0.5, 1, (1, 1), turns(100.0, 2), routed(16, 2, 3, 1)),
                 state_space(1, 8, 4, 1, 1, 1, None),
                 shared_attention(1, 1, 8, 0.4, None, routed(16, 2, 3, 1))]}

# no routed experts (in bfloat16 nothing is decided by a hair, so every row is held to the
# bound): a window of 40 that keeps two tokens, no convolution in the first attention, a window
# without kept tokens in the second, a state space that forgets slowly
T5 = {"architecture": "Tirudra", "vocab": 384, "width": 128, "norm": {"eps": 1e-5},
      "logit_scale": 1.0,
      "layers": [
          conv_attention(4, 2, 64, 64, 0.125, None, (40, 2), turns(8000.0, 64), None),
          state_space(4, 32, 64, 2, 3, 2, None),
          shared_attention(4, 1, 48, 0.14, waves(8000.0, 48, 8.0, 128, 1.0, 4.0), None),
          conv_attention(2, 2, 32, 32, 0.2, 3, (33, None), turns(8000.0, 32, 8.0, 32, 4.0, 1.0), None)]}

CONFIGS = {"T5": (T5, 35, 16), "T1": (T1, 31, 4), "T2": (T2, 32, 8), "T3": (T3, 33, 16),
           "T4": (T4, 34, 2)}   # config, seed, page


def draw_tensors(config: dict, seed: int) -> dict[str, torch.Tensor]:
    """Weights for ``config``, by the names and shapes of the engine's weight contract: matrices
    ~ N(0, 1/in) (the embedding N(0, 1), routers three times as wide so that scores differ),
    norm weights around 0 (those of queries, keys and the state space's output around 1),
    convolutions ~ N(0, 0.5), biases ~ N(0, 0.3), corrections ~ N(0, 0.05); A_log around -2 and
    dt_bias around -1, so that a state keeps what it saw for tens of tokens."""
    from mlx_one_b200.architectures.tirudra import describe
    from mlx_one_b200.config.tirudra import TirudraConfig
    from mlx_one_b200.parts import expected_tensors

    generator = torch.Generator().manual_seed(seed)
    out = {}
    for name, want in expected_tensors(describe(TirudraConfig.from_dict(config))).items():
        values = torch.randn(want.shape, generator=generator)
        if name.endswith(".A_log"):
            values = -2.0 + 0.7 * values
        elif name.endswith(".dt_bias"):
            values = -1.0 + 0.5 * values
        elif name.endswith(".correction"):
            values = 0.05 * values
        elif want.init == "norm":
            values = 1.0 + 0.2 * values
        elif want.init == "norm0":
            values = 0.2 * values
        elif name.endswith(".router"):
            values = 3.0 * values / want.shape[1] ** 0.5
        elif name == "embed":
            pass
        elif name.endswith(".conv"):
            values = 0.5 * values
        elif len(want.shape) == 2:
            values = values / want.shape[1] ** 0.5
        else:
            values = 0.3 * values
        out[name] = values.to(torch.bfloat16)
    return out


def write_model(folder: Path, config: dict, seed: int) -> Path:
    from mlx_one_b200.weights.safetensors_io import write_safetensors

    write_safetensors(folder / "model.safetensors", draw_tensors(config, seed), {"format": "pt"})
    (folder / "config.json").write_text(json.dumps(config, indent=1))
    return folder


def make_model_dir(name: str, root: Path | None = None, config: dict | None = None) -> Path:
    """Writes the tiny model ``name`` into a fresh temporary folder (never into the repo)."""
    base, seed, _ = CONFIGS[name]
    folder = Path(tempfile.mkdtemp(prefix=f"tiny_{name}_", dir=root))
    return write_model(folder, base if config is None else config, seed)


# bfloat16: a row's error is the root mean square over the vocabulary of (engine - plain), its
# mean taken off, relative to the spread of the plain logits. Rounding alone gives a few percent
# on these models; a wrong key, a lost state or a token fed twice gives 15 % and more.
BF16_ROW_ERROR = 0.12
USUAL_NOISE = 5e-6
# The bfloat16 engine routes what its own 16-bit arithmetic has made of the stream, so a
# position whose routing margin is below this may go to other experts than in the plain model;
# its logits are then others, and so, a little, are those of every later position of the request
# (a state space forgets slowly). Rows from the first such position on are not compared in
# bfloat16; the 32-bit engine is compared everywhere, and so is bfloat16 on models without
# routed experts.
ROUTING_MARGIN = 0.02


def assert_rows_close(got: torch.Tensor, want: torch.Tensor, dtype, what: str = "") -> None:
    """float32: every logit within 1e-4 + 1e-4 |plain| + 4 x the position's noise (positions with
    a routing margin below 1e-5 left out, and those behind them in their request). bfloat16:
    every row's error (see above) within ``BF16_ROW_ERROR`` up to the request's first position
    that is routed by a hair."""
    noise, margin = getattr(want, "noise", None), getattr(want, "margin", None)
    got, want = got.float().cpu(), want.float().cpu()
    assert got.shape == want.shape, f"{what}: {tuple(got.shape)} against {tuple(want.shape)}"
    noise = torch.zeros(want.shape[0]) if noise is None else noise.float().cpu()
    margin = torch.full((want.shape[0],), float("inf")) if margin is None else margin.float().cpu()
    if dtype == torch.float32:
        excess = (got - want).abs() - (1e-4 + 1e-4 * want.abs() + 4 * noise[:, None])
        settled = torch.cumsum((margin < 1e-5).float(), 0) == 0
        excess[~settled] = 0
        assert excess.max() <= 0, (f"{what}: logits differ by {(got - want).abs().max():.3e}; rows "
                                   f"{torch.nonzero((excess > 0).any(-1)).flatten().tolist()[:8]}")
        return
    difference = got - want
    difference = difference - difference.mean(-1, keepdim=True)
    spread = (want - want.mean(-1, keepdim=True)).pow(2).mean().sqrt()
    rows = difference.pow(2).mean(-1).sqrt() / spread
    allowed = BF16_ROW_ERROR * torch.clamp(noise / USUAL_NOISE, min=1.0)
    settled = torch.cumsum((margin < ROUTING_MARGIN).float(), 0) == 0
    bad = (rows > allowed) & settled
    assert not bad.any(), (f"{what}: row error {rows[settled].max():.3f} of the spread; rows "
                           f"{torch.nonzero(bad).flatten().tolist()[:8]}")


def sliced(want: torch.Tensor, count: int) -> torch.Tensor:
    """The first ``count`` rows of a plain model's logits, with their noise and margins."""
    out = want[:count]
    out.noise, out.margin = want.noise[:count], want.margin[:count]
    return out
