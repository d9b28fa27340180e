"""Plain, slow Tirudra written from the design's equations: whole sequences, no cache, one
function per mechanism. It shares no code with the engine: it reads config.json and the
safetensors file by itself and computes everything in one floating type (float64 by default).

Notation: x [T, W] the stream, h the normed input of a part, T tokens at positions 0..T-1.
"""

from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch

_KINDS = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32}


def read_tensors(path):
    """A safetensors file: 8 bytes little-endian header length, the JSON header, the data."""
    raw = Path(path).read_bytes()
    (length,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + length])
    data = raw[8 + length:]
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        out[name] = torch.frombuffer(bytearray(data[lo:hi]), dtype=_KINDS[info["dtype"]]) \
            .reshape(info["shape"]).clone()
    return out


# --------------------------------------------------------------------------- small pieces


def unit_rms(x, eps):
    """x divided by its root mean square over the last axis, eps under the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z / (1 + torch.exp(-z))


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def conv_over_time(u, kernel, bias=None):
    """u [T, C], kernel [C, taps]: y_t = sum_j kernel[:, j] u_(t - taps + 1 + j), nothing before
    the sequence's first token; the last column weighs the token itself."""
    T, taps = u.shape[0], kernel.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, u.shape[1], dtype=u.dtype), u], 0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + padded[j:j + T] * kernel[:, j]
    return y if bias is None else y + bias


def stretched_frequencies(rot, kind):
    """f_i = base^(-2i/dims); with ``fast``/``slow`` turns of the original context the pairs
    between them are slowed gradually by ``factor`` (returns also the amplitude 0.1 ln(factor) +
    1); with ``low``/``high`` the wavelength decides: short ones stay, long ones are divided by
    ``factor``, those between are blended."""
    dims, base = rot["dims"], rot["base"]
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    s = rot.get("scaling")
    amplitude = 1.0
    if s and "fast" in s:
        at = lambda turns: dims * math.log(s["original"] / (2 * math.pi * turns)) / (2 * math.log(base))
        lo, hi = max(math.floor(at(s["fast"])), 0), min(math.ceil(at(s["slow"])), dims - 1)
        for i in range(dims // 2):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            f[i] = f[i] / s["factor"] * ramp + f[i] * (1 - ramp)
        amplitude = 0.1 * math.log(s["factor"]) + 1.0
    elif s:
        for i in range(dims // 2):
            wave = 2 * math.pi / f[i]
            if wave > s["original"] / s["low"]:
                f[i] = f[i] / s["factor"]
            elif wave >= s["original"] / s["high"]:
                t = (s["original"] / wave - s["low"]) / (s["high"] - s["low"])
                f[i] = (1 - t) * f[i] / s["factor"] + t * f[i]
    return torch.tensor(f, dtype=kind), amplitude


def rotate_halves(x, positions, rot):
    """x [T, heads, D]: within the first dims dimensions, i and i + dims/2 are turned by
    position * f_i (cosine and sine times the amplitude); the other dimensions pass."""
    if not rot:
        return x
    f, amplitude = stretched_frequencies(rot, x.dtype)
    dims = rot["dims"]
    angle = positions.to(x.dtype)[:, None] * f[None, :]
    cos, sin = amplitude * torch.cos(angle)[:, None, :], amplitude * torch.sin(angle)[:, None, :]
    u, v = x[..., :dims // 2], x[..., dims // 2:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], -1)


def masked_attention(q, k, v, scale, window=None, keep_first=0):
    """q [T, H, D], k [T, G, D], v [T, G, V] -> [T, H, V]. Query i sees key j <= i if
    i - j < window or j < keep_first (no window: every j <= i)."""
    T, H, _ = q.shape
    G = k.shape[1]
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    visible = j <= i
    if window is not None:
        visible = visible & ((i - j < window) | (j < keep_first))
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~visible, -math.inf)
        out[:, h] = torch.softmax(s, -1) @ v[:, g]
    return out


def selective_state_space(x, B, C, dt, A, D):
    """x [T, H, P], B, C [T, G, N], dt [T, H], A [H] (positive), D [H] -> y [T, H, P], from a
    zero state. Per head (group g of the head): S = exp(-A dt) S + dt B x^T; y = S^T C + D x."""
    T, H, P = x.shape
    G, N = B.shape[1], B.shape[2]
    y = torch.zeros_like(x)
    for h in range(H):
        g = h // (H // G)
        S = torch.zeros(N, P, dtype=x.dtype)
        for t in range(T):
            S = torch.exp(-A[h] * dt[t, h]) * S + dt[t, h] * torch.outer(B[t, g], x[t, h])
            y[t, h] = S.T @ C[t, g] + D[h] * x[t, h]
    return y


def routing(h, router, correction, top, margins=None):
    """Weights [T, outputs of the router]: softmax scores over all of them; the ``top`` with
    the largest score + correction are chosen and keep their scores (no renormalisation)."""
    s = torch.softmax(h @ router.T, -1)
    choice = s + correction
    chosen = choice.topk(top, dim=-1).indices
    weights = torch.zeros_like(s)
    weights.scatter_(1, chosen, s.gather(1, chosen))
    if margins is not None and top < s.shape[1]:
        ranked = choice.sort(dim=-1, descending=True).values
        margins.append(ranked[:, top - 1] - ranked[:, top])
    return weights


# --------------------------------------------------------------------------- parts


def attention_mixer(h, w, p, c, eps):
    """Convolutions on q, k, v; normed, rotated q and k; window that keeps the first tokens; a
    sigmoid gate on every value of the heads' outputs."""
    T = h.shape[0]
    H, G, D, V = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    positions = torch.arange(T)
    q, k, v = h @ w[p + "q"].T, h @ w[p + "k"].T, h @ w[p + "v"].T
    if c.get("conv"):
        q, k, v = (conv_over_time(u, w[p + name + ".conv"]) for u, name in ((q, "q"), (k, "k"), (v, "v")))
    q = unit_rms(q.view(T, H, D), eps) * w[p + "q.norm"]
    k = unit_rms(k.view(T, G, D), eps) * w[p + "k.norm"]
    q, k = rotate_halves(q, positions, c.get("rot")), rotate_halves(k, positions, c.get("rot"))
    mask = c.get("mask") or {}
    mixed = masked_attention(q, k, v.view(T, G, V), c["scale"], mask.get("size"),
                             mask.get("keep_first", 0))
    mixed = mixed.reshape(T, H * V) * torch.sigmoid(h @ w[p + "g"].T)
    return mixed @ w[p + "o"].T


def attention_2_mixer(h, w, p, c, eps):
    """Biased q and k; the values are the keys as projected; causal; one gate number per head."""
    T = h.shape[0]
    H, G, D = c["heads"], c["kv_heads"], c["dim"]
    positions = torch.arange(T)
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, D)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, D)
    v = k
    q = rotate_halves(unit_rms(q, eps) * w[p + "q.norm"], positions, c.get("rot"))
    k = rotate_halves(unit_rms(k, eps) * w[p + "k.norm"], positions, c.get("rot"))
    mixed = masked_attention(q, k, v, c["scale"])
    mixed = mixed * torch.sigmoid(h @ w[p + "g"].T)[:, :, None]
    return mixed.reshape(T, H * D) @ w[p + "o"].T


def mamba2_mixer(h, w, p, c, eps):
    T = h.shape[0]
    H, P, N, G = c["heads"], c["vdim"], c["state"], c["groups"]
    inner = H * P
    z, xBC, dt = torch.split(h @ w[p + "in"].T, [inner, inner + 2 * G * N, H], dim=-1)
    xBC = silu(conv_over_time(xBC, w[p + "conv"], w[p + "conv.b"]))
    x, B, C = torch.split(xBC, [inner, G * N, G * N], dim=-1)
    dt = softplus(dt + w[p + "dt_bias"])
    y = selective_state_space(x.view(T, H, P), B.view(T, G, N), C.view(T, G, N), dt,
                              torch.exp(w[p + "A_log"]), w[p + "D"])
    y = y.reshape(T, inner) * silu(z)
    parts = c["norm_groups"]
    y = unit_rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def gated_feed_forward(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def routed_feed_forward(h, w, p, c, margins=None):
    r = c["router"]
    weights = routing(h, w[p + "router"], w[p + "correction"], r["top"], margins)
    out = torch.zeros_like(h)
    for e in range(r["experts"]):
        out = out + weights[:, e:e + 1] * gated_feed_forward(h, w, f"{p}e{e}.")
    for e in range(r["experts"], r["experts"] + r.get("identity", 0)):
        out = out + weights[:, e:e + 1] * h
    if c.get("shared"):
        out = out + torch.sigmoid(h @ w[p + "shared.sg"].T) * gated_feed_forward(h, w, p + "shared.")
    return out


MIXERS = {"attention": attention_mixer, "attention_2": attention_2_mixer, "mamba2": mamba2_mixer}


# --------------------------------------------------------------------------- the model


def forward(cfg, w, tokens, states=None, margins=None):
    """Logits [T, vocab] of a whole sequence; ``states`` collects the stream after each layer,
    ``margins`` the routing margins of every routed feed-forward."""
    eps = cfg["norm"]["eps"]
    norm = lambda x, name: unit_rms(x, eps) * (1 + w[name])
    x = w["embed"][torch.as_tensor(tokens)]
    for index, layer in enumerate(cfg["layers"]):
        p = f"l{index}."
        mixed = MIXERS[layer["type"]](norm(x, p + "norm1"), w, p + "mix.", layer["mixer"], eps)
        x = x + norm(mixed, p + "norm1b")
        mlp = layer.get("mlp")
        if mlp:
            if mlp["kind"] != "moe":
                raise ValueError(mlp["kind"])
            out = routed_feed_forward(norm(x, p + "norm2"), w, p + "mlp.", mlp, margins)
            x = x + norm(out, p + "norm2b")
        if states is not None:
            states.append(x.clone())
    return norm(x, "final.norm") @ w["head"].T * cfg.get("logit_scale", 1.0)


class PlainModel:
    def __init__(self, model_dir, kind=torch.float64):
        self.cfg = json.loads((Path(model_dir) / "config.json").read_text())
        self.w = {name: t.to(kind) for name, t in
                  read_tensors(Path(model_dir) / "model.safetensors").items()}
        self.w32 = {name: t.to(torch.float32) for name, t in self.w.items()} \
            if kind == torch.float64 else None

    def logits(self, tokens, states=None):
        """Logits [T, vocab]. The result carries ``noise`` [T], how far the same equations in
        32-bit arithmetic land from the 64-bit ones at each position (largest difference of a
        logit), and ``margin`` [T], the smallest routing margin of the position (infinite
        without routed layers): a position whose margin is tiny is decided by rounding."""
        margins = []
        out = forward(self.cfg, self.w, tokens, states, margins).float()
        out.margin = torch.stack(margins).amin(0).float() if margins \
            else torch.full((len(tokens),), math.inf)
        if self.w32 is not None:
            out.noise = (forward(self.cfg, self.w32, tokens) - out).abs().amax(dim=-1)
        return out

    def greedy(self, prompt, count):
        tokens = list(prompt)
        for _ in range(count):
            tokens.append(int(torch.argmax(self.logits(tokens)[-1])))
        return tokens[len(prompt):]
