"""Plain, slow Lamisun written from the design's equations: whole sequences, no cache, one
function per mechanism. It shares no code with the engine: it reads config.json and the
safetensors file by itself and computes everything in one floating type (float64 by default).

Notation: x [T, W] the stream, h the input of a sublayer, T tokens at positions 0..T-1.
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


def rms(x, eps):
    return torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return x / rms(x, eps) * w


def softplus(z):
    return math.log1p(math.exp(z))


def xielu(z, p, q):
    """Above zero softplus(p) z^2 + z/2; at and below zero (1/2 + softplus(q)) (e^z - 1 - z) + z/2."""
    up = softplus(p) * z * z + 0.5 * z
    down = (0.5 + softplus(q)) * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z
    return torch.where(z > 0, up, down)


def embed(tokens, table, scale, bigram=None, rule=None):
    """Row of each token times ``scale``; plus the pair table's row (31-style hash of the token
    before and the token), the table's last row for the first token."""
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x = table[ids] * scale
    if bigram is not None:
        buckets = rule["buckets"]
        rows = [buckets]
        for t in range(1, len(tokens)):
            rows.append((int(tokens[t - 1]) * rule["mul_prev"] + int(tokens[t]) * rule["mul_cur"])
                        % buckets)
        x = x + bigram[torch.tensor(rows)]
    return x


def input_convolution(h, w):
    """h + conv(h): conv(h)_t = sum_j w[:, j] h_(t - taps + 1 + j), nothing before the start."""
    taps = w.shape[1]
    out = h.clone()
    for t in range(h.shape[0]):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] = out[t] + w[:, j] * h[s]
    return out


def rotate_pairs(x, positions, base, dims):
    """x [T, heads, D]: within the first ``dims`` dimensions the neighbours (2i, 2i+1) are turned
    by position * base^(-2i/dims); the others pass."""
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=x.dtype)
    angle = positions.to(x.dtype)[:, None] * f[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def visible(T, chunk=None):
    """[T, T] True where query i may read key j: j <= i, and with ``chunk`` both in one chunk."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    mask = j <= i
    if chunk is not None:
        mask = mask & (i // chunk == j // chunk)
    return mask


def softmax_rows(scores, mask):
    scores = scores.masked_fill(~mask, float("-inf"))
    scores = scores - scores.max(-1, keepdim=True).values
    e = torch.exp(scores)
    return e / e.sum(-1, keepdim=True)


# --------------------------------------------------------------------------- mixers


def latent_attention(h, w, m, eps, prefix):
    """Keys and values of all heads come from one small latent per token; a part of every key
    is one rotated vector that all heads share; a sigmoid gate on the heads' outputs."""
    T = h.shape[0]
    H, D, R, V, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    positions = torch.arange(T)
    q = (h @ w[prefix + "q"].T).view(T, H, D + R)
    q_plain, q_rot = q[..., :D], q[..., D:]
    down = h @ w[prefix + "dkv"].T
    latent = rms_norm(down[:, :C], w[prefix + "dkv.norm"], eps)
    k_rot = down[:, C:].view(T, 1, R)
    rot = m["rot"]
    q_rot = rotate_pairs(q_rot, positions, rot["base"], rot["dims"])
    k_rot = rotate_pairs(k_rot, positions, rot["base"], rot["dims"])
    k_plain = (latent @ w[prefix + "uk"].T).view(T, H, D)
    v = (latent @ w[prefix + "uv"].T).view(T, H, V)
    mask = visible(T)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for head in range(H):
        scores = (q_plain[:, head] @ k_plain[:, head].T + q_rot[:, head] @ k_rot[:, 0].T) * m["scale"]
        out[:, head] = softmax_rows(scores, mask) @ v[:, head]
    gate = torch.sigmoid(h @ w[prefix + "g"].T)
    return (out.reshape(T, H * V) * gate) @ w[prefix + "o"].T


def differential_attention(h, w, m, eps, prefix):
    """Two score maps per head over the same values, within chunks of the sequence; the second
    map's output is taken off the first's with one learned factor, and the difference is divided
    by its root mean square."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[prefix + "q"].T).view(T, H, 2, D)
    k = (h @ w[prefix + "k"].T).view(T, G, 2, D)
    v = (h @ w[prefix + "v"].T).view(T, G, V)
    q = rms_norm(q, w[prefix + "q.norm"], eps)
    k = rms_norm(k, w[prefix + "k.norm"], eps)
    chunk = (m.get("mask") or {}).get("size")
    mask = visible(T, chunk)
    lam = (math.exp(float((w[prefix + "lq1"] * w[prefix + "lk1"]).sum()))
           - math.exp(float((w[prefix + "lq2"] * w[prefix + "lk2"]).sum())) + m["diff"])
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for head in range(H):
        group = head // (H // G)
        maps = []
        for which in range(2):
            scores = (q[:, head, which] @ k[:, group, which].T) * m["scale"]
            maps.append(softmax_rows(scores, mask) @ v[:, group])
        o = maps[0] - lam * maps[1]
        out[:, head] = o / rms(o, eps) * (1 - m["diff"])
    return out.reshape(T, H * V) @ w[prefix + "o"].T


MIXERS = {"latent_attention": latent_attention, "attention": differential_attention}


def feed_forward(h, w, prefix):
    p, q = (float(value) for value in w[prefix + "act"])
    return xielu(h @ w[prefix + "up"].T, p, q) @ w[prefix + "down"].T


# --------------------------------------------------------------------------- the model


def forward(config, weights, tokens, kind=torch.float64, streams=None):
    """Logits [T, vocab] of one sequence. ``streams``: a list that receives the stream after the
    embedding and after every layer."""
    w = {name: (t.to(kind) if t.is_floating_point() else t) for name, t in weights.items()}
    eps = config["norm"]["eps"]
    emb = config["embedding"]
    rule = emb.get("bigram")
    x = embed(tokens, w["embed"], emb["scale"], w["bigram"] if rule else None, rule)
    canon = config.get("canon")
    results = [x]
    if streams is not None:
        streams.append(x.clone())
    for index, layer in enumerate(config["layers"]):
        prefix = f"l{index}."
        h = input_convolution(x, w[prefix + "canon1"]) if canon else x
        mixed = MIXERS[layer["type"]](h, w, layer["mixer"], eps, prefix + "mix.")
        x = x + rms_norm(mixed, w[prefix + "norm1"], eps)
        if layer.get("mlp") is not None:
            h = input_convolution(x, w[prefix + "canon2"]) if canon else x
            x = x + rms_norm(feed_forward(h, w, prefix + "mlp."), w[prefix + "norm2"], eps)
        results.append(x)
        if prefix + "dwa" in w:
            x = sum(w[prefix + "dwa"][j] * results[j] for j in range(index + 2))
        if streams is not None:
            streams.append(x.clone())
    x = rms_norm(x, w["final.norm"], eps)
    return x @ w["head"].T


def load(model_dir):
    path = Path(model_dir)
    return json.loads((path / "config.json").read_text()), read_tensors(path / "model.safetensors")
