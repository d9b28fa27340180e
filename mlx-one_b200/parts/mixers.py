"""Sequence mixers: grouped-query attention over paged keys and values, the gated short
convolution with a fixed-size state, the gated delta rule with a matrix state per head,
several mixers side by side on one input, attention over one latent row per token, and
attention with two score maps per head."""

from __future__ import annotations

import torch

from .base import FixedState, Mixer, PagedKeyValues
from .registry import MIXERS, NORMS, POSITIONS
from .spec import PartSpec, TensorSpec


@MIXERS.register("attention")
class Attention(Mixer):
    """Grouped-query attention. Parameters: ``hidden``, ``heads``, ``kv_heads``,
    ``head_dim`` (size of a query and key head), ``value_dim`` (size of a value head; None =
    head_dim), ``bias`` (the three input projections have biases), ``qk_norm_eps`` (None = no
    per-head RMSNorm of queries and keys), ``qk_norm`` (``weighted_before``: with a stored
    weight, before the rotation; ``plain_after``: without a weight, after the rotation),
    ``position`` (a position-encoding PartSpec), ``window`` (None = all keys), ``scale`` (None =
    head_dim^-0.5), ``sink`` (a stored number per query head, ``sink`` [heads], that stands in
    the softmax's denominator as exp(sink) beside the keys' terms: it has no key and no value
    and is not scaled), ``keep_first`` (with a window: the sequence's first ``keep_first``
    positions stay visible to every later query, at their true positions), ``values``
    (``projected``, the default, or ``keys``: the values are the keys as projected, before norm
    and rotation, and there is no value matrix; a bias then belongs to queries and keys),
    ``conv_taps`` (None: none; else queries, keys and values pass, right after their projection,
    a causal convolution over the last ``conv_taps`` tokens of their request on every channel,
    with the stored ``q_conv``, ``k_conv``, ``v_conv`` [channels, taps], last column the current
    token's; the last taps - 1 projected rows of a request are kept in a state slot), ``gate``
    (None; ``values``: the heads' outputs are multiplied value by value with sigmoid(W_g x),
    ``gate.weight`` [heads * value_dim, hidden]; ``heads``: one number per head, ``gate.weight``
    [heads, hidden]; the gate reads the mixer's input and is applied before the output matrix).

    q, k, v projections (one fused matrix product), per-head RMSNorm of q and k, rotation,
    keys and values appended to the request's pages, causal softmax(q k^T scale) v where
    query head h reads key head h // (heads / kv_heads), output projection. Keys and values
    share pages whose rows have max(head_dim, value_dim) entries: the shorter of the two is
    padded with zeros (as are the queries), and the output matrix gets zero columns for the
    padding of the values, so the attention kernels see one head size.
    Reference: src/mlx_one/models/language/lfm2/reference_math.py:52-111; window mask
    src/mlx_one/models/shared/hybrid.py:14-20."""

    @staticmethod
    def _sizes(spec):
        head_dim = spec["head_dim"]
        value_dim = spec.get("value_dim") or head_dim
        return head_dim, value_dim, max(head_dim, value_dim)

    @staticmethod
    def _norm_kind(spec):
        if spec.get("qk_norm_eps") is None:
            return None
        kind = spec.get("qk_norm") or "weighted_before"
        if kind not in ("weighted_before", "plain_after"):
            raise ValueError(f"unknown qk_norm {kind!r}")
        return kind

    @classmethod
    def tensors(cls, spec):
        hidden = spec["hidden"]
        hd, vd, _ = cls._sizes(spec)
        q_dim, k_dim, v_dim = spec["heads"] * hd, spec["kv_heads"] * hd, spec["kv_heads"] * vd
        own_values = cls._own_values(spec)
        # (stored tensors keep their order from version to version: weights drawn in order by a
        # seeded generator stay what they were)
        out = {
            "q_proj.weight": TensorSpec((q_dim, hidden)),
            "k_proj.weight": TensorSpec((k_dim, hidden)),
        }
        if own_values:
            out["v_proj.weight"] = TensorSpec((v_dim, hidden))
        out["out_proj.weight"] = TensorSpec((hidden, spec["heads"] * vd))
        if spec.get("bias"):
            out["q_proj.bias"] = TensorSpec((q_dim,), "bias")
            out["k_proj.bias"] = TensorSpec((k_dim,), "bias")
            if own_values:
                out["v_proj.bias"] = TensorSpec((v_dim,), "bias")
        if spec.get("conv_taps"):
            for name, size in (("q_conv", q_dim), ("k_conv", k_dim), ("v_conv", v_dim)):
                out[name] = TensorSpec((size, spec["conv_taps"]), "wide")
        gate = cls._gate_kind(spec)
        if gate is not None:
            out["gate.weight"] = TensorSpec((spec["heads"] * (vd if gate == "values" else 1), hidden))
        if cls._norm_kind(spec) == "weighted_before":
            out["q_layernorm.weight"] = TensorSpec((hd,), "norm")
            out["k_layernorm.weight"] = TensorSpec((hd,), "norm")
        if spec.get("sink"):
            out["sink"] = TensorSpec((spec["heads"],), "wide")
        return out

    @staticmethod
    def _own_values(spec):
        kind = spec.get("values") or "projected"
        if kind not in ("projected", "keys"):
            raise ValueError(f"unknown values {kind!r}")
        if kind == "keys" and (spec.get("value_dim") or spec["head_dim"]) != spec["head_dim"]:
            raise ValueError("values that are the keys have the keys' size")
        return kind == "projected"

    @staticmethod
    def _gate_kind(spec):
        kind = spec.get("gate")
        if kind not in (None, "values", "heads"):
            raise ValueError(f"unknown gate {kind!r}")
        return kind

    @classmethod
    def cache_need(cls, spec):
        hd, vd, row = cls._sizes(spec)
        window = spec.get("window")
        pages = PagedKeyValues(spec["kv_heads"], row, window,
                               keep_first=int(spec.get("keep_first") or 0) if window else 0)
        taps = spec.get("conv_taps") or 0
        if taps < 2:
            return pages
        channels = (spec["heads"] + spec["kv_heads"]) * hd + spec["kv_heads"] * vd
        return {"pages": pages, "inputs": FixedState((taps - 1, channels))}

    def _reordered(self, weight, heads, order):
        """The rows of a projection [heads * head_dim, hidden] in another order within each
        head (queries and keys alike, so that their products stay what they were)."""
        if order is None:
            return weight
        index = (torch.arange(heads)[:, None] * self.head_dim + order[None, :]).reshape(-1)
        return weight[index.to(weight.device)]

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.heads, self.kv_heads = spec["heads"], spec["kv_heads"]
        self.head_dim, self.value_dim, self.row_dim = self._sizes(spec)
        if self.heads % self.kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        self.window = spec.get("window")
        scale = spec.get("scale")
        self.scale = float(self.head_dim ** -0.5 if scale is None else scale)
        position: PartSpec = spec.get("position") or PartSpec("none")
        self.position = POSITIONS.get(position.kind)(position, {}, runtime)
        # an encoding that pairs neighbouring dimensions: the kernels pair halves, so the rows
        # of the query and key projections (and their biases) are put into that order once
        order = getattr(self.position, "row_order", lambda size: None)(self.head_dim)
        reorder = lambda name, heads: self._reordered(tensors[name], heads, order)
        # values that are the keys as projected: the key matrix (in its stored order) once more
        # in the values' place, so that everything behind the projection stays as it is
        values = "v_proj" if self._own_values(spec) else "k_proj"
        self.gate_kind = self._gate_kind(spec)
        self.taps = int(spec.get("conv_taps") or 0)
        self.keep_first = int(spec.get("keep_first") or 0) if self.window else 0
        stacked = [reorder("q_proj.weight", self.heads), reorder("k_proj.weight", self.kv_heads),
                   tensors[values + ".weight"]]
        self.qkv_width = sum(weight.shape[0] for weight in stacked)
        # The gate reads the same input: its rows follow those of q, k and v where what comes
        # next takes a slice of wider rows (the convolution, the general preparation); the plain
        # preparation kernels want rows of their own, and the gate is then a second product.
        self.gate = None
        biases = []
        if spec.get("bias"):
            biases = [reorder("q_proj.bias", self.heads), reorder("k_proj.bias", self.kv_heads),
                      tensors[values + ".bias"]]
        if self.gate_kind is not None:
            general = (self.value_dim != self.head_dim or self._norm_kind(spec) == "plain_after"
                       or self.position.amplitude() != 1.0)
            if self.taps or general:
                stacked.append(tensors["gate.weight"])
                if biases:
                    biases.append(torch.zeros(tensors["gate.weight"].shape[0],
                                              dtype=biases[0].dtype, device=biases[0].device))
            else:
                self.gate = self.matrix(tensors["gate.weight"])
        self.qkv = self.matrix(torch.cat(stacked, dim=0))
        self.qkv_bias = self.vector(torch.cat(biases, dim=0)) if biases else None
        self.conv = None
        if self.taps:
            self.conv = self.vector(torch.cat([reorder("q_conv", self.heads),
                                               reorder("k_conv", self.kv_heads),
                                               tensors["v_conv"]], dim=0))
        out = tensors["out_proj.weight"]
        if self.value_dim < self.row_dim and self.gate_kind is None:
            # zero columns where the values' rows are padded
            wide = out.new_zeros((out.shape[0], self.heads, self.row_dim))
            wide[:, :, :self.value_dim] = out.view(out.shape[0], self.heads, self.value_dim)
            out = wide.view(out.shape[0], self.heads * self.row_dim)
        self.out = self.matrix(out)
        self.norm_kind = self._norm_kind(spec)
        self.eps = spec.get("qk_norm_eps")
        self.q_norm = self.k_norm = None
        if self.norm_kind == "weighted_before":
            self.q_norm = self.vector(tensors["q_layernorm.weight"])
            self.k_norm = self.vector(tensors["k_layernorm.weight"])
            if order is not None:
                self.q_norm = self.q_norm[order.to(self.q_norm.device)].contiguous()
                self.k_norm = self.k_norm[order.to(self.k_norm.device)].contiguous()
        self.ops.check_attention_sizes(self.heads, self.kv_heads, self.row_dim)
        # what the plain form of the operation (one head size, weighted norm before a pure
        # rotation) does not cover goes to the kernels as extra arguments
        self.extra = {}
        if (self.value_dim != self.head_dim or self.norm_kind == "plain_after"
                or self.position.amplitude() != 1.0):
            self.extra = dict(value_dim=self.value_dim, amplitude=self.position.amplitude(),
                              norm_after=self.norm_kind == "plain_after")
        self.sinks = {}
        if spec.get("sink"):
            self.sinks = dict(sinks=self.vector(tensors["sink"]))
        if self.keep_first:
            self.sinks["keep_first"] = self.keep_first
        # (with a second product for the gate the input is read twice: it is normed once, ahead)
        self.accepts_normed_input = self.gate is None

    fuses_residual = True
    scales_residual = True
    accepts_normed_input = True

    def inner_parts(self):
        return (self.position,)

    def input_projection(self):
        # (the plain form's kernels want rows of their own, the general preparation takes slices)
        return (self.qkv, self.qkv_bias) if self.extra and self.gate is None else None

    def forward(self, x, ctx, cache, write, residual=None):
        gate = None if self.gate is None else self.ops.linear(x, self.gate)
        return self.forward_projected(self.ops.linear(x, self.qkv, self.qkv_bias), ctx, cache,
                                      write, residual, gate=gate)

    def forward_projected(self, projected, ctx, cache, write, residual=None, gate=None):
        qkv = projected if projected.shape[1] == self.qkv_width else projected[:, :self.qkv_width]
        if self.gate_kind is not None and gate is None:
            gate = projected[:, self.qkv_width:]
        pages = cache
        if self.taps:
            pages = cache if self.taps < 2 else cache["pages"]
            qkv = self.ops.channel_conv(qkv, self.conv, None, taps=self.taps, activation=None,
                                        ctx=ctx, view=None if self.taps < 2 else cache["inputs"],
                                        write=write)
        mixed = self.ops.qkv_attention(
            qkv, heads=self.heads, kv_heads=self.kv_heads, head_dim=self.head_dim,
            q_weight=self.q_norm, k_weight=self.k_norm, eps=self.eps,
            rotary=self.position.rotary_table(), scale=self.scale, window=self.window, ctx=ctx,
            view=pages, write=write, **self.sinks, **self.extra)
        if self.gate_kind is not None:
            # (the heads' outputs may have rows of the pages' size: the gate leaves the values)
            mixed = self.ops.gate_heads(mixed, gate, heads=self.heads, row_dim=self.row_dim,
                                        value_dim=self.value_dim,
                                        per_head=self.gate_kind == "heads")
        if residual is None:
            return self.ops.linear(mixed, self.out)
        if self.residual_scale != 1.0:
            return self.ops.linear_add(mixed, self.out, None, residual, scale=self.residual_scale)
        return self.ops.linear_add(mixed, self.out, None, residual)


@MIXERS.register("short_conv")
class ShortConv(Mixer):
    """Gated short convolution. Parameters: ``hidden``, ``taps`` (kernel width), ``bias``.

    BCx = in_proj(x) split in the order B, C, x; g = B * x; y[t] = sum_k conv[:, k] *
    g[t - (taps-1) + k] over this request's tokens (zero before its first token), + bias;
    output = out_proj(C * y). The state is the last taps-1 rows of g.
    Reference: src/mlx_one/models/language/lfm2/reference_math.py:19-49; state
    src/mlx_one/core/cache.py:476-491; batched carry src/mlx_one/engine/hybrid.py:67-82."""

    @classmethod
    def tensors(cls, spec):
        hidden, taps = spec["hidden"], spec["taps"]
        out = {
            "in_proj.weight": TensorSpec((3 * hidden, hidden)),
            "conv": TensorSpec((hidden, taps)),
            "out_proj.weight": TensorSpec((hidden, hidden)),
        }
        if spec.get("bias"):
            out["in_proj.bias"] = TensorSpec((3 * hidden,), "bias")
            out["conv_bias"] = TensorSpec((hidden,), "bias")
            out["out_proj.bias"] = TensorSpec((hidden,), "bias")
        return out

    @classmethod
    def cache_need(cls, spec):
        return FixedState((max(spec["taps"] - 1, 1), spec["hidden"]))

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.hidden, self.taps = spec["hidden"], spec["taps"]
        self.in_proj = self.matrix(tensors["in_proj.weight"])
        self.out_proj = self.matrix(tensors["out_proj.weight"])
        self.kernel = self.vector(tensors["conv"])
        bias = bool(spec.get("bias"))
        self.in_bias = self.vector(tensors["in_proj.bias"]) if bias else None
        self.conv_bias = self.vector(tensors["conv_bias"]) if bias else None
        self.out_bias = self.vector(tensors["out_proj.bias"]) if bias else None

    fuses_residual = True
    accepts_normed_input = True

    def forward(self, x, ctx, cache, write, residual=None):
        gated = self.ops.linear_short_conv(x, self.in_proj, self.in_bias, kernel=self.kernel,
                                           bias=self.conv_bias, taps=self.taps, ctx=ctx,
                                           view=cache, write=write)
        if residual is None:
            return self.ops.linear(gated, self.out_proj, self.out_bias)
        return self.ops.linear_add(gated, self.out_proj, self.out_bias, residual)


@MIXERS.register("gated_delta")
class GatedDeltaRule(Mixer):
    """A linear-attention mixer whose state is one matrix S [key_dim, value_dim] per value head,
    kept in 32-bit from token to token. Parameters: ``hidden``, ``heads`` (value heads),
    ``kv_heads`` (query/key heads; value head h reads query/key head h // (heads / kv_heads)),
    ``key_dim``, ``value_dim``, ``taps``, ``eps`` (of the output norm).

    q, k = W x [kv_heads * key_dim], v = W x [heads * value_dim]; each channel passes a causal
    convolution over the last ``taps`` tokens of its request (``conv`` [channels, taps], last
    column the current token's) and silu. Per head q and k become unit vectors,
    x / sqrt(sum x^2 + 1e-6), and q is scaled by key_dim^-0.5. beta = sigmoid(W_b x) and the decay
    g = exp(-exp(A_log) softplus(W_a x + dt_bias)) are one number per value head. Then, per
    token and head: S = g S; u = beta (v - S^T k); S = S + k u^T; o = S^T q. The output is
    o / rms(o) (over value_dim, with ``eps``) * norm * silu(W_g x), projected by W_o.
    Everything after the convolutions' silu is 32-bit. The state of a request is S of every
    head and the last inputs of every convolution (a ring of ``taps`` rows, row = position %
    taps, of which a step reads the taps - 1 before its own), in one 32-bit slot."""

    UNIT_EPS = 1e-6

    @classmethod
    def _channels(cls, spec):
        qk = spec["kv_heads"] * spec["key_dim"]
        return qk, spec["heads"] * spec["value_dim"]

    @classmethod
    def tensors(cls, spec):
        hidden, heads, taps = spec["hidden"], spec["heads"], spec["taps"]
        qk, inner = cls._channels(spec)
        return {
            "q": TensorSpec((qk, hidden)), "q.conv": TensorSpec((qk, taps), "wide"),
            "k": TensorSpec((qk, hidden)), "k.conv": TensorSpec((qk, taps), "wide"),
            "v": TensorSpec((inner, hidden)), "v.conv": TensorSpec((inner, taps), "wide"),
            "b": TensorSpec((heads, hidden)), "a": TensorSpec((heads, hidden)),
            "A_log": TensorSpec((heads,), "wide"), "dt_bias": TensorSpec((heads,), "wide"),
            "norm": TensorSpec((spec["value_dim"],), "norm"),
            "g": TensorSpec((inner, hidden)), "o": TensorSpec((hidden, inner)),
        }

    @classmethod
    def state_size(cls, spec):
        qk, inner = cls._channels(spec)
        matrices = spec["heads"] * spec["key_dim"] * spec["value_dim"]
        return matrices + spec["taps"] * (2 * qk + inner)

    @classmethod
    def cache_need(cls, spec):
        return FixedState((cls.state_size(spec),), "float32")

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.sizes = dict(heads=spec["heads"], kv_heads=spec["kv_heads"], key_dim=spec["key_dim"],
                          value_dim=spec["value_dim"], taps=spec["taps"])
        if spec["heads"] % spec["kv_heads"]:
            raise ValueError("heads must be a multiple of kv_heads")
        # one product for everything that reads x: q | k | v | gate | beta | decay
        self.project = self.matrix(torch.cat([tensors[name] for name in
                                              ("q", "k", "v", "g", "b", "a")], dim=0))
        self.conv = self.vector(torch.cat([tensors[name] for name in
                                           ("q.conv", "k.conv", "v.conv")], dim=0))
        self.a_log = self.vector(tensors["A_log"])
        self.dt_bias = self.vector(tensors["dt_bias"])
        self.norm = self.vector(tensors["norm"])
        self.out = self.matrix(tensors["o"])
        self.eps = float(spec["eps"])

    fuses_residual = True
    accepts_normed_input = True

    def input_projection(self):
        return self.project, None

    def forward(self, x, ctx, cache, write, residual=None):
        return self.forward_projected(self.ops.linear(x, self.project), ctx, cache, write, residual)

    def forward_projected(self, projected, ctx, cache, write, residual=None):
        mixed = self.ops.gated_delta_rule(
            projected, conv=self.conv, a_log=self.a_log, dt_bias=self.dt_bias,
            norm_weight=self.norm, eps=self.eps, unit_eps=self.UNIT_EPS, ctx=ctx, view=cache,
            write=write, **self.sizes)
        if residual is None:
            return self.ops.linear(mixed, self.out)
        return self.ops.linear_add(mixed, self.out, None, residual)


@MIXERS.register("lightning")
class LightningAttention(Mixer):
    """Linear attention with a constant decay per head. Parameters: ``hidden``, ``heads``,
    ``key_dim``, ``value_dim``, ``decay`` (one number per head), ``eps`` (of the output norm).

    q, k = silu(W x) [heads * key_dim], v = silu(W x) [heads * value_dim], head by head. Per
    token and head S = decay_h S + k v^T and o = S^T q, with S [key_dim, value_dim] in 32-bit,
    zero at a request's start and carried from token to token in the request's state slot. The
    heads' outputs side by side are divided by their common root mean square (with ``eps``),
    multiplied by ``norm`` [heads * value_dim] and by sigmoid(W_g x), and projected by W_o.
    Everything after the projections' silu is 32-bit."""

    @classmethod
    def tensors(cls, spec):
        hidden = spec["hidden"]
        qk, inner = spec["heads"] * spec["key_dim"], spec["heads"] * spec["value_dim"]
        return {"q": TensorSpec((qk, hidden)), "k": TensorSpec((qk, hidden)),
                "v": TensorSpec((inner, hidden)), "g": TensorSpec((inner, hidden)),
                "norm": TensorSpec((inner,), "norm"), "o": TensorSpec((hidden, inner))}

    @classmethod
    def cache_need(cls, spec):
        return FixedState((spec["heads"] * spec["key_dim"] * spec["value_dim"],), "float32")

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.sizes = dict(heads=spec["heads"], key_dim=spec["key_dim"], value_dim=spec["value_dim"])
        decay = [float(value) for value in spec["decay"]]
        if len(decay) != spec["heads"]:
            raise ValueError("one decay per head")
        self.decay = torch.tensor(decay, dtype=torch.float64).to(torch.float32).to(runtime.device)
        # one product for everything that reads x: q | k | v | gate
        self.project = self.matrix(torch.cat([tensors[name] for name in ("q", "k", "v", "g")], dim=0))
        self.norm = self.vector(tensors["norm"])
        self.out = self.matrix(tensors["o"])
        self.eps = float(spec["eps"])

    fuses_residual = True
    scales_residual = True
    accepts_normed_input = True

    def input_projection(self):
        return self.project, None

    def forward(self, x, ctx, cache, write, residual=None):
        return self.forward_projected(self.ops.linear(x, self.project), ctx, cache, write, residual)

    def forward_projected(self, projected, ctx, cache, write, residual=None):
        mixed = self.ops.lightning_attention(
            projected, decay=self.decay, norm_weight=self.norm, eps=self.eps, ctx=ctx, view=cache,
            write=write, **self.sizes)
        if residual is None:
            return self.ops.linear(mixed, self.out)
        if self.residual_scale != 1.0:
            return self.ops.linear_add(mixed, self.out, None, residual, scale=self.residual_scale)
        return self.ops.linear_add(mixed, self.out, None, residual)


@MIXERS.register("parallel")
class ParallelMixers(Mixer):
    """Several mixers side by side on the same input. Parameters: ``hidden``, ``eps``,
    ``branches``: a tuple of (name, mixer PartSpec, stored name of the branch's output weight);
    ``shared_projection`` (True): one product for the input projections of all branches.
    Every branch's output is divided by its root mean square over the model width (with
    ``eps``) and multiplied by its weight [hidden]; the mixer's output is the mean of these,
    added to the 32-bit stream without being rounded first. Each branch keeps what its mixer
    needs (pages, a state slot) under its name."""

    @classmethod
    def _branches(cls, spec):
        return [(name, part, MIXERS.get(part.kind), weight)
                for name, part, weight in spec["branches"]]

    @classmethod
    def tensors(cls, spec):
        out = {}
        for name, part, kind, weight in cls._branches(spec):
            for local, want in kind.tensors(part).items():
                out[part.stored_name(local)] = want
            out[weight] = TensorSpec((spec["hidden"],), "norm")
        return out

    @classmethod
    def cache_need(cls, spec):
        needs = {name: kind.cache_need(part) for name, part, kind, _ in cls._branches(spec)}
        return {name: need for name, need in needs.items() if need is not None} or None

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.eps = float(spec["eps"])
        self.names, self.branches, self.weights = [], [], []
        for name, part, kind, weight in self._branches(spec):
            local = {key: tensors[part.stored_name(key)] for key in kind.tensors(part)}
            self.names.append(name)
            self.branches.append(kind(part, local, runtime))
            self.weights.append(self.vector(tensors[weight]))
        # One product for all branches where each reads its input through one projection: the
        # weights stacked, the branches take column ranges of the result. The input is then used
        # by that product only, so the norm before it may be applied inside it.
        self.project = self.project_bias = None
        self.columns: list[tuple[int, int]] = []
        projections = [branch.input_projection() for branch in self.branches]
        if spec.get("shared_projection", True) and all(p is not None for p in projections):
            self.project = torch.cat([weight for weight, _ in projections], dim=0).contiguous()
            if any(bias is not None for _, bias in projections):
                self.project_bias = torch.cat([
                    bias if bias is not None else torch.zeros(weight.shape[0], dtype=torch.float32,
                                                              device=weight.device)
                    for weight, bias in projections]).contiguous()
            at = 0
            for weight, _ in projections:
                self.columns.append((at, at + weight.shape[0]))
                at += weight.shape[0]
            for branch in self.branches:        # the stacked copy is the one that is read
                for name in ("qkv", "project"):
                    if hasattr(branch, name):
                        setattr(branch, name, None)
            self.accepts_normed_input = True

    fuses_residual = True

    def inner_parts(self):
        parts = list(self.branches)
        for branch in self.branches:
            parts += list(getattr(branch, "inner_parts", lambda: ())())
        return parts

    def forward(self, x, ctx, cache, write, residual=None):
        cache = cache or {}
        if self.project is not None:
            projected = self.ops.linear(x, self.project, self.project_bias)
            outputs = [branch.forward_projected(projected[:, lo:hi], ctx, cache.get(name), write)
                       for name, branch, (lo, hi) in zip(self.names, self.branches, self.columns)]
        else:
            outputs = [branch.forward(x, ctx, cache.get(name), write)
                       for name, branch in zip(self.names, self.branches)]
        if residual is None:
            raise ValueError("side-by-side mixers add their mean into the stream themselves")
        self.ops.normed_mean_add(residual, outputs, self.weights, self.eps)
        return None


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    """Softmax attention whose keys and values of all heads come from one small latent per
    token. Parameters: ``hidden``, ``heads``, ``head_dim`` (unrotated query/key dimensions of a
    head), ``rot_dim`` (rotated ones), ``value_dim``, ``latent`` (size of the latent), ``eps`` (of
    the latent's norm), ``position`` (a position-encoding PartSpec for the rotated part), ``scale``,
    ``gate`` (a sigmoid gate on the heads' outputs, computed from the mixer's input).

    q = W_q x, head by head [head_dim unrotated | rot_dim rotated]. W_down x has latent + rot_dim
    rows: the first ``latent``, divided by their root mean square and multiplied by ``down_norm``,
    are the latent c; the last rot_dim are one rotated key part r that all heads share. Per head
    h the key is [W_uk,h c | r] and the value W_uv,h c; causal softmax(q k^T scale) v; the heads
    side by side are multiplied by sigmoid(W_g x) and projected by W_o.

    Only c and r are kept per token: one row [c | r] in single-plane pages. The up-projections
    move to the query's side: q_h . (W_uk,h c) = (W_uk,h^T q_h) . c, so every head's query becomes
    [W_uk,h^T q_h | rotated part] against the one shared row, the attention's output is the
    weights' average of c, and the head's value is W_uv,h applied to that average. Scores,
    weights, the norm and the rotation are 32-bit."""

    @classmethod
    def tensors(cls, spec):
        hidden, heads, latent = spec["hidden"], spec["heads"], spec["latent"]
        inner = heads * spec["value_dim"]
        out = {"q": TensorSpec((heads * (spec["head_dim"] + spec["rot_dim"]), hidden)),
               "down": TensorSpec((latent + spec["rot_dim"], hidden)),
               "down_norm": TensorSpec((latent,), "norm"),
               "up_k": TensorSpec((heads * spec["head_dim"], latent)),
               "up_v": TensorSpec((inner, latent)),
               "out": TensorSpec((hidden, inner))}
        if spec.get("gate", True):
            out["gate"] = TensorSpec((inner, hidden))
        return out

    @classmethod
    def cache_need(cls, spec):
        return PagedKeyValues(1, spec["latent"] + spec["rot_dim"], planes=1)

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.heads, self.head_dim, self.rot_dim = spec["heads"], spec["head_dim"], spec["rot_dim"]
        self.value_dim, self.latent = spec["value_dim"], spec["latent"]
        self.scale, self.eps = float(spec["scale"]), float(spec["eps"])
        position: PartSpec = spec.get("position") or PartSpec("none")
        self.position = POSITIONS.get(position.kind)(position, {}, runtime)
        self.neighbours = getattr(self.position, "layout", "halves") == "neighbours"
        self.gated = bool(spec.get("gate", True))
        # one product for everything that reads x: q | latent and shared key part | gate
        names = ["q", "down"] + (["gate"] if self.gated else [])
        self.project = self.matrix(torch.cat([tensors[name] for name in names], dim=0))
        self.down_norm = self.vector(tensors["down_norm"])
        # per head: [latent, head_dim] (the key's up-projection, transposed) and [value_dim, latent]
        up_k = tensors["up_k"].view(self.heads, self.head_dim, self.latent)
        self.up_k = self.matrix(up_k.transpose(1, 2))
        self.up_v = self.matrix(tensors["up_v"].view(self.heads, self.value_dim, self.latent))
        self.out = self.matrix(tensors["out"])
        self.ops.check_attention_sizes(self.heads, 1, self.latent + self.rot_dim)

    def inner_parts(self):
        return (self.position,)

    def forward(self, x, ctx, cache, write):
        heads, latent, rot = self.heads, self.latent, self.rot_dim
        projected = self.ops.linear(x, self.project)
        tokens = projected.shape[0]
        queries = torch.empty((tokens, heads, latent + rot), dtype=projected.dtype,
                              device=projected.device)
        # the latent's norm, the rotation of the shared key part and of the queries' rotated
        # parts, the row [c | r] appended to the request's pages
        self.ops.latent_prepare(projected, queries, heads=heads, head_dim=self.head_dim,
                                rot_dim=rot, latent=latent, norm_weight=self.down_norm,
                                eps=self.eps, rotary=self.position.rotary_table(),
                                neighbours=self.neighbours, ctx=ctx, view=cache, write=write)
        plain = projected[:, :heads * (self.head_dim + rot)].view(tokens, heads, -1)
        self.ops.linear_heads(plain[:, :, :self.head_dim], self.up_k, out=queries[:, :, :latent])
        mixed = self.ops.latent_attention(queries, heads=heads, latent=latent, scale=self.scale,
                                          ctx=ctx, view=cache)
        values = self.ops.linear_heads(mixed[:, :, :latent], self.up_v)
        values = values.view(tokens, heads * self.value_dim)
        if self.gated:
            gate = projected[:, heads * (self.head_dim + rot) + latent + rot:]
            values = self.ops.sigmoid_gate(values, gate)
        return self.ops.linear(values, self.out)


@MIXERS.register("differential_attention")
class DifferentialAttention(Mixer):
    """Grouped-query attention with two score maps per head over the same values. Parameters:
    ``hidden``, ``heads``, ``kv_heads``, ``head_dim`` (of one map's queries and keys),
    ``value_dim``, ``eps``, ``scale``, ``diff`` (a constant of the mixing factor), ``chunk`` (None:
    every earlier position is seen; else only those of the query's own chunk of ``chunk``
    positions, counted from 0).

    q = W_q x has heads * 2 * head_dim rows, k = W_k x kv_heads * 2 * head_dim, head by head as
    [map 1 | map 2]; v = W_v x. Queries and keys are divided by their root mean square per head and
    map and multiplied by ``q_norm`` / ``k_norm`` [head_dim]; no rotation. Each map is a causal
    softmax attention of its own; with a1, a2 their outputs and lambda = exp(lq1 . lk1) -
    exp(lq2 . lk2) + diff (one number), o = a1 - lambda a2, divided by its root mean square over
    value_dim, times (1 - diff); W_o on the heads side by side.

    The two maps run as twice as many heads of one attention: the rows of W_q and W_k are put
    map by map at load time (query head m * heads + h, key head m * kv_heads + g), so that the
    grouping of query heads over key heads holds within each map, and W_v is stacked twice so that
    both maps' key heads find their values in the pages."""

    @classmethod
    def tensors(cls, spec):
        hidden, dim = spec["hidden"], spec["head_dim"]
        out = {"q": TensorSpec((spec["heads"] * 2 * dim, hidden)),
               "k": TensorSpec((spec["kv_heads"] * 2 * dim, hidden)),
               "v": TensorSpec((spec["kv_heads"] * spec["value_dim"], hidden)),
               "q_norm": TensorSpec((dim,), "norm"), "k_norm": TensorSpec((dim,), "norm"),
               "out": TensorSpec((hidden, spec["heads"] * spec["value_dim"]))}
        for name in ("lq1", "lk1", "lq2", "lk2"):
            out[name] = TensorSpec((dim,), "wide")
        return out

    @classmethod
    def cache_need(cls, spec):
        return PagedKeyValues(2 * spec["kv_heads"], max(spec["head_dim"], spec["value_dim"]),
                              chunk=spec.get("chunk"))

    @staticmethod
    def _by_map(weight, heads, dim):
        """Rows [head][map][dim] -> [map][head][dim]."""
        return weight.view(heads, 2, dim, -1).transpose(0, 1).reshape(2 * heads * dim, -1)

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.heads, self.kv_heads = spec["heads"], spec["kv_heads"]
        self.head_dim, self.value_dim = spec["head_dim"], spec["value_dim"]
        if self.heads % self.kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        self.row_dim = max(self.head_dim, self.value_dim)
        self.scale, self.eps = float(spec["scale"]), float(spec["eps"])
        self.diff = float(spec["diff"])
        self.chunk = spec.get("chunk")
        self.qkv = self.matrix(torch.cat([
            self._by_map(tensors["q"], self.heads, self.head_dim),
            self._by_map(tensors["k"], self.kv_heads, self.head_dim),
            tensors["v"], tensors["v"]], dim=0))
        self.q_norm = self.vector(tensors["q_norm"])
        self.k_norm = self.vector(tensors["k_norm"])
        dot = lambda a, b: (tensors[a].to(torch.float32) * tensors[b].to(torch.float32)).sum()
        self.mix = float(torch.exp(dot("lq1", "lk1")) - torch.exp(dot("lq2", "lk2"))) + self.diff
        self.out = self.matrix(tensors["out"])
        self.ops.check_attention_sizes(2 * self.heads, 2 * self.kv_heads, self.row_dim)
        self.extra = {}
        if self.value_dim != self.head_dim:
            self.extra = dict(value_dim=self.value_dim, amplitude=1.0, norm_after=False)

    def forward(self, x, ctx, cache, write):
        qkv = self.ops.linear(x, self.qkv)
        maps = self.ops.qkv_attention(
            qkv, heads=2 * self.heads, kv_heads=2 * self.kv_heads, head_dim=self.head_dim,
            q_weight=self.q_norm, k_weight=self.k_norm, eps=self.eps, rotary=None,
            scale=self.scale, window=None, chunk=self.chunk, ctx=ctx, view=cache, write=write,
            **self.extra)
        mixed = self.ops.differential_combine(maps, heads=self.heads, row_dim=self.row_dim,
                                              value_dim=self.value_dim, mix=self.mix, eps=self.eps,
                                              factor=1.0 - self.diff)
        return self.ops.linear(mixed, self.out)


@MIXERS.register("mamba2")
class SelectiveStateSpace(Mixer):
    """A selective state space in the form of Mamba-2: one matrix state S [state, value_dim] per
    head, kept in 32-bit from token to token. Parameters: ``hidden``, ``heads``, ``value_dim``,
    ``state`` (N), ``groups`` (G; head h reads group h // (heads / groups)), ``taps``,
    ``norm_groups``, ``eps``.

    With inner = heads * value_dim, W_in x is laid out as [z: inner | x: inner | B: G N | C: G N |
    dt: heads]. x, B and C together pass a causal convolution over the last ``taps`` tokens of
    their request on every channel (``conv`` [channels, taps], last column the current token's,
    ``conv_bias``) and silu. dt = softplus(dt + dt_bias). Per token and head: S = exp(-exp(A_log)
    dt) S + dt B x^T; y = S^T C + D x. The heads' outputs side by side are multiplied by silu(z),
    divided by their root mean square in ``norm_groups`` equal parts (each part by its own, with
    ``eps``), multiplied by ``norm`` and projected by W_o. Everything after the convolution's
    silu is 32-bit. A request keeps S of every head in a 32-bit slot and the convolution's last
    taps - 1 inputs in a slot of the compute dtype."""

    @classmethod
    def _sizes(cls, spec):
        inner = spec["heads"] * spec["value_dim"]
        return inner, inner + 2 * spec["groups"] * spec["state"]

    @classmethod
    def tensors(cls, spec):
        hidden, heads = spec["hidden"], spec["heads"]
        inner, channels = cls._sizes(spec)
        return {"in": TensorSpec((inner + channels + heads, hidden)),
                "conv": TensorSpec((channels, spec["taps"]), "wide"),
                "conv_bias": TensorSpec((channels,), "bias"),
                "dt_bias": TensorSpec((heads,), "wide"), "A_log": TensorSpec((heads,), "wide"),
                "D": TensorSpec((heads,), "norm"), "norm": TensorSpec((inner,), "norm"),
                "o": TensorSpec((hidden, inner))}

    @classmethod
    def cache_need(cls, spec):
        _, channels = cls._sizes(spec)
        need = {"state": FixedState((spec["heads"] * spec["state"] * spec["value_dim"],), "float32")}
        if spec["taps"] > 1:
            need["inputs"] = FixedState((spec["taps"] - 1, channels))
        return need

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.sizes = dict(heads=spec["heads"], value_dim=spec["value_dim"], state_dim=spec["state"],
                          groups=spec["groups"])
        if spec["heads"] % spec["groups"]:
            raise ValueError("heads must be a multiple of groups")
        self.inner, self.channels = self._sizes(spec)
        self.taps, self.norm_groups = int(spec["taps"]), int(spec["norm_groups"])
        if self.inner % self.norm_groups:
            raise ValueError("the heads' outputs must split into equal parts for the norm")
        self.project = self.matrix(tensors["in"])
        self.conv = self.vector(tensors["conv"])
        self.conv_bias = self.vector(tensors["conv_bias"])
        self.dt_bias = self.vector(tensors["dt_bias"])
        self.a_log = self.vector(tensors["A_log"])
        self.skip = self.vector(tensors["D"])
        self.norm = self.vector(tensors["norm"])
        self.out = self.matrix(tensors["o"])
        self.eps = float(spec["eps"])

    accepts_normed_input = True

    def input_projection(self):
        return self.project, None

    def forward(self, x, ctx, cache, write):
        return self.forward_projected(self.ops.linear(x, self.project), ctx, cache, write)

    def forward_projected(self, projected, ctx, cache, write, residual=None):
        inner, channels = self.inner, self.channels
        mixed = self.ops.channel_conv(projected[:, inner:inner + channels], self.conv,
                                      self.conv_bias, taps=self.taps, activation="silu", ctx=ctx,
                                      view=cache.get("inputs"), write=write)
        y = self.ops.state_space_scan(mixed, projected[:, inner + channels:], a_log=self.a_log,
                                      dt_bias=self.dt_bias, skip=self.skip, ctx=ctx,
                                      view=cache["state"], write=write, **self.sizes)
        gated = self.ops.gated_group_norm(y, projected[:, :inner], self.norm,
                                          groups=self.norm_groups, eps=self.eps,
                                          dtype=self.runtime.dtype)
        out = self.ops.linear(gated, self.out)
        if residual is not None:
            raise ValueError("this mixer hands its output back")
        return out
