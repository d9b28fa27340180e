"""Feed-forward parts."""

from __future__ import annotations

import torch

from .base import FeedForward
from .registry import FEED_FORWARDS
from .spec import TensorSpec


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    """w2(act(w1 x) * w3 x), no biases. Parameters: ``hidden``, ``width``, ``activation`` of the
    gate (``silu``, the default, or ``gelu_tanh``, ``relu``, ``relu2``). The gate and up matrices
    are stacked at load time so that one matrix product feeds the gate kernel.
    Reference: src/mlx_one/models/language/lfm2/reference_math.py:114-135."""

    @classmethod
    def tensors(cls, spec):
        hidden, width = spec["hidden"], spec["width"]
        return {
            "w1.weight": TensorSpec((width, hidden)),
            "w3.weight": TensorSpec((width, hidden)),
            "w2.weight": TensorSpec((hidden, width)),
        }

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.width = spec["width"]
        self.activation = spec.get("activation") or "silu"
        self.gate_up = self.matrix(torch.cat([tensors["w1.weight"], tensors["w3.weight"]], dim=0))
        self.down = self.matrix(tensors["w2.weight"])

    fuses_residual = True
    scales_residual = True
    accepts_normed_input = True

    def forward(self, x, ctx, residual=None):
        if self.activation == "silu":
            gated = self.ops.linear_swiglu(x, self.gate_up)
        else:
            gated = self.ops.linear_gated(x, self.gate_up, self.activation)
        if residual is None:
            return self.ops.linear(gated, self.down)
        if self.residual_scale != 1.0:
            return self.ops.linear_add(gated, self.down, None, residual, scale=self.residual_scale)
        return self.ops.linear_add(gated, self.down, None, residual)


@FEED_FORWARDS.register("dense")
class DenseFeedForward(FeedForward):
    """down(act(up x)), no gate, no biases. Parameters: ``hidden``, ``width``, ``activation``:
    ``relu2`` (the square of max(z, 0)), ``gelu_tanh`` (0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715
    z^3)))), ``silu``, ``relu``, or ``xielu``: with the two stored numbers ``act`` = (p, q), a =
    softplus(p) and b = 1/2 + softplus(q), a z^2 + z / 2 above zero and b (e^z - 1 - z) + z / 2 at
    and below it. The activation is the up product's epilogue where the kernels have one."""

    ACTIVATIONS = ("relu2", "gelu_tanh", "silu", "relu", "xielu")

    @classmethod
    def tensors(cls, spec):
        hidden, width = spec["hidden"], spec["width"]
        out = {"up.weight": TensorSpec((width, hidden)),
               "down.weight": TensorSpec((hidden, width))}
        if spec.get("activation") == "xielu":
            out["act"] = TensorSpec((2,), "wide")
        return out

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.activation = spec.get("activation", "relu2")
        if self.activation not in self.ACTIVATIONS:
            raise ValueError(f"unknown activation {self.activation!r}")
        self.up = self.matrix(tensors["up.weight"])
        self.down = self.matrix(tensors["down.weight"])
        self.shape = {}
        if self.activation == "xielu":
            # the two factors, worked out once in 32-bit
            p, q = tensors["act"].to(torch.float32).cpu()
            softplus = torch.nn.functional.softplus
            self.shape = dict(params=(float(softplus(p)), float(0.5 + softplus(q))))

    fuses_residual = True
    accepts_normed_input = True

    def forward(self, x, ctx, residual=None):
        hidden = self.ops.linear_act(x, self.up, self.activation, **self.shape)
        if residual is None:
            return self.ops.linear(hidden, self.down)
        return self.ops.linear_add(hidden, self.down, None, residual)


@FEED_FORWARDS.register("routed")
class RoutedExperts(FeedForward):
    """A mixture of gated feed-forwards. Parameters: ``hidden``, ``width`` (of an expert),
    ``experts``, ``top`` (experts a token uses), ``groups`` and ``keep`` (experts form ``groups``
    equal runs of neighbours; a group's score is the sum of its ``group_score`` largest scores,
    and only experts of the ``keep`` best groups can be chosen), ``shared_width`` (None: no
    shared expert), ``activation`` of the gates, ``scores`` (``sigmoid``, or ``softmax`` over all
    outputs of the router), ``correction`` (True: the stored ``correction``, one number per
    output of the router, is added to the scores where experts are chosen, and only there),
    ``normalize`` (True; False: the chosen experts keep their scores as weights), ``identity``
    (0: that many further outputs of the router, behind the experts', stand for experts without
    tensors whose output is the input itself), ``shared_gate`` (True: the shared expert's output
    is multiplied by sigmoid(w x), one number per token, with the stored ``shared.sg`` [1,
    hidden]).

    Router logits W_r x are 32-bit, scores s = sigmoid of them; the ``top`` allowed experts
    with the largest scores are chosen and weighted with s / (sum of the chosen s + 1e-20). The
    output is the weighted sum of the chosen experts' down(act(gate x) * up x), plus the shared
    expert's, which every token uses with weight 1. The options above (softmax scores, a
    correction, weights that are not normalised, identity outputs, a gated shared expert) go
    through a second routing kernel that has no groups.

    The experts' gate and up matrices are stacked into one matrix and their down matrices side
    by side into another (the shared expert last). Small steps run every token through all of
    it: one product with the gate, the routing weights multiplied into the expert's columns
    (zero for experts that were not chosen), one down product; at those sizes every expert's
    weights are read anyway. Where the kernel set offers it (``sorts_experts``) larger steps sort
    their (token, expert) pairs by expert and run one grouped product per matrix over the same
    stacked weights, so that a token costs only the experts it uses."""

    @classmethod
    def tensors(cls, spec):
        hidden, width = spec["hidden"], spec["width"]
        outputs = spec["experts"] + int(spec.get("identity") or 0)
        out = {"router": TensorSpec((outputs, hidden), "wide")}
        if spec.get("correction"):
            out["correction"] = TensorSpec((outputs,), "norm0")
        if spec.get("shared_gate"):
            if not spec.get("shared_width"):
                raise ValueError("a gate of the shared expert needs a shared expert")
            out["shared.sg"] = TensorSpec((1, hidden), "wide")
        for e in range(spec["experts"]):
            out[f"e{e}.gate"] = TensorSpec((width, hidden))
            out[f"e{e}.up"] = TensorSpec((width, hidden))
            out[f"e{e}.down"] = TensorSpec((hidden, width))
        if spec.get("shared_width"):
            shared = spec["shared_width"]
            out["shared.gate"] = TensorSpec((shared, hidden))
            out["shared.up"] = TensorSpec((shared, hidden))
            out["shared.down"] = TensorSpec((hidden, shared))
        return out

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.experts, self.width = spec["experts"], spec["width"]
        self.shared_width = spec.get("shared_width") or 0
        self.activation = spec.get("activation") or "silu"
        scores = spec.get("scores") or "sigmoid"
        if scores not in ("sigmoid", "softmax"):
            raise ValueError(f"unknown routing scores {scores!r}")
        self.identity = int(spec.get("identity") or 0)
        self.shared_gate = bool(spec.get("shared_gate"))
        normalize = spec.get("normalize", True)
        self.routing = dict(experts=self.experts, top=spec["top"], groups=spec.get("groups") or 1,
                            keep=spec.get("keep") or 1, group_score=spec.get("group_score") or 2)
        if self.experts % self.routing["groups"]:
            raise ValueError("experts must form equal groups")
        # what the first routing kernel does not know goes to the second one
        self.general = None
        if (scores != "sigmoid" or spec.get("correction") or not normalize or self.identity
                or self.shared_gate):
            if self.routing["groups"] != 1:
                raise ValueError("groups of experts go with sigmoid scores, normalised weights "
                                 "and no identity outputs")
            self.general = dict(experts=self.experts, identity=self.identity, top=spec["top"],
                                scores=scores, normalize=bool(normalize),
                                shared_gate=self.shared_gate)
            self.correction = None
            if spec.get("correction"):
                self.correction = tensors["correction"].to(torch.float32).contiguous()
        names = [f"e{e}." for e in range(self.experts)] + (["shared."] if self.shared_width else [])
        self.gate_up = self.matrix(torch.cat([tensors[name + "gate"] for name in names] +
                                             [tensors[name + "up"] for name in names], dim=0))
        self.down = self.matrix(torch.cat([tensors[name + "down"] for name in names], dim=1))
        self.router = tensors["router"].to(torch.float32).contiguous()
        if self.shared_gate:
            # the gate's row behind the router's: one pass over the token serves both
            self.router = torch.cat([self.router, tensors["shared.sg"].to(torch.float32)
                                     .reshape(1, -1)], dim=0).contiguous()
        # the shared expert once more on its own, for steps that sort their tokens by expert
        self.shared = {}
        self.sortable = (self.activation == "silu" and hasattr(self.ops, "sorts_experts")
                         and runtime.dtype == torch.bfloat16)
        if self.sortable and self.shared_width:
            self.shared = dict(
                shared_gate_up=self.matrix(torch.cat([tensors["shared.gate"], tensors["shared.up"]], dim=0)),
                shared_down=self.matrix(tensors["shared.down"]))

    fuses_residual = True
    scales_residual = True

    def _forward_general(self, x, ctx):
        """Routing with the second kernel: weights [tokens, experts] of the experts that have
        tensors, and per token the sum of the chosen identity outputs' weights and the shared
        expert's gate."""
        weights, others = self.ops.route_general(x, self.router, self.correction, **self.general)
        shared_scale = others[1] if self.shared_gate else None
        if self.sortable and self.ops.sorts_experts(x, experts=self.experts, width=self.width,
                                                    top=self.routing["top"],
                                                    stack=self.gate_up.shape[0] // 2):
            out = self.ops.routed_experts_sorted(
                x, weights, self.gate_up, self.down, experts=self.experts, width=self.width,
                top=self.routing["top"], shared_scale=shared_scale, **self.shared)
        else:
            if self.activation == "silu":
                gated = self.ops.linear_swiglu(x, self.gate_up)
            else:
                gated = self.ops.linear_gated(x, self.gate_up, self.activation)
            # (the shared expert's columns, behind the experts', times its gate in the same pass)
            self.ops.scale_expert_columns(gated, weights, self.width, tail=shared_scale)
            out = self.ops.linear(gated, self.down)
        if self.identity:
            self.ops.add_scaled_rows(out, x, others[0])
        return out

    def forward(self, x, ctx, residual=None):
        if self.general is not None:
            out = self._forward_general(x, ctx)
            return out          # (the caller adds it, with its factor, where it norms next)
        weights = self.ops.route_experts(x, self.router, **self.routing)
        if self.sortable and self.ops.sorts_experts(x, experts=self.experts, width=self.width,
                                                    top=self.routing["top"],
                                                    stack=self.gate_up.shape[0] // 2):
            return self.ops.routed_experts_sorted(
                x, weights, self.gate_up, self.down, experts=self.experts, width=self.width,
                top=self.routing["top"], **self.shared)
        if self.activation == "silu":
            gated = self.ops.linear_swiglu(x, self.gate_up)
        else:
            gated = self.ops.linear_gated(x, self.gate_up, self.activation)
        self.ops.scale_expert_columns(gated, weights, self.width)
        if residual is None:
            return self.ops.linear(gated, self.down)
        if self.residual_scale != 1.0:
            return self.ops.linear_add(gated, self.down, None, residual, scale=self.residual_scale)
        return self.ops.linear_add(gated, self.down, None, residual)
