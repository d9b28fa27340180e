"""Normalisation parts."""

from __future__ import annotations

from .base import Norm, NormedInput
from .registry import NORMS
from .spec import TensorSpec


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    """v * rsqrt(mean(v^2) + eps) * weight over the last axis, computed in 32-bit, fused
    with the residual add that precedes it. Parameters: ``size``, ``eps``, ``offset`` (0; a
    weight stored around zero has offset 1 and the norm multiplies by offset + weight).
    Reference: nn.RMSNorm at src/mlx_one/models/language/lfm2/reference_math.py:156-157."""

    supports_lazy = True

    @classmethod
    def tensors(cls, spec):
        return {"weight": TensorSpec((spec["size"],), "norm0" if spec.get("offset") else "norm")}

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.weight = self.vector(tensors["weight"])
        if spec.get("offset"):
            self.weight = (self.weight + float(spec["offset"])).contiguous()
        self.eps = float(spec["eps"])

    def forward(self, residual, delta, lazy=False, delta_scale=1.0):
        can_fuse = getattr(self.ops, "can_fuse_norm", None)
        if lazy and delta is None and can_fuse is not None and can_fuse(residual, self.runtime.dtype):
            return NormedInput(residual, self.weight, self.eps, self.runtime.dtype, self.ops)
        if delta is None or delta_scale == 1.0:
            return self.ops.add_rmsnorm(residual, delta, self.weight, self.eps, self.runtime.dtype)
        return self.ops.add_rmsnorm(residual, delta, self.weight, self.eps, self.runtime.dtype,
                                    delta_scale=delta_scale)

    def add_normed(self, residual, x):
        """In place: residual += x * rsqrt(mean(x^2) + eps) * weight, the norm taken over a part's
        output ``x`` (compute dtype) and everything in 32-bit."""
        self.ops.normed_mean_add(residual, [x], [self.weight], self.eps)
