"""RMSNorm with its eps as a parameter.

``y = x · w / sqrt(mean(x²) + eps)``: eps inside the root, added after the mean; the
weight multiplies directly (src/compute/Norm.cpp:21-37).  The residual add that precedes
a norm is fused into it, as the reference's add+norm kernel does
(kernels/cuda/common/add_rmsnorm.cu:32-81).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..config.spec import PartSpec, TensorSpec
from ..kernels import ops
from ..registry import NORMS
from .base import NativeDesc, Norm, Runtime, WeightView


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    """spec params: width, eps, weight (tensor name under the prefix), offset (default 0: the stored weight multiplies
    directly; 1: the weight is stored around zero and ``1 + w`` multiplies, formed once at load in fp32), streams (default
    1; S: the residual holds S streams per token, ``[n, S * width]``, and the norm is taken of their sum)."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> List[TensorSpec]:
        return [TensorSpec(prefix + spec["weight"], (spec["width"],), role="norm0" if float(spec.get("offset", 0.0)) else "norm")]

    def __init__(self, spec: PartSpec, weights: WeightView, rt: Runtime):
        super().__init__(spec, weights, rt)
        self.width = int(spec["width"])
        self.eps = float(spec["eps"])
        self.offset = float(spec.get("offset", 0.0))
        self.streams = int(spec.get("streams", 1) or 1)
        self.weight = weights.get(spec["weight"]).contiguous()
        if self.offset:
            self.weight = (self.weight.float() + self.offset).contiguous()
        self._ones = torch.ones(self.streams, dtype=torch.float32, device=rt.device) if self.streams > 1 else None

    def factors(self):
        return (self.weight, self.eps) if self.streams == 1 else None

    def native(self):
        if type(self) is not RMSNorm or self.offset or self.streams != 1:
            return None
        return NativeDesc("rmsnorm", {"width": self.width, "eps": self.eps}, {"weight": self.weight})

    def forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor], rows: Optional[torch.Tensor] = None,
                n_rows: Optional[int] = None) -> torch.Tensor:
        n = residual.shape[0] if rows is None else (n_rows if n_rows is not None else rows.numel())
        if rows is not None and rows.numel() != n:
            rows = rows[:n]
        if self.streams > 1:
            if delta is not None:
                raise ValueError("rmsnorm over several streams: nothing can be pending, the streams are complete")
            return ops.hc_read(residual, self.streams, self._ones, self.weight, self.eps, self.rt.dtype, rows, n if rows is not None else None)
        out = torch.empty((n, self.width), dtype=self.rt.dtype, device=residual.device)
        return ops.add_rmsnorm(residual, delta, self.weight, self.eps, out, rows)


@NORMS.register("group_rmsnorm")
class GroupRMSNorm(Norm):
    """RMS norm in groups: a row is cut into ``groups`` equal consecutive parts, each divided by its own
    ``sqrt(mean(part^2) + eps)``, and the whole multiplied by the weight.  One group is the plain RMS norm.

    spec params: width, eps, groups, weight (tensor name under the prefix)."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> List[TensorSpec]:
        return [TensorSpec(prefix + spec["weight"], (spec["width"],), role="norm")]

    def __init__(self, spec: PartSpec, weights: WeightView, rt: Runtime):
        super().__init__(spec, weights, rt)
        self.width, self.eps, self.groups = int(spec["width"]), float(spec["eps"]), int(spec.get("groups", 1))
        if self.groups < 1 or self.width % self.groups:
            raise ValueError(f"group norm: {self.groups} groups do not divide the width {self.width}")
        self.weight = weights.get(spec["weight"]).contiguous()

    def factors(self):
        return (self.weight, self.eps) if self.groups == 1 else None

    def same_shape(self, other) -> bool:
        """True if ``other`` is a grouped norm that one launch can chain with this one."""
        return (isinstance(other, GroupRMSNorm) and other.width == self.width and other.groups == self.groups
                and other.eps == self.eps and other.weight.dtype == self.weight.dtype)

    def forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor], rows: Optional[torch.Tensor] = None,
                n_rows: Optional[int] = None) -> torch.Tensor:
        n = residual.shape[0] if rows is None else (n_rows if n_rows is not None else rows.numel())
        out = torch.empty((n, self.width), dtype=self.rt.dtype, device=residual.device)
        if rows is not None:
            if delta is not None:
                ops.add_residual(residual, delta)
            return ops.group_norm_chain(residual, None, None, self.weight, self.groups, self.eps, out, rows[:n] if rows.numel() != n else rows)
        return ops.group_norm_chain(residual, delta, None, self.weight, self.groups, self.eps, out)

    def add_normed(self, residual: torch.Tensor, branch: torch.Tensor, then: Optional["GroupRMSNorm"] = None) -> Optional[torch.Tensor]:
        """``residual += norm(branch)`` with this norm; with ``then`` (a norm of the same shape) also returns
        ``then(residual)`` from the same launch."""
        if then is None:
            ops.group_norm_chain(residual, branch, self.weight, None, self.groups, self.eps)
            return None
        if not self.same_shape(then):
            ops.group_norm_chain(residual, branch, self.weight, None, self.groups, self.eps)
            return then.forward(residual, None)
        out = torch.empty((residual.shape[0], self.width), dtype=self.rt.dtype, device=residual.device)
        return ops.group_norm_chain(residual, branch, self.weight, then.weight, self.groups, self.eps, out)


@NORMS.register("none")
class NoNorm(Norm):
    """Stands where a layer has no such norm (a layer without a feed-forward); never run."""
