"""Two mixers side by side on the same input.  ``combine``:

* ``normed_mean`` (the default): each output is RMS-normed over the model width with a plain weight of its own, and the
  mixer's result is ``scale`` times their sum (one half: the mean);
* ``sum``: the result is ``left_scale * left + right_scale * right``, no norms.  A block that adds scaled branches itself
  asks for them with :meth:`ParallelMixers.forward_branches` and the sum is never formed.

The two sides are built from their own part specs through the mixer registry, so any pair of registered mixers can stand
here; a side that keeps keys and values and a side that keeps a state share the layer's cache entry (the paged arrays go
to the one, the state slot to the other).  Two sides that keep a state share the slot: the left side's numbers stand first
(both states must be flat and of one dtype).  Two sides that keep a paged cache are refused.
"""
from __future__ import annotations

import dataclasses
from typing import List, Optional, Tuple

import torch

from ..config.spec import PartSpec, TensorSpec
from ..kernels import ops
from ..registry import MIXERS
from .base import KVCacheSpec, LayerCache, Mixer, Runtime, StateSpec, StepContext, WeightView


@MIXERS.register("parallel_mixers")
class ParallelMixers(Mixer):
    """spec params: hidden, left and right (PartSpecs of mixers), combine; for ``normed_mean``: eps, scale, left_out and
    right_out (names of the two norm weights); for ``sum``: left_scale, right_scale."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> List[TensorSpec]:
        out = []
        for side in ("left", "right"):
            out += MIXERS.get(spec[side].kind).tensor_specs(spec[side], prefix)
            if spec.get("combine", "normed_mean") == "normed_mean":
                out.append(TensorSpec(prefix + spec[side + "_out"], (spec["hidden"],), role="norm"))
        return out

    def __init__(self, spec: PartSpec, weights: WeightView, rt: Runtime):
        super().__init__(spec, weights, rt)
        self.hidden = int(spec["hidden"])
        self.combine = spec.get("combine", "normed_mean")
        if self.combine not in ("normed_mean", "sum"):
            raise ValueError("parallel mixers: combine is 'normed_mean' or 'sum'")
        self.left = MIXERS.get(spec["left"].kind)(spec["left"], weights, rt)
        self.right = MIXERS.get(spec["right"].kind)(spec["right"], weights, rt)
        if self.combine == "normed_mean":
            self.eps, self.scale = float(spec["eps"]), float(spec.get("scale", 0.5))
            self.w_left = weights.take(spec["left_out"]).float().contiguous()
            self.w_right = weights.take(spec["right_out"]).float().contiguous()
        else:
            self.left_scale, self.right_scale = float(spec.get("left_scale", 1.0)), float(spec.get("right_scale", 1.0))
        if self.left.kv_cache_spec() is not None and self.right.kv_cache_spec() is not None:
            raise ValueError("parallel mixers: both sides keep a paged cache; a layer has one")
        ls, rs = self.left.state_spec(), self.right.state_spec()
        self._split = None           # where the right side's numbers start when both sides keep a state
        if ls is not None and rs is not None:
            if len(ls.shape) != 1 or len(rs.shape) != 1 or ls.dtype != rs.dtype:
                raise ValueError("parallel mixers: two sides that keep a state need flat states of one dtype")
            self._split = int(ls.shape[0])

    def kv_cache_spec(self) -> Optional[KVCacheSpec]:
        return self.left.kv_cache_spec() or self.right.kv_cache_spec()

    def state_spec(self) -> Optional[StateSpec]:
        ls, rs = self.left.state_spec(), self.right.state_spec()
        if self._split is not None:
            return StateSpec((int(ls.shape[0]) + int(rs.shape[0]),), ls.dtype)
        return ls or rs

    def _sides(self, x: torch.Tensor, ctx: StepContext, cache: LayerCache) -> Tuple[torch.Tensor, torch.Tensor]:
        if self._split is None:
            return self.left.forward(x, ctx, cache), self.right.forward(x, ctx, cache)
        a = self.left.forward(x, ctx, dataclasses.replace(cache, state=cache.state[:, :self._split]))
        b = self.right.forward(x, ctx, dataclasses.replace(cache, state=cache.state[:, self._split:]))
        return a, b

    def forward_branches(self, x: torch.Tensor, ctx: StepContext, cache: LayerCache):
        """The mixer's result as a list of (tensor, factor) whose weighted sum it is, or None when it is not such a sum."""
        if self.combine != "sum":
            return None
        a, b = self._sides(x, ctx, cache)
        return [(a, self.left_scale), (b, self.right_scale)]

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        a, b = self._sides(x, ctx, cache)
        if self.combine == "sum":
            return ops.scaled_sum2(a, b, self.left_scale, self.right_scale)
        return ops.normed_mean2(a, b, self.w_left, self.w_right, self.eps, self.scale)
