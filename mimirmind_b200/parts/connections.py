"""Residual connections: how a sublayer reads its input from the residual stream and how its result goes back.

``hyper_connection`` keeps ``S`` copies ("streams") of the residual per token, fp32 ``[n, S * D]``.  A sublayer reads
``u = sum_s read[s] x_s`` (which the layer's norm then norms) and its result ``y`` goes back into every stream at once,
``x_t <- sum_s mix[s, t] x_s + write[t] (scale . y)``, each new stream made from the old ones (``mix`` is indexed
[from, to]); ``scale`` is an optional per-channel factor on the sublayer's result ("layer scale").  ``streams`` 0 is the
ordinary residual sum ``x <- x + scale . y`` over one stream and names no stream tensors.

The write of one sublayer and the read and norm of the next are one launch (``csrc/hyper_connections.cu``), so the
streams are read and written once per sublayer.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..config.spec import PartSpec, TensorSpec
from ..kernels import ops
from ..registry import CONNECTIONS
from .base import Norm, Part, Runtime, WeightView


@CONNECTIONS.register("hyper_connection")
class HyperConnection(Part):
    """spec params: width, streams (0: one stream, plain sum), read, mix, write (tensor names; not needed with streams 0),
    scale (tensor name of the per-channel factor, or None)."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> List[TensorSpec]:
        s, out = int(spec.get("streams", 0) or 0), []
        if s:
            out += [TensorSpec(prefix + spec["read"], (s,), role="stream_read"), TensorSpec(prefix + spec["write"], (s,), role="norm"),
                    TensorSpec(prefix + spec["mix"], (s, s), role="stream_mix")]
        if spec.get("scale"):
            out.append(TensorSpec(prefix + spec["scale"], (int(spec["width"]),), role="norm"))
        return out

    def __init__(self, spec: PartSpec, weights: WeightView, rt: Runtime):
        super().__init__(spec, weights, rt)
        self.width = int(spec["width"])
        declared = int(spec.get("streams", 0) or 0)
        self.streams = max(1, declared)
        if declared:
            self.w_read = weights.take(spec["read"]).float().contiguous()
            self.w_write = weights.take(spec["write"]).float().contiguous()
            self.w_mix = weights.take(spec["mix"]).float().contiguous()
        else:
            self.w_read = torch.ones(1, dtype=torch.float32, device=rt.device)
            self.w_write = torch.ones(1, dtype=torch.float32, device=rt.device)
            self.w_mix = torch.ones((1, 1), dtype=torch.float32, device=rt.device)
        self.scale = weights.take(spec["scale"]).float().contiguous() if spec.get("scale") else None

    @staticmethod
    def _factors(norm: Norm):
        f = norm.factors()
        if f is None:
            raise ValueError("a stream connection needs a norm of the form x * w / rms(x) behind it")
        return f

    def read(self, residual: torch.Tensor, norm: Norm) -> torch.Tensor:
        """The sublayer's normed input from the streams."""
        w, eps = self._factors(norm)
        return ops.hc_read(residual, self.streams, self.w_read, w, eps, self.rt.dtype)

    def write(self, residual: torch.Tensor, y: torch.Tensor, then: Optional["HyperConnection"] = None,
              then_norm: Optional[Norm] = None) -> Optional[torch.Tensor]:
        """The sublayer's result into the streams (in place); with ``then`` also the next sublayer's normed input."""
        if then is None:
            return ops.hc_write(residual, self.streams, y, self.scale, self.w_mix, self.w_write)
        if then.streams != self.streams:
            raise ValueError("consecutive stream connections differ in their number of streams")
        w, eps = self._factors(then_norm)
        return ops.hc_write(residual, self.streams, y, self.scale, self.w_mix, self.w_write, then.w_read, w, eps, self.rt.dtype)

    def total(self, residual: torch.Tensor) -> torch.Tensor:
        """The sum of the streams, fp32 [n, D] (diagnostics)."""
        ones = torch.ones(self.streams, dtype=torch.float32, device=residual.device)
        return ops.hc_read(residual, self.streams, ones, None, 0.0, torch.float32)


@CONNECTIONS.register("unused_sublayer")
class UnusedSublayer(Part):
    """The tensors of a sublayer that a layer does not have (a layer without a feed-forward whose checkpoint still carries
    the norm, scale and stream weights of one): declared so that the checkpoint passes the check at load, allowed to be
    absent, never read.  spec params: tensors, a list of (name, shape)."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> List[TensorSpec]:
        return [TensorSpec(prefix + name, tuple(int(x) for x in shape), role="norm", optional=True) for name, shape in spec["tensors"]]
