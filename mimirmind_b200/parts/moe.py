"""Mixture of experts with a softmax (or sigmoid) router and a choice limited to the best runs of experts.

``s = softmax(h·W_routerᵀ)`` over all ``experts`` in fp32; the experts stand in ``groups`` equal runs of neighbours, a run is
scored by its best expert and only the ``keep`` best runs are eligible; the ``top`` eligible experts with the largest ``s``
are chosen and weighted by ``s / (sum of the chosen s + 1e-20)``.  Expert: ``W_down (silu(W_gate h) ⊙ W_up h)``, no biases.
The output is the weighted sum of the chosen experts' outputs.

Further options, each a parameter.  ``scoring`` ``sigmoid``: ``s = sigmoid(z)`` and the chosen experts are weighted by their
``s`` as it is.  ``weight_on`` ``input``: the weight multiplies the expert's input, the output is ``sum_e expert_e(w_e h)``
(both of an expert's first products are linear, so the weight is applied to their results in fp32).  ``activation``
``clamped`` with ``limit``: ``g = min(W_gate h, limit)``, ``u = clamp(W_up h, -limit, limit)``, ``y = g sigmoid(1.702 g) (u + 1)``.
``shared``: the PartSpec of a feed-forward that every token goes through beside its routed experts; the two results add up.

The experts' matrices are stacked at load (``[E, 2F, D]`` gate and up rows, ``[E, D, F]``).  A step routes on the
device, puts the rows of every expert side by side, and runs two grouped products over them: for prompt-sized steps in
bfloat16 the tcgen05 product over row tiles laid out on the device (``csrc/gemm_tcgen05.cu``, SwiGLU in its epilogue),
otherwise the ``mma.sync`` or fp32 kernels of ``csrc/moe.cu``.  Nothing waits for the host, so a decode step with this
feed-forward can be captured.
"""
from __future__ import annotations

from typing import List

import torch

from ..config.spec import PartSpec, TensorSpec
from ..kernels import ops
from ..registry import FEED_FORWARDS
from .base import FeedForward, Runtime, StepContext, WeightView
from .linear import linear


GROUPED_MIN_ROWS = 1024      # (token, choice) rows from which a step's expert products run on tensor memory


def ctx_plain(ctx) -> bool:
    return ctx is not None and getattr(ctx, "plain_only", False)


@FEED_FORWARDS.register("routed_experts")
class RoutedExperts(FeedForward):
    """spec params: hidden, ff, experts, top, groups, keep, router (tensor name), expert (a name pattern with ``{}`` for
    the expert's number, e.g. ``mlp.e{}``; its matrices are ``.gate``, ``.up``, ``.down``), scoring (``softmax`` or
    ``sigmoid``), weight_on (``output`` or ``input``), activation (``silu`` or ``clamped``), limit, shared (PartSpec or None)."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> List[TensorSpec]:
        d, f = spec["hidden"], spec["ff"]
        out = [TensorSpec(prefix + spec["router"], (spec["experts"], d), role="router")]
        for e in range(spec["experts"]):
            stem = prefix + spec["expert"].format(e)
            out += [TensorSpec(stem + ".gate", (f, d)), TensorSpec(stem + ".up", (f, d)), TensorSpec(stem + ".down", (d, f))]
        if spec.get("shared") is not None:
            out += FEED_FORWARDS.get(spec["shared"].kind).tensor_specs(spec["shared"], prefix)
        return out

    def __init__(self, spec: PartSpec, weights: WeightView, rt: Runtime):
        super().__init__(spec, weights, rt)
        self.hidden, self.ff = int(spec["hidden"]), int(spec["ff"])
        self.experts, self.top = int(spec["experts"]), int(spec["top"])
        self.groups, self.keep = int(spec.get("groups", 1)), int(spec.get("keep", 1))
        if self.experts % self.groups or not (0 < self.keep <= self.groups) or not (0 < self.top <= self.keep * (self.experts // self.groups)):
            raise ValueError("routed experts: the experts split into equal runs, 0 < keep <= runs, and top fits into the kept runs")
        self.scoring, self.weight_on = spec.get("scoring", "softmax"), spec.get("weight_on", "output")
        self.activation, self.limit = spec.get("activation", "silu"), float(spec.get("limit", 0.0) or 0.0)
        if self.scoring not in ops.ROUTER_SCORINGS or self.weight_on not in ("output", "input") or self.activation not in ops.GLU_ACTIVATIONS:
            raise ValueError("routed experts: scoring is 'softmax' or 'sigmoid', weight_on 'output' or 'input', activation 'silu' or 'clamped'")
        self.shared = FEED_FORWARDS.get(spec["shared"].kind)(spec["shared"], weights, rt) if spec.get("shared") is not None else None
        self.w_router = weights.take(spec["router"]).float().contiguous()        # the router runs in fp32
        stacked_in, stacked_out = [], []
        f, d = self.ff, self.hidden
        # bfloat16 with sizes the tensor-memory product takes: gate and up rows alternate in blocks of 8, so that a tile of
        # the product holds a gate value beside its up value and the activation is the product's epilogue
        self.interleaved = (rt.dtype == torch.bfloat16 and rt.matmul != "simt" and f % 8 == 0 and d % 8 == 0)
        for e in range(self.experts):
            stem = spec["expert"].format(e)
            gate, up = weights.take(stem + ".gate"), weights.take(stem + ".up")
            if self.interleaved:
                stacked_in.append(torch.stack([gate.view(f // 8, 8, d), up.view(f // 8, 8, d)], dim=1).reshape(2 * f, d))
            else:
                stacked_in.append(torch.cat([gate, up], dim=0))
            stacked_out.append(weights.take(stem + ".down"))
        self.w_in = torch.stack(stacked_in).to(rt.dtype).contiguous()       # [E, 2F, D]
        self.w_out = torch.stack(stacked_out).to(rt.dtype).contiguous()     # [E, D, F]
        del stacked_in, stacked_out

    def forward_branches(self, x: torch.Tensor, ctx: StepContext):
        """The feed-forward's result as a list of (tensor, factor) whose weighted sum it is: the routed experts and, if the
        layer has one, the shared expert."""
        out = [(self._routed(x, ctx), 1.0)]
        if self.shared is not None:
            out.append((self.shared.forward(x, ctx), 1.0))
        return out

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        y = self._routed(x, ctx)
        return y if self.shared is None else ops.scaled_sum2(y, self.shared.forward(x, ctx), 1.0, 1.0)

    def _routed(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        n = x.shape[0]
        idx, wts = ops.moe_router(x, self.w_router, self.top, self.groups, self.keep, scoring=self.scoring)
        n_rows = n * self.top
        on_input = self.weight_on == "input"
        if self.interleaved and n_rows >= GROUPED_MIN_ROWS and not ctx_plain(ctx):
            # prompt-sized: the rows are copied into sorted order once, and both products run on tensor memory over tiles of
            # 128 rows of one expert; the outputs stay in sorted order and the weighted sum fetches them by place
            rows = ops.moe_sort(idx, self.experts, with_tiles=True)
            if on_input:        # the weight rides on the copy: expert(w h) with w h rounded to the rows' dtype
                sorted_x = ops.moe_gather_scaled(x, rows, wts)
            else:
                sorted_x = torch.empty((n_rows, self.hidden), dtype=x.dtype, device=x.device)
                ops.gather_rows(x, rows.row_token, sorted_x)
            hidden = ops.moe_gemm_grouped(sorted_x, self.w_in, rows, swiglu=True, activation=self.activation, limit=self.limit)
            y = ops.moe_gemm_grouped(hidden, self.w_out, rows, swiglu=False)
            return ops.moe_combine(y, None if on_input else wts, self.rt.dtype, place=rows.place, top=self.top)
        rows = ops.moe_sort(idx, self.experts)
        tc = self.rt.matmul != "simt"
        hidden = ops.moe_gemm(x, self.w_in, rows, n_rows, self.top, True, self.rt.dtype, tensor_cores=tc, interleaved=self.interleaved,
                              activation=self.activation, limit=self.limit, row_scale=wts if on_input else None)
        y = ops.moe_gemm(hidden, self.w_out, rows, n_rows, self.top, False, torch.float32, tensor_cores=tc)
        return ops.moe_combine(y, None if on_input else wts, self.rt.dtype, top=self.top)


@FEED_FORWARDS.register("gated_mlp")
class GatedMLP(FeedForward):
    """A two-matrix gated feed-forward with its activation as a parameter: ``y = W_down act(W_gate h, W_up h)``, no biases.
    ``activation`` ``silu``: ``silu(g) u``; ``clamped`` with ``limit``: ``g = min(g, limit)``, ``u = clamp(u, -limit, limit)``,
    ``g sigmoid(1.702 g) (u + 1)``.  The gate's and the up projection's rows are one product with an fp32 result, the
    activation a pass of its own.

    spec params: hidden, intermediate, activation, limit, gate, up, down (tensor names under the prefix)."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> List[TensorSpec]:
        d, f = spec["hidden"], spec["intermediate"]
        return [TensorSpec(prefix + spec["gate"], (f, d)), TensorSpec(prefix + spec["up"], (f, d)), TensorSpec(prefix + spec["down"], (d, f))]

    def __init__(self, spec: PartSpec, weights: WeightView, rt: Runtime):
        super().__init__(spec, weights, rt)
        self.hidden, self.intermediate = int(spec["hidden"]), int(spec["intermediate"])
        self.activation, self.limit = spec.get("activation", "silu"), float(spec.get("limit", 0.0) or 0.0)
        if self.activation not in ops.GLU_ACTIVATIONS:
            raise ValueError("gated mlp: activation is 'silu' or 'clamped'")
        gate, up = weights.take(spec["gate"]), weights.take(spec["up"])
        if gate.dtype != up.dtype:
            gate, up = gate.float(), up.float()
        self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()          # [2F, D]
        del gate, up
        self.w_down = weights.take(spec["down"]).contiguous()               # [D, F]

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        gu = linear(x, self.w_gate_up, None, self.rt, out_dtype=torch.float32)
        return linear(ops.glu_rows(gu, self.rt.dtype, self.activation, self.limit), self.w_down, None, self.rt)
