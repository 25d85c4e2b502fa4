"""Token embedding and output head.

Embedding: ``x[t,:] = E[id_t,:]`` with an optional scale (none for this architecture,
src/runtime/arch/Qwen2Backend.hpp:50); an id outside the table gives a zero row
(src/compute/Embedding.cpp:46-67).  Head: ``logits = n·Wᵀ`` with W the ``lm_head`` tensor
if the checkpoint has one, else the embedding table (src/runtime/InferenceEngine.cpp:1374-1377),
computed only for the rows whose logits are wanted and returned as fp32.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..config.spec import PartSpec, TensorSpec
from ..kernels import ops
from ..registry import EMBEDDINGS, HEADS
from .base import Embedding, NativeDesc, Part, Runtime, StateSpec, StepContext, WeightView
from .linear import linear


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Embedding):
    """spec params: vocab, width, scale, weight (full tensor name), copies (default 1: how many residual streams the
    model keeps per token; each starts as a copy of the row, side by side in ``[n, copies * width]``)."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> List[TensorSpec]:
        return [TensorSpec(spec["weight"], (spec["vocab"], spec["width"]), role="table")]

    def __init__(self, spec: PartSpec, weights: WeightView, rt: Runtime):
        super().__init__(spec, weights, rt)
        self.vocab = int(spec["vocab"])
        self.width = int(spec["width"])
        self.scale = float(spec.get("scale", 1.0))
        self.copies = int(spec.get("copies", 1) or 1)
        self.table = weights.get(spec["weight"]).contiguous()

    def native(self):
        if type(self) is not TokenEmbedding or self.copies != 1:
            return None
        return NativeDesc("token_embedding", {"vocab": self.vocab, "width": self.width, "scale": self.scale}, {"table": self.table})

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        out = torch.empty((token_ids.numel(), self.width), dtype=torch.float32, device=token_ids.device)
        ops.embedding(token_ids, self.table, out, self.scale)
        return ops.stream_copies(out, self.copies) if self.copies > 1 else out


@EMBEDDINGS.register("bigram_embedding")
class BigramEmbedding(Embedding):
    """Token row plus a hashed row for the pair (previous token, token):
    ``x = E[id] + B[(prev * mul_prev + id * mul_cur) mod buckets]``, and the table's extra row ``buckets`` for a
    sequence's first token.  The previous token of a portion's first token is per-request state (one int32).

    spec params: vocab, width, buckets, mul_prev, mul_cur, weight, pairs (full tensor names)."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> List[TensorSpec]:
        return [TensorSpec(spec["weight"], (spec["vocab"], spec["width"]), role="table"),
                TensorSpec(spec["pairs"], (spec["buckets"] + 1, spec["width"]), role="table")]

    def __init__(self, spec: PartSpec, weights: WeightView, rt: Runtime):
        super().__init__(spec, weights, rt)
        self.vocab, self.width = int(spec["vocab"]), int(spec["width"])
        self.buckets, self.mul_prev, self.mul_cur = int(spec["buckets"]), int(spec["mul_prev"]), int(spec["mul_cur"])
        if self.buckets < 1:
            raise ValueError("bigram embedding: buckets must be positive")
        self.table = weights.get(spec["weight"]).contiguous()
        self.pairs = weights.get(spec["pairs"]).contiguous()
        if self.pairs.dtype != self.table.dtype:
            self.table, self.pairs = self.table.float(), self.pairs.float()

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((1,), torch.int32)

    def embed(self, ctx: StepContext, state: Optional[torch.Tensor]) -> torch.Tensor:
        if state is None:
            raise RuntimeError("the bigram embedding needs its per-request state")
        out = torch.empty((ctx.n_tokens, self.width), dtype=torch.float32, device=ctx.token_ids.device)
        return ops.embedding_bigram(ctx.token_ids, ctx.positions, ctx.token_req, ctx.req_meta, ctx.state_slots, state, self.table,
                                    self.pairs, out, self.buckets, self.mul_prev, self.mul_cur)


@HEADS.register("lm_head")
class LMHead(Part):
    """spec params: vocab, width, weight (full tensor name), tied_to (embedding tensor name or None)."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> List[TensorSpec]:
        tied = spec.get("tied_to") is not None
        return [TensorSpec(spec["weight"], (spec["vocab"], spec["width"]), optional=tied)]

    def __init__(self, spec: PartSpec, weights: WeightView, rt: Runtime):
        super().__init__(spec, weights, rt)
        self.vocab = int(spec["vocab"])
        if weights.has(spec["weight"]):
            self.weight = weights.get(spec["weight"]).contiguous()
        elif spec.get("tied_to") is not None:
            self.weight = weights.get(spec["tied_to"]).contiguous()
        else:
            raise KeyError(f"tensor '{spec['weight']}' not in model")

    def native(self):
        return NativeDesc("lm_head", {"vocab": self.vocab}, {"weight": self.weight}) if type(self) is LMHead else None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return linear(x, self.weight, None, self.rt, out_dtype=torch.float32)
