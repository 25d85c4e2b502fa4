"""Latent attention: the keys and values of all heads are made from one low-rank vector per token.

``q = h Wq^T`` holds, per head, ``dk`` plain and ``dr`` rotated numbers.  ``h Wd^T`` holds ``rank`` numbers, which are
RMS-normed with a weight into the latent ``c``, and ``dr`` more, one rotated key part shared by all heads.  Per head the
plain key is ``Wuk_h c`` and the value ``Wuv_h c``; the score of a query at position ``a`` and a key at ``j <= a`` is
``(q_plain . Wuk_h c_j + q_rot . k_rot_j) scale``; softmax over all earlier tokens; the head's result times
``sigmoid(h Wg^T)_h``; the output projection.  Rotation: dimension ``i`` pairs with ``i + dims/2``,
``(u, v) -> (u cos a - v sin a, v cos a + u sin a)``, ``a = position * base^(-2i/dims)``.

Only ``c`` and the rotated key part are cached, as one per-token array of ``rank + dr`` numbers.  The up-projections are
absorbed: ``q_plain . Wuk_h c = (Wuk_h^T q_plain) . c``, so the kernel runs H query heads of size ``rank + dr`` over ONE
key head, whose first ``rank`` numbers are also the value; the per-head ``Wuv_h`` is applied to the attention's
``rank``-wide result afterwards.  Both absorbed products are a matrix per head (``head_matmul``).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..config.spec import PartSpec, TensorSpec
from ..kernels import ops
from ..registry import MIXERS
from .base import CacheArray, KVCacheSpec, LayerCache, Mixer, Runtime, StepContext, WeightView
from .linear import linear


def split_frequencies(base: float, dims: int, device):
    """``base^(-2i/dims)`` for ``i < dims/2``, made in float64 and kept as two fp32 words (value and remainder)."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims)
    hi = f.to(torch.float32)
    lo = (f - hi.to(torch.float64)).to(torch.float32)
    return hi.to(device), lo.to(device)


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    """spec params: hidden, heads, key_dim (plain), rot_dim (rotated), value_dim, rank, scale, eps, rotary ({"dims", "base"} or
    None), and the tensor names q, down, down_norm, up_k, up_v, o, g (the gate's projection, or None)."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> List[TensorSpec]:
        d, H, dk, dr, dv, r = spec["hidden"], spec["heads"], spec["key_dim"], spec["rot_dim"], spec["value_dim"], spec["rank"]
        out = [TensorSpec(prefix + spec["q"], (H * (dk + dr), d)), TensorSpec(prefix + spec["down"], (r + dr, d)),
               TensorSpec(prefix + spec["down_norm"], (r,), role="norm"), TensorSpec(prefix + spec["up_k"], (H * dk, r)),
               TensorSpec(prefix + spec["up_v"], (H * dv, r)), TensorSpec(prefix + spec["o"], (d, H * dv))]
        if spec.get("g"):
            out.append(TensorSpec(prefix + spec["g"], (H, d)))
        return out

    def __init__(self, spec: PartSpec, weights: WeightView, rt: Runtime):
        super().__init__(spec, weights, rt)
        self.hidden, self.heads = int(spec["hidden"]), int(spec["heads"])
        self.key_dim, self.rot_dim, self.value_dim, self.rank = int(spec["key_dim"]), int(spec["rot_dim"]), int(spec["value_dim"]), int(spec["rank"])
        self.scale, self.eps = float(spec["scale"]), float(spec["eps"])
        H, dk, dr, dv, r = self.heads, self.key_dim, self.rot_dim, self.value_dim, self.rank
        rot = spec.get("rotary")
        self.rot_dims, self.f_hi, self.f_lo, self.rot_key = 0, None, None, None
        if rot and int(rot["dims"]):
            self.rot_dims = int(rot["dims"])
            if self.rot_dims % 2 or self.rot_dims > dr:
                raise ValueError("latent attention: the rotated dimensions must be even and at most rot_dim")
            self.f_hi, self.f_lo = split_frequencies(float(rot["base"]), self.rot_dims, rt.device)
            self.rot_key = ("rope_half_exact", self.rot_dims, float(rot["base"]))
        self.has_gate = bool(spec.get("g"))
        ws = [weights.take(spec["q"]), weights.take(spec["down"])] + ([weights.take(spec["g"])] if self.has_gate else [])
        if len({w.dtype for w in ws}) > 1:
            ws = [w.float() for w in ws]
        self.w_in = torch.cat(ws, dim=0).contiguous()            # [H (dk + dr) + rank + dr (+ H), hidden]
        del ws
        self.q_cols, self.c_off = H * (dk + dr), H * (dk + dr)
        self.g_off = self.c_off + r + dr
        self.norm_weight = weights.take(spec["down_norm"]).contiguous()
        act = torch.float32 if rt.dtype == torch.float32 else None
        up_k, up_v = weights.take(spec["up_k"]), weights.take(spec["up_v"])
        # a matrix per head, [K, N] each: the key up-projection as it stands (dk -> rank), the value's transposed (rank -> dv)
        self.m_key = up_k.reshape(H, dk, r).to(act or up_k.dtype).contiguous()
        self.m_value = up_v.reshape(H, dv, r).transpose(1, 2).to(act or up_v.dtype).contiguous()
        self.w_o = weights.take(spec["o"]).contiguous()

    def kv_cache_spec(self) -> Optional[KVCacheSpec]:
        return KVCacheSpec(1, self.rank + self.rot_dim, 0, arrays=(CacheArray("latent", (1, self.rank + self.rot_dim)),))

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        n = x.shape[0]
        H, dk, dr, dv, r = self.heads, self.key_dim, self.rot_dim, self.value_dim, self.rank
        wide = r + dr
        a = linear(x, self.w_in, None, self.rt, out_dtype=torch.float32)
        rot = None
        if self.rot_dims:
            if self.rot_key not in ctx.derived:
                ctx.derived[self.rot_key] = ops.rope_half_table(ctx.positions, self.f_hi, self.f_lo)
            rot = ctx.derived[self.rot_key]
        pages = cache.arrays["latent"]
        slots = None
        if cache.writes:
            skey = ("slots", cache.block_table.data_ptr(), cache.page_size)
            if skey not in ctx.derived:
                ctx.derived[skey] = ops.slot_mapping(ctx.positions, ctx.token_req, cache.block_table, cache.page_size)
            slots = ctx.derived[skey]
        q_plain = torch.empty((n, H * dk), dtype=self.rt.dtype, device=a.device)
        q_full = torch.empty((n, H * wide), dtype=self.rt.dtype, device=a.device)
        ops.latent_prep(a, 0, self.c_off, self.norm_weight, self.eps, rot, self.rot_dims, q_plain, q_full, pages if cache.writes else None,
                        slots, cache.page_size, H, dk, dr, r)
        ops.head_matmul(q_plain, self.m_key, q_full, H)                      # each head's first `rank` places: Wuk_h^T q_plain
        att = torch.empty((n, H * r), dtype=self.rt.dtype, device=a.device)
        from ..kernels import attention as attn_kernels
        attn_kernels.paged_latent_attention(q_full, pages, cache, att, ctx, H, wide, r, 0, self.scale)
        o = torch.empty((n, H * dv), dtype=self.rt.dtype, device=a.device)
        ops.head_matmul(att, self.m_value, o, H)
        if self.has_gate:
            o = ops.head_finish(o, H, dv, gate=a[:, self.g_off:self.g_off + H])
        return linear(o, self.w_o, None, self.rt)
