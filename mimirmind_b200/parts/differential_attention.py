"""Differential attention: two softmax maps per head over the same values, the second subtracted from the first.

``q = h Wq^T + bq`` has ``H * 2 * dk`` numbers, ``k`` has ``G * 2 * dk`` (head by head: map 1, map 2), ``v`` has ``G * dv``;
query head ``h`` reads key/value head ``h // (H/G)``.  A short causal convolution over time runs on every channel of q, k
and v directly behind the projection (``y_t = sum_j w[:, j] u_(t-K+1+j)``, zeros before the sequence); the last ``K-1``
projected rows of a request are its state.  Per map ``m``: ``s = (q_m . k_m) scale``, then ``s <- cap tanh(s / cap)``
(``softcap`` 0: not capped), a sliding window of ``window`` keys (0: all), softmax, ``a_m = sum p v``.  Then
``o = a_1 - lambda a_2`` with ``lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff`` (one number for the layer),
``o <- o / sqrt(mean(o^2) + eps) (1 - diff)`` per head, times ``sigmoid(h Wg^T)_h`` (one gate per head), and the output
projection.  No position enters the scores.

How it runs: the weights' rows are reordered at load so that all first maps stand before all second maps; q then has
``2H`` heads of ``dk`` and k ``2G``, query head ``j`` reads key head ``j // (H/G)`` as in any grouped attention, and the
value head is the key head modulo ``G``.  The windowed attention kernels of :mod:`..kernels.attention` run the ``2H``
maps with that head mapping and the soft cap; ``head_finish`` (``csrc/attention_parts.cu``) takes the difference, the
norm, the factor and the gate.  One product makes q, k, v and the gates (fp32 result); the convolution is the one of the
matrix-state mixers (``csrc/linear_state.cu``), without its activation.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..config.spec import PartSpec, TensorSpec
from ..kernels import ops
from ..registry import MIXERS
from .base import CacheArray, KVCacheSpec, LayerCache, Mixer, Runtime, StateSpec, StepContext, WeightView
from .linear import linear

CONV_BY_TOKEN_FROM = 32      # a step whose longest portion has at least this many tokens runs the convolution per (token, channel)


def maps_first(t: torch.Tensor, heads: int, dim: int) -> torch.Tensor:
    """Rows ``[heads, 2, dim, ...]`` (head by head: map 1, map 2) reordered to ``[2, heads, dim, ...]``."""
    rest = t.shape[1:]
    return t.reshape(heads, 2, dim, *rest).transpose(0, 1).reshape(2 * heads * dim, *rest).contiguous()


@MIXERS.register("differential_attention")
class DifferentialAttention(Mixer):
    """spec params: hidden, heads, kv_heads, key_dim, value_dim, window (0: all), scale, softcap (0: none), diff, eps,
    conv (taps; 0: no convolution), bias (bool: q, k and v), and the tensor names q, k, v, o, g (the gate's projection, or
    None), lq1, lk1, lq2, lk2; biases are the name + ``bias_suffix``, taps the name + ``conv_suffix``."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> List[TensorSpec]:
        d, H, G, dk, dv = spec["hidden"], spec["heads"], spec["kv_heads"], spec["key_dim"], spec["value_dim"]
        rows = {"q": H * 2 * dk, "k": G * 2 * dk, "v": G * dv}
        out = [TensorSpec(prefix + spec[n], (r, d)) for n, r in rows.items()] + [TensorSpec(prefix + spec["o"], (d, H * dv))]
        if spec.get("bias", False):
            out += [TensorSpec(prefix + spec[n] + spec.get("bias_suffix", ".b"), (r,), role="bias") for n, r in rows.items()]
        if spec.get("conv"):
            out += [TensorSpec(prefix + spec[n] + spec.get("conv_suffix", ".conv"), (r, int(spec["conv"])), role="taps") for n, r in rows.items()]
        if spec.get("g"):
            out.append(TensorSpec(prefix + spec["g"], (H, d)))
        out += [TensorSpec(prefix + spec[n], (dk,), role="bias") for n in ("lq1", "lk1", "lq2", "lk2")]
        return out

    def __init__(self, spec: PartSpec, weights: WeightView, rt: Runtime):
        super().__init__(spec, weights, rt)
        self.hidden = int(spec["hidden"])
        self.heads, self.kv_heads = int(spec["heads"]), int(spec["kv_heads"])
        self.key_dim, self.value_dim = int(spec["key_dim"]), int(spec["value_dim"])
        if self.heads % self.kv_heads:
            raise ValueError("differential attention: heads must be a multiple of kv_heads")
        self.window = int(spec.get("window", 0) or 0)
        self.scale, self.softcap = float(spec["scale"]), float(spec.get("softcap", 0.0) or 0.0)
        self.diff, self.eps = float(spec["diff"]), float(spec["eps"])
        self.taps = int(spec.get("conv", 0) or 0)
        H, G, dk, dv = self.heads, self.kv_heads, self.key_dim, self.value_dim
        self.channels = 2 * H * dk + 2 * G * dk + G * dv

        def ordered(suffix: str):
            return [maps_first(weights.take(spec["q"] + suffix), H, dk), maps_first(weights.take(spec["k"] + suffix), G, dk),
                    weights.take(spec["v"] + suffix)]

        ws = ordered("")
        self.has_gate = bool(spec.get("g"))
        if self.has_gate:
            ws.append(weights.take(spec["g"]))
        if len({w.dtype for w in ws}) > 1:
            ws = [w.float() for w in ws]
        self.w_in = torch.cat(ws, dim=0).contiguous()                  # [channels (+ H), hidden]
        del ws
        self.b_in = None
        if spec.get("bias", False):
            bs = [b.float() for b in ordered(spec.get("bias_suffix", ".b"))]
            if self.has_gate:
                bs.append(torch.zeros(H, dtype=torch.float32, device=bs[0].device))
            self.b_in = torch.cat(bs, dim=0).contiguous()
        self.conv_taps = None
        if self.taps:
            self.conv_taps = torch.cat([t.float() for t in ordered(spec.get("conv_suffix", ".conv"))], dim=0).contiguous()
        lam = [weights.take(spec[n]).float() for n in ("lq1", "lk1", "lq2", "lk2")]
        # one number for the layer, made once at load in fp32 and handed to the kernel by value
        self.lam = float((torch.exp(torch.sum(lam[0] * lam[1])) - torch.exp(torch.sum(lam[2] * lam[3])) + self.diff).item())
        self.w_o = weights.take(spec["o"]).contiguous()
        self.tail_size = (self.taps - 1) * self.channels if self.taps > 1 else 0
        self._no_tail = torch.zeros((1, 1), dtype=torch.float32, device=rt.device) if self.taps == 1 else None

    def kv_cache_spec(self) -> Optional[KVCacheSpec]:
        return KVCacheSpec(2 * self.kv_heads, self.key_dim, self.window,
                           arrays=(CacheArray("k", (2 * self.kv_heads, self.key_dim)), CacheArray("v", (self.kv_heads, self.value_dim))))

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((self.tail_size,), torch.float32) if self.tail_size else None

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        n = x.shape[0]
        H, G, dk, dv, C = self.heads, self.kv_heads, self.key_dim, self.value_dim, self.channels
        a = linear(x, self.w_in, self.b_in, self.rt, out_dtype=torch.float32)
        rows = a
        if self.taps:
            tail = cache.state if self.tail_size else self._no_tail
            if ctx.max_q_len >= CONV_BY_TOKEN_FROM:
                rows = ops.causal_conv_tokens(a, C, self.conv_taps, tail, ctx.token_req, ctx.req_meta, ctx.state_slots, ctx.positions,
                                              ctx.n_requests, silu=False)
            else:
                ops.causal_conv_walk(a, C, self.conv_taps, tail, ctx.req_meta, ctx.state_slots, ctx.positions, ctx.n_requests, silu=False)
        k_pages, v_pages = (cache.arrays["k"], cache.arrays["v"]) if cache.writes else (None, None)
        slots = None
        if k_pages is not None:
            skey = ("slots", cache.block_table.data_ptr(), cache.page_size)
            if skey not in ctx.derived:
                ctx.derived[skey] = ops.slot_mapping(ctx.positions, ctx.token_req, cache.block_table, cache.page_size)
            slots = ctx.derived[skey]
        q = torch.empty((n, 2 * H * dk), dtype=self.rt.dtype, device=a.device)
        ops.qkv_split_post(rows, 0, 2 * H * dk, 2 * (H + G) * dk, q, k_pages, v_pages, slots, cache.page_size, 2 * H, 2 * G, dk, G, dv)
        # both maps' results stay fp32: their difference is normed to unit size, which would magnify a rounding of the maps
        att = torch.empty((n, 2 * H * dv), dtype=torch.float32, device=a.device)
        from ..kernels import attention as attn_kernels
        attn_kernels.paged_sink_attention(q, cache, att, ctx, 2 * H, 2 * G, dk, dv, self.window, self.scale, False,
                                          softcap=self.softcap, value_heads=G)
        o = ops.head_finish(att, H, dv, pair=True, lam=self.lam, eps=self.eps, post=1.0 - self.diff,
                            gate=a[:, C:C + H] if self.has_gate else None, out_dtype=self.rt.dtype)
        return linear(o, self.w_o, None, self.rt)
