"""Attention whose heads talk to one another before the softmax.

``q, k, v = h W^T`` with ``H`` query heads and ``G`` key/value heads (query head ``h`` reads key/value head ``h // (H/G)``),
keys of size ``key_dim`` and values of size ``value_dim``.  Options, each a parameter:

* ``conv``: taps of a short causal convolution over time on every channel of q, k and v directly behind the projection
  (``y_t = sum_j w[:, j] u_(t-K+1+j)``, zeros before the sequence); the last ``K-1`` projected rows of a request are
  its state;
* ``qk_norm``: every q and k head is RMS-normed over ``key_dim`` with one plain weight for all heads (``q_norm``, ``k_norm``);
* ``rotary``: ``{"dims", "base"}``: the first ``dims`` numbers of every q and k head turn by position, number ``i`` paired
  with ``i + dims/2``, angle ``p base^(-2i/dims)``;
* ``v_unit``: every value head is divided by its root mean square (no weight) and cached so;
* ``talk``: a matrix ``[H, H]``; the scaled scores of one (query, key) pair are mixed, ``s_h = sum_g talk[h, g] r_g``;
* ``sink``: one learned logit per head whose ``exp`` joins the softmax's denominator: it stands for no token, so nothing
  is added to the output for it, and the score scale does not touch it;
* ``window``: 0 (causal over everything) or the number of keys a query sees, itself included.

One product makes q, k and v as fp32 rows; convolution, norms and rotation read those (``csrc/linear_state.cu``,
``csrc/attention_talking.cu``); scores, mixing and softmax are fp32.  Keys and values are two per-token arrays of the paged
cache.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..config.spec import PartSpec, TensorSpec
from ..kernels import ops
from ..registry import MIXERS
from .base import CacheArray, KVCacheSpec, LayerCache, Mixer, Runtime, StateSpec, StepContext, WeightView
from .latent_attention import split_frequencies
from .linear import linear

CONV_BY_TOKEN_FROM = 32      # a step whose longest portion has at least this many tokens runs the convolution per (token, channel)


@MIXERS.register("talking_attention")
class TalkingAttention(Mixer):
    """spec params: hidden, heads, kv_heads, key_dim, value_dim, window (0: all), scale, eps, conv (taps; 0: none), qk_norm
    (bool), rotary ({"dims", "base"} or None), v_unit (bool), and the tensor names q, k, v, o, q_norm, k_norm, talk (or
    None), sink (or None); taps are the projection's name + ``conv_suffix``."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> List[TensorSpec]:
        d, H, G, dk, dv = spec["hidden"], spec["heads"], spec["kv_heads"], spec["key_dim"], spec["value_dim"]
        rows = {"q": H * dk, "k": G * dk, "v": G * dv}
        out = [TensorSpec(prefix + spec[n], (r, d)) for n, r in rows.items()] + [TensorSpec(prefix + spec["o"], (d, H * dv))]
        if spec.get("conv"):
            out += [TensorSpec(prefix + spec[n] + spec.get("conv_suffix", ".conv"), (r, int(spec["conv"])), role="taps") for n, r in rows.items()]
        if spec.get("qk_norm"):
            out += [TensorSpec(prefix + spec["q_norm"], (dk,), role="norm"), TensorSpec(prefix + spec["k_norm"], (dk,), role="norm")]
        if spec.get("talk"):
            out.append(TensorSpec(prefix + spec["talk"], (H, H), role="head_mix"))
        if spec.get("sink"):
            out.append(TensorSpec(prefix + spec["sink"], (H,), role="bias"))
        return out

    def __init__(self, spec: PartSpec, weights: WeightView, rt: Runtime):
        super().__init__(spec, weights, rt)
        self.hidden = int(spec["hidden"])
        self.heads, self.kv_heads = int(spec["heads"]), int(spec["kv_heads"])
        self.key_dim, self.value_dim = int(spec["key_dim"]), int(spec["value_dim"])
        if self.heads % self.kv_heads:
            raise ValueError("talking attention: heads must be a multiple of kv_heads")
        self.window = int(spec.get("window", 0) or 0)
        self.scale, self.eps = float(spec["scale"]), float(spec.get("eps", 0.0))
        self.taps = int(spec.get("conv", 0) or 0)
        if self.taps > 8:
            raise ValueError("talking attention: convolutions of more than 8 taps are not supported")
        H, G, dk, dv = self.heads, self.kv_heads, self.key_dim, self.value_dim
        self.channels = H * dk + G * dk + G * dv
        ws = [weights.take(spec[n]) for n in ("q", "k", "v")]
        if len({w.dtype for w in ws}) > 1:
            ws = [w.float() for w in ws]
        self.w_in = torch.cat(ws, dim=0).contiguous()                  # [channels, hidden]
        del ws
        self.conv_taps = None
        if self.taps:
            sfx = spec.get("conv_suffix", ".conv")
            self.conv_taps = torch.cat([weights.take(spec[n] + sfx).float() for n in ("q", "k", "v")], dim=0).contiguous()
        self.q_norm = self.k_norm = None
        if spec.get("qk_norm"):
            self.q_norm = weights.take(spec["q_norm"]).float().contiguous()
            self.k_norm = weights.take(spec["k_norm"]).float().contiguous()
        self.v_unit = bool(spec.get("v_unit", False))
        rot = spec.get("rotary")
        self.rot_dims, self.f_hi, self.f_lo, self.rot_key = 0, None, None, None
        if rot and int(rot["dims"]):
            self.rot_dims = int(rot["dims"])
            if self.rot_dims % 2 or self.rot_dims > dk:
                raise ValueError("talking attention: the rotated dimensions must be even and at most the key size")
            self.f_hi, self.f_lo = split_frequencies(float(rot["base"]), self.rot_dims, rt.device)
            self.rot_key = ("rope_half_exact", self.rot_dims, float(rot["base"]))
        self.talk = weights.take(spec["talk"]).float().contiguous() if spec.get("talk") else None
        self.sink = weights.take(spec["sink"]).float().contiguous() if spec.get("sink") else None
        self.w_o = weights.take(spec["o"]).contiguous()
        self.tail_size = (self.taps - 1) * self.channels if self.taps > 1 else 0
        self._no_tail = torch.zeros((1, 1), dtype=torch.float32, device=rt.device) if self.taps == 1 else None

    def kv_cache_spec(self) -> Optional[KVCacheSpec]:
        return KVCacheSpec(self.kv_heads, self.key_dim, self.window,
                           arrays=(CacheArray("k", (self.kv_heads, self.key_dim)), CacheArray("v", (self.kv_heads, self.value_dim))))

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((self.tail_size,), torch.float32) if self.tail_size else None

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        n = x.shape[0]
        H, G, dk, dv, C = self.heads, self.kv_heads, self.key_dim, self.value_dim, self.channels
        a = linear(x, self.w_in, None, self.rt, out_dtype=torch.float32)
        rows = a
        if self.taps:
            tail = cache.state if self.tail_size else self._no_tail
            if ctx.max_q_len >= CONV_BY_TOKEN_FROM:
                rows = ops.causal_conv_tokens(a, C, self.conv_taps, tail, ctx.token_req, ctx.req_meta, ctx.state_slots, ctx.positions,
                                              ctx.n_requests, silu=False)
            else:
                ops.causal_conv_walk(a, C, self.conv_taps, tail, ctx.req_meta, ctx.state_slots, ctx.positions, ctx.n_requests, silu=False)
        rot = None
        if self.rot_dims:
            if self.rot_key not in ctx.derived:
                ctx.derived[self.rot_key] = ops.rope_half_table(ctx.positions, self.f_hi, self.f_lo)
            rot = ctx.derived[self.rot_key]
        k_pages, v_pages = (cache.arrays["k"], cache.arrays["v"]) if cache.writes else (None, None)
        slots = None
        if k_pages is not None:
            skey = ("slots", cache.block_table.data_ptr(), cache.page_size)
            if skey not in ctx.derived:
                ctx.derived[skey] = ops.slot_mapping(ctx.positions, ctx.token_req, cache.block_table, cache.page_size)
            slots = ctx.derived[skey]
        q = torch.empty((n, H * dk), dtype=self.rt.dtype, device=a.device)
        ops.talking_prep(rows, 0, H * dk, (H + G) * dk, self.q_norm, self.k_norm, self.eps, rot, self.rot_dims, self.v_unit, q, k_pages, v_pages,
                         slots, cache.page_size, H, G, dk, dv)
        out = torch.empty((n, H * dv), dtype=self.rt.dtype, device=a.device)
        from ..kernels import attention as attn_kernels
        attn_kernels.paged_talking_attention(q, cache, out, ctx, H, G, dk, dv, self.window, self.scale, self.talk, self.sink)
        return linear(out, self.w_o, None, self.rt)
