"""Mixers that keep a matrix per head instead of keys and values (linear attention and its gated, delta-rule kin).

Per head, with ``S`` a ``[key_dim, value_dim]`` matrix in fp32 that starts at zero and is carried per request in the
engine's state slots::

    S <- g_t S;    u_t = v_t   or, with the delta rule,   u_t = beta_t (v_t - S^T k_t);    S <- S + k_t u_t^T;    o_t = S^T q_t

One class covers the family; what differs between its members is a parameter:

* ``decay``: a list with one constant per head (retention, lightning attention), or the name stem of a learned decay per
  token, ``g = exp(-exp(A_log) softplus(W_a h + dt_bias))`` (gated delta rule), or ``"forget_gate"`` (HGRN2): the decay is a
  vector over the key channels whose complement is the write strength, ``f = l + (1 - l) sigmoid(W_k h + f_bias)`` with a lower
  bound ``l`` per channel (``lower``), ``S <- diag(f) S + (1 - f) v^T``: the ``k`` projection is the gate's, there is no key
  of its own, q and k have as many heads as v, and of the activation only q's part applies;
* ``g``: the name of the output gate's projection, or None for no gate;
* ``delta``: the name of the projection of the write strength ``beta = sigmoid(W_b h)``, or None for the plain update;
* ``conv``: taps of a short causal convolution per channel on q, k and v before the activation (its last inputs are
  state too), or 0;
* ``activation``: ``silu`` on q, k and v, or None;
* ``rotary``: ``{"dims", "base"}`` for a rotation of half-split pairs of q and k by position, or None;
* ``unit_eps``: q and k heads are brought to unit length ``x / sqrt(sum x^2 + unit_eps)``, or None;
* ``q_scale``, ``k_scale``: constants;
* ``out_norm``: ``"head"`` (every head's output divided by its root mean square) or ``"all"`` (the joined heads as one
  vector), ``out_weight``: the name of a weight of ``value_dim`` (``head``, shared by the heads) or of
  ``heads * value_dim`` (``all``) numbers, or None; ``gate_activation``: ``silu`` or ``sigmoid`` on ``W_g h``.

All input projections are one product with an fp32 result; everything between it and the output projection is fp32
(``csrc/linear_state.cu``, ``csrc/norm_gated.cu``).  A request's tokens are walked in order from its slot's state; long
portions without the delta rule (whose update is a scaling and an addition) are cut into chunks that are walked side by
side, except in float32 runs, which keep one order of operations whatever the cutting.  q and k have ``qk_heads`` heads; head h reads q/k head ``h // (heads / qk_heads)``.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..config.spec import PartSpec, TensorSpec
from ..kernels import ops
from ..registry import MIXERS
from .base import LayerCache, Mixer, Runtime, StateSpec, StepContext, WeightView
from .chunks import token_chunks
from .linear import linear


CHUNK = 64                   # tokens per chunk of the three-pass walk
CHUNKED_FROM = 256           # a step whose longest portion has at least this many tokens walks its chunks side by side (not in float32)
CONV_BY_TOKEN_FROM = 32      # a step whose longest portion has at least this many tokens runs the convolution per (token, channel)


@MIXERS.register("linear_state")
class LinearStateMixer(Mixer):
    """spec params: hidden, heads, qk_heads, key_dim, value_dim, eps, the options of the module's text, and the tensor
    names q, k, v, g, o (weights; a convolution's taps are the projection's name + ``conv_suffix``), and for a learned
    decay ``a`` (projection), ``A_log``, ``dt_bias``."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> List[TensorSpec]:
        d, H, G, dk, dv = spec["hidden"], spec["heads"], spec["qk_heads"], spec["key_dim"], spec["value_dim"]
        out = [TensorSpec(prefix + spec["q"], (G * dk, d)), TensorSpec(prefix + spec["k"], (G * dk, d)),
               TensorSpec(prefix + spec["v"], (H * dv, d)), TensorSpec(prefix + spec["o"], (d, H * dv))]
        if spec.get("g"):
            out.append(TensorSpec(prefix + spec["g"], (H * dv, d)))
        if spec["decay"] == "forget_gate":
            out += [TensorSpec(prefix + spec["f_bias"], (G * dk,), role="bias"), TensorSpec(prefix + spec["lower"], (G * dk,), role="lower_bound")]
        taps = int(spec.get("conv", 0) or 0)
        if taps:
            sfx = spec.get("conv_suffix", ".conv")
            out += [TensorSpec(prefix + spec["q"] + sfx, (G * dk, taps), role="taps"), TensorSpec(prefix + spec["k"] + sfx, (G * dk, taps), role="taps"),
                    TensorSpec(prefix + spec["v"] + sfx, (H * dv, taps), role="taps")]
        if spec.get("delta"):
            out.append(TensorSpec(prefix + spec["delta"], (H, d)))
        if not isinstance(spec["decay"], (list, tuple)) and spec["decay"] != "forget_gate":
            out += [TensorSpec(prefix + spec["a"], (H, d)), TensorSpec(prefix + spec["A_log"], (H,), role="bias"),
                    TensorSpec(prefix + spec["dt_bias"], (H,), role="bias")]
        if spec.get("out_weight"):
            out.append(TensorSpec(prefix + spec["out_weight"], (dv if spec.get("out_norm", "head") == "head" else H * dv,), role="norm"))
        return out

    def __init__(self, spec: PartSpec, weights: WeightView, rt: Runtime):
        super().__init__(spec, weights, rt)
        self.hidden, self.heads, self.qk_heads = int(spec["hidden"]), int(spec["heads"]), int(spec["qk_heads"])
        self.dk, self.dv, self.eps = int(spec["key_dim"]), int(spec["value_dim"]), float(spec["eps"])
        H, G, dk, dv = self.heads, self.qk_heads, self.dk, self.dv
        if H % G:
            raise ValueError("linear state: heads must be a multiple of the q/k heads")
        if dk > 256:
            raise ValueError("linear state: key sizes above 256 are not supported")
        self.taps = int(spec.get("conv", 0) or 0)
        if self.taps > 8:
            raise ValueError("linear state: convolutions of more than 8 taps are not supported")
        self.activation = spec.get("activation")
        if self.activation not in (None, "silu"):
            raise ValueError("linear state: the activation is 'silu' or None")
        self.forget_gate = spec["decay"] == "forget_gate"
        self.learned_decay = not isinstance(spec["decay"], (list, tuple)) and not self.forget_gate
        self.delta = bool(spec.get("delta"))
        self.has_gate = bool(spec.get("g"))
        if self.forget_gate and (G != H or self.delta or spec.get("conv") or spec.get("rotary") or spec.get("unit_eps") is not None):
            raise ValueError("linear state: a forget gate per channel goes with as many q/k heads as heads, and without the delta rule, "
                             "convolution, rotation or unit length")
        names = ["q", "k", "v"] + (["delta"] if self.delta else []) + (["a"] if self.learned_decay else []) + (["g"] if self.has_gate else [])
        ws = [weights.take(spec[n]) for n in names]
        if len({w.dtype for w in ws}) > 1:
            ws = [w.float() for w in ws]
        self.w_in = torch.cat(ws, dim=0).contiguous()
        del ws
        self.q_off, self.k_off, self.v_off = 0, G * dk, 2 * G * dk
        off = 2 * G * dk + H * dv
        self.b_off = self.a_off = -1
        if self.delta:
            self.b_off, off = off, off + H
        if self.learned_decay:
            self.a_off, off = off, off + H
        self.g_off = off
        self.channels = 2 * G * dk + H * dv
        self.conv_taps = None
        if self.taps:
            sfx = spec.get("conv_suffix", ".conv")
            self.conv_taps = torch.cat([weights.take(spec[n] + sfx).float() for n in ("q", "k", "v")], dim=0).contiguous()
        self.head_decay = self.A_log = self.dt_bias = self.f_bias = self.lower = None
        if self.forget_gate:
            self.f_bias = weights.take(spec["f_bias"]).float().contiguous()
            self.lower = weights.take(spec["lower"]).float().contiguous()
        elif self.learned_decay:
            self.A_log = weights.take(spec["A_log"]).float().contiguous()
            self.dt_bias = weights.take(spec["dt_bias"]).float().contiguous()
        else:
            if len(spec["decay"]) != H:
                raise ValueError(f"linear state: {len(spec['decay'])} decay constants for {H} heads")
            self.head_decay = torch.tensor([float(x) for x in spec["decay"]], dtype=torch.float32, device=rt.device)
        rot = spec.get("rotary")
        self.rot_dims, self.freq, self.rot_key = 0, None, None
        if rot and int(rot["dims"]):
            self.rot_dims = int(rot["dims"])
            if self.rot_dims % 2 or self.rot_dims > dk:
                raise ValueError("linear state: the rotated dimensions must be even and at most the key size")
            i = torch.arange(self.rot_dims // 2, dtype=torch.float64)
            self.freq = torch.pow(torch.tensor(float(rot["base"]), dtype=torch.float64), -2.0 * i / self.rot_dims).to(torch.float32).to(rt.device)
            self.rot_key = ("half_pair_angles", self.rot_dims, float(rot["base"]))
        self.unit_eps = spec.get("unit_eps")
        self.q_scale, self.k_scale = float(spec.get("q_scale", 1.0)), float(spec.get("k_scale", 1.0))
        self.out_norm = spec.get("out_norm", "head")
        if self.out_norm not in ("head", "all"):
            raise ValueError("linear state: out_norm is 'head' or 'all'")
        self.out_weight = weights.take(spec["out_weight"]).float().contiguous() if spec.get("out_weight") else None
        self.gate_activation = spec.get("gate_activation", "silu")
        if self.gate_activation not in ops.GATE_ACTIVATIONS:
            raise ValueError("linear state: the gate's activation is 'silu' or 'sigmoid'")
        self.w_o = weights.take(spec["o"]).contiguous()
        self.state_size = H * dv * dk
        self.tail_size = (self.taps - 1) * self.channels if self.taps else 0

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((self.state_size + self.tail_size,), torch.float32)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        H, G, dk, dv = self.heads, self.qk_heads, self.dk, self.dv
        a = linear(x, self.w_in, None, self.rt, out_dtype=torch.float32)
        state = cache.state
        if self.forget_gate:
            ops.forget_gate_prep(a, self.q_off, self.k_off, H * dk, self.f_bias, self.lower, silu_q=self.activation == "silu")
            qs, fs, vs = a[:, self.q_off:self.q_off + H * dk], a[:, self.k_off:self.k_off + H * dk], a[:, self.v_off:self.v_off + H * dv]
            # the 32-bit path keeps one order of operations whatever the cutting: it always walks token by token
            if ctx.max_q_len >= CHUNKED_FROM and self.rt.dtype != torch.float32:
                chunk_meta, req_chunks = token_chunks(ctx, CHUNK)
                o = ops.forget_gate_chunked(qs, fs, vs, state, chunk_meta, req_chunks, ctx.state_slots, ctx.positions, H, dk, dv)
            else:
                o = ops.forget_gate_walk(qs, fs, vs, state, ctx.req_meta, ctx.state_slots, ctx.positions, ctx.n_requests, H, dk, dv)
            return self._finish(o, a)
        qkv, gate_rows = a, None          # where q, k and v stand, and (if elsewhere) the rows with the gates' columns
        if self.taps and ctx.max_q_len >= CONV_BY_TOKEN_FROM:
            qkv, gate_rows = ops.causal_conv_tokens(a, self.channels, self.conv_taps, state[:, self.state_size:], ctx.token_req, ctx.req_meta,
                                                    ctx.state_slots, ctx.positions, ctx.n_requests, silu=self.activation == "silu"), a
        elif self.taps:
            ops.causal_conv_walk(a, self.channels, self.conv_taps, state[:, self.state_size:], ctx.req_meta, ctx.state_slots, ctx.positions,
                                 ctx.n_requests, silu=self.activation == "silu")
        rot = None
        if self.rot_dims:
            if self.rot_key not in ctx.derived:
                ctx.derived[self.rot_key] = ops.angle_table(ctx.positions, self.freq)
            rot = ctx.derived[self.rot_key]
        gate, beta = ops.linear_state_prep(
            qkv, self.q_off, self.k_off, self.v_off, G, dk, H * dv, silu=self.activation == "silu" and not self.taps, rot=rot,
            rot_dims=self.rot_dims, unit=self.unit_eps is not None, unit_eps=float(self.unit_eps or 0.0), q_scale=self.q_scale,
            k_scale=self.k_scale, a_off=self.a_off if self.learned_decay else -1, b_off=self.b_off, heads=H, A_log=self.A_log,
            dt_bias=self.dt_bias, gate_rows=gate_rows)
        qs, ks_, vs = qkv[:, self.q_off:self.q_off + G * dk], qkv[:, self.k_off:self.k_off + G * dk], qkv[:, self.v_off:self.v_off + H * dv]
        # the 32-bit path keeps one order of operations whatever the cutting: it always walks; so does the delta rule,
        # whose update of the state is not a scaling and an addition
        if not self.delta and ctx.max_q_len >= CHUNKED_FROM and self.rt.dtype != torch.float32:
            chunk_meta, req_chunks = token_chunks(ctx, CHUNK)
            o = ops.linear_state_chunked(qs, ks_, vs, state, chunk_meta, req_chunks, ctx.state_slots, ctx.positions, H, G, dk, dv,
                                         gate=gate, head_decay=self.head_decay)
        else:
            o = ops.linear_state_walk(qs, ks_, vs, state, ctx.req_meta, ctx.state_slots, ctx.positions, ctx.n_requests, H, G, dk, dv,
                                      gate=gate, beta=beta, head_decay=self.head_decay)
        return self._finish(o, a)

    def _finish(self, o: torch.Tensor, a: torch.Tensor) -> torch.Tensor:
        """The norm behind the heads, the output gate (its columns stand in the projection's rows ``a``) and the output projection."""
        H, dv = self.heads, self.dv
        g = a[:, self.g_off:self.g_off + H * dv] if self.has_gate else None
        if self.out_norm == "head":
            y = ops.gated_group_norm(o, H, dv, self.rt.dtype, eps=self.eps, weight=self.out_weight, gate=g, activation=self.gate_activation)
        else:
            y = ops.gated_group_norm(o, 1, H * dv, self.rt.dtype, eps=self.eps, weight=self.out_weight, gate=g, activation=self.gate_activation)
        return linear(y, self.w_o, None, self.rt)
