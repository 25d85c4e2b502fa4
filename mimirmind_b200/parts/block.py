"""Pre-norm residual block: ``x += mixer(norm1(x)); x += ffn(norm2(x))``.

Order per layer in the reference: norm → QKV(+bias) → RoPE → cache write → attention → O
→ (+residual, fused with the next norm) → gate, up → SiLU·up → down → (+residual)
(src/runtime/arch/Qwen2Backend.cpp:203-461).  The last add of a layer is left pending so
that it fuses into the norm that follows, whichever layer that norm belongs to.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..registry import BLOCKS
from .base import Block, FactoredRows, LayerCache, NativeDesc, NormedRows, ResidualSink, StepContext


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    """With parts that fuse (a few tokens in bfloat16), the residual add and the norm move into the epilogue of
    the branch's last matrix product and the 1/rms into the next product: a layer is five launches."""

    def entry_norm(self, n_tokens: int):
        f = self.mixer_norm.factors()
        return f if f is not None and self.mixer.fuses(n_tokens) else None

    def native(self):
        parts = {"mixer_norm": self.mixer_norm.native(), "mixer": self.mixer.native(), "ffn_norm": self.ffn_norm.native(),
                 "feed_forward": self.feed_forward.native()}
        if type(self) is not PreNormBlock or any(p is None for p in parts.values()):
            return None
        return NativeDesc("pre_norm", {}, {}, parts)

    def forward(self, residual: torch.Tensor, pending, ctx: StepContext, cache: LayerCache,
                successor: Optional[Block] = None):
        n = residual.shape[0]
        if ctx.plain_only:
            return self._forward_plain(residual, pending, ctx, cache)
        mixer_fuses, ffn_fuses = self.mixer.fuses(n), self.feed_forward.fuses(n)
        h = pending if isinstance(pending, FactoredRows) else self.mixer_norm.forward(residual, pending)
        between = self.ffn_norm.factors() if (mixer_fuses and ffn_fuses) else None
        if between is not None:
            h = self.mixer.forward(h, ctx, cache, sink=ResidualSink(residual, between[0], between[1]))
        else:
            h = self.ffn_norm.forward(residual, self.mixer.forward(h, ctx, cache))
        if not ffn_fuses:
            return self.feed_forward.forward(h, ctx)
        after = successor.entry_norm(n) if successor is not None else None
        if successor is not None and after is None:
            return self.feed_forward.forward(h, ctx)       # the next block wants a plain pending sum
        sink = ResidualSink(residual, after[0], after[1]) if after is not None else ResidualSink(residual)
        return self.feed_forward.forward(h, ctx, sink=sink)

    def _forward_plain(self, residual: torch.Tensor, pending, ctx: StepContext, cache: LayerCache):
        """Every stage as a tensor of its own, with the stage dumps of the reference
        (src/runtime/arch/Qwen2Backend.cpp:207, 431, 458, 462): the normalised input of the mixer, the two branch
        outputs, and the layer's output (the residual stream with both branches added)."""
        dump = ctx.dump or (lambda stage, t: None)
        h = self.mixer_norm.forward(residual, pending)
        dump("attn_norm", h)
        branch = self.mixer.forward(h, ctx, cache)
        dump("attn_out", branch)
        h = self.ffn_norm.forward(residual, branch)
        out = self.feed_forward.forward(h, ctx)
        dump("ffn_mlp", out)
        if ctx.dump is not None:
            dump("l_out", residual + out.to(residual.dtype))
        return out


@BLOCKS.register("sandwich_norm")
class SandwichNormBlock(Block):
    """A norm before and after each sublayer: ``x += post1(mixer(pre1(x)))``, then ``x += post2(ffn(pre2(x)))``; a layer
    whose feed-forward is of kind ``none`` has the first sublayer only.  The two post norms are the layer's extra parts
    ``mixer_post_norm`` and ``ffn_post_norm``.

    The branch is normed, added into the fp32 residual stream and the sum normed for the next sublayer in one launch
    where the two norms are grouped RMS norms of one shape; the last add of the layer does so for the first norm of
    the block that follows and hands its rows over as ``NormedRows``.  The residual stream is complete when the block
    returns."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        from .mlp import NoFeedForward
        self.has_ffn = not isinstance(self.feed_forward, NoFeedForward)
        for name in ("mixer_post_norm",) + (("ffn_post_norm",) if self.has_ffn else ()):
            if name not in self.extras:
                raise ValueError(f"sandwich_norm block: the layer has no '{name}'")
        self.mixer_post = self.extras["mixer_post_norm"]
        self.ffn_post = self.extras.get("ffn_post_norm")

    def accepts_normed_rows(self) -> bool:
        """True if a predecessor may run this block's first norm for it."""
        return hasattr(self.mixer_norm, "same_shape")

    @staticmethod
    def _add(post, residual: torch.Tensor, branch: torch.Tensor, then):
        """residual += post(branch); returns then(residual) if ``then`` is given."""
        if hasattr(post, "add_normed") and (then is None or hasattr(then, "same_shape")):
            return post.add_normed(residual, branch, then)
        zero = torch.zeros_like(residual)
        normed = post.forward(zero, branch)                    # any other norm: through its plain interface
        if then is None:
            ops_add(residual, normed)
            return None
        return then.forward(residual, normed)

    def forward(self, residual: torch.Tensor, pending, ctx: StepContext, cache: LayerCache,
                successor: Optional[Block] = None):
        dump = ctx.dump or (lambda stage, t: None)
        h = pending.x if isinstance(pending, NormedRows) else self.mixer_norm.forward(residual, pending)
        dump("attn_norm", h)
        branch = self.mixer.forward(h, ctx, cache)
        dump("attn_out", branch)
        hand_over = None
        if successor is not None and isinstance(successor, SandwichNormBlock) and successor.accepts_normed_rows() and not ctx.plain_only:
            hand_over = successor.mixer_norm
        if self.has_ffn:
            h = self._add(self.mixer_post, residual, branch, self.ffn_norm)
            branch = self.feed_forward.forward(h, ctx)
            dump("ffn_mlp", branch)
            post = self.ffn_post
        else:
            post = self.mixer_post
        made = self._add(post, residual, branch, hand_over)
        if ctx.dump is not None:
            dump("l_out", residual)
        return NormedRows(made) if made is not None else None


@BLOCKS.register("parallel_branches")
class ParallelBranchesBlock(Block):
    """Mixer and feed-forward side by side, each behind a norm of its own over the same stream:
    ``x += mixer(norm1(x)) + ffn(norm2(x))``; a layer whose feed-forward is of kind ``none`` has the first branch only.
    The mixer's branch is added into the fp32 residual stream here, the feed-forward's is left pending so that the add
    fuses into the norm that follows, whichever layer owns it."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        from .mlp import NoFeedForward
        self.has_ffn = not isinstance(self.feed_forward, NoFeedForward)

    def forward(self, residual: torch.Tensor, pending, ctx: StepContext, cache: LayerCache,
                successor: Optional[Block] = None):
        dump = ctx.dump or (lambda stage, t: None)
        h = self.mixer_norm.forward(residual, pending)           # the stream is complete from here on
        dump("attn_norm", h)
        branch = self.mixer.forward(h, ctx, cache)
        dump("attn_out", branch)
        if not self.has_ffn:
            if ctx.dump is not None:
                dump("l_out", residual + branch.to(residual.dtype))
            return branch
        out = self.feed_forward.forward(self.ffn_norm.forward(residual, None), ctx)
        dump("ffn_mlp", out)
        ops_add(residual, branch)
        if ctx.dump is not None:
            dump("l_out", residual + out.to(residual.dtype))
        return out


@BLOCKS.register("stream_connections")
class StreamConnectionsBlock(Block):
    """Pre-norm sublayers whose way in and out of the residual stream is a part of its own (``parts/connections.py``):
    ``h = norm1(read1(x)); x <- write1(x, mixer(h)); h = norm2(read2(x)); x <- write2(x, ffn(h))``, with one or several
    copies of the residual stream per token.  The connections are the layer's extra parts ``mixer_connection`` and
    ``ffn_connection``; a layer whose feed-forward is of kind ``none`` has the first sublayer only.

    A write and the read and norm that follow it are one launch, also across the border to the next block of this
    kind, which gets its first normed rows as ``NormedRows``.  The streams are complete when the block returns."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        from .mlp import NoFeedForward
        self.has_ffn = not isinstance(self.feed_forward, NoFeedForward)
        for name in ("mixer_connection",) + (("ffn_connection",) if self.has_ffn else ()):
            if name not in self.extras:
                raise ValueError(f"stream_connections block: the layer has no '{name}'")
        self.mixer_connection = self.extras["mixer_connection"]
        self.ffn_connection = self.extras.get("ffn_connection")

    def forward(self, residual: torch.Tensor, pending, ctx: StepContext, cache: LayerCache,
                successor: Optional[Block] = None):
        dump = ctx.dump or (lambda stage, t: None)
        first = self.mixer_connection
        h = pending.x if isinstance(pending, NormedRows) else first.read(residual, self.mixer_norm)
        dump("attn_norm", h)
        branch = self.mixer.forward(h, ctx, cache)
        dump("attn_out", branch)
        last = first
        if self.has_ffn:
            h = first.write(residual, branch, self.ffn_connection, self.ffn_norm)
            branch = self.feed_forward.forward(h, ctx)
            dump("ffn_mlp", branch)
            last = self.ffn_connection
        made = None
        if (isinstance(successor, StreamConnectionsBlock) and successor.mixer_connection.streams == last.streams
                and successor.mixer_norm.factors() is not None and not ctx.plain_only):
            made = last.write(residual, branch, successor.mixer_connection, successor.mixer_norm)
        else:
            last.write(residual, branch)
        if ctx.dump is not None:
            dump("l_out", last.total(residual))
        return NormedRows(made) if made is not None else None


@BLOCKS.register("post_norm")
class PostNormBlock(Block):
    """The norm after the sum: ``x <- norm1(alpha x + mixer(x))``, then ``x <- norm2(alpha x + ffn(x))``; the sublayers read the
    stream itself, and a layer whose feed-forward is of kind ``none`` has the first sublayer only.  Both norms are of the kind
    ``y w / sqrt(mean(y^2) + eps)`` (``Norm.factors``).

    The scaling of the stream, the sum and the norm are one launch that leaves the fp32 stream and its rounding to the
    activation dtype, which is what the next sublayer's products read.  A mixer or feed-forward whose result is a weighted
    sum of two branches (``forward_branches``) hands the branches over and the same launch adds them.  The block that follows,
    if it is of this kind, gets the rounded stream as ``NormedRows``.

    spec params: alpha."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        from .mlp import NoFeedForward
        self.alpha = float(self.spec.get("alpha", 1.0))
        self.has_ffn = not isinstance(self.feed_forward, NoFeedForward)
        self.norms = []
        for norm in (self.mixer_norm,) + ((self.ffn_norm,) if self.has_ffn else ()):
            f = norm.factors()
            if f is None:
                raise ValueError("post_norm block: its norms must be of the kind y * w / sqrt(mean(y^2) + eps)")
            self.norms.append((f[0].float().contiguous(), float(f[1])))

    @staticmethod
    def _branches(part, *args):
        many = part.forward_branches(*args) if hasattr(part, "forward_branches") else None
        if many is None:
            return [(part.forward(*args), 1.0)]
        if len(many) > 2:
            raise ValueError("post_norm block: a sublayer hands over at most two branches")
        return many

    def _sublayer(self, residual: torch.Tensor, branches, which: int):
        from ..kernels import ops
        w, eps = self.norms[which]
        (a, ca), (b, cb) = branches[0], (branches[1] if len(branches) > 1 else (None, 1.0))
        if self.rt.dtype == torch.float32:
            ops.post_norm(residual, a, b, w, eps, self.alpha, ca, cb)
            return residual                          # a float32 run reads the stream itself
        out = torch.empty(residual.shape, dtype=self.rt.dtype, device=residual.device)
        return ops.post_norm(residual, a, b, w, eps, self.alpha, ca, cb, out=out)

    def forward(self, residual: torch.Tensor, pending, ctx: StepContext, cache: LayerCache,
                successor: Optional[Block] = None):
        from ..kernels import ops
        dump = ctx.dump or (lambda stage, t: None)
        if isinstance(pending, NormedRows):
            h = pending.x
        else:
            if pending is not None:
                ops.add_residual(residual, pending)
            h = residual if self.rt.dtype == torch.float32 else ops.cast_rows(residual, self.rt.dtype)
        dump("attn_norm", h)
        h = self._sublayer(residual, self._branches(self.mixer, h, ctx, cache), 0)
        dump("attn_out", residual)               # the stream behind the mixer's sublayer
        if self.has_ffn:
            h = self._sublayer(residual, self._branches(self.feed_forward, h, ctx), 1)
        if ctx.dump is not None:
            dump("l_out", residual)
        return NormedRows(h) if isinstance(successor, PostNormBlock) else None


def ops_add(residual: torch.Tensor, delta: torch.Tensor) -> None:
    from ..kernels import ops
    ops.add_residual(residual, delta)
