"""Pre-norm residual block: h += mixer(norm(h)); h += feed_forward(norm(h))
(src/model.py:113-127 of the reference). Each add is fused with the norm that follows it, so a
branch output travels to the next norm as `pending`."""
from __future__ import annotations

import torch

from ..kernels import ops, trace
from .base import Block, DeferredBranchAdd, ScaledDelta, call_branch, register_block, single_delta


class PreNormBlock(Block):
    """Roles: mixer, feed_forward and a norm in front of each. A branch whose part declares
    `accepts_deferred_norm` gets the norm as a promise and folds it into its first kernel; one that declares
    `adds_to_residual` gets the residual stream and may add its output there itself (parts/base.py)."""
    ROLES = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "feed_forward_norm": "norm"}

    def forward(self, h, pending, ctx, unit, owns_cache):
        tracing = trace.active()
        if tracing:
            trace.push(f"Attn_{ctx.entry}")           # the reference's range names (src/model.py:112,126)
        x = None
        if pending is None and self.mixer.accepts_deferred_norm:
            x = self.mixer_norm.defer(h)              # the mixer's first kernel applies the norm
        if x is None:
            x = self.mixer_norm.forward(h, pending)
        mixed = call_branch(self.mixer, x, ctx, unit, owns_cache, residual=h)
        if tracing:
            trace.pop()
            trace.push(f"FFN_{ctx.entry}")
        x = None
        if mixed is None and self.feed_forward.accepts_deferred_norm:
            x = self.feed_forward_norm.defer(h)
        if x is None:
            x = self.feed_forward_norm.forward(h, mixed)
        out = call_branch(self.feed_forward, x, ctx, residual=h)
        if tracing:
            trace.pop()
        return h, out


register_block("pre_norm", PreNormBlock)


class BranchNormBlock(Block):
    """h += norm(mixer(h)); h += norm(feed_forward(h)): the branches read the residual stream itself and the norm
    sits on each branch's OUTPUT. The sum stays float32; a bfloat16 engine's products read the stream rounded to
    bfloat16, and that rounded copy is written by the same kernel that adds the branch (it travels to the next
    layer in `ctx.carry["h_act"]`). A feed-forward that declares `down_bias` has it added inside the norm's
    kernel. In one-token steps of one or two rows of a bfloat16 engine the add is not done here at all: it is handed
    on as a `DeferredBranchAdd` to the part that opens the next branch (the feed-forward, or the next layer's
    mixer, which gets it as `pending`), whose first product does it while it stages its input."""
    ROLES = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "feed_forward_norm": "norm"}
    leaves_rounded_stream = True
    accepts_deferred_branch_add = True

    def _rounded(self, h, ctx):
        """The stream as the products read it: itself in a float32 engine, else its bfloat16 copy."""
        if self.runtime.dtype == torch.float32:
            return h
        act = ctx.carry.pop("h_act", None)
        if act is None:
            act = ops.cast_rows(h, torch.empty(h.shape, dtype=self.runtime.dtype, device=h.device))
        return act

    def _new_rounded(self, h):
        return None if self.runtime.dtype == torch.float32 else torch.empty(h.shape, dtype=self.runtime.dtype,
                                                                            device=h.device)

    def _defers(self, h, ctx) -> bool:
        """Whether the adds of this step are handed on instead of done: one-token steps the fused product takes."""
        return (self.runtime.dtype == torch.bfloat16 and ctx.decode and h.shape[0] <= ops.BRANCH_FOLD_BEST_ROWS
                and ops.norm_gemm_supported(h.shape[0], h.shape[1]))

    def _close(self, h, y, bias, norm, ctx, nxt):
        """Ends a branch: h += norm(y + bias), here, or handed to `nxt` (the part that opens the next branch, None =
        unknown) when it can fold the add into its first product. Returns (h, x for the next branch, pending)."""
        if self._defers(h, ctx) and y.dtype == torch.float32 and (nxt is None or getattr(nxt, "accepts_deferred_branch_add", False)):
            d = DeferredBranchAdd(norm, h, y, bias)
            return h, d, d
        act = self._new_rounded(h)
        norm.add_normed(h, y, bias, act)
        return h, (h if act is None else act), None

    def _open(self, h, pending, ctx):
        """What the mixer reads: the deferred add of the layer before, or the (rounded) stream."""
        if isinstance(pending, DeferredBranchAdd):
            if self.mixer.accepts_deferred_branch_add:
                return pending
            h = pending.apply()
            pending = None
        if pending is not None:
            ops.residual_add(h, pending)
            ctx.carry.pop("h_act", None)
        return self._rounded(h, ctx)

    def forward(self, h, pending, ctx, unit, owns_cache):
        tracing = trace.active()
        if tracing:
            trace.push(f"Attn_{ctx.entry}")
        x = self._open(h, pending, ctx)
        y = call_branch(self.mixer, x, ctx, unit, owns_cache)
        if isinstance(x, DeferredBranchAdd):
            h = x.apply()                      # the new stream (the mixer's first product has made it)
        ff = self.feed_forward
        h, x, _ = self._close(h, y, None, self.mixer_norm, ctx, ff)
        if tracing:
            trace.pop()
            trace.push(f"FFN_{ctx.entry}")
        deferred = getattr(ff, "down_bias", None)
        y = ff.forward(x, ctx, defer_bias=True) if deferred is not None else call_branch(ff, x, ctx)
        if isinstance(x, DeferredBranchAdd):
            h = x.apply()
        h, x, handed_on = self._close(h, y, deferred, self.feed_forward_norm, ctx, None)
        if handed_on is None and x is not h:
            ctx.carry["h_act"] = x
        if tracing:
            trace.pop()
        return h, handed_on


class BranchNormMixerBlock(BranchNormBlock):
    """The same arrangement for a layer without a feed-forward: h += norm(mixer(h))."""
    ROLES = {"mixer": "mixer", "mixer_norm": "norm"}

    def forward(self, h, pending, ctx, unit, owns_cache):
        x = self._open(h, pending, ctx)
        y = call_branch(self.mixer, x, ctx, unit, owns_cache)
        if isinstance(x, DeferredBranchAdd):
            h = x.apply()
        h, x, handed_on = self._close(h, y, None, self.mixer_norm, ctx, None)
        if handed_on is None and x is not h:
            ctx.carry["h_act"] = x
        return h, handed_on


register_block("branch_norm", BranchNormBlock)
register_block("branch_norm_mixer", BranchNormMixerBlock)


class ParallelBlock(Block):
    """u = norm(h); h += mixer(u) + feed_forward(u): ONE norm, both branches read its output, and both are added to
    the stream together. The two branch outputs travel on as a pair and the next norm's kernel adds them while it
    reads the stream (the float32 sum h + y1 + y2 is formed there); a branch whose part declares `adds_to_residual`
    may instead add its output into the stream inside its own last product, which is safe because both branches read
    the norm's output and not the stream."""
    ROLES = {"mixer": "mixer", "feed_forward": "feed_forward", "norm": "norm"}

    def forward(self, h, pending, ctx, unit, owns_cache):
        tracing = trace.active()
        u = self.norm.forward(h, pending)
        if tracing:
            trace.push(f"Attn_{ctx.entry}")
        y1 = call_branch(self.mixer, u, ctx, unit, owns_cache, residual=h)
        if tracing:
            trace.pop()
            trace.push(f"FFN_{ctx.entry}")
        y2 = call_branch(self.feed_forward, u, ctx, residual=h)
        if tracing:
            trace.pop()
        left = tuple(y for y in (y1, y2) if y is not None)
        return h, (left if len(left) > 1 else (left[0] if left else None))


class ParallelMixerBlock(Block):
    """The same arrangement for a layer without a feed-forward: h += mixer(norm(h))."""
    ROLES = {"mixer": "mixer", "norm": "norm"}

    def forward(self, h, pending, ctx, unit, owns_cache):
        u = self.norm.forward(h, pending)
        return h, call_branch(self.mixer, u, ctx, unit, owns_cache, residual=h)


register_block("parallel", ParallelBlock)
register_block("parallel_mixer", ParallelMixerBlock)


class PreNormScaledBlock(Block):
    """h += s1 (.) mixer(norm(h)); h += s2 (.) feed_forward(norm(h)): the pre-norm block with a learned scale per
    channel on each branch's output (the roles `mixer_scale` and `feed_forward_scale`, pointwise parts of kind
    "layer_scale"). The scaled output travels to the next norm as a `ScaledDelta`, whose kernel multiplies and adds
    while it reads the stream, so the scale costs no launch; a mixer made of two mixers hands over both outputs with
    their constants and they are added in the same pass."""
    ROLES = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "feed_forward_norm": "norm",
             "mixer_scale": "pointwise", "feed_forward_scale": "pointwise"}

    def forward(self, h, pending, ctx, unit, owns_cache):
        tracing = trace.active()
        if tracing:
            trace.push(f"Attn_{ctx.entry}")
        x = self.mixer_norm.forward(h, pending)
        mixed = ScaledDelta.of(call_branch(self.mixer, x, ctx, unit, owns_cache), self.mixer_scale.vector)
        if tracing:
            trace.pop()
            trace.push(f"FFN_{ctx.entry}")
        x = self.feed_forward_norm.forward(h, mixed)
        out = ScaledDelta.of(call_branch(self.feed_forward, x, ctx), self.feed_forward_scale.vector)
        if tracing:
            trace.pop()
        return h, out


class PreNormScaledMixerBlock(Block):
    """The same arrangement for a layer without a feed-forward: h += s1 (.) mixer(norm(h))."""
    ROLES = {"mixer": "mixer", "mixer_norm": "norm", "mixer_scale": "pointwise"}

    def forward(self, h, pending, ctx, unit, owns_cache):
        x = self.mixer_norm.forward(h, pending)
        return h, ScaledDelta.of(call_branch(self.mixer, x, ctx, unit, owns_cache), self.mixer_scale.vector)


register_block("pre_norm_scaled", PreNormScaledBlock)
register_block("pre_norm_scaled_mixer", PreNormScaledMixerBlock)


class PostNormScaledBlock(BranchNormBlock):
    """h = norm(alpha h + s1 (.) mixer(h)); h = norm(alpha h + s2 (.) feed_forward(h)): the norm comes AFTER the residual
    sum, so the stream itself is what every norm returns, and the branches read the stream. alpha is a constant of the
    norm parts (`residual_scale`), s a learned scale per channel (the roles `mixer_scale` and `feed_forward_scale`,
    pointwise parts of kind "layer_scale"). Scale, sum and norm are one kernel (`Norm.norm_sum`), which also writes the
    copy of the new stream that a bfloat16 engine's next product reads; the stream stays float32."""
    ROLES = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "feed_forward_norm": "norm",
             "mixer_scale": "pointwise", "feed_forward_scale": "pointwise"}
    accepts_deferred_branch_add = False

    def _start(self, h, pending, ctx):
        """Whatever the layer before has left unadded goes into the stream first."""
        if isinstance(pending, DeferredBranchAdd):
            h, pending = pending.apply(), None
        pending = single_delta(pending)
        if pending is not None:
            ops.residual_add(h, pending)
            ctx.carry.pop("h_act", None)
        return h

    def _branch(self, h, x, y, norm, scale):
        """Closes a branch; returns what the next branch reads."""
        if isinstance(y, ScaledDelta):
            y = y.materialize()
        act = self._new_rounded(h)
        norm.norm_sum(h, y, scale.vector, act)
        return h if act is None else act

    def forward(self, h, pending, ctx, unit, owns_cache):
        tracing = trace.active()
        h = self._start(h, pending, ctx)
        if tracing:
            trace.push(f"Attn_{ctx.entry}")
        x = self._rounded(h, ctx)
        x = self._branch(h, x, call_branch(self.mixer, x, ctx, unit, owns_cache), self.mixer_norm, self.mixer_scale)
        if tracing:
            trace.pop()
            trace.push(f"FFN_{ctx.entry}")
        x = self._branch(h, x, call_branch(self.feed_forward, x, ctx), self.feed_forward_norm, self.feed_forward_scale)
        if x is not h:
            ctx.carry["h_act"] = x
        if tracing:
            trace.pop()
        return h, None


class PostNormScaledMixerBlock(PostNormScaledBlock):
    """The same arrangement for a layer without a feed-forward: h = norm(alpha h + s1 (.) mixer(h))."""
    ROLES = {"mixer": "mixer", "mixer_norm": "norm", "mixer_scale": "pointwise"}

    def forward(self, h, pending, ctx, unit, owns_cache):
        h = self._start(h, pending, ctx)
        x = self._rounded(h, ctx)
        x = self._branch(h, x, call_branch(self.mixer, x, ctx, unit, owns_cache), self.mixer_norm, self.mixer_scale)
        if x is not h:
            ctx.carry["h_act"] = x
        return h, None


register_block("post_norm_scaled", PostNormScaledBlock)
register_block("post_norm_scaled_mixer", PostNormScaledMixerBlock)
