"""Pre-norm arrangement: ``x += mixer(norm(x)); x += feed_forward(norm(x))``.

The reference defers each layer's last residual add to the next layer
(gllm/model/transformer.py:58-78): a layer receives the previous feed-forward
output and the residual, adds them, and returns its own feed-forward output
un-added.  The same protocol is kept here because it lets every add fuse into
the norm kernel that follows it.
"""

from __future__ import annotations

from gllm_b200 import ops
from gllm_b200.parts.base import Block, register_block


@register_block("prenorm")
class PreNormBlock(Block):
    graph_safe_portions = True
    part_kinds = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}
    # a layer may have a mixer only
    optional_parts = frozenset({"feed_forward_norm", "feed_forward"})

    def forward(self, branch, resid, ctx, cache):
        # a part may add its result into the residual itself (its last product's epilogue) and say so
        ctx.residual_sink = resid
        x = self.mixer_norm.forward(None if branch is ops.ADDED else branch, resid, ctx.dtype)
        out = self.mixer.forward(x, ctx, cache)
        if self.feed_forward is not None:
            x = self.feed_forward_norm.forward(None if out is ops.ADDED else out, resid, ctx.dtype)
            out = self.feed_forward.forward(x, ctx)
        ctx.residual_sink = None
        return out, resid


@register_block("shared_norm")
class SharedNormBlock(Block):
    """One norm, two branches that both read its output: ``h = norm(x); x += mixer(h) + feed_forward(h)``.
    The mixer's result is added into the fp32 residual at once (by its last product where that adds itself,
    by ``ops.residual_add`` otherwise); the feed-forward's result is handed on un-added, as the pre-norm block
    does, so that the next norm's kernel adds it.  A layer may have no feed-forward."""

    graph_safe_portions = True
    part_kinds = {"norm": "norm", "mixer": "mixer", "feed_forward": "feed_forward"}
    optional_parts = frozenset({"feed_forward"})

    def forward(self, branch, resid, ctx, cache):
        ctx.residual_sink = resid
        x = self.norm.forward(None if branch is ops.ADDED else branch, resid, ctx.dtype)
        out = self.mixer.forward(x, ctx, cache)
        if self.feed_forward is not None:
            if out is not ops.ADDED:
                ops.residual_add(resid, out)
            out = self.feed_forward.forward(x, ctx)
        ctx.residual_sink = None
        return out, resid


@register_block("sandwich")
class SandwichBlock(Block):
    """A norm before and a norm after each sublayer: ``x += post_a(mixer(pre_a(x))); x += post_b(ff(pre_b(x)))``.
    A sublayer's result is not normed and added by a kernel of its own: it travels on as ``ops.Pending`` (the
    result with the post-norm's weight) and the NEXT pre-norm's kernel does the post-norm, the add and its own
    norm in one pass, as the pre-norm block defers its plain adds.  The sublayers' last products cannot add
    themselves into the residual (their result is normed first).  A layer may have no feed-forward."""

    graph_safe_portions = True
    part_kinds = {"mixer_norm": "norm", "mixer": "mixer", "mixer_post_norm": "norm",
                  "feed_forward_norm": "norm", "feed_forward": "feed_forward", "feed_forward_post_norm": "norm"}
    optional_parts = frozenset({"feed_forward_norm", "feed_forward", "feed_forward_post_norm"})

    def forward(self, branch, resid, ctx, cache):
        ctx.residual_sink = None
        x = self.mixer_norm.forward(None if branch is ops.ADDED else branch, resid, ctx.dtype)
        out = self.mixer_post_norm.pending(self.mixer.forward(x, ctx, cache))
        if self.feed_forward is not None:
            x = self.feed_forward_norm.forward(out, resid, ctx.dtype)
            out = self.feed_forward_post_norm.pending(self.feed_forward.forward(x, ctx))
        return out, resid
