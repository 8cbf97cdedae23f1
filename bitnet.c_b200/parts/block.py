"""How a mixer, a feed-forward and their norms are arranged into one block."""
from __future__ import annotations

from ..csrc import ops
from .base import Block, Cast, Normed
from .registry import build_part, register_block


@register_block("pre_norm")
class PreNormBlock(Block):
    """x += mixer(norm(x)); x += ffn(norm(x))   (src/transformer/cpu.c:491-987).

    Each delta is handed to the next norm, which adds it to the residual while it reads
    it anyway; the block's last delta is returned as ``pending`` for whoever norms next.
    Where a part's last product can do that norm's work in its epilogue (few rows, bfloat16:
    ``Norm.sink``), the part gets a sink, adds to the residual itself and returns the norm's
    output; what the block then returns is ``Normed`` for the block after it.
    """

    graph_safe = True  # as far as its parts are
    accepts_normed = True

    def entry_norm(self):
        return self.mixer_norm

    def __init__(self, spec, build):
        super().__init__(spec, build)
        self.mixer_norm = build_part("norm", spec.mixer_norm, build)
        self.mixer = build_part("mixer", spec.mixer, build)
        self.ffn_norm = build_part("norm", spec.ffn_norm, build)
        self.ffn = build_part("ffn", spec.ffn, build)

    def children(self):
        return {"mixer_norm": self.mixer_norm, "mixer": self.mixer, "ffn_norm": self.ffn_norm, "ffn": self.ffn}

    def cache_request(self):
        return self.mixer.cache_request()

    def state_request(self):
        return self.mixer.state_request()

    @staticmethod
    def _input_for(part, h):
        if isinstance(h, ops.RowScaled) and not getattr(part, "accepts_sink", False):
            return h.dense()
        return h

    def forward(self, x, pending, ctx, kv, state, next_norm=None):
        h = pending.value if isinstance(pending, Normed) else self.mixer_norm.add_norm(x, pending, ctx)
        ctx.tap("attn_norm", h)
        sink = self.ffn_norm.sink(x, ctx) if getattr(self.mixer, "accepts_sink", False) else None
        if sink is not None:
            h = self.mixer.forward(self._input_for(self.mixer, h), ctx, kv, state, sink=sink)
        else:
            d = self.mixer.forward(self._input_for(self.mixer, h), ctx, kv, state)
            ctx.tap("attn_proj", d)
            h = self.ffn_norm.add_norm(x, d, ctx)
        ctx.tap("ffn_norm", h)
        sink = next_norm.sink(x, ctx) if next_norm is not None and getattr(self.ffn, "accepts_sink", False) else None
        if sink is not None:
            return Normed(self.ffn.forward(self._input_for(self.ffn, h), ctx, sink=sink))
        d = self.ffn.forward(self._input_for(self.ffn, h), ctx)
        ctx.tap("ffn_out", d)
        return d


@register_block("post_norm")
class PostNormBlock(Block):
    """x <- norm(alpha x + mixer(x)); x <- norm(alpha x + ffn(x)): the norms follow the sums, and their
    output is the residual stream itself (float32), which the sublayers read as it is.  Each norm
    also leaves a copy of its output in the compute type for the products that come next; the last
    copy goes to the next block as ``Cast``.  Without a feed-forward the second step is skipped, unless
    the block has a second norm, which then norms alpha x."""

    graph_safe = True  # as far as its parts are
    accepts_cast = True

    def __init__(self, spec, build):
        super().__init__(spec, build)
        self.mixer_norm = build_part("norm", spec.mixer_norm, build)
        self.mixer = build_part("mixer", spec.mixer, build)
        self.ffn = build_part("ffn", spec.ffn, build) if spec.ffn is not None else None
        self.ffn_norm = build_part("norm", spec.ffn_norm, build) if spec.ffn_norm is not None else None

    def children(self):
        c = {"mixer_norm": self.mixer_norm, "mixer": self.mixer}
        if self.ffn_norm is not None:
            c["ffn_norm"] = self.ffn_norm
        if self.ffn is not None:
            c["ffn"] = self.ffn
        return c

    def cache_request(self):
        return self.mixer.cache_request()

    def state_request(self):
        return self.mixer.state_request()

    def _as_input(self, x):
        return x if self.build.dtype == x.dtype else x.to(self.build.dtype)

    def forward(self, x, pending, ctx, kv, state):
        alpha = self.spec.alpha
        h = pending.value if isinstance(pending, Cast) else self._as_input(x)
        d = self.mixer.forward(h, ctx, kv, state)
        ctx.tap("attn_proj", d)
        h = self.mixer_norm.scaled_add_norm(x, alpha, d)
        ctx.tap("attn_norm", h)
        if self.ffn is not None:
            d = self.ffn.forward(h, ctx)
            ctx.tap("ffn_out", d)
            h = self.ffn_norm.scaled_add_norm(x, alpha, d)
        elif self.ffn_norm is not None and self.ffn_norm.weight is not None:
            h = self.ffn_norm.scaled_add_norm(x, alpha, None)
        return Cast(h)


@register_block("parallel")
class ParallelBlock(Block):
    """x <- x + (mixer(h) + ffn(h)) with h = norm(x): one norm, both sublayers read its output, and their deltas
    are summed before they meet the float32 stream.  Then, if the block has a ``side`` part, its input by token
    id: x <- x + norm'(side(x)).  The norm of whoever reads the stream next is taken in the same pass as the
    last addition when that reader says which it is (``next_norm``).  With a second norm (``ffn_norm``) the
    feed-forward reads that norm of the same x instead: x <- x + (mixer(norm(x)) + ffn(ffn_norm(x)))."""

    graph_safe = True  # as far as its parts are
    accepts_normed = True

    def __init__(self, spec, build):
        super().__init__(spec, build)
        self.norm = build_part("norm", spec.norm, build)
        self.mixer = build_part("mixer", spec.mixer, build)
        self.ffn = build_part("ffn", spec.ffn, build) if spec.ffn is not None else None
        self.side = build_part("side", spec.side, build) if spec.side is not None else None
        ffn_norm = getattr(spec, "ffn_norm", None)
        self.ffn_norm = build_part("norm", ffn_norm, build) if ffn_norm is not None else None
        if self.ffn is not None and self.ffn_norm is not None:
            self.norm.sibling = self.ffn_norm  # who prepares this block's first norm can prepare its second in the same pass

    def children(self):
        c = {"norm": self.norm, "mixer": self.mixer}
        if self.ffn_norm is not None:
            c["ffn_norm"] = self.ffn_norm
        if self.ffn is not None:
            c["ffn"] = self.ffn
        if self.side is not None:
            c["side"] = self.side
        return c

    def entry_norm(self):
        return self.norm

    def cache_request(self):
        return self.mixer.cache_request()

    def state_request(self):
        return self.mixer.state_request()

    def forward(self, x, pending, ctx, kv, state, next_norm=None):
        if isinstance(pending, Normed):
            h = pending.value.dense() if isinstance(pending.value, ops.RowScaled) else pending.value
        else:
            h = self.norm.add_norm(x, pending, ctx)
        ctx.tap("attn_norm", h)
        h2 = h
        if self.ffn is not None and self.ffn_norm is not None:
            h2 = pending.second if isinstance(pending, Normed) and pending.second is not None else None
            if h2 is None:
                h2 = self.ffn_norm.add_norm(x, None, ctx)  # the second norm of the same rows (the delta is in them by now)
            ctx.tap("ffn_norm", h2)
        d = self.mixer.forward(h, ctx, kv, state)
        ctx.tap("attn_proj", d)
        f = self.ffn.forward(h2, ctx) if self.ffn is not None else None
        if f is not None:
            ctx.tap("ffn_out", f)
        if self.side is None:
            w1 = getattr(next_norm, "weight", None) if next_norm is not None else None
            if w1 is None or x.shape[1] > ops.RESIDUAL_NORMS_MAX_WIDTH:
                ops.residual_add(x, d, f)
                return None
            # the sum of the deltas and the norms that read the stream next (the next block's, both of them where
            # it has two: they share their statistics) in one pass
            sib = getattr(next_norm, "sibling", None)
            w2 = getattr(sib, "weight", None) if sib is not None and sib.spec.eps == next_norm.spec.eps else None
            h1, h2n = ops.residual_add_norms(x, d, f, w1, w2.to(w1.dtype) if w2 is not None and w2.dtype != w1.dtype else w2,
                                             next_norm.spec.eps, self.build.dtype)
            return Normed(h1, second=h2n)
        xc = ops.residual_add(x, d, f, cast=self.build.dtype)
        y = self.side.delta(xc, ctx)
        ctx.tap("side_out", y)
        fused = next_norm if next_norm is not None and getattr(next_norm, "weight", None) is not None else None
        s = self.side.spec
        if fused is None:
            ops.add_normed(x, y, self.side.gain, s.eps)
            return None
        return Normed(ops.add_normed(x, y, self.side.gain, s.eps, fused.weight, fused.spec.eps, self.build.dtype))


@register_block("sandwich")
class SandwichBlock(Block):
    """x <- x + post(mixer(pre(x))); x <- x + ffn_post(ffn(ffn_pre(x))): a norm before and after each sublayer.
    The sublayers leave their products in float32; one pass divides a sublayer's output by its root mean square,
    multiplies by the gain, adds it to the float32 stream and takes the norm that reads the new rows next (this
    block's second pre-norm, or the next block's first when that reader says which it is).  Without a feed-forward
    the second step is left out."""

    graph_safe = True  # as far as its parts are
    accepts_normed = True

    def __init__(self, spec, build):
        super().__init__(spec, build)
        self.mixer_norm = build_part("norm", spec.mixer_norm, build)
        self.mixer = build_part("mixer", spec.mixer, build)
        self.mixer_post_norm = build_part("norm", spec.mixer_post_norm, build)
        self.ffn = build_part("ffn", spec.ffn, build) if spec.ffn is not None else None
        if self.ffn is not None and (spec.ffn_norm is None or spec.ffn_post_norm is None):
            raise ValueError("a sandwich block with a feed-forward needs both of its norms")
        self.ffn_norm = build_part("norm", spec.ffn_norm, build) if self.ffn is not None else None
        self.ffn_post_norm = build_part("norm", spec.ffn_post_norm, build) if self.ffn is not None else None

    def children(self):
        c = {"mixer_norm": self.mixer_norm, "mixer": self.mixer, "mixer_post_norm": self.mixer_post_norm}
        if self.ffn is not None:
            c.update(ffn_norm=self.ffn_norm, ffn=self.ffn, ffn_post_norm=self.ffn_post_norm)
        return c

    def entry_norm(self):
        return self.mixer_norm

    def cache_request(self):
        return self.mixer.cache_request()

    def state_request(self):
        return self.mixer.state_request()

    def _add(self, x, y, post, reader):
        """x += post(y); the reader's norm of the new rows, if there is a reader whose gain is at hand."""
        w = getattr(reader, "weight", None) if reader is not None else None
        if w is None:
            ops.add_normed(x, y, post.weight, post.spec.eps)
            return None
        return ops.add_normed(x, y, post.weight, post.spec.eps, w, reader.spec.eps, self.build.dtype)

    def forward(self, x, pending, ctx, kv, state, next_norm=None):
        if isinstance(pending, Normed):
            h = pending.value.dense() if isinstance(pending.value, ops.RowScaled) else pending.value
        else:
            h = self.mixer_norm.add_norm(x, pending, ctx)
        ctx.tap("attn_norm", h)
        d = self.mixer.forward(h, ctx, kv, state)
        ctx.tap("attn_proj", d)
        h = self._add(x, d, self.mixer_post_norm, self.ffn_norm if self.ffn is not None else next_norm)
        if self.ffn is None:
            return Normed(h) if h is not None else None
        ctx.tap("ffn_norm", h)
        f = self.ffn.forward(h, ctx)
        ctx.tap("ffn_out", f)
        h = self._add(x, f, self.ffn_post_norm, next_norm)
        return Normed(h) if h is not None else None
