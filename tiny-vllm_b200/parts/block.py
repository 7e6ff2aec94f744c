"""Arrangement of a layer's parts: pre-norm with a deferred residual sum.

The first layer keeps its input as the residual stream and norms it; every
later norm first adds the previous part's output to the stream.  The
feed-forward output is NOT added here: the next block's first norm (or the
model's final norm) adds it (tinyvllm/models/qwen3.py:386-412).
"""

from __future__ import annotations

import torch

from ..ops import kernels, linear
from .base import Block, BuildContext, ParamSpec
from .registry import register_part


class PreNormResidualBlock(Block):
    """x <- x + mixer(norm1(x)), then x <- x + feed_forward(norm2(x)); a layer may have no feed-forward
    (``feed_forward`` None: the layer ends after its mixer and declares no second norm).
    ``bare_norm_names``: the norms' weights are stored as "<layer>.<norm name>" instead of
    "<layer>.<norm name>.weight"."""

    def __init__(self, ctx: BuildContext, *, mixer, feed_forward, norm, mixer_norm_name: str,
                 feed_forward_norm_name: str, mixer_name: str, feed_forward_name: str,
                 bare_norm_names: bool = False) -> None:
        def build_norm(name):
            if bare_norm_names:
                return ctx.build("norm", norm.with_params(name=f"{ctx.prefix}.{name}"), ctx)
            return ctx.build("norm", norm, ctx.child(name))

        self.mixer_norm = build_norm(mixer_norm_name)
        self.mixer = ctx.build("mixer", mixer, ctx.child(mixer_name))
        self.feed_forward_norm = self.feed_forward = None
        if feed_forward is not None:
            self.feed_forward_norm = build_norm(feed_forward_norm_name)
            self.feed_forward = ctx.build("feed_forward", feed_forward, ctx.child(feed_forward_name))

    def children(self):
        return [part for part in (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward)
                if part is not None]

    def forward(self, hidden, residual, ctx, run: int):
        # a part that can take its norm into its first projection does so (forward_normed
        # returns its output and the new residual stream); the others get a normalised input
        # A forward_normed may return None as its output: it has added it to the stream already.
        if hasattr(self.mixer, "forward_normed"):
            mixed, residual = self.mixer.forward_normed(hidden, residual, self.mixer_norm, ctx, run)
        else:
            x, residual = _normed(self.mixer_norm, hidden, residual)
            mixed = self.mixer.forward(x, ctx, run)
        if self.feed_forward is None:
            return mixed, residual
        if hasattr(self.feed_forward, "forward_normed"):
            return self.feed_forward.forward_normed(mixed, residual, self.feed_forward_norm, ctx)
        x, residual = _normed(self.feed_forward_norm, mixed, residual)
        return self.feed_forward.forward(x, ctx), residual


def _normed(norm, hidden, residual):
    """(norm(hidden + residual), hidden + residual); either of the two may be missing: the first
    layer has no residual yet, and a part that added its output to the stream returns no output."""
    if hidden is None:
        return norm.forward(residual), residual
    if residual is None:
        return norm.forward(hidden), hidden
    return norm.add(hidden, residual)


class ParallelResidualBlock(Block):
    """One norm, and mixer and feed-forward side by side: with h = norm(x), x <- x + (mixer(h) +
    feed_forward(h)).  The residual stream x is float32 whatever the storage type; the sum of the
    two outputs is float32 and is added to the stream by the next norm (or the model's last one).

    Parts that can be a block's guests (``input_rows``, ``output_cols``, ``between``) share two
    products: all input projections are the rows of one weight [sum of rows, width], all output
    projections stand side by side in one weight [width, sum of columns], whose product with the
    concatenated inner activations is the float32 sum mixer(h) + feed_forward(h) itself.  Parts
    that cannot are run through their ``forward`` and their outputs are added.  A layer may have
    no feed-forward."""

    def __init__(self, ctx: BuildContext, *, mixer, feed_forward, norm, norm_name: str, mixer_name: str,
                 feed_forward_name: str, share_products: bool = True) -> None:
        self.norm = ctx.build("norm", norm, ctx.child(norm_name))
        self.width = norm.params["width"]
        self.shared = share_products
        hosted = {"hosted": True} if share_products else {}
        self.mixer = ctx.build("mixer", mixer.with_params(**hosted), ctx.child(mixer_name))
        self.feed_forward = None
        if feed_forward is not None:
            self.feed_forward = ctx.build("feed_forward", feed_forward.with_params(**hosted),
                                          ctx.child(feed_forward_name))
        self.guests = [part for part in (self.mixer, self.feed_forward) if part is not None]
        if share_products and not all(hasattr(part, "between") for part in self.guests):
            raise ValueError("a block shares its products only among parts that can be its guests")
        self.in_weight = self.out_weight = None

    def children(self):
        return [self.norm] + self.guests

    def param_specs(self):
        if not self.shared:
            return []
        rows = [pair for part in self.guests for pair in part.input_rows()]
        cols = [part.output_cols() for part in self.guests]
        return [ParamSpec.packed("in_weight", rows, self.width),
                ParamSpec.side_by_side("out_weight", self.width, cols)]

    def streamed_weights(self):
        return [self.in_weight, self.out_weight] if self.shared else []

    def forward(self, hidden, residual, ctx, run: int):
        x, residual = self.norm.add(hidden, residual)
        if not self.shared:
            update = self.mixer.forward(x, ctx, run)
            if self.feed_forward is not None:
                update = kernels.sum_pair(update, self.feed_forward.forward(x, ctx))
            return update, residual
        projected = linear(x, self.in_weight)
        inner = torch.empty((x.shape[0], self.out_weight.shape[1]), dtype=x.dtype, device=x.device)
        at_in = at_out = 0
        for part in self.guests:
            columns = part.output_cols()[1]
            out = inner[:, at_out:at_out + columns]
            if part is self.mixer:
                part.between(projected, at_in, ctx, out, run)
            else:
                part.between(projected, at_in, ctx, out)
            at_in += sum(rows for _, rows in part.input_rows())
            at_out += columns
        return linear(inner, self.out_weight, out_dtype=torch.float32), residual


class PostNormResidualBlock(Block):
    """The norm follows the residual sum: x <- norm1(alpha * x + mixer(x)), then x <- norm2(alpha * x +
    feed_forward(x)); both sublayers read x itself.  A layer may have no feed-forward: it then has no
    second step, unless its checkpoint holds the second norm, which is then applied to alpha * x.  The stream x is float32 whatever the storage type; the norms hand on, beside it,
    its one rounding to the storage type (``stream.rounded``), which is what the next products read.
    The block returns (None, stream): nothing is left to add."""

    def __init__(self, ctx: BuildContext, *, mixer, feed_forward, norm, alpha: float, mixer_norm_name: str,
                 feed_forward_norm_name: str, mixer_name: str, feed_forward_name: str) -> None:
        self.alpha = float(alpha)
        # the norms' weights are stored under the norms' own names, "<layer>.<norm name>"
        self.mixer_norm = ctx.build("norm", norm.with_params(name=f"{ctx.prefix}.{mixer_norm_name}"), ctx)
        self.mixer = ctx.build("mixer", mixer, ctx.child(mixer_name))
        self.feed_forward = None
        # a layer without a feed-forward has no second step; if its checkpoint holds the second norm all the
        # same, the step is x <- norm2(alpha x), the formula with nothing added
        self.feed_forward_norm = ctx.build(
            "norm", norm.with_params(name=f"{ctx.prefix}.{feed_forward_norm_name}",
                                     **({"optional": True} if feed_forward is None else {})), ctx)
        if feed_forward is not None:
            self.feed_forward = ctx.build("feed_forward", feed_forward, ctx.child(feed_forward_name))
        for part in (self.mixer_norm, self.feed_forward_norm):
            if part is not None and not hasattr(part, "post"):
                raise ValueError("a post-norm block needs norms that offer post(x, y, alpha)")

    def children(self):
        return [part for part in (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward)
                if part is not None]

    def forward(self, hidden, residual, ctx, run: int):
        if residual is None:                 # the first block: the embedding starts the stream
            stream, x = hidden, hidden
        else:
            if hidden is not None:
                raise ValueError("a post-norm block follows blocks that leave nothing to add to the stream")
            stream = residual
            x = getattr(stream, "rounded", None)
            if x is None:
                x = stream if stream.dtype == self.mixer_norm.out_dtype else stream.to(self.mixer_norm.out_dtype)
        x, stream = self.mixer_norm.post(stream, self.mixer.forward(x, ctx, run), self.alpha)
        if self.feed_forward is not None:
            x, stream = self.feed_forward_norm.post(stream, self.feed_forward.forward(x, ctx), self.alpha)
        elif self.feed_forward_norm.weight is not None:
            x, stream = self.feed_forward_norm.post(stream, None, self.alpha)
        if x is not stream:
            stream.rounded = x
        return None, stream


class SandwichResidualBlock(Block):
    """A norm before and a norm behind every sublayer: x <- x + post1(mixer(pre1(x))), then, where the layer has a
    feed-forward, x <- x + post2(feed_forward(pre2(x))).  The stream x is float32 whatever the storage type.

    A norm behind a sublayer and the norm in front of the next run as one kernel (``norm.after``); what the
    block's last sublayer leaves is handed on as ``stream.pending`` (:class:`parts.norm.PendingUpdate`), which
    the next block's first norm, or the model's last norm, adds in its own pass.  A feed-forward that offers
    ``forward_carried(x, ctx) -> (y, row_scale)`` stands for y + row_scale[:, None] * x (experts that hand
    their input on): the scaled term joins inside the norm kernel.  The block returns (None, stream)."""

    def __init__(self, ctx: BuildContext, *, mixer, feed_forward, norm, mixer_norm_name: str,
                 mixer_post_norm_name: str, feed_forward_norm_name: str, feed_forward_post_norm_name: str,
                 mixer_name: str, feed_forward_name: str) -> None:
        def build_norm(name):
            return ctx.build("norm", norm.with_params(name=f"{ctx.prefix}.{name}"), ctx)

        self.mixer_norm, self.mixer_post_norm = build_norm(mixer_norm_name), build_norm(mixer_post_norm_name)
        self.mixer = ctx.build("mixer", mixer, ctx.child(mixer_name))
        self.feed_forward_norm = self.feed_forward_post_norm = self.feed_forward = None
        if feed_forward is not None:
            self.feed_forward_norm = build_norm(feed_forward_norm_name)
            self.feed_forward_post_norm = build_norm(feed_forward_post_norm_name)
            self.feed_forward = ctx.build("feed_forward", feed_forward, ctx.child(feed_forward_name))
        for part in (self.mixer_norm, self.mixer_post_norm):
            if not hasattr(part, "after") or not hasattr(part, "resume"):
                raise ValueError("a sandwich block needs norms over a float32 stream that offer after() and resume()")

    def children(self):
        return [part for part in (self.mixer_norm, self.mixer_post_norm, self.mixer, self.feed_forward_norm,
                                  self.feed_forward_post_norm, self.feed_forward) if part is not None]

    def forward(self, hidden, residual, ctx, run: int):
        from .norm import PendingUpdate

        if residual is None:                 # the first block: the embedding starts the stream
            x, stream = self.mixer_norm.add(hidden, None)
        else:
            if hidden is not None:
                raise ValueError("a sandwich block follows blocks that leave nothing but the stream")
            stream = residual
            if getattr(stream, "pending", None) is not None:
                x, _ = self.mixer_norm.resume(stream)
            else:
                x = self.mixer_norm.forward(stream)
        mixed = self.mixer.forward(x, ctx, run)
        if self.feed_forward is None:
            stream.pending = PendingUpdate(mixed, self.mixer_post_norm)
            return None, stream
        x, stream = self.mixer_post_norm.after(stream, mixed, self.feed_forward_norm)
        if hasattr(self.feed_forward, "forward_carried"):
            y, row_scale = self.feed_forward.forward_carried(x, ctx)
            stream.pending = PendingUpdate(y, self.feed_forward_post_norm, row_scale, x if row_scale is not None else None)
        else:
            stream.pending = PendingUpdate(self.feed_forward.forward(x, ctx), self.feed_forward_post_norm)
        return None, stream


register_part("block", "prenorm_residual", PreNormResidualBlock)
register_part("block", "sandwich_residual", SandwichResidualBlock)
register_part("block", "postnorm_residual", PostNormResidualBlock)
register_part("block", "parallel_residual", ParallelResidualBlock)
