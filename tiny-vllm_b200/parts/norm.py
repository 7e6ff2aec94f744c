"""RMSNorm with float32 statistics.

y = round(round(x * (mean(x^2) + eps)^-1/2) * w); ``add`` first forms the rounded
sum with the residual stream and returns it as the new stream
(tinyvllm/layers.py:129-164; tinyvllm/kernels/pointwise.cu:153-211).
"""

from __future__ import annotations

import torch

from ..ops import kernels
from .base import BuildContext, ParamSpec, Part
from .registry import register_part


class RMSNorm(Part):
    # y = x * rsqrt(mean(x^2) + eps) * weight: a projection behind it may apply it in its own kernel
    folds_into_product = True

    def __init__(self, ctx: BuildContext, *, width: int, eps: float, name: str | None = None) -> None:
        self.width = width
        self.eps = float(eps)
        self.name = name if name is not None else f"{ctx.prefix}.weight"
        self.weight = None

    def param_specs(self):
        return [ParamSpec.single("weight", self.name, (self.width,), role="vector", init="around_one")]

    def forward(self, x):
        return kernels.rms_norm(x, self.weight, self.eps)

    def add(self, x, residual):
        """(norm(x + residual), x + residual)"""
        return kernels.rms_norm(x, self.weight, self.eps, residual=residual)

    def add_rows(self, x, residual, rows):
        """norm(x + residual) on the rows named by ``rows`` only."""
        return kernels.rms_norm(x, self.weight, self.eps, residual=residual, rows=rows)


class PendingUpdate:
    """What a block left for the next norm to add to the float32 stream: norm(y + row_scale * x), with ``norm`` a
    :class:`StreamRMSNorm` (or None: y + row_scale * x as it is) and the scaled term optional.  It rides on the
    stream tensor as ``stream.pending``; whoever norms the stream next adds it in the same pass."""

    __slots__ = ("y", "norm", "row_scale", "x")

    def __init__(self, y, norm=None, row_scale=None, x=None) -> None:
        self.y, self.norm, self.row_scale, self.x = y, norm, row_scale, x


class StreamRMSNorm(Part):
    """RMSNorm in front of a float32 residual stream: y = s * rsqrt(mean(s^2) + eps) * weight with
    statistics, scaling and the product with the weight in float32 and one rounding, to the
    storage type, at the end.  ``add`` first forms s = residual + x in float32 (x may be of the
    storage type or float32) and keeps s, in place, as the new stream.  The stream is float32
    also where activations and weights are bfloat16."""

    def __init__(self, ctx: BuildContext, *, width: int, eps: float, name: str | None = None,
                 unit_offset: bool = False) -> None:
        self.width = width
        self.eps = float(eps)
        self.name = name if name is not None else f"{ctx.prefix}.weight"
        self.out_dtype = ctx.dtype
        self.unit_offset = bool(unit_offset)   # the checkpoint stores w around zero and the norm multiplies by 1 + w
        self.weight = None

    def param_specs(self):
        return [ParamSpec.single("weight", self.name, (self.width,), role="vector",
                                 init="normal" if self.unit_offset else "around_one")]

    def finalize(self) -> None:
        if self.unit_offset and self.weight is not None and not getattr(self, "_offset_applied", False):
            self.weight = (self.weight.to(torch.float32) + 1.0).contiguous()      # 1 + w, once, in float32
            self._offset_applied = True

    def start(self, x):
        """norm(x) in float32: the first tensor of a float32 stream (a normed embedding)."""
        if x.dtype == torch.float32:
            return kernels.stream_norm(x, self.weight, self.eps, out_dtype=torch.float32, rows=None)[0]
        return kernels.stream_norm(None, self.weight, self.eps, add=x, out_dtype=torch.float32)[0]

    def forward(self, x):
        """norm(x) for a float32 stream or for activations that start one."""
        if getattr(x, "pending", None) is not None:
            return self.resume(x)[0]
        if x.dtype == torch.float32:
            return kernels.stream_norm(x, self.weight, self.eps, out_dtype=self.out_dtype)[0]
        return kernels.stream_norm(None, self.weight, self.eps, add=x, out_dtype=self.out_dtype)[0]

    def resume(self, stream, rows=None):
        """(norm(s'), s') with s' = stream + what the block before left pending on it (:class:`PendingUpdate`:
        a sublayer's output with a norm of its own behind it), in one pass; the stream is updated in place and
        nothing is pending afterwards.  With ``rows`` only those rows of the result, and nothing is written."""
        pending = stream.pending
        post = pending.norm
        out, updated = kernels.sandwich_norm(
            stream, pending.y, post_weight=None if post is None else post.weight,
            post_eps=0.0 if post is None else post.eps, pre_weight=self.weight, pre_eps=self.eps,
            row_scale=pending.row_scale, x=pending.x, rows=rows, out_dtype=self.out_dtype)
        if rows is None:
            stream.pending = None
        return out, updated

    def after(self, stream, y, following=None, row_scale=None, x=None):
        """This norm behind a sublayer: (following(s'), s') with s' = stream + norm(y + row_scale * x), the stream
        updated in place; ``following`` is the norm in front of the next sublayer (None: no first result)."""
        return kernels.sandwich_norm(
            stream, y, post_weight=self.weight, post_eps=self.eps,
            pre_weight=None if following is None else following.weight,
            pre_eps=0.0 if following is None else following.eps, row_scale=row_scale, x=x,
            out_dtype=self.out_dtype)

    def add(self, x, residual):
        """(norm(residual + x), residual + x); without a residual x starts the stream, without x
        the stream holds the sum already."""
        if residual is not None and residual.dtype != torch.float32:
            raise kernels.KernelError("this norm keeps its residual stream in float32")
        return kernels.stream_norm(residual, self.weight, self.eps, add=x, out_dtype=self.out_dtype)

    def add_rows(self, x, residual, rows):
        """norm(residual + x) on the rows named by ``rows`` only; nothing is written back."""
        if residual is None and x.dtype == torch.float32:
            x, residual = None, x
        if x is None and getattr(residual, "pending", None) is not None:
            return self.resume(residual, rows=rows)[0]
        return kernels.stream_norm(residual, self.weight, self.eps, add=x, rows=rows,
                                   out_dtype=self.out_dtype)[0]


class StreamLayerNorm(Part):
    """Layer norm with a weight and no bias over a float32 residual stream, for blocks that norm after
    the sum: out = (s - mean(s)) / sqrt(mean((s - mean)^2) + eps) * weight with s = alpha * x + y, all
    in float32.  ``post`` returns (out rounded once to the storage type, out in float32): the first
    feeds the next products, the second is the stream.  In the float32 path both are one tensor."""

    def __init__(self, ctx: BuildContext, *, width: int, eps: float, name: str | None = None,
                 optional: bool = False) -> None:
        self.width = width
        self.eps = float(eps)
        self.name = name if name is not None else f"{ctx.prefix}.weight"
        self.out_dtype = ctx.dtype
        self.optional = optional          # the checkpoint may lack the weight: ``weight`` stays None
        self.weight = None

    def param_specs(self):
        return [ParamSpec.single("weight", self.name, (self.width,), role="vector", init="around_one",
                                 optional=self.optional)]

    def post(self, x, y, alpha: float = 1.0):
        """(LN(alpha * x + y) in the storage type, the same in float32); y may be None."""
        return kernels.post_layer_norm(x, self.weight, self.eps, alpha=alpha, add=y, out_dtype=self.out_dtype)

    def forward(self, x):
        return self.post(x, None)[0]

    def add(self, x, residual):
        """(LN(residual + x), the same in float32)."""
        if residual is None:
            return self.post(x, None)
        return self.post(residual, x)

    def add_rows(self, x, residual, rows):
        """LN(residual + x) on the rows named by ``rows`` only (x alone without a residual)."""
        if residual is None:
            x, residual = None, x
        return kernels.post_layer_norm(residual, self.weight, self.eps, add=x, rows=rows,
                                       out_dtype=self.out_dtype)[0]


register_part("norm", "rms_norm", RMSNorm)
register_part("norm", "layer_norm_stream32", StreamLayerNorm)
register_part("norm", "rms_norm_stream32", StreamRMSNorm)
