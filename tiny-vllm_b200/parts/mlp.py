"""Dense gated feed-forward: down(act(gate(x)) * up(x)), no biases; act is SiLU (SwiGLU) or the
tanh form of GELU.

gate and up are one packed projection [gate | up]
(tinyvllm/models/qwen3.py:316-346; activation tinyvllm/kernels/pointwise.cu:274-285).

A block that computes the input projections of all its parts as one product, and their output
projections as one product too, builds the part with ``hosted=True``: the part then declares no
matrices of its own, tells the block which checkpoint tensors make up its share
(``input_rows``, ``output_cols``) and only turns its columns of the common projection into
its columns of the common input of the output product (``between``).
"""

from __future__ import annotations

import torch

from ..ops import kernels, linear, linear_into_stream, linear_norm, linear_silu
from .base import BuildContext, ParamSpec, Part
from .registry import register_part


class SwiGLU(Part):
    def __init__(self, ctx: BuildContext, *, hidden_size: int, intermediate_size: int,
                 names: dict | None = None, activation: str = "silu", hosted: bool = False,
                 float32_output: bool = False) -> None:
        if activation not in kernels.ACTIVATIONS:
            raise ValueError(f"activation is one of {', '.join(kernels.ACTIVATIONS)}, not {activation!r}")
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.activation = activation
        self.hosted = hosted
        # the down projection leaves its float32 sums unrounded (for a float32 residual sum)
        self.out_dtype = torch.float32 if float32_output else None
        n = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight",
             **(names or {})}
        self.names = {key: f"{ctx.prefix}.{value}" for key, value in n.items()}
        self.gate_up_weight = self.down_weight = None

    def param_specs(self):
        if self.hosted:
            return []
        return [
            ParamSpec.packed("gate_up_weight", [(self.names["gate"], self.intermediate_size),
                                                (self.names["up"], self.intermediate_size)],
                             self.hidden_size),
            ParamSpec.single("down_weight", self.names["down"],
                             (self.hidden_size, self.intermediate_size)),
        ]

    def streamed_weights(self):
        return [] if self.hosted else [self.gate_up_weight, self.down_weight]

    # ------------------------------------------------- as a guest of a block
    def input_rows(self):
        """(checkpoint tensor, rows) of the input projections, in the order of their columns."""
        return [(self.names["gate"], self.intermediate_size), (self.names["up"], self.intermediate_size)]

    def output_cols(self):
        """(checkpoint tensor, columns) of the output projection."""
        return (self.names["down"], self.intermediate_size)

    def between(self, projected, at: int, ctx, out) -> None:
        """act(gate) * up from the columns ``at ...`` of the common projection into ``out``."""
        kernels.gated_act(projected, at, at + self.intermediate_size, self.intermediate_size,
                          self.activation, out=out)

    # ------------------------------------------------------------ on its own
    def _activated(self, x):
        if self.activation == "silu":
            return linear_silu(x, self.gate_up_weight)
        return kernels.gated_act(linear(x, self.gate_up_weight), 0, self.intermediate_size,
                                 self.intermediate_size, self.activation)

    def forward(self, x, ctx):
        return linear(self._activated(x), self.down_weight, out_dtype=self.out_dtype)

    def forward_normed(self, hidden, residual, norm, ctx):
        """forward(norm(hidden + residual)) and the new residual stream; the output is None when
        the down projection has added it to the stream itself."""
        if self.activation != "silu" or self.out_dtype is not None:
            if hidden is None:
                x = norm.forward(residual)
            elif residual is None:
                x, residual = norm.forward(hidden), hidden
            else:
                x, residual = norm.add(hidden, residual)
            return self.forward(x, ctx), residual
        activated, residual = linear_norm(hidden, residual, norm, self.gate_up_weight, silu=True)
        return linear_into_stream(activated, self.down_weight, residual)


register_part("feed_forward", "swiglu", SwiGLU)
register_part("feed_forward", "gated_mlp", SwiGLU)


class RoutedExperts(Part):
    """A mixture of small feed-forward experts, down_e(act(up_e h)), without biases.

    Router logits z = W_router h are float32; each token uses the ``top`` experts with the largest
    logits, weighted by the softmax over those logits alone; a shared expert of the same form (size
    ``shared_ff``, 0 for none) runs for every token and is added.

    The experts' up-projections are the rows of one weight [experts * ff + shared_ff, width] and their
    down-projections stand side by side in one weight [width, experts * ff + shared_ff]: between the
    two products one kernel picks the experts, turns their logits into weights and stores act(up) *
    weight (0 for experts that were not chosen), so that the second product is the weighted sum of
    the chosen experts' outputs plus the shared expert's, accumulated in float32.  Every token pays
    for all experts' columns: the form for few, small experts."""

    def __init__(self, ctx: BuildContext, *, hidden_size: int, experts: int, top: int, ff: int,
                 shared_ff: int = 0, activation: str = "relu_squared", float32_output: bool = False,
                 names: dict | None = None) -> None:
        if activation not in kernels.EXPERT_ACTIVATIONS:
            raise ValueError(f"activation is one of {', '.join(kernels.EXPERT_ACTIVATIONS)}, not {activation!r}")
        if not 0 < top <= experts or experts > kernels.ROUTE_MAX_EXPERTS:
            raise ValueError(f"a token uses between 1 and all of at most {kernels.ROUTE_MAX_EXPERTS} experts")
        self.hidden_size, self.experts, self.top, self.ff, self.shared_ff = hidden_size, experts, top, ff, shared_ff
        self.activation = activation
        self.out_dtype = torch.float32 if float32_output else None
        n = {"router": "router", "expert": "e{index}", "shared": "shared", "up": "up", "down": "down",
             **(names or {})}
        self.router_name = f"{ctx.prefix}.{n['router']}"
        stems = [f"{ctx.prefix}.{n['expert'].format(index=index)}" for index in range(experts)]
        if shared_ff:
            stems.append(f"{ctx.prefix}.{n['shared']}")
        sizes = [ff] * experts + ([shared_ff] if shared_ff else [])
        self.up_sources = [(f"{stem}.{n['up']}", size) for stem, size in zip(stems, sizes)]
        self.down_sources = [(f"{stem}.{n['down']}", size) for stem, size in zip(stems, sizes)]
        self.router_weight = self.up_weight = self.down_weight = None

    def param_specs(self):
        return [ParamSpec.single("router_weight", self.router_name, (self.experts, self.hidden_size)),
                ParamSpec.packed("up_weight", self.up_sources, self.hidden_size),
                ParamSpec.side_by_side("down_weight", self.hidden_size, self.down_sources)]

    def streamed_weights(self):
        return [self.up_weight, self.down_weight]

    def forward(self, x, ctx):
        logits = linear(x, self.router_weight, out_dtype=torch.float32)
        inner = kernels.route_act(logits, linear(x, self.up_weight), experts=self.experts, top=self.top,
                                  ff=self.ff, shared_ff=self.shared_ff, activation=self.activation)
        return linear(inner, self.down_weight, out_dtype=self.out_dtype)


register_part("feed_forward", "routed_experts", RoutedExperts)


class GatedRoutedExperts(Part):
    """A mixture of gated experts with sigmoid routing, without biases.

    An expert: g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit), y = g * sigmoid(alpha * g) *
    (u + 1), output W_down y.  Router logits z = W_router h are float32, the scores s = sigmoid(z).  A token
    uses the ``top`` experts with the largest choice scores s + correction (tensor ``correction``, with
    ``correction=True``); the experts form ``groups`` equal groups of neighbours, a group's score is the
    sum of its two largest choice scores, and only experts of the ``keep`` best groups can be chosen.  The
    chosen experts' weights are their scores s divided by their sum (+ 1e-20), times ``route_scale``.  A
    shared expert of the same form (``shared_ff`` wide, 0 for none, with ``shared_limit``) runs for every
    token and is added, multiplied by sigmoid(W_sg h), one number a token (``shared_gate``).

    As in :class:`RoutedExperts` the experts are two products: [gate_e | up_e] of all experts and of the
    shared one are the rows of one weight, the down-projections stand side by side in another, and one
    kernel between the two routes, activates and weights (exactly 0 for experts not chosen).  The
    router's rows and the shared expert's gate row are one small float32-result product."""

    def __init__(self, ctx: BuildContext, *, hidden_size: int, experts: int, top: int, ff: int, limit: float,
                 alpha: float, route_scale: float = 1.0, correction: bool = False, groups: int = 1, keep: int = 1,
                 shared_ff: int = 0, shared_limit: float | None = None, shared_gate: bool = False,
                 float32_output: bool = False, names: dict | None = None) -> None:
        if not 0 < top <= experts or experts > kernels.ROUTE_MAX_EXPERTS:
            raise ValueError(f"a token uses between 1 and all of at most {kernels.ROUTE_MAX_EXPERTS} experts")
        if groups <= 0 or experts % groups or not 0 < keep <= groups:
            raise ValueError("experts form equal groups of which at least one and at most all are kept")
        if shared_gate and not shared_ff:
            raise ValueError("a gate of the shared expert needs a shared expert")
        self.hidden_size, self.experts, self.top, self.ff, self.shared_ff = hidden_size, experts, top, ff, shared_ff
        self.limit, self.alpha, self.route_scale = float(limit), float(alpha), float(route_scale)
        self.shared_limit = float(limit if shared_limit is None else shared_limit)
        self.has_correction, self.groups, self.keep, self.shared_gate = bool(correction), groups, keep, bool(shared_gate)
        self.out_dtype = torch.float32 if float32_output else None
        n = {"router": "router", "correction": "correction", "expert": "e{index}", "shared": "shared",
             "gate": "gate", "up": "up", "down": "down", "shared_gate": "sg", **(names or {})}
        self.router_sources = [(f"{ctx.prefix}.{n['router']}", experts)]
        if shared_gate:
            self.router_sources.append((f"{ctx.prefix}.{n['shared']}.{n['shared_gate']}", 1))
        self.correction_name = f"{ctx.prefix}.{n['correction']}"
        stems = [f"{ctx.prefix}.{n['expert'].format(index=index)}" for index in range(experts)]
        if shared_ff:
            stems.append(f"{ctx.prefix}.{n['shared']}")
        sizes = [ff] * experts + ([shared_ff] if shared_ff else [])
        self.in_sources = [(f"{stem}.{n[which]}", size) for stem, size in zip(stems, sizes) for which in ("gate", "up")]
        self.down_sources = [(f"{stem}.{n['down']}", size) for stem, size in zip(stems, sizes)]
        self.router_weight = self.in_weight = self.down_weight = self.correction = None

    def param_specs(self):
        specs = [ParamSpec.packed("router_weight", self.router_sources, self.hidden_size),
                 ParamSpec.packed("in_weight", self.in_sources, self.hidden_size),
                 ParamSpec.side_by_side("down_weight", self.hidden_size, self.down_sources)]
        if self.has_correction:
            specs.append(ParamSpec.single("correction", self.correction_name, (self.experts,), role="vector"))
        return specs

    def finalize(self) -> None:
        if self.correction is not None:
            self.correction = self.correction.to(torch.float32).contiguous()

    def streamed_weights(self):
        return [self.in_weight, self.down_weight]

    def forward(self, x, ctx):
        logits = linear(x, self.router_weight, out_dtype=torch.float32)
        inner = kernels.route_gated_act(
            logits, linear(x, self.in_weight), experts=self.experts, top=self.top, ff=self.ff,
            shared_ff=self.shared_ff, limit=self.limit, shared_limit=self.shared_limit, alpha=self.alpha,
            route_scale=self.route_scale, correction=self.correction, groups=self.groups, keep=self.keep,
            shared_gated=self.shared_gate)
        return linear(inner, self.down_weight, out_dtype=self.out_dtype)


register_part("feed_forward", "gated_routed_experts", GatedRoutedExperts)


class SoftmaxRoutedExperts(Part):
    """A mixture of gated experts, down_e(silu(gate_e h) * (up_e h)), routed by a softmax over all slots, some of
    which may hand their input on unchanged.

    Router logits z = W_router h are float32 and have ``experts + identity`` entries; the scores are s =
    softmax(z) over all of them.  A token uses the ``top`` slots with the largest choice scores s + correction
    (tensor ``correction``, with ``correction=True``; the weights use s without it), weighted by s as it is
    (``renormalise``: divided by the sum of the chosen scores).  The last ``identity`` slots are experts without
    tensors whose output is h itself.

    As in :class:`RoutedExperts` the experts are two products: [gate_e | up_e] of all experts are the rows of
    one weight, the down-projections stand side by side in another, and one kernel between the two routes,
    activates and weights (exactly 0 for experts not chosen).  The pass-through slots cost one number a token:
    the sum of their weights, times which h is added (``forward``), or which a norm kernel behind the part adds
    for it (``forward_carried``)."""

    def __init__(self, ctx: BuildContext, *, hidden_size: int, experts: int, top: int, ff: int, identity: int = 0,
                 correction: bool = False, renormalise: bool = False, float32_output: bool = False,
                 names: dict | None = None) -> None:
        if experts <= 0 or identity < 0 or experts + identity > kernels.ROUTE_MAX_EXPERTS or not 0 < top <= experts + identity:
            raise ValueError(f"a token uses between 1 and all of at most {kernels.ROUTE_MAX_EXPERTS} slots")
        self.hidden_size, self.experts, self.identity, self.top, self.ff = hidden_size, experts, identity, top, ff
        self.has_correction, self.renormalise = bool(correction), bool(renormalise)
        self.out_dtype = torch.float32 if float32_output else None
        n = {"router": "router", "correction": "correction", "expert": "e{index}", "gate": "gate", "up": "up",
             "down": "down", **(names or {})}
        self.router_name = f"{ctx.prefix}.{n['router']}"
        self.correction_name = f"{ctx.prefix}.{n['correction']}"
        stems = [f"{ctx.prefix}.{n['expert'].format(index=index)}" for index in range(experts)]
        self.in_sources = [(f"{stem}.{n[which]}", ff) for stem in stems for which in ("gate", "up")]
        self.down_sources = [(f"{stem}.{n['down']}", ff) for stem in stems]
        self.router_weight = self.in_weight = self.down_weight = self.correction = None

    @property
    def slots(self) -> int:
        return self.experts + self.identity

    def param_specs(self):
        specs = [ParamSpec.single("router_weight", self.router_name, (self.slots, self.hidden_size)),
                 ParamSpec.packed("in_weight", self.in_sources, self.hidden_size),
                 ParamSpec.side_by_side("down_weight", self.hidden_size, self.down_sources)]
        if self.has_correction:
            specs.append(ParamSpec.single("correction", self.correction_name, (self.slots,), role="vector"))
        return specs

    def finalize(self) -> None:
        if self.correction is not None:
            self.correction = self.correction.to(torch.float32).contiguous()

    def streamed_weights(self):
        return [self.in_weight, self.down_weight]

    def forward_carried(self, x, ctx):
        """(y, row_scale): the part's output is y + row_scale[:, None] * x; ``row_scale`` (float32 [tokens], the
        weights of the chosen pass-through slots) is None where the part has no such slots."""
        logits = linear(x, self.router_weight, out_dtype=torch.float32)
        inner, passed = kernels.route_softmax_gated(
            logits, linear(x, self.in_weight), experts=self.experts, identity=self.identity, top=self.top,
            ff=self.ff, correction=self.correction, renormalise=self.renormalise)
        return linear(inner, self.down_weight, out_dtype=self.out_dtype), passed

    def forward(self, x, ctx):
        y, passed = self.forward_carried(x, ctx)
        if passed is None:
            return y
        if y.dtype != torch.float32:
            raise kernels.KernelError("experts that hand their input on leave a float32 result (float32_output)")
        return kernels.add_scaled_rows(y, x, passed)


register_part("feed_forward", "softmax_routed_experts", SoftmaxRoutedExperts)
