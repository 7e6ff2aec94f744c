"""Retention: linear attention with a fixed decay a head, no softmax and no denominator.

q = W_q h and k = W_k h (``num_heads`` heads of ``key_dim``), v = W_v h (heads of ``value_dim``), no
biases.  A position part (or none) turns the first dimensions of every q and k head; k is then
multiplied by ``key_scale``.  Per head and request a float32 state S [key_dim, value_dim] runs along the
tokens: S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t.  With ``unit_norm`` every head's o is divided
by its root mean square (``eps`` inside the root, no weight); the concatenated heads are multiplied by
act(W_g h) (``gate``: "silu", "sigmoid" or None for no gate) and projected by W_o.

The state is the mixer's whole memory: a slot a request in the cache storage's state arena, zero when
the request starts, read at the start of every step and left as the state after the step's last
token.  Angles, rotated q and k, outer products, state and sums are float32 whatever the storage type.
"""

from __future__ import annotations

import torch

from ..ops import kernels, linear
from .base import BuildContext, ParamSpec, Part, StateNeed
from .registry import register_part


class Retention(Part):
    def __init__(self, ctx: BuildContext, *, hidden_size: int, num_heads: int, key_dim: int, value_dim: int,
                 decay, key_scale: float | None = None, position=None, unit_norm: bool = True, eps: float = 0.0,
                 gate: str | None = "silu", float32_output: bool = False, names: dict | None = None) -> None:
        decay = [float(d) for d in decay]
        if len(decay) != num_heads:
            raise ValueError(f"retention wants one decay a head: {num_heads}, not {len(decay)}")
        if not 0 < key_dim <= kernels.RETENTION_MAX_DIM or value_dim <= 0:
            raise ValueError(f"retention takes key sizes up to {kernels.RETENTION_MAX_DIM}, not {key_dim}")
        if gate not in kernels.RETENTION_ACTS:
            raise ValueError(f"gate is 'silu', 'sigmoid' or None, not {gate!r}")
        self.hidden_size, self.num_heads = hidden_size, num_heads
        self.key_dim, self.value_dim = key_dim, value_dim
        self.decay_values = decay
        self.key_scale = float(key_dim) ** -0.5 if key_scale is None else float(key_scale)
        self.unit_norm, self.eps = bool(unit_norm), float(eps)
        self.gate = gate
        self.out_dtype = torch.float32 if float32_output else None
        self.device = ctx.device
        n = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", **(names or {})}
        self.names = {key: f"{ctx.prefix}.{value}" for key, value in n.items()}
        self.position = ctx.build("position", position, ctx) if position is not None else None
        if self.position is not None and (not hasattr(self.position, "inv_freq")
                                          or getattr(self.position, "magnitude", 1.0) != 1.0
                                          or self.position.rot_dims > key_dim):
            raise ValueError("retention turns q and k by position * frequency over at most the head's size")
        self.in_weight = self.o_weight = self.decay = None

    # ------------------------------------------------------------ declaration
    @property
    def qk_cols(self) -> int:
        return self.num_heads * self.key_dim

    @property
    def out_cols(self) -> int:
        return self.num_heads * self.value_dim

    def param_specs(self):
        rows = [(self.names["q"], self.qk_cols), (self.names["k"], self.qk_cols), (self.names["v"], self.out_cols)]
        if self.gate is not None:
            rows.append((self.names["g"], self.out_cols))
        return [ParamSpec.packed("in_weight", rows, self.hidden_size),
                ParamSpec.single("o_weight", self.names["o"], (self.hidden_size, self.out_cols))]

    def children(self):
        return [self.position] if self.position is not None else []

    def finalize(self) -> None:
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=self.device)

    def streamed_weights(self):
        return [self.in_weight, self.o_weight]

    def cache_need(self):
        return StateNeed((self.num_heads, self.key_dim, self.value_dim), torch.float32)

    def takes_tensor_memory_tiles(self, page_size: int) -> bool:
        return True                  # no attention over pages: any cutting of a step into tiles will do

    # ---------------------------------------------------------------- running
    def forward(self, x, ctx, run: int):
        projected = linear(x, self.in_weight)
        position = self.position
        v_at = 2 * self.qk_cols
        gated = kernels.retention(
            projected, q_at=0, k_at=self.qk_cols, v_at=v_at,
            g_at=v_at + self.out_cols if self.gate is not None else None, heads=self.num_heads,
            dim=self.key_dim, vdim=self.value_dim, decay=self.decay, state=ctx.storage.state_of(run),
            row_starts=ctx.row_starts, state_slots=ctx.state_slots, token_row=ctx.token_row,
            positions=ctx.positions, inv_freq=None if position is None else position.inv_freq,
            rot_dims=0 if position is None else position.rot_dims,
            pairing="half_split" if position is None else position.pairing, key_scale=self.key_scale,
            unit_norm=self.unit_norm, eps=self.eps, gate_act=self.gate)
        return linear(gated, self.o_weight, out_dtype=self.out_dtype)


class GatedRecurrence(Part):
    """A linear recurrence with a gate a token, head and key channel: a channel keeps its state times the gate and
    writes with one minus the gate.

    q = act(W_q h) (``query_act``: "silu" or None; ``num_heads`` heads of ``key_dim``), v = W_v h (heads of
    ``value_dim``), and the gate g = l + (1 - l) * sigmoid(W_f h + b), with a bias b (``gate_bias``) and a lower
    bound l (``lower_bound``: a stored vector of heads * key_dim numbers below which the gate never falls).
    Per head and request a float32 state S [key_dim, value_dim] runs along the tokens: S_t = diag(g_t) S_(t-1)
    + (1 - g_t) v_t^T, o_t = S_t^T q_t: there is no key of its own, what a channel does not keep it writes.
    Every head's o is divided by its root mean square (``eps`` inside the root) and multiplied by one weight
    of ``value_dim`` numbers that all heads share (``out_norm``: "weight", "unit" for no weight, None for no
    norm); the concatenated heads are projected by W_o.

    The state is the mixer's whole memory: a slot a request in the cache storage's state arena, zero when the
    request starts, read at the start of every step and left as the state after the step's last token.
    Gates, products, state and sums are float32 whatever the storage type."""

    def __init__(self, ctx: BuildContext, *, hidden_size: int, num_heads: int, key_dim: int, value_dim: int,
                 query_act: str | None = "silu", gate_bias: bool = True, lower_bound: bool = True,
                 out_norm: str | None = "weight", eps: float = 0.0, float32_output: bool = False,
                 names: dict | None = None) -> None:
        if not 0 < key_dim <= kernels.RETENTION_MAX_DIM or value_dim <= 0:
            raise ValueError(f"the recurrence takes key sizes up to {kernels.RETENTION_MAX_DIM}, not {key_dim}")
        if query_act not in kernels.GATED_QUERY_ACTS:
            raise ValueError(f"query_act is 'silu' or None, not {query_act!r}")
        if out_norm not in (None, "unit", "weight"):
            raise ValueError(f"out_norm is None, 'unit' or 'weight', not {out_norm!r}")
        self.hidden_size, self.num_heads = hidden_size, num_heads
        self.key_dim, self.value_dim = key_dim, value_dim
        self.query_act, self.has_bias, self.has_lower = query_act, bool(gate_bias), bool(lower_bound)
        self.out_norm, self.eps = out_norm, float(eps)
        self.out_dtype = torch.float32 if float32_output else None
        n = {"q": "q", "f": "f", "f_bias": "f.b", "lower": "lower", "v": "v", "norm": "norm", "o": "o", **(names or {})}
        self.names = {key: f"{ctx.prefix}.{value}" for key, value in n.items()}
        self.in_weight = self.o_weight = self.gate_bias = self.lower = self.norm_weight = None

    @property
    def qk_cols(self) -> int:
        return self.num_heads * self.key_dim

    @property
    def out_cols(self) -> int:
        return self.num_heads * self.value_dim

    def param_specs(self):
        rows = [(self.names["q"], self.qk_cols), (self.names["f"], self.qk_cols), (self.names["v"], self.out_cols)]
        specs = [ParamSpec.packed("in_weight", rows, self.hidden_size),
                 ParamSpec.single("o_weight", self.names["o"], (self.hidden_size, self.out_cols))]
        if self.has_bias:
            specs.append(ParamSpec.single("gate_bias", self.names["f_bias"], (self.qk_cols,), role="vector"))
        if self.has_lower:
            specs.append(ParamSpec.single("lower", self.names["lower"], (self.qk_cols,), role="vector",
                                          init="unit_interval"))
        if self.out_norm == "weight":
            specs.append(ParamSpec.single("norm_weight", self.names["norm"], (self.value_dim,), role="vector",
                                          init="around_one"))
        return specs

    def finalize(self) -> None:
        for attr in ("gate_bias", "lower", "norm_weight"):
            tensor = getattr(self, attr)
            if tensor is not None:
                setattr(self, attr, tensor.to(torch.float32).contiguous())

    def streamed_weights(self):
        return [self.in_weight, self.o_weight]

    def cache_need(self):
        return StateNeed((self.num_heads, self.key_dim, self.value_dim), torch.float32)

    def takes_tensor_memory_tiles(self, page_size: int) -> bool:
        return True                  # no attention over pages: any cutting of a step into tiles will do

    def forward(self, x, ctx, run: int):
        projected = linear(x, self.in_weight)
        normed = kernels.gated_recurrence(
            projected, q_at=0, g_at=self.qk_cols, v_at=2 * self.qk_cols, heads=self.num_heads, dim=self.key_dim,
            vdim=self.value_dim, state=ctx.storage.state_of(run), row_starts=ctx.row_starts,
            state_slots=ctx.state_slots, token_row=ctx.token_row, bias=self.gate_bias, lower=self.lower,
            query_act=self.query_act, unit_norm=self.out_norm is not None, norm_weight=self.norm_weight,
            eps=self.eps)
        return linear(normed, self.o_weight, out_dtype=self.out_dtype)


register_part("mixer", "retention", Retention)
register_part("mixer", "gated_recurrence", GatedRecurrence)
