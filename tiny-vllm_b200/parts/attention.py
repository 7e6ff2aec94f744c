"""Grouped-query attention over the paged cache, with per-head q/k RMSNorm.

qkv = x . Wqkv^T packed as [q | k | v] (tinyvllm/models/qwen3.py:230-240,
:273-280); q and k are normalised per head and rotated, k and v go to their
cache pages (:284-299; tinyvllm/kernels/kv_store.cu:26-90); every query attends
the keys of its request up to its own position, at most ``window`` of them
(tinyvllm/runtime/attention.py:34-55; tinyvllm/kernels/paged_decode.cu:85-466);
then the output projection (:303).  All sizes, the scale, the eps and the window
are parameters; the position encoding is a part of its own.
"""

from __future__ import annotations

import torch

from ..ops import attention as attention_ops
from ..ops import kernels, linear, linear_into_stream, linear_norm
from .base import BuildContext, KVNeed, ParamSpec, Part
from .registry import register_part


class GQAAttention(Part):
    def __init__(self, ctx: BuildContext, *, hidden_size: int, num_heads: int, num_kv_heads: int,
                 head_dim: int, scale: float, qk_norm_eps: float | None, window: int | None,
                 position=None, names: dict | None = None) -> None:
        if num_heads % num_kv_heads:
            raise ValueError("query heads must be a multiple of key-value heads")
        if head_dim % 16 or head_dim > 256:
            raise ValueError(f"the attention kernels take head sizes in steps of 16 up to 256, not {head_dim}")
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.scale = float(scale)
        self.qk_norm_eps = qk_norm_eps
        self.window = window
        self.prefix = ctx.prefix
        n = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
             "q_norm": "q_norm.weight", "k_norm": "k_norm.weight", **(names or {})}
        self.names = {key: f"{ctx.prefix}.{value}" for key, value in n.items()}
        self.position = ctx.build("position", position, ctx) if position is not None else None
        self.qkv_weight = self.o_weight = self.q_norm_weight = self.k_norm_weight = None

    # ------------------------------------------------------------ declaration
    def param_specs(self):
        q_rows, kv_rows = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        specs = [
            ParamSpec.packed("qkv_weight", [(self.names["q"], q_rows), (self.names["k"], kv_rows),
                                            (self.names["v"], kv_rows)], self.hidden_size),
            ParamSpec.single("o_weight", self.names["o"], (self.hidden_size, q_rows)),
        ]
        if self.qk_norm_eps is not None:
            specs += [
                ParamSpec.single("q_norm_weight", self.names["q_norm"], (self.head_dim,),
                                 role="vector", init="around_one"),
                ParamSpec.single("k_norm_weight", self.names["k_norm"], (self.head_dim,),
                                 role="vector", init="around_one"),
            ]
        return specs

    def children(self):
        return [self.position] if self.position is not None else []

    def streamed_weights(self):
        return [self.qkv_weight, self.o_weight]

    def cache_need(self):
        return KVNeed(self.num_kv_heads, self.head_dim, self.window)

    def takes_tensor_memory_tiles(self, page_size: int) -> bool:
        """Whether this mixer's prefill may run on the tcgen05 tile kernel; the step cuts its
        tile lists for that kernel only if every mixer of the model says so."""
        return kernels.attention_prefill_tc_supports(self.head_dim, self.num_heads, self.num_kv_heads,
                                                     page_size)

    def scratch_floats(self, rows: int, chunks: int) -> int:
        """float32 scratch the row kernel asks for when it spreads ``chunks`` key chunks of
        ``rows`` single tokens over the grid."""
        return kernels.attention_rows_scratch_floats(rows, self.num_heads, self.head_dim, chunks)

    # ---------------------------------------------------------------- running
    def forward(self, x, ctx, run: int):
        qkv = linear(x, self.qkv_weight)
        attended = attention_ops.mixer_attention(ctx, self, qkv, run)
        return linear(attended, self.o_weight)

    def forward_normed(self, hidden, residual, norm, ctx, run: int):
        """forward(norm(hidden + residual)) and the new residual stream; the output is None when
        the output projection has added it to the stream itself."""
        qkv, residual = linear_norm(hidden, residual, norm, self.qkv_weight)
        attended = attention_ops.mixer_attention(ctx, self, qkv, run)
        return linear_into_stream(attended, self.o_weight, residual)


def distance_buckets(rows: int, far: float) -> list[int]:
    """The bucket of every distance 0 .. ceil(far): n itself below rows / 2, then logarithmic steps that
    reach the last bucket, rows - 1, at ``far``; evaluated in double precision."""
    import math

    half = rows // 2
    buckets = []
    for n in range(int(math.ceil(far)) + 1):
        if n < half:
            buckets.append(n)
        else:
            step = int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half)))
            buckets.append(min(rows - 1, half + step))
    return buckets


class WindowedAttention(Part):
    """Grouped-query attention with every size and step a parameter.

    Keys (``key_dim``) and values (``value_dim``) may differ in size.  ``qk_norm``: None, "unit"
    (q and k divided by their root mean square over the head, no weight) or "weight" (with
    tensors ``q_norm`` / ``k_norm``); ``position``: a position part whose ``inv_freq``, ``rot_dims``
    and ``pairing`` the preparing kernel applies to q and k, or None (positions then do not enter
    the scores).  ``window``: query i sees the keys j with 0 <= i - j < window, and with
    ``keep_first`` also the keys j < keep_first.  ``gate``: the concatenated heads are multiplied
    by sigmoid(W_g x) before the output projection.  ``value_mix``: "first" hands this layer's
    values on to the later layers of the step under ``value_mix_key``; "blend" replaces v by
    (1 - l) v + l v_first, with the scalar tensor ``vmix`` as l, before it is cached.

    ``qk_norm="whole"``: q and k are divided by their root mean square over the whole projection,
    all heads at once, and multiplied by weights of that size (``q_norm`` / ``k_norm``).
    ``query_temperature`` (coef, every): q at position p is multiplied by 1 + coef * ln(floor((p + 1) /
    every) + 1).  ``distance_slope_exponent`` = c: head h takes 2^(-c (h + 1) / heads) * (i - j) off
    the score of key j for query i.  ``sink``: a learned number a head (tensor ``sink``) whose
    exponential is added to the softmax's denominator and to nothing else.  ``gate="head"``:
    the gate is one number a head, sigmoid(W_g x)_h with W_g [heads, width].  ``float32_output``: the
    output projection leaves its float32 sums unrounded (for a float32 residual sum).

    ``qk_bias``: q and k have biases (tensors ``q_bias`` / ``k_bias``), added to the projection in float32
    before anything else.  ``values_are_keys``: there is no value projection; a token's values are its
    keys as projected (bias included), before their norm and rotation.  ``distance_table`` (rows, far):
    a learned number a head and distance bucket (tensor ``rel`` [rows, heads]; a checkpoint's tensor
    decides ``rows`` by its shape) is added to the scaled score; distance n < rows / 2 has the bucket n, a larger one min(rows - 1, rows / 2 + floor(ln(n /
    (rows / 2)) / ln(far / (rows / 2)) * (rows - rows / 2))).  ``segment``: the positions form segments
    of so many, counted from position 0, and a query sees only the keys of its own.  ``sink`` may also be
    a number: a sink of that fixed score for every head.

    ``hosted=True``: a block computes the input projections of all its parts as one product and
    the output projections as another; the mixer then owns no matrices, names its share
    (``input_rows``, ``output_cols``) and works between the two products (``between``)."""

    def __init__(self, ctx: BuildContext, *, hidden_size: int, num_heads: int, num_kv_heads: int,
                 key_dim: int, value_dim: int, scale: float, window: int | None = None,
                 keep_first: int = 0, qk_norm: str | None = None, qk_norm_eps: float = 0.0,
                 position=None, gate: bool | str = False, value_mix: str | None = None,
                 value_mix_key: str = "v_first", names: dict | None = None, hosted: bool = False,
                 query_temperature: tuple | None = None, distance_slope_exponent: float | None = None,
                 sink: bool | float = False, float32_output: bool = False, qk_bias: bool = False,
                 values_are_keys: bool = False, distance_table: tuple | None = None,
                 segment: int | None = None) -> None:
        if num_heads % num_kv_heads:
            raise ValueError("query heads must be a multiple of key-value heads")
        limit = kernels.ATTENTION_ROWS_MAX_DIM
        if not 0 < key_dim <= limit or not 0 < value_dim <= limit:
            raise ValueError(f"the attention kernels take key and value sizes up to {limit}, not {key_dim} / {value_dim}")
        if qk_norm not in (None, "unit", "weight", "whole"):
            raise ValueError(f"qk_norm is None, 'unit', 'weight' or 'whole', not {qk_norm!r}")
        if gate not in (False, True, "head"):
            raise ValueError(f"gate is False, True or 'head', not {gate!r}")
        if query_temperature is not None and qk_norm != "whole":
            raise ValueError("the query temperature is applied by the norm over the whole projection")
        if value_mix not in (None, "first", "blend"):
            raise ValueError(f"value_mix is None, 'first' or 'blend', not {value_mix!r}")
        if window is not None and window <= 0:
            raise ValueError("a window holds at least one key")
        if keep_first < 0:
            raise ValueError("keep_first must not be negative")
        if values_are_keys and (value_dim != key_dim or value_mix is not None):
            raise ValueError("values that are the keys have the keys' size and are not blended")
        if segment is not None and segment <= 0:
            raise ValueError("a segment holds at least one position")
        if distance_table is not None:
            # the checkpoint's table decides the rows (finalize checks those against ``far``); the count given
            # here only sizes random weights, and gives way where ``far`` lies inside its linear half
            rows, far = int(distance_table[0]), float(distance_table[1])
            if rows < 2 or not far > 1.0:
                raise ValueError("a distance table has at least two rows and reaches beyond distance 1")
            while rows > 2 and not far > rows // 2:
                rows -= 1
            distance_table = (rows, far)
        self.qk_bias, self.values_are_keys = bool(qk_bias), bool(values_are_keys)
        self.distance_table, self.segment = distance_table, segment
        self.hidden_size = hidden_size
        self.num_heads, self.num_kv_heads = num_heads, num_kv_heads
        self.key_dim, self.value_dim = key_dim, value_dim
        self.scale = float(scale)
        self.window = window
        self.keep_first = keep_first if window is not None else 0
        self.qk_norm, self.qk_norm_eps = qk_norm, float(qk_norm_eps)
        self.gate = gate
        self.value_mix, self.value_mix_key = value_mix, value_mix_key
        self.hosted = hosted
        self.query_temperature = None if query_temperature is None else (float(query_temperature[0]),
                                                                          int(query_temperature[1]))
        if self.query_temperature is not None and self.query_temperature[1] <= 0:
            raise ValueError("the query temperature's period must be positive")
        self.distance_slope_exponent = None if distance_slope_exponent is None else float(distance_slope_exponent)
        self.has_sink = sink is True
        self.fixed_sink = None if isinstance(sink, bool) else float(sink)
        self.out_dtype = torch.float32 if float32_output else None
        self.device = ctx.device
        self.slopes = self.sinks = self.sink = None
        self.q_bias = self.k_bias = self.rel = self.bias_table = None
        n = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "vmix": "vmix", "q_norm": "q_norm",
             "k_norm": "k_norm", "sink": "sink", "q_bias": "q.b", "k_bias": "k.b", "rel": "rel", **(names or {})}
        self.names = {key: f"{ctx.prefix}.{value}" for key, value in n.items()}
        self.position = ctx.build("position", position, ctx) if position is not None else None
        self.in_weight = self.o_weight = self.vmix = self.q_norm_weight = self.k_norm_weight = None

    # ------------------------------------------------------------ declaration
    @property
    def q_cols(self) -> int:
        return self.num_heads * self.key_dim

    @property
    def k_cols(self) -> int:
        return self.num_kv_heads * self.key_dim

    @property
    def v_cols(self) -> int:
        """Columns of the value projection (none when the values are the keys)."""
        return 0 if self.values_are_keys else self.num_kv_heads * self.value_dim

    @property
    def out_cols(self) -> int:
        return self.num_heads * self.value_dim

    @property
    def gate_cols(self) -> int:
        return 0 if not self.gate else self.num_heads if self.gate == "head" else self.out_cols

    @property
    def plain(self) -> bool:
        """No distance bias, no sink, a gate (if any) of one number a value, keys and values apart:
        what the tensor-core kernels of the windowed attention take."""
        return (self.distance_slope_exponent is None and not self.has_sink and self.fixed_sink is None
                and self.gate != "head" and self.distance_table is None and self.segment is None)

    def input_rows(self):
        """(checkpoint tensor, rows) of the input projections, in the order of their columns:
        q heads, k heads, v heads and, with a gate, the gate."""
        rows = [(self.names["q"], self.q_cols), (self.names["k"], self.k_cols)]
        if not self.values_are_keys:
            rows.append((self.names["v"], self.v_cols))
        if self.gate:
            rows.append((self.names["g"], self.gate_cols))
        return rows

    def output_cols(self):
        return (self.names["o"], self.out_cols)

    def param_specs(self):
        specs = []
        if not self.hosted:
            specs += [ParamSpec.packed("in_weight", self.input_rows(), self.hidden_size),
                      ParamSpec.single("o_weight", self.names["o"], (self.hidden_size, self.out_cols))]
        if self.value_mix is not None:
            # every layer that takes part stores the scalar; the one that hands its values on ignores it
            specs.append(ParamSpec.scalar("vmix", self.names["vmix"]))
        if self.qk_norm == "weight":
            specs += [ParamSpec.single("q_norm_weight", self.names["q_norm"], (self.key_dim,),
                                       role="vector", init="around_one"),
                      ParamSpec.single("k_norm_weight", self.names["k_norm"], (self.key_dim,),
                                       role="vector", init="around_one")]
        if self.qk_norm == "whole":
            specs += [ParamSpec.single("q_norm_weight", self.names["q_norm"], (self.q_cols,),
                                       role="vector", init="around_one"),
                      ParamSpec.single("k_norm_weight", self.names["k_norm"], (self.k_cols,),
                                       role="vector", init="around_one")]
        if self.has_sink:
            specs.append(ParamSpec.single("sink", self.names["sink"], (self.num_heads,), role="vector"))
        if self.qk_bias:
            specs += [ParamSpec.single("q_bias", self.names["q_bias"], (self.q_cols,), role="vector"),
                      ParamSpec.single("k_bias", self.names["k_bias"], (self.k_cols,), role="vector")]
        if self.distance_table is not None:
            # the table's own shape says how many buckets there are; distance_table[0] only sizes random weights
            specs.append(ParamSpec.single("rel", self.names["rel"], (self.distance_table[0], self.num_heads),
                                          role="table", free_rows=True))
        return specs

    def finalize(self) -> None:
        """The per-head constants of the attention kernels, float32 on the device."""
        if self.distance_slope_exponent is not None:
            heads = torch.arange(1, self.num_heads + 1, dtype=torch.float64)
            self.slopes = (2.0 ** (-self.distance_slope_exponent * heads / self.num_heads)).to(
                torch.float32).to(self.device)
        if self.has_sink and self.sink is not None:
            self.sinks = self.sink.to(torch.float32).contiguous()
        if self.fixed_sink is not None:
            self.sinks = torch.full((self.num_heads,), self.fixed_sink, dtype=torch.float32, device=self.device)
        if self.qk_bias and self.q_bias is not None:
            self.q_bias = self.q_bias.to(torch.float32).contiguous()
            self.k_bias = self.k_bias.to(torch.float32).contiguous()
        if self.distance_table is not None and self.rel is not None:
            # one row a distance: the kernels read table[min(distance, rows - 1)], and every distance from
            # ``far`` on has the last bucket
            if self.rel.shape[0] < 2 or not self.distance_table[1] > self.rel.shape[0] // 2:
                raise ValueError("a distance table has at least two rows and reaches beyond its linear half")
            buckets = distance_buckets(self.rel.shape[0], self.distance_table[1])
            index = torch.tensor(buckets, dtype=torch.long, device=self.rel.device)
            self.bias_table = self.rel.to(torch.float32).index_select(0, index).contiguous()

    def children(self):
        return [self.position] if self.position is not None else []

    def streamed_weights(self):
        return [] if self.hosted else [self.in_weight, self.o_weight]

    def cache_need(self):
        return KVNeed(self.num_kv_heads, self.key_dim, self.window, self.value_dim, self.keep_first)

    def takes_tensor_memory_tiles(self, page_size: int) -> bool:
        return False

    def scratch_floats(self, rows: int, chunks: int) -> int:
        """float32 scratch for ``rows`` single tokens whose keys span ``chunks`` chunks: what the row
        kernel or the tensor-core kernel for single tokens asks for, whichever is more."""
        span = chunks * kernels.attention_chunk_keys()
        return max(kernels.attention_rows_scratch_floats(rows, self.num_heads, self.value_dim, chunks),
                   kernels.attention_tiles_singles_floats(rows, self.num_heads, self.value_dim,
                                                          self.segment or self.window, self.keep_first, span))

    # ---------------------------------------------------------------- running
    def between(self, projected, at: int, ctx, out, run: int) -> None:
        """From this mixer's columns of a projection (from ``at`` on) to the gated, concatenated
        heads in ``out``; writes the step's keys and values."""
        attention_ops.windowed_attention(ctx, self, projected, at, run, out)

    def forward(self, x, ctx, run: int):
        projected = linear(x, self.in_weight)
        attended = torch.empty((x.shape[0], self.out_cols), dtype=x.dtype, device=x.device)
        self.between(projected, 0, ctx, attended, run)
        return linear(attended, self.o_weight, out_dtype=self.out_dtype)


class LatentAttention(Part):
    """Attention whose queries, keys and values come through low-rank latents.

    c_q = RMSnorm(W_dq x) (weight ``dq.norm``), q = W_uq c_q, a head being [``key_dim`` plain |
    ``rot_dim`` rotated] dimensions.  W_dkv x has ``kv_rank + rot_dim`` rows: the first, RMS-normed
    (weight ``dkv.norm``), are the latent c, the rest one rotated key part that all heads share.  A
    head's plain key is W_uk c and its value W_uv c; the score is (q_plain . k_plain + q_rot . k_rot) *
    scale, softmax over the causal keys.  The concatenated heads are multiplied by sigmoid(W_g x)
    (``gate``) and projected by W_o.  ``window``: query i sees the keys j with 0 <= i - j < window.  ``sink``: a
    learned number a head (tensor ``sink``) whose exponential is added to the softmax's denominator and to
    nothing else.  ``gate="head"``: the gate is one number a head, sigmoid(W_g x)_h with W_g [heads, width].  The
    rotated part turns as neighbouring pairs or as pairs of its two halves, as the position part says.

    Only [c | rotated key part] is cached, as one key row a token of one kv head.  The up-projections
    never touch the cache: W_uk is folded into the query (q_plain^T W_uk is a query over c itself,
    so every head attends rows [c | k_rot] with the query [W_uk^T q_plain | q_rot]), the attention's
    values are the first ``kv_rank`` elements of the same rows, and W_uv is applied to the attended
    latent afterwards, a head at a time."""

    def __init__(self, ctx: BuildContext, *, hidden_size: int, num_heads: int, key_dim: int, rot_dim: int,
                 value_dim: int, q_rank: int, kv_rank: int, scale: float, eps: float, position=None,
                 gate: bool | str = True, float32_output: bool = False, names: dict | None = None,
                 window: int | None = None, sink: bool = False) -> None:
        if gate not in (False, True, "head"):
            raise ValueError(f"gate is False, True or 'head', not {gate!r}")
        if window is not None and window <= 0:
            raise ValueError("a window holds at least one key")
        if rot_dim % 2:
            raise ValueError("the rotated part of a head has an even size")
        if (rot_dim > 0) != (position is not None):
            raise ValueError("a rotated part needs a position part, and only then")
        if kv_rank + rot_dim > kernels.ATTENTION_ROWS_MAX_DIM:
            raise ValueError(f"latent and rotated part together may hold up to {kernels.ATTENTION_ROWS_MAX_DIM} "
                             f"elements, not {kv_rank + rot_dim}")
        self.hidden_size, self.num_heads = hidden_size, num_heads
        self.key_dim, self.rot_dim, self.value_dim = key_dim, rot_dim, value_dim
        self.q_rank, self.kv_rank = q_rank, kv_rank
        self.scale, self.eps = float(scale), float(eps)
        self.gate = gate
        self.window, self.has_sink = window, bool(sink)
        self.sink = self.sinks = None
        self.out_dtype = torch.float32 if float32_output else None
        n = {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk",
             "uv": "uv", "g": "g", "o": "o", "sink": "sink", **(names or {})}
        self.names = {key: f"{ctx.prefix}.{value}" for key, value in n.items()}
        self.position = ctx.build("position", position, ctx) if position is not None else None
        if self.position is not None and (getattr(self.position, "pairing", None) not in ("interleaved", "half_split")
                                          or not hasattr(self.position, "inv_freq")
                                          or self.position.rot_dims != rot_dim):
            raise ValueError("the rotated part is turned over its whole size, by position * frequency")
        self.in_weight = self.uq_weight = self.uk_weight = self.uv_weight = self.o_weight = None
        self.dq_norm_weight = self.dkv_norm_weight = None
        self.uk_by_head = self.uv_by_head = None

    @property
    def out_cols(self) -> int:
        return self.num_heads * self.value_dim

    @property
    def row_dim(self) -> int:
        """Size of a cached row: the latent and the rotated key part."""
        return self.kv_rank + self.rot_dim

    @property
    def gate_cols(self) -> int:
        return 0 if not self.gate else self.num_heads if self.gate == "head" else self.out_cols

    def param_specs(self):
        rows = [(self.names["dq"], self.q_rank), (self.names["dkv"], self.row_dim)]
        if self.gate:
            rows.append((self.names["g"], self.gate_cols))
        sink = [ParamSpec.single("sink", self.names["sink"], (self.num_heads,), role="vector")] if self.has_sink else []
        return sink + [
            ParamSpec.packed("in_weight", rows, self.hidden_size),
            ParamSpec.single("dq_norm_weight", self.names["dq_norm"], (self.q_rank,), role="vector", init="around_one"),
            ParamSpec.single("dkv_norm_weight", self.names["dkv_norm"], (self.kv_rank,), role="vector",
                             init="around_one"),
            ParamSpec.single("uq_weight", self.names["uq"], (self.num_heads * (self.key_dim + self.rot_dim), self.q_rank)),
            ParamSpec.single("uk_weight", self.names["uk"], (self.num_heads * self.key_dim, self.kv_rank)),
            ParamSpec.single("uv_weight", self.names["uv"], (self.out_cols, self.kv_rank)),
            ParamSpec.single("o_weight", self.names["o"], (self.hidden_size, self.out_cols)),
        ]

    def children(self):
        return [self.position] if self.position is not None else []

    def finalize(self) -> None:
        """The up-projections a head at a time, as the head products read them: W_uk transposed
        ([heads, kv_rank, key_dim]: the product with it folds W_uk into the query), W_uv as it is."""
        self.uk_by_head = self.uk_weight.view(self.num_heads, self.key_dim, self.kv_rank).transpose(1, 2).contiguous()
        self.uv_by_head = self.uv_weight.view(self.num_heads, self.value_dim, self.kv_rank)
        if self.has_sink and self.sink is not None:
            self.sinks = self.sink.to(torch.float32).contiguous()

    def streamed_weights(self):
        return [self.in_weight, self.uq_weight, self.o_weight]

    def cache_need(self):
        return KVNeed(1, self.row_dim, self.window, self.kv_rank, 0, value_offset=0)

    def takes_tensor_memory_tiles(self, page_size: int) -> bool:
        return False

    def scratch_floats(self, rows: int, chunks: int) -> int:
        span = chunks * kernels.attention_chunk_keys()
        return max(kernels.attention_rows_scratch_floats(rows, self.num_heads, self.kv_rank, chunks),
                   kernels.attention_tiles_singles_floats(rows, self.num_heads, self.kv_rank, self.window, 0, span))

    def forward(self, x, ctx, run: int):
        projected = linear(x, self.in_weight)
        gated = attention_ops.latent_attention(ctx, self, projected, run)
        return linear(gated, self.o_weight, out_dtype=self.out_dtype)


register_part("mixer", "gqa_attention", GQAAttention)
register_part("mixer", "latent_attention", LatentAttention)
register_part("mixer", "windowed_attention", WindowedAttention)
