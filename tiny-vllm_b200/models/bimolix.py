"""Bimolix: typed configuration and its description as parts.

A decoder whose config.json lists its layers one by one.  The embedding is normed at once; a layer is
x <- x + mixer(norm1(x)), then, where it has a feed-forward, x <- x + ff(norm2(x)); the norms are RMS
norms whose stored weight w multiplies as 1 + w, and the stream x is float32 also in the bfloat16 path.
A layer with ``weights_of: j`` has no tensors of its own: it runs layer j's parts again, with a state
or cache of its own.  Two mixers:

``retention``  linear attention with a fixed decay a head (``decay``), no softmax and no denominator: a
               float32 state [dim, vdim] a head runs along a request's tokens.  q and k are rotated
               (halves paired, ``rot.dims`` dimensions, ``rot.base``), k is multiplied by dim^(-1/2); every
               head's output is divided by its root mean square, the heads are multiplied by silu(W_g h).
``attention``  grouped-query attention whose values are the keys as projected (no value projection): q
               and k have biases and a weighted RMS norm a head; no rotation; a learned bias a head and
               distance bucket (``rel``, logarithmic buckets up to ``bias_max``) is added to the scaled score;
               a query sees only the keys of its own chunk of ``mask.size`` positions; the softmax has
               one more term of score 0 in its denominator; the heads are multiplied by sigmoid(W_g h).

The feed-forward is dense, down(silu(gate h) * (up h)), or a mixture of gated experts with sigmoid
routing, a choice correction, groups of experts and a gated shared expert, or absent.  All of it maps
onto parts of the package with these numbers as parameters; nothing here computes.

Checkpoint names: ``embed``, ``embed.norm``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.{q,k,v,g,o}`` or
``l<i>.mix.{q,q.b,k,k.b,q.norm,k.norm,rel,g,o}``, ``l<i>.mlp.{gate,up,down}`` or ``l<i>.mlp.{router,
correction,e<j>.gate,e<j>.up,e<j>.down,shared.gate,shared.up,shared.down,shared.sg}``, ``final.norm``, ``head``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from ..config.registry import ConfigError, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunStep

MIXER_TYPES = ("retention", "attention")
# the experts' activation is g * sigmoid(EXPERT_ALPHA * g) * (u + 1)
EXPERT_ALPHA = 1.702
# the score of the softmax's extra term
SINK_SCORE = 0.0
# positions enter through computed angles, distances and chunk numbers, none tabulated: the engine's own
# max_model_len bounds a request
UNBOUNDED_POSITIONS = 1 << 20
# rows of a distance table where no checkpoint says (random weights): a checkpoint's ``rel`` tensor decides
DEFAULT_DISTANCE_ROWS = 32


def _positive_int(name: str, value: Any) -> int:
    if type(value) is not int or value <= 0:
        raise ConfigError(f"{name} must be a positive integer, got {value!r}")
    return value


def _number(name: str, value: Any) -> float:
    if type(value) not in (int, float):
        raise ConfigError(f"{name} must be a number, got {value!r}")
    return float(value)


def _need(where: str, data: Any, keys) -> Mapping[str, Any]:
    if not isinstance(data, Mapping):
        raise ConfigError(f"{where} must be an object")
    missing = [key for key in keys if key not in data]
    if missing:
        raise ConfigError(f"{where} lacks " + ", ".join(missing))
    return data


@dataclass(frozen=True)
class BimolixFeedForward:
    kind: str                              # "dense" or "moe"
    ff: int                                # dense: the inner size; moe: an expert's
    limit: float = 0.0                     # moe from here on
    experts: int = 0
    top: int = 0
    route_scale: float = 1.0
    groups: int = 1
    keep: int = 1
    shared_ff: int = 0                     # 0: no shared expert
    shared_limit: float = 0.0

    def __post_init__(self) -> None:
        if self.kind not in ("dense", "moe"):
            raise ConfigError(f"mlp.kind is 'dense' or 'moe', not {self.kind!r}")
        _positive_int("mlp.ff", self.ff)
        if self.kind == "moe":
            _positive_int("mlp.router.experts", self.experts)
            _positive_int("mlp.router.top", self.top)
            _positive_int("mlp.router.groups.count", self.groups)
            _positive_int("mlp.router.groups.keep", self.keep)
            if self.top > self.experts:
                raise ConfigError("mlp.router.top must not exceed mlp.router.experts")
            if self.experts % self.groups or self.keep > self.groups:
                raise ConfigError("mlp.router.groups must divide the experts, and keep at most all groups")
            if type(self.shared_ff) is not int or self.shared_ff < 0:
                raise ConfigError("mlp.shared.ff must be a non-negative integer")

    @classmethod
    def from_json(cls, where: str, data: Any) -> "BimolixFeedForward":
        data = _need(where, data, ("kind",))
        if data["kind"] == "dense":
            return cls(kind="dense", ff=_need(where, data, ("ff",))["ff"])
        if data["kind"] != "moe":
            raise ConfigError(f"{where}.kind is 'dense' or 'moe', not {data['kind']!r}")
        data = _need(where, data, ("expert", "router"))
        expert = _need(f"{where}.expert", data["expert"], ("ff", "limit"))
        router = _need(f"{where}.router", data["router"], ("experts", "top"))
        groups = router.get("groups")
        count = keep = 1
        if groups is not None:
            groups = _need(f"{where}.router.groups", groups, ("count", "keep"))
            count, keep = groups["count"], groups["keep"]
        shared = data.get("shared")
        shared_ff, shared_limit = 0, 0.0
        if shared is not None:
            shared = _need(f"{where}.shared", shared, ("ff", "limit"))
            shared_ff, shared_limit = shared["ff"], _number("mlp.shared.limit", shared["limit"])
        return cls(kind="moe", ff=expert["ff"], limit=_number("mlp.expert.limit", expert["limit"]),
                   experts=router["experts"], top=router["top"],
                   route_scale=_number("mlp.router.scale", router.get("scale", 1.0)), groups=count, keep=keep,
                   shared_ff=shared_ff, shared_limit=shared_limit)

    def to_json(self) -> dict[str, Any]:
        if self.kind == "dense":
            return {"ff": self.ff, "kind": "dense"}
        data: dict[str, Any] = {
            "expert": {"ff": self.ff, "limit": self.limit}, "kind": "moe",
            "router": {"experts": self.experts, "groups": {"count": self.groups, "keep": self.keep},
                       "scale": self.route_scale, "top": self.top}}
        if self.shared_ff:
            data["shared"] = {"ff": self.shared_ff, "limit": self.shared_limit}
        return data


@dataclass(frozen=True)
class BimolixLayer:
    type: str
    heads: int
    dim: int
    vdim: int
    decay: tuple[float, ...] = ()          # retention
    rot_dims: int = 0                      # retention: 0 for no rotation
    rot_base: float = 0.0
    kv_heads: int = 1                      # attention from here on
    scale: float = 1.0
    bias_max: float = 0.0
    chunk: int | None = None
    mlp: BimolixFeedForward | None = None
    weights_of: int | None = None
    rel_rows: int = DEFAULT_DISTANCE_ROWS  # not in config.json: the rows random weights give ``rel``

    def __post_init__(self) -> None:
        if self.type not in MIXER_TYPES:
            raise ConfigError(f"a layer's type is one of {', '.join(MIXER_TYPES)}, not {self.type!r}")
        for name in ("heads", "dim", "vdim", "kv_heads"):
            _positive_int(f"mixer.{name}", getattr(self, name))
        if self.type == "retention":
            if len(self.decay) != self.heads:
                raise ConfigError("mixer.decay must list one number a head")
            if type(self.rot_dims) is not int or self.rot_dims < 0 or self.rot_dims % 2 or self.rot_dims > self.dim:
                raise ConfigError("mixer.rot.dims must be even and at most mixer.dim")
            if self.rot_dims and not self.rot_base > 0:
                raise ConfigError("mixer.rot.base must be positive")
        else:
            if self.heads % self.kv_heads:
                raise ConfigError("mixer.heads must be a multiple of mixer.kv_heads")
            if self.vdim != self.dim:
                raise ConfigError("mixer.vdim must equal mixer.dim: the values are the keys")
            if self.chunk is not None:
                _positive_int("mixer.mask.size", self.chunk)

    @classmethod
    def from_json(cls, index: int, data: Any) -> "BimolixLayer":
        where = f"layers[{index}]"
        data = _need(where, data, ("type", "mixer"))
        kind = data["type"]
        mlp = data.get("mlp")
        feed_forward = None if mlp is None else BimolixFeedForward.from_json(f"{where}.mlp", mlp)
        weights_of = data.get("weights_of")
        if weights_of is not None and (type(weights_of) is not int or not 0 <= weights_of < index):
            raise ConfigError(f"{where}.weights_of must name an earlier layer")
        if kind == "retention":
            mixer = _need(f"{where}.mixer", data["mixer"], ("heads", "dim", "vdim", "decay"))
            rot = mixer.get("rot")
            rot_dims, rot_base = 0, 0.0
            if rot is not None:
                rot = _need(f"{where}.mixer.rot", rot, ("dims", "base"))
                rot_dims, rot_base = rot["dims"], _number("mixer.rot.base", rot["base"])
            if not isinstance(mixer["decay"], list):
                raise ConfigError(f"{where}.mixer.decay must be a list")
            return cls(type=kind, heads=mixer["heads"], dim=mixer["dim"], vdim=mixer["vdim"],
                       decay=tuple(_number("mixer.decay", d) for d in mixer["decay"]), rot_dims=rot_dims,
                       rot_base=rot_base, mlp=feed_forward, weights_of=weights_of)
        if kind == "attention":
            mixer = _need(f"{where}.mixer", data["mixer"], ("heads", "kv_heads", "dim", "vdim", "scale", "bias_max"))
            mask = mixer.get("mask")
            chunk = None if mask is None else _need(f"{where}.mixer.mask", mask, ("size",))["size"]
            return cls(type=kind, heads=mixer["heads"], kv_heads=mixer["kv_heads"], dim=mixer["dim"],
                       vdim=mixer["vdim"], scale=_number("mixer.scale", mixer["scale"]),
                       bias_max=_number("mixer.bias_max", mixer["bias_max"]), chunk=chunk, mlp=feed_forward,
                       weights_of=weights_of)
        raise ConfigError(f"{where}.type is one of {', '.join(MIXER_TYPES)}, not {kind!r}")

    def to_json(self) -> dict[str, Any]:
        if self.type == "retention":
            mixer: dict[str, Any] = {"decay": list(self.decay), "dim": self.dim, "heads": self.heads, "vdim": self.vdim}
            if self.rot_dims:
                mixer["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        else:
            mixer = {"bias_max": self.bias_max, "dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads,
                     "scale": self.scale, "vdim": self.vdim}
            if self.chunk is not None:
                mixer["mask"] = {"size": self.chunk}
        data = {"mixer": mixer, "mlp": None if self.mlp is None else self.mlp.to_json(), "type": self.type}
        if self.weights_of is not None:
            data["weights_of"] = self.weights_of
        return data


@dataclass(frozen=True)
class BimolixConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple[BimolixLayer, ...]
    eos_token_ids: tuple[int, ...] = ()

    architecture = "Bimolix"

    def __post_init__(self) -> None:
        _positive_int("vocab", self.vocab)
        _positive_int("width", self.width)
        if not self.norm_eps > 0:
            raise ConfigError("norm.eps must be positive")
        if not self.layers:
            raise ConfigError("a model needs at least one layer")
        for index, layer in enumerate(self.layers):
            if layer.weights_of is not None and self.layers[self.owner(index)].type != layer.type:
                raise ConfigError(f"layers[{index}] uses the weights of a layer with another mixer")

    def owner(self, index: int) -> int:
        """The layer whose tensors layer ``index`` runs with (itself, unless it names another)."""
        while self.layers[index].weights_of is not None:
            index = self.layers[index].weights_of
        return index

    @classmethod
    def from_json(cls, data: Mapping[str, Any]) -> "BimolixConfig":
        missing = [key for key in ("vocab", "width", "norm", "layers") if key not in data]
        if missing:
            raise ConfigError("missing config.json keys: " + ", ".join(missing))
        norm = data["norm"]
        if not isinstance(norm, Mapping) or "eps" not in norm:
            raise ConfigError("config.json 'norm' must give 'eps'")
        if not isinstance(data["layers"], list):
            raise ConfigError("config.json 'layers' must be a list")
        eos = data.get("eos_token_id")
        eos_ids = () if eos is None else (eos,) if type(eos) is int else tuple(eos)
        return cls(vocab=data["vocab"], width=data["width"], norm_eps=_number("norm.eps", norm["eps"]),
                   layers=tuple(BimolixLayer.from_json(i, layer) for i, layer in enumerate(data["layers"])),
                   eos_token_ids=eos_ids)

    def to_json(self) -> dict[str, Any]:
        data: dict[str, Any] = {"architecture": self.architecture,
                                "layers": [layer.to_json() for layer in self.layers],
                                "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.eos_token_ids:
            data["eos_token_id"] = list(self.eos_token_ids)
        return data

    # ------------------------------------------------------------------ spec
    def _mixer_spec(self, layer: BimolixLayer) -> PartSpec:
        if layer.type == "retention":
            position = None
            if layer.rot_dims:
                position = PartSpec("rope_half_split_computed", {"dims": layer.rot_dims, "base": layer.rot_base})
            return PartSpec("retention", {
                "hidden_size": self.width, "num_heads": layer.heads, "key_dim": layer.dim,
                "value_dim": layer.vdim, "decay": layer.decay, "key_scale": float(layer.dim) ** -0.5,
                "position": position, "unit_norm": True, "eps": self.norm_eps, "gate": "silu",
                "float32_output": True})
        return PartSpec("windowed_attention", {
            "hidden_size": self.width, "num_heads": layer.heads, "num_kv_heads": layer.kv_heads,
            "key_dim": layer.dim, "value_dim": layer.vdim, "scale": layer.scale, "window": None,
            "qk_norm": "weight", "qk_norm_eps": self.norm_eps, "qk_bias": True, "values_are_keys": True,
            "distance_table": (layer.rel_rows, layer.bias_max), "segment": layer.chunk,
            "sink": SINK_SCORE, "gate": True, "float32_output": True,
            "names": {"q_norm": "q.norm", "k_norm": "k.norm"}})

    def _feed_forward_spec(self, mlp: BimolixFeedForward | None) -> PartSpec | None:
        if mlp is None:
            return None
        if mlp.kind == "dense":
            return PartSpec("gated_mlp", {
                "hidden_size": self.width, "intermediate_size": mlp.ff, "activation": "silu",
                "float32_output": True, "names": {"gate": "gate", "up": "up", "down": "down"}})
        return PartSpec("gated_routed_experts", {
            "hidden_size": self.width, "experts": mlp.experts, "top": mlp.top, "ff": mlp.ff, "limit": mlp.limit,
            "alpha": EXPERT_ALPHA, "route_scale": mlp.route_scale, "correction": True, "groups": mlp.groups,
            "keep": mlp.keep, "shared_ff": mlp.shared_ff, "shared_limit": mlp.shared_limit,
            "shared_gate": bool(mlp.shared_ff), "float32_output": True})

    def to_spec(self) -> ModelSpec:
        norm = PartSpec("rms_norm_stream32", {"width": self.width, "eps": self.norm_eps, "unit_offset": True})
        block = PartSpec("prenorm_residual", {"mixer_norm_name": "norm1", "feed_forward_norm_name": "norm2",
                                              "mixer_name": "mix", "feed_forward_name": "mlp",
                                              "bare_norm_names": True})
        # layers that own tensors become layers of the spec; one that names another's is a further run of
        # that layer, with a state or cache of its own
        spec_index: dict[int, int] = {}
        layers = []
        for index, layer in enumerate(self.layers):
            if layer.weights_of is not None:
                continue
            spec_index[index] = len(layers)
            layers.append(LayerSpec(prefix=f"l{index}", block=block, mixer=self._mixer_spec(layer),
                                    feed_forward=self._feed_forward_spec(layer.mlp), norm=norm))
        order = tuple(RunStep(spec_index[self.owner(index)]) for index in range(len(self.layers)))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width,
            max_positions=UNBOUNDED_POSITIONS,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "width": self.width, "name": "embed",
                                                   "norm": norm.with_params(name="embed.norm")}),
            layers=tuple(layers), order=order, final_norm=norm.with_params(name="final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "width": self.width, "tied_to": None,
                                      "name": "head"}),
            eos_token_ids=self.eos_token_ids)


register_architecture(BimolixConfig.architecture, BimolixConfig)
