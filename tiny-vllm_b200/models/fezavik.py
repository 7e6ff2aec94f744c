"""Fezavik: typed configuration and its description as parts.

A decoder whose config.json lists its layers one by one.  A layer norms before and behind each sublayer,
x <- x + norm1b(mixer(norm1(x))), then, where it has a feed-forward, x <- x + norm2b(ff(norm2(x))); the norms
are RMS norms with plain weights and the stream x is float32 also in the bfloat16 path.  Three mixers:

``attention``         grouped-query attention: q and k are RMS-normed over the whole projection (weights of
                      that size), then the first ``rot.dims`` dimensions of every head turn as neighbouring
                      pairs (``rot.base``; ``rot.scaling`` slows the long waves down, by wavelength bands);
                      a sliding window of ``mask.size`` keys; the softmax's denominator holds a learned sink
                      a head
``latent_attention``  queries through a latent of ``q_rank``, keys and values through one of ``kv_rank``; a
                      head is ``dim`` plain and ``rot_dim`` rotated dimensions (the halves of the rotated
                      part are paired), the rotated key part is shared by all heads; window and sink as
                      above; every head's output is multiplied by one gate number, sigmoid(W_g x)_h
``hgrn2``             a linear recurrence a head with a gate a key channel that never falls below a stored
                      bound; a channel keeps its state times the gate and writes the value times one minus
                      the gate (there is no key); q = silu(W_q x); every head's output is RMS-normed with
                      one weight for all heads

The feed-forward is a mixture of gated SiLU experts routed by a softmax over all slots, with a choice
correction and without renormalising the chosen weights; the last ``router.identity`` slots hand their
input on unchanged.  All of it maps onto parts of the package with these numbers as parameters; nothing here
computes.

Checkpoint names: ``embed``, ``l<i>.norm1``, ``l<i>.norm1b``, ``l<i>.norm2``, ``l<i>.norm2b``,
``l<i>.mix.{q,k,v,q.norm,k.norm,sink,o}`` or ``l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,sink,g,o}`` or
``l<i>.mix.{q,f,f.b,lower,v,norm,o}``, ``l<i>.mlp.{router,correction,e<j>.gate,e<j>.up,e<j>.down}``,
``final.norm``, ``head``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from ..config.registry import ConfigError, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunStep

MIXER_TYPES = ("attention", "latent_attention", "hgrn2")
# positions enter through computed angles and distances, none tabulated: the engine's own max_model_len
# bounds a request
UNBOUNDED_POSITIONS = 1 << 20
SCALING_KEYS = ("factor", "low", "high", "original")


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
class FezavikRotation:
    dims: int
    base: float
    scaling: tuple[float, float, float, float] | None = None      # (factor, low, high, original)

    def __post_init__(self) -> None:
        if type(self.dims) is not int or self.dims <= 0 or self.dims % 2:
            raise ConfigError("rot.dims must be an even, positive integer")
        if not self.base > 0:
            raise ConfigError("rot.base must be positive")
        if self.scaling is not None:
            factor, low, high, original = self.scaling
            if not (factor > 0 and 0 < low < high and original > 0):
                raise ConfigError("rot.scaling wants a positive factor and original length and 0 < low < high")

    @classmethod
    def from_json(cls, where: str, data: Any) -> "FezavikRotation":
        data = _need(where, data, ("dims", "base"))
        scaling = data.get("scaling")
        if scaling is not None:
            scaling = _need(f"{where}.scaling", scaling, SCALING_KEYS)
            scaling = tuple(_number(f"{where}.scaling.{key}", scaling[key]) for key in SCALING_KEYS)
        return cls(dims=data["dims"], base=_number(f"{where}.base", data["base"]), scaling=scaling)

    def to_json(self) -> dict[str, Any]:
        data: dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            data["scaling"] = dict(zip(SCALING_KEYS, self.scaling))
        return data

    def to_spec(self, kind: str) -> PartSpec:
        scaling = None if self.scaling is None else dict(zip(SCALING_KEYS, self.scaling))
        return PartSpec(kind, {"dims": self.dims, "base": self.base, "scaling": scaling})


@dataclass(frozen=True)
class FezavikExperts:
    experts: int
    top: int
    ff: int
    identity: int = 0                  # slots behind the experts that hand their input on

    def __post_init__(self) -> None:
        for name in ("experts", "top", "ff"):
            _positive_int(f"mlp.{name}", getattr(self, name))
        if type(self.identity) is not int or self.identity < 0:
            raise ConfigError("mlp.router.identity must be a non-negative integer")
        if self.top > self.experts + self.identity:
            raise ConfigError("mlp.router.top must not exceed the router's slots")

    @classmethod
    def from_json(cls, where: str, data: Any) -> "FezavikExperts":
        data = _need(where, data, ("kind", "expert", "router"))
        if data["kind"] != "moe":
            raise ConfigError(f"{where}.kind must be 'moe', not {data['kind']!r}")
        expert = _need(f"{where}.expert", data["expert"], ("ff",))
        router = _need(f"{where}.router", data["router"], ("experts", "top"))
        return cls(experts=router["experts"], top=router["top"], ff=expert["ff"], identity=router.get("identity", 0))

    def to_json(self) -> dict[str, Any]:
        return {"expert": {"ff": self.ff}, "kind": "moe",
                "router": {"experts": self.experts, "identity": self.identity, "top": self.top}}


@dataclass(frozen=True)
class FezavikLayer:
    type: str
    heads: int
    dim: int
    vdim: int
    scale: float = 1.0                 # the two attention mixers from here on
    window: int | None = None
    rot: FezavikRotation | None = None
    kv_heads: int = 1                  # attention
    q_rank: int | None = None          # latent_attention
    kv_rank: int | None = None
    rot_dim: int = 0
    mlp: FezavikExperts | None = None

    def __post_init__(self) -> None:
        if self.type not in MIXER_TYPES:
            raise ConfigError(f"a layer's type is one of {', '.join(MIXER_TYPES)}, not {self.type!r}")
        for name in ("heads", "dim", "vdim", "kv_heads"):
            _positive_int(f"mixer.{name}", getattr(self, name))
        if self.window is not None:
            _positive_int("mixer.mask.size", self.window)
        if self.type == "attention":
            if self.heads % self.kv_heads:
                raise ConfigError("mixer.heads must be a multiple of mixer.kv_heads")
            if self.rot is not None and self.rot.dims > self.dim:
                raise ConfigError("mixer.rot.dims must not exceed mixer.dim")
        elif self.type == "latent_attention":
            _positive_int("mixer.q_rank", self.q_rank)
            _positive_int("mixer.kv_rank", self.kv_rank)
            if type(self.rot_dim) is not int or self.rot_dim < 0 or self.rot_dim % 2:
                raise ConfigError("mixer.rot_dim must be an even, non-negative integer")
            if (self.rot_dim > 0) != (self.rot is not None) or (self.rot is not None and self.rot.dims != self.rot_dim):
                raise ConfigError("mixer.rot.dims must equal mixer.rot_dim")

    @classmethod
    def from_json(cls, index: int, data: Any) -> "FezavikLayer":
        where = f"layers[{index}]"
        data = _need(where, data, ("type", "mixer"))
        kind = data["type"]
        mlp = data.get("mlp")
        experts = None if mlp is None else FezavikExperts.from_json(f"{where}.mlp", mlp)
        if kind == "hgrn2":
            mixer = _need(f"{where}.mixer", data["mixer"], ("heads", "dim", "vdim"))
            return cls(type=kind, heads=mixer["heads"], dim=mixer["dim"], vdim=mixer["vdim"], mlp=experts)
        if kind not in MIXER_TYPES:
            raise ConfigError(f"{where}.type is one of {', '.join(MIXER_TYPES)}, not {kind!r}")
        mixer = _need(f"{where}.mixer", data["mixer"], ("heads", "dim", "vdim", "scale"))
        mask = mixer.get("mask")
        window = None if mask is None else _need(f"{where}.mixer.mask", mask, ("size",))["size"]
        rot = mixer.get("rot")
        rot = None if rot is None else FezavikRotation.from_json(f"{where}.mixer.rot", rot)
        common = dict(type=kind, heads=mixer["heads"], dim=mixer["dim"], vdim=mixer["vdim"],
                      scale=_number("mixer.scale", mixer["scale"]), window=window, rot=rot, mlp=experts)
        if kind == "attention":
            return cls(kv_heads=_need(f"{where}.mixer", mixer, ("kv_heads",))["kv_heads"], **common)
        mixer = _need(f"{where}.mixer", mixer, ("q_rank", "kv_rank", "rot_dim"))
        return cls(q_rank=mixer["q_rank"], kv_rank=mixer["kv_rank"], rot_dim=mixer["rot_dim"], **common)

    def to_json(self) -> dict[str, Any]:
        mixer: dict[str, Any] = {"dim": self.dim, "heads": self.heads, "vdim": self.vdim}
        if self.type != "hgrn2":
            mixer["scale"] = self.scale
            if self.window is not None:
                mixer["mask"] = {"size": self.window}
            if self.rot is not None:
                mixer["rot"] = self.rot.to_json()
            if self.type == "attention":
                mixer["kv_heads"] = self.kv_heads
            else:
                mixer.update(kv_rank=self.kv_rank, q_rank=self.q_rank, rot_dim=self.rot_dim)
        return {"mixer": mixer, "mlp": None if self.mlp is None else self.mlp.to_json(), "type": self.type}


@dataclass(frozen=True)
class FezavikConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple[FezavikLayer, ...]
    eos_token_ids: tuple[int, ...] = ()

    architecture = "Fezavik"

    def __post_init__(self) -> None:
        _positive_int("vocab", self.vocab)
        _positive_int("width", self.width)
        if not self.norm_eps > 0:
            raise ConfigError("norm.eps must be positive")
        if not self.layers:
            raise ConfigError("a model needs at least one layer")

    @classmethod
    def from_json(cls, data: Mapping[str, Any]) -> "FezavikConfig":
        data = _need("config.json", data, ("vocab", "width", "norm", "layers"))
        norm = _need("config.json 'norm'", data["norm"], ("eps",))
        if not isinstance(data["layers"], list):
            raise ConfigError("config.json 'layers' must be a list")
        eos = data.get("eos_token_id")
        eos_ids = () if eos is None else (eos,) if type(eos) is int else tuple(eos)
        return cls(vocab=data["vocab"], width=data["width"], norm_eps=_number("norm.eps", norm["eps"]),
                   layers=tuple(FezavikLayer.from_json(i, layer) for i, layer in enumerate(data["layers"])),
                   eos_token_ids=eos_ids)

    def to_json(self) -> dict[str, Any]:
        data: dict[str, Any] = {"architecture": self.architecture,
                                "layers": [layer.to_json() for layer in self.layers],
                                "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.eos_token_ids:
            data["eos_token_id"] = list(self.eos_token_ids)
        return data

    # ------------------------------------------------------------------ spec
    def _mixer_spec(self, layer: FezavikLayer) -> PartSpec:
        if layer.type == "hgrn2":
            return PartSpec("gated_recurrence", {
                "hidden_size": self.width, "num_heads": layer.heads, "key_dim": layer.dim, "value_dim": layer.vdim,
                "query_act": "silu", "gate_bias": True, "lower_bound": True, "out_norm": "weight",
                "eps": self.norm_eps, "float32_output": True})
        if layer.type == "attention":
            return PartSpec("windowed_attention", {
                "hidden_size": self.width, "num_heads": layer.heads, "num_kv_heads": layer.kv_heads,
                "key_dim": layer.dim, "value_dim": layer.vdim, "scale": layer.scale, "window": layer.window,
                "qk_norm": "whole", "qk_norm_eps": self.norm_eps,
                "position": None if layer.rot is None else layer.rot.to_spec("rope_interleaved"),
                "sink": True, "float32_output": True, "names": {"q_norm": "q.norm", "k_norm": "k.norm"}})
        return PartSpec("latent_attention", {
            "hidden_size": self.width, "num_heads": layer.heads, "key_dim": layer.dim, "rot_dim": layer.rot_dim,
            "value_dim": layer.vdim, "q_rank": layer.q_rank, "kv_rank": layer.kv_rank, "scale": layer.scale,
            "eps": self.norm_eps, "window": layer.window, "sink": True, "gate": "head", "float32_output": True,
            "position": None if layer.rot is None else layer.rot.to_spec("rope_half_split_computed")})

    def to_spec(self) -> ModelSpec:
        norm = PartSpec("rms_norm_stream32", {"width": self.width, "eps": self.norm_eps})
        block = PartSpec("sandwich_residual", {
            "mixer_norm_name": "norm1", "mixer_post_norm_name": "norm1b", "feed_forward_norm_name": "norm2",
            "feed_forward_post_norm_name": "norm2b", "mixer_name": "mix", "feed_forward_name": "mlp"})
        layers = []
        for index, layer in enumerate(self.layers):
            feed_forward = None
            if layer.mlp is not None:
                feed_forward = PartSpec("softmax_routed_experts", {
                    "hidden_size": self.width, "experts": layer.mlp.experts, "identity": layer.mlp.identity,
                    "top": layer.mlp.top, "ff": layer.mlp.ff, "correction": True, "renormalise": False,
                    "float32_output": True})
            layers.append(LayerSpec(prefix=f"l{index}", block=block, mixer=self._mixer_spec(layer),
                                    feed_forward=feed_forward, norm=norm))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width,
            max_positions=UNBOUNDED_POSITIONS,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "width": self.width, "name": "embed"}),
            layers=tuple(layers), order=tuple(RunStep(i) for i in range(len(self.layers))),
            final_norm=norm.with_params(name="final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "width": self.width, "tied_to": None,
                                      "name": "head"}),
            eos_token_ids=self.eos_token_ids)


register_architecture(FezavikConfig.architecture, FezavikConfig)
