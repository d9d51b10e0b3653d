"""Kelasun: typed configuration and its description as parts.

A decoder whose config.json lists its layers one by one.  A layer norms after the sum,
x <- LN(a x + mixer(x)) and then x <- LN(a x + ff(x)) with a = ``postln_alpha`` (layer norms with a
weight and no bias, the stream in float32), and has one of two mixers:

``attention``         grouped-query attention without a position encoding: q and k are RMS-normed over
                      the whole projection (weights of that size), q is multiplied by a temperature that
                      grows with the logarithm of the position (``q_temp``), head h takes 2^(-8 (h + 1) /
                      heads) * (i - j) off its scores, the softmax's denominator holds a learned sink a
                      head, and every head's output is multiplied by one gate number, sigmoid(W_g x)_h
``latent_attention``  queries through a latent of ``q_rank``, keys and values through one of ``kv_rank``;
                      a head is ``dim`` plain and ``rot_dim`` rotated dimensions, the rotated key part is
                      shared by all heads; neighbouring dimensions are paired and the frequencies are
                      stretched for long contexts (``rot.scaling``); a gate sigmoid(W_g x) on the
                      concatenated heads

The feed-forward is a mixture of experts (``router.experts`` experts of size ``expert.ff`` with
act = relu^2, of which a token uses ``router.top``, weighted by the softmax over the chosen logits)
plus a shared expert, or absent.  The last norm is a layer norm too, and the logits are multiplied by
``logit_scale``.  All of it maps onto parts of the package with these numbers as parameters; nothing
here computes.

Checkpoint names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.{q,k,v,q.norm,k.norm,sink,g,o}`` or
``l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,g,o}``, ``l<i>.mlp.{router,e<j>.up,e<j>.down,shared.up,
shared.down}``, ``final.norm``, ``head``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from ..config.registry import ConfigError, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunStep

MIXER_TYPES = ("attention", "latent_attention")
# the distance bias of the 'attention' mixer: head h has the slope 2^(-SLOPE_EXPONENT (h + 1) / heads)
SLOPE_EXPONENT = 8.0
# positions enter through computed angles, logarithms and distances, none tabulated: the engine's own
# max_model_len bounds a request
UNBOUNDED_POSITIONS = 1 << 20


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
class KelasunExperts:
    experts: int
    top: int
    ff: int
    shared_ff: int = 0                 # 0: no shared expert

    def __post_init__(self) -> None:
        for name in ("experts", "top", "ff"):
            _positive_int(f"mlp.{name}", getattr(self, name))
        if self.top > self.experts:
            raise ConfigError("mlp.router.top must not exceed mlp.router.experts")
        if type(self.shared_ff) is not int or self.shared_ff < 0:
            raise ConfigError("mlp.shared.ff must be a non-negative integer")

    @classmethod
    def from_json(cls, where: str, data: Any) -> "KelasunExperts":
        data = _need(where, data, ("kind", "expert", "router"))
        if data["kind"] != "moe":
            raise ConfigError(f"{where}.kind must be 'moe', not {data['kind']!r}")
        expert = _need(f"{where}.expert", data["expert"], ("ff",))
        router = _need(f"{where}.router", data["router"], ("experts", "top"))
        shared = data.get("shared")
        shared_ff = 0 if shared is None else _need(f"{where}.shared", shared, ("ff",))["ff"]
        return cls(experts=router["experts"], top=router["top"], ff=expert["ff"], shared_ff=shared_ff)

    def to_json(self) -> dict[str, Any]:
        data: dict[str, Any] = {"expert": {"ff": self.ff}, "kind": "moe",
                                "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff:
            data["shared"] = {"ff": self.shared_ff}
        return data


@dataclass(frozen=True)
class KelasunLayer:
    type: str
    heads: int
    dim: int
    vdim: int
    scale: float
    kv_heads: int = 1                      # attention
    q_temp: tuple[float, int] | None = None    # attention: (coef, every)
    q_rank: int | None = None              # latent_attention
    kv_rank: int | None = None
    rot_dim: int = 0
    rot_base: float | None = None
    rot_scaling: tuple | None = None       # (factor, original, fast, slow)
    mlp: KelasunExperts | None = None

    def __post_init__(self) -> None:
        if self.type not in MIXER_TYPES:
            raise ConfigError(f"a layer's type is one of {', '.join(MIXER_TYPES)}, not {self.type!r}")
        for name in ("heads", "dim", "vdim", "kv_heads"):
            _positive_int(f"mixer.{name}", getattr(self, name))
        if self.heads % self.kv_heads:
            raise ConfigError("mixer.heads must be a multiple of mixer.kv_heads")
        if self.type == "attention":
            if self.q_temp is not None and (self.q_temp[1] <= 0 or type(self.q_temp[1]) is not int):
                raise ConfigError("mixer.q_temp.every must be a positive integer")
        else:
            _positive_int("mixer.q_rank", self.q_rank)
            _positive_int("mixer.kv_rank", self.kv_rank)
            if type(self.rot_dim) is not int or self.rot_dim < 0 or self.rot_dim % 2:
                raise ConfigError("mixer.rot_dim must be an even, non-negative integer")
            if self.rot_dim and (self.rot_base is None or not self.rot_base > 0):
                raise ConfigError("mixer.rot.base must be positive")

    @classmethod
    def from_json(cls, index: int, data: Any) -> "KelasunLayer":
        where = f"layers[{index}]"
        data = _need(where, data, ("type", "mixer"))
        kind = data["type"]
        mlp = data.get("mlp")
        experts = None if mlp is None else KelasunExperts.from_json(f"{where}.mlp", mlp)
        if kind == "attention":
            mixer = _need(f"{where}.mixer", data["mixer"], ("heads", "kv_heads", "dim", "vdim", "scale"))
            temp = mixer.get("q_temp")
            q_temp = None
            if temp is not None:
                temp = _need(f"{where}.mixer.q_temp", temp, ("coef", "every"))
                q_temp = (_number("mixer.q_temp.coef", temp["coef"]), temp["every"])
            return cls(type=kind, heads=mixer["heads"], kv_heads=mixer["kv_heads"], dim=mixer["dim"],
                       vdim=mixer["vdim"], scale=_number("mixer.scale", mixer["scale"]), q_temp=q_temp, mlp=experts)
        if kind == "latent_attention":
            mixer = _need(f"{where}.mixer", data["mixer"],
                          ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "scale"))
            rot_base = rot_scaling = None
            if mixer["rot_dim"]:
                rot = _need(f"{where}.mixer.rot", mixer.get("rot"), ("base", "dims"))
                if rot["dims"] != mixer["rot_dim"]:
                    raise ConfigError(f"{where}.mixer.rot.dims must equal mixer.rot_dim")
                rot_base = _number("mixer.rot.base", rot["base"])
                scaling = rot.get("scaling")
                if scaling is not None:
                    scaling = _need(f"{where}.mixer.rot.scaling", scaling, ("factor", "original", "fast", "slow"))
                    rot_scaling = tuple(_number(f"mixer.rot.scaling.{key}", scaling[key])
                                        for key in ("factor", "original", "fast", "slow"))
            return cls(type=kind, heads=mixer["heads"], dim=mixer["dim"], vdim=mixer["vdim"],
                       scale=_number("mixer.scale", mixer["scale"]), q_rank=mixer["q_rank"],
                       kv_rank=mixer["kv_rank"], rot_dim=mixer["rot_dim"], rot_base=rot_base,
                       rot_scaling=rot_scaling, mlp=experts)
        raise ConfigError(f"{where}.type is one of {', '.join(MIXER_TYPES)}, not {kind!r}")

    def to_json(self) -> dict[str, Any]:
        mixer: dict[str, Any] = {"dim": self.dim, "heads": self.heads, "scale": self.scale, "vdim": self.vdim}
        if self.type == "attention":
            mixer["kv_heads"] = self.kv_heads
            if self.q_temp is not None:
                mixer["q_temp"] = {"coef": self.q_temp[0], "every": self.q_temp[1]}
        else:
            mixer.update(kv_rank=self.kv_rank, q_rank=self.q_rank, rot_dim=self.rot_dim)
            if self.rot_dim:
                rot: dict[str, Any] = {"base": self.rot_base, "dims": self.rot_dim}
                if self.rot_scaling is not None:
                    rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), self.rot_scaling))
                mixer["rot"] = rot
        return {"mixer": mixer, "mlp": None if self.mlp is None else self.mlp.to_json(), "type": self.type}


@dataclass(frozen=True)
class KelasunConfig:
    vocab: int
    width: int
    norm_eps: float
    postln_alpha: float
    logit_scale: float
    layers: tuple[KelasunLayer, ...]
    eos_token_ids: tuple[int, ...] = ()

    architecture = "Kelasun"

    def __post_init__(self) -> None:
        _positive_int("vocab", self.vocab)
        _positive_int("width", self.width)
        if not self.norm_eps > 0:
            raise ConfigError("norm.eps must be positive")
        if not self.layers:
            raise ConfigError("a model needs at least one layer")

    @classmethod
    def from_json(cls, data: Mapping[str, Any]) -> "KelasunConfig":
        data = _need("config.json", data, ("vocab", "width", "norm", "layers", "postln_alpha", "logit_scale"))
        norm = _need("config.json 'norm'", data["norm"], ("eps",))
        if not isinstance(data["layers"], list):
            raise ConfigError("config.json 'layers' must be a list")
        eos = data.get("eos_token_id")
        eos_ids = () if eos is None else (eos,) if type(eos) is int else tuple(eos)
        return cls(vocab=data["vocab"], width=data["width"], norm_eps=_number("norm.eps", norm["eps"]),
                   postln_alpha=_number("postln_alpha", data["postln_alpha"]),
                   logit_scale=_number("logit_scale", data["logit_scale"]),
                   layers=tuple(KelasunLayer.from_json(i, layer) for i, layer in enumerate(data["layers"])),
                   eos_token_ids=eos_ids)

    def to_json(self) -> dict[str, Any]:
        data: dict[str, Any] = {"architecture": self.architecture,
                                "layers": [layer.to_json() for layer in self.layers],
                                "logit_scale": self.logit_scale, "norm": {"eps": self.norm_eps},
                                "postln_alpha": self.postln_alpha, "vocab": self.vocab, "width": self.width}
        if self.eos_token_ids:
            data["eos_token_id"] = list(self.eos_token_ids)
        return data

    # ------------------------------------------------------------------ spec
    def to_spec(self) -> ModelSpec:
        norm = PartSpec("layer_norm_stream32", {"width": self.width, "eps": self.norm_eps})
        block = PartSpec("postnorm_residual", {"alpha": self.postln_alpha, "mixer_norm_name": "norm1",
                                               "feed_forward_norm_name": "norm2", "mixer_name": "mix",
                                               "feed_forward_name": "mlp"})
        layers = []
        for index, layer in enumerate(self.layers):
            if layer.type == "attention":
                mixer = PartSpec("windowed_attention", {
                    "hidden_size": self.width, "num_heads": layer.heads, "num_kv_heads": layer.kv_heads,
                    "key_dim": layer.dim, "value_dim": layer.vdim, "scale": layer.scale, "window": None,
                    "qk_norm": "whole", "qk_norm_eps": self.norm_eps, "query_temperature": layer.q_temp,
                    "distance_slope_exponent": SLOPE_EXPONENT, "sink": True, "gate": "head",
                    "float32_output": True, "names": {"q_norm": "q.norm", "k_norm": "k.norm"}})
            else:
                position = None
                if layer.rot_dim:
                    scaling = None if layer.rot_scaling is None else dict(
                        zip(("factor", "original", "fast", "slow"), layer.rot_scaling))
                    position = PartSpec("rope_interleaved", {"dims": layer.rot_dim, "base": layer.rot_base,
                                                             "scaling": scaling})
                mixer = PartSpec("latent_attention", {
                    "hidden_size": self.width, "num_heads": layer.heads, "key_dim": layer.dim,
                    "rot_dim": layer.rot_dim, "value_dim": layer.vdim, "q_rank": layer.q_rank,
                    "kv_rank": layer.kv_rank, "scale": layer.scale, "eps": self.norm_eps, "position": position,
                    "gate": True, "float32_output": True})
            feed_forward = None
            if layer.mlp is not None:
                feed_forward = PartSpec("routed_experts", {
                    "hidden_size": self.width, "experts": layer.mlp.experts, "top": layer.mlp.top,
                    "ff": layer.mlp.ff, "shared_ff": layer.mlp.shared_ff, "activation": "relu_squared",
                    "float32_output": True})
            layers.append(LayerSpec(prefix=f"l{index}", block=block, mixer=mixer, feed_forward=feed_forward,
                                    norm=norm))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width,
            max_positions=UNBOUNDED_POSITIONS,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "width": self.width, "name": "embed"}),
            layers=tuple(layers), order=tuple(RunStep(i) for i in range(len(self.layers))),
            final_norm=norm.with_params(name="final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "width": self.width, "tied_to": None,
                                      "name": "head", "scale": self.logit_scale}),
            eos_token_ids=self.eos_token_ids)


register_architecture(KelasunConfig.architecture, KelasunConfig)
