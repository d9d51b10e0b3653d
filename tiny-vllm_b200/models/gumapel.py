"""Gumapel: typed configuration and its description as parts.

A decoder whose config.json lists its layers one by one.  Every layer is a parallel block (one
norm; mixer and feed-forward both read its output and their sum joins a float32 residual stream)
with one of two attention mixers:

``attention``     q and k divided by their root mean square over the head (no weight), no position
                  encoding, a plain sliding window, an output gate sigmoid(W_g h) on the
                  concatenated heads
``attention_2``   rotary positions on the first ``rot.dims`` dimensions of q and k (neighbouring
                  dimensions paired, frequency ``rot.base``^(-2i / dims)), a sliding window that also
                  keeps the first ``mask.keep_first`` tokens

Both take key and value sizes of their own (``dim``, ``vdim``), a score scale from the
configuration, and may blend their values with those of the first layer that says ``v_mix``
(scalar tensor ``vmix``).  The feed-forward is down(gelu_tanh(gate h) * (up h)) or absent.  All of
it maps onto parts of the package with these numbers as parameters; nothing here computes.

Checkpoint names: ``embed``, ``l<i>.norm1``, ``l<i>.mix.{q,k,v,g,o,vmix}``,
``l<i>.mlp.{gate,up,down}``, ``final.norm``, ``head``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from ..config.registry import ConfigError, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunStep

MIXER_TYPES = ("attention", "attention_2")
# the design sets no limit on positions (angles are computed, not tabulated); the engine's own
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


@dataclass(frozen=True)
class GumapelLayer:
    type: str
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int | None = None          # mask.size
    keep_first: int = 0                # mask.keep_first (attention_2)
    rot_dims: int | None = None        # rot.dims (attention_2)
    rot_base: float | None = None      # rot.base
    v_mix: bool = False
    ff: int | None = None              # mlp.ff; None: no feed-forward

    def __post_init__(self) -> None:
        if self.type not in MIXER_TYPES:
            raise ConfigError(f"a layer's type is one of {', '.join(MIXER_TYPES)}, not {self.type!r}")
        for name in ("heads", "kv_heads", "dim", "vdim"):
            _positive_int(f"mixer.{name}", getattr(self, name))
        if self.heads % self.kv_heads:
            raise ConfigError("mixer.heads must be a multiple of mixer.kv_heads")
        if self.window is not None:
            _positive_int("mixer.mask.size", self.window)
        if type(self.keep_first) is not int or self.keep_first < 0:
            raise ConfigError("mixer.mask.keep_first must be a non-negative integer")
        if self.type == "attention_2":
            _positive_int("mixer.rot.dims", self.rot_dims)
            if self.rot_dims % 2 or self.rot_dims > self.dim:
                raise ConfigError("mixer.rot.dims must be even and at most mixer.dim")
            if self.rot_base is None or not self.rot_base > 0:
                raise ConfigError("mixer.rot.base must be positive")
        if self.ff is not None:
            _positive_int("mlp.ff", self.ff)

    @classmethod
    def from_json(cls, index: int, data: Any) -> "GumapelLayer":
        if not isinstance(data, Mapping) or not isinstance(data.get("mixer"), Mapping):
            raise ConfigError(f"layers[{index}] must be an object with 'type' and 'mixer'")
        mixer = data["mixer"]
        missing = [key for key in ("heads", "kv_heads", "dim", "vdim", "scale") if key not in mixer]
        if missing:
            raise ConfigError(f"layers[{index}].mixer lacks " + ", ".join(missing))
        mask = mixer.get("mask") or {}
        rot = mixer.get("rot") or {}
        kind = data.get("type")
        mlp = data.get("mlp")
        if mlp is not None:
            if not isinstance(mlp, Mapping) or mlp.get("kind") != "dense":
                raise ConfigError(f"layers[{index}].mlp must be null or of kind 'dense'")
        v_mix = mixer.get("v_mix", False)
        if type(v_mix) is not bool:
            raise ConfigError(f"layers[{index}].mixer.v_mix must be true or false")
        return cls(
            type=kind, heads=mixer["heads"], kv_heads=mixer["kv_heads"], dim=mixer["dim"], vdim=mixer["vdim"],
            scale=_number("mixer.scale", mixer["scale"]), window=mask.get("size"),
            keep_first=mask.get("keep_first", 0) if kind == "attention_2" else 0,
            rot_dims=rot.get("dims") if kind == "attention_2" else None,
            rot_base=_number("mixer.rot.base", rot["base"]) if kind == "attention_2" and "base" in rot else None,
            v_mix=v_mix, ff=None if mlp is None else mlp.get("ff"))

    def to_json(self) -> dict[str, Any]:
        mixer: dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads,
                                 "scale": self.scale, "v_mix": self.v_mix, "vdim": self.vdim}
        mask: dict[str, Any] = {}
        if self.window is not None:
            mask["size"] = self.window
        if self.type == "attention_2":
            mask["keep_first"] = self.keep_first
            mixer["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        if mask:
            mixer["mask"] = mask
        return {"mixer": mixer, "mlp": None if self.ff is None else {"ff": self.ff, "kind": "dense"},
                "type": self.type}


@dataclass(frozen=True)
class GumapelConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple[GumapelLayer, ...]
    eos_token_ids: tuple[int, ...] = ()

    architecture = "Gumapel"

    def __post_init__(self) -> None:
        _positive_int("vocab", self.vocab)
        _positive_int("width", self.width)
        if not self.norm_eps > 0:
            raise ConfigError("norm.eps must be positive")
        if not self.layers:
            raise ConfigError("a model needs at least one layer")
        mixing = [layer for layer in self.layers if layer.v_mix]
        for layer in mixing[1:]:
            if (layer.kv_heads, layer.vdim) != (mixing[0].kv_heads, mixing[0].vdim):
                raise ConfigError("layers that blend their values with the first such layer's must have "
                                  "its kv_heads and vdim")

    @classmethod
    def from_json(cls, data: Mapping[str, Any]) -> "GumapelConfig":
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
                   layers=tuple(GumapelLayer.from_json(i, layer) for i, layer in enumerate(data["layers"])),
                   eos_token_ids=eos_ids)

    def to_json(self) -> dict[str, Any]:
        data: dict[str, Any] = {"architecture": self.architecture,
                                "layers": [layer.to_json() for layer in self.layers],
                                "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.eos_token_ids:
            data["eos_token_id"] = list(self.eos_token_ids)
        return data

    # ------------------------------------------------------------------ spec
    def to_spec(self) -> ModelSpec:
        norm = PartSpec("rms_norm_stream32", {"width": self.width, "eps": self.norm_eps})
        block = PartSpec("parallel_residual", {"norm_name": "norm1", "mixer_name": "mix",
                                               "feed_forward_name": "mlp"})
        layers, mixing_seen = [], False
        for index, layer in enumerate(self.layers):
            params: dict[str, Any] = {
                "hidden_size": self.width, "num_heads": layer.heads, "num_kv_heads": layer.kv_heads,
                "key_dim": layer.dim, "value_dim": layer.vdim, "scale": layer.scale, "window": layer.window,
            }
            if layer.type == "attention":
                params.update(qk_norm="unit", qk_norm_eps=self.norm_eps, gate=True)
            else:
                params.update(keep_first=layer.keep_first,
                              position=PartSpec("rope_interleaved", {"dims": layer.rot_dims, "base": layer.rot_base}))
            if layer.v_mix:
                params["value_mix"] = "blend" if mixing_seen else "first"
                mixing_seen = True
            feed_forward = None
            if layer.ff is not None:
                feed_forward = PartSpec("gated_mlp", {
                    "hidden_size": self.width, "intermediate_size": layer.ff, "activation": "gelu_tanh",
                    "names": {"gate": "gate", "up": "up", "down": "down"}})
            layers.append(LayerSpec(prefix=f"l{index}", block=block,
                                    mixer=PartSpec("windowed_attention", params),
                                    feed_forward=feed_forward, norm=norm.with_params(name=f"l{index}.norm1")))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width,
            max_positions=UNBOUNDED_POSITIONS,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "width": self.width, "name": "embed"}),
            layers=tuple(layers), order=tuple(RunStep(i) for i in range(len(self.layers))),
            final_norm=norm.with_params(name="final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "width": self.width, "tied_to": None,
                                      "name": "head"}),
            eos_token_ids=self.eos_token_ids)


register_architecture(GumapelConfig.architecture, GumapelConfig)
