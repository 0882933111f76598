"""The typed configuration of the Gaperax design, read from config.json's own keys.

A Gaperax config.json names the design under `architecture` and gives `vocab`, `width`, `norm.eps` and `layers`. A
layer entry has `type` ("latent_attention" or "attention"), the mixer's sizes and constants under `mixer`, the
feed-forward under `mlp` (kind "dense" with `ff`, or null for a layer without one), and optionally `weights_of`: the
index of another layer whose tensors this layer runs with (its cache is its own). Nothing here is a size of a
particular model."""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Mapping

from .registry import ConfigError

MIXER_TYPES = ("latent_attention", "attention")
DEFAULT_MAX_POSITION = 32768
"""The design has no longest sequence; this bounds the rotary table and the cache unless `max_position` is given."""


def _need(where: str, mapping: Any, keys) -> None:
    if not isinstance(mapping, Mapping):
        raise ConfigError(f"{where} must be an object")
    missing = [k for k in keys if k not in mapping]
    if missing:
        raise ConfigError(f"{where} has no {', '.join(missing)}")


def _positive(where: str, mapping: Mapping, keys) -> None:
    for key in keys:
        if not isinstance(mapping[key], int) or isinstance(mapping[key], bool) or mapping[key] <= 0:
            raise ConfigError(f"{where}.{key} must be a positive integer, not {mapping[key]!r}")


def _check_mixer(where: str, kind: str, mixer: Any) -> None:
    if kind == "latent_attention":
        _need(where, mixer, ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "scale"))
        _positive(where, mixer, ("heads", "dim", "vdim", "q_rank", "kv_rank"))
        rot_dim = mixer["rot_dim"]
        if not isinstance(rot_dim, int) or isinstance(rot_dim, bool) or rot_dim < 0 or rot_dim % 2:
            raise ConfigError(f"{where}.rot_dim must be even and not negative, not {rot_dim!r}")
        if rot_dim:
            _need(where, mixer, ("rot",))
            _need(f"{where}.rot", mixer["rot"], ("base", "dims"))
            if mixer["rot"]["dims"] != rot_dim:
                raise ConfigError(f"{where}.rot.dims ({mixer['rot']['dims']!r}) must equal rot_dim ({rot_dim}): the "
                                  "rotated part turns as a whole")
            if not float(mixer["rot"]["base"]) > 1:
                raise ConfigError(f"{where}.rot.base must be above 1")
            scaling = mixer["rot"].get("scaling")
            if scaling is not None:
                _need(f"{where}.rot.scaling", scaling, ("factor", "original", "fast", "slow"))
                for key in ("factor", "original", "fast", "slow"):
                    if not float(scaling[key]) > 0:
                        raise ConfigError(f"{where}.rot.scaling.{key} must be positive")
    else:
        _need(where, mixer, ("heads", "kv_heads", "dim", "vdim", "scale", "mask"))
        _positive(where, mixer, ("heads", "kv_heads", "dim", "vdim"))
        if mixer["heads"] % mixer["kv_heads"]:
            raise ConfigError(f"{where}: {mixer['heads']} heads are not a multiple of {mixer['kv_heads']} kv_heads")
        _need(f"{where}.mask", mixer["mask"], ("size", "keep_first"))
        _positive(f"{where}.mask", mixer["mask"], ("size",))
        keep = mixer["mask"]["keep_first"]
        if not isinstance(keep, int) or isinstance(keep, bool) or keep < 0:
            raise ConfigError(f"{where}.mask.keep_first must be an integer and not negative, not {keep!r}")
    if not float(mixer["scale"]) > 0:
        raise ConfigError(f"{where}.scale must be positive")


@dataclass(frozen=True)
class GaperaxConfig:
    model_type = "Gaperax"

    vocab: int
    width: int
    norm_eps: float
    layers: tuple = field(default_factory=tuple)
    """The layer entries as config.json gives them (checked)."""
    max_position: int = DEFAULT_MAX_POSITION
    eos_token_ids: tuple[int, ...] = field(default_factory=tuple)

    def __post_init__(self) -> None:
        for name in ("vocab", "width", "max_position"):
            if int(getattr(self, name)) <= 0:
                raise ConfigError(f"{name} must be positive, not {getattr(self, name)}")
        if not self.norm_eps > 0:
            raise ConfigError(f"norm.eps must be positive, not {self.norm_eps}")
        if not self.layers:
            raise ConfigError("layers is empty")
        for index, layer in enumerate(self.layers):
            where = f"layers[{index}]"
            _need(where, layer, ("type", "mixer"))
            if layer["type"] not in MIXER_TYPES:
                raise ConfigError(f"{where}.type {layer['type']!r} is not supported (supported: "
                                  f"{', '.join(MIXER_TYPES)})")
            _check_mixer(f"{where}.mixer", layer["type"], layer["mixer"])
            mlp = layer.get("mlp")
            if mlp is not None:
                _need(f"{where}.mlp", mlp, ("kind", "ff"))
                if mlp["kind"] != "dense":
                    raise ConfigError(f"{where}.mlp.kind {mlp['kind']!r} is not supported (supported: dense)")
                _positive(f"{where}.mlp", mlp, ("ff",))
        for index in range(len(self.layers)):
            self.weights_layer(index)

    def weights_layer(self, index: int) -> int:
        """The layer whose tensors layer `index` runs with: itself, or where its `weights_of` leads."""
        seen = {index}
        at = index
        while self.layers[at].get("weights_of") is not None:
            source = self.layers[at]["weights_of"]
            if not isinstance(source, int) or isinstance(source, bool) or not 0 <= source < len(self.layers):
                raise ConfigError(f"layers[{at}].weights_of {source!r} is no layer of the model")
            if source in seen:
                raise ConfigError(f"layers[{index}].weights_of leads back to itself")
            seen.add(source)
            at = source
        ours, theirs = self.layers[index], self.layers[at]
        if ours["type"] != theirs["type"] or ours["mixer"] != theirs["mixer"] or ours.get("mlp") != theirs.get("mlp"):
            raise ConfigError(f"layers[{index}] runs with the weights of layers[{at}] but has other sizes")
        return at

    @classmethod
    def from_hf(cls, config: Mapping[str, Any], generation: Mapping[str, Any] | None = None) -> "GaperaxConfig":
        if config.get("architecture") != "Gaperax":
            raise ConfigError(f"architecture {config.get('architecture')!r} is not 'Gaperax'")
        _need("config.json", config, ("vocab", "width", "norm", "layers"))
        _need("norm", config["norm"], ("eps",))
        if not isinstance(config["layers"], (list, tuple)):
            raise ConfigError("layers must be a list")
        eos = config.get("eos_token_id")
        eos = [] if eos is None else ([int(t) for t in eos] if isinstance(eos, (list, tuple)) else [int(eos)])
        return cls(
            vocab=int(config["vocab"]), width=int(config["width"]), norm_eps=float(config["norm"]["eps"]),
            layers=tuple(copy.deepcopy(layer) for layer in config["layers"]),
            max_position=int(config.get("max_position", DEFAULT_MAX_POSITION)),
            eos_token_ids=tuple(eos),
        )

    def to_hf(self) -> dict:
        """The config.json that reads back as this configuration."""
        out: dict[str, Any] = {
            "architecture": "Gaperax", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
            "layers": [copy.deepcopy(layer) for layer in self.layers],
        }
        if self.max_position != DEFAULT_MAX_POSITION:
            out["max_position"] = self.max_position
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out
