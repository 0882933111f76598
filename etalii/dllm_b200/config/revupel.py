"""The typed configuration of the Revupel design, read from config.json's own keys.

A Revupel config.json names the design under `architecture` and gives `vocab`, `width`, `norm.eps`, `canon.taps` (the
taps of the causal convolution in front of every mixer), optionally `token_side.dim` (the part of the tokens' second
embedding that each layer takes), `layers` and optionally `loop` (`start`, `stop`, `times`: layers start .. stop - 1
run `times` times in a row). A layer entry has `type` ("latent_attention" or "mlstm"), the mixer's sizes and constants
under `mixer`, and the feed-forward under `mlp` (kind "dense": `ff`; kind "moe": `expert.ff`, `router.experts`,
`router.top`, optionally `shared.ff`; or null for a layer without one). Nothing here is a size of a particular model."""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Mapping

from .registry import ConfigError

MIXER_TYPES = ("latent_attention", "mlstm")
MLP_KINDS = ("dense", "moe")
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
        _need(where, mixer, ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "scale", "rot"))
        _positive(where, mixer, ("heads", "dim", "vdim", "q_rank", "kv_rank"))
        rot_dim = mixer["rot_dim"]
        if not isinstance(rot_dim, int) or isinstance(rot_dim, bool) or rot_dim < 0 or rot_dim % 2:
            raise ConfigError(f"{where}.rot_dim must be even and not negative, not {rot_dim!r}")
        _need(f"{where}.rot", mixer["rot"], ("base", "dims"))
        if mixer["rot"]["dims"] != rot_dim:
            raise ConfigError(f"{where}.rot.dims ({mixer['rot']['dims']!r}) must equal rot_dim ({rot_dim}): the "
                              "rotated part turns as a whole")
        if rot_dim and not float(mixer["rot"]["base"]) > 0:
            raise ConfigError(f"{where}.rot.base must be positive")
        if not float(mixer["scale"]) > 0:
            raise ConfigError(f"{where}.scale must be positive")
    else:
        _need(where, mixer, ("heads", "dim", "vdim", "gate_cap"))
        _positive(where, mixer, ("heads", "dim", "vdim"))
        if not float(mixer["gate_cap"]) > 0:
            raise ConfigError(f"{where}.gate_cap must be positive")


def _check_mlp(where: str, mlp: Any) -> None:
    _need(where, mlp, ("kind",))
    if mlp["kind"] not in MLP_KINDS:
        raise ConfigError(f"{where}.kind {mlp['kind']!r} is not supported (supported: {', '.join(MLP_KINDS)})")
    if mlp["kind"] == "dense":
        _need(where, mlp, ("ff",))
        _positive(where, mlp, ("ff",))
        return
    _need(where, mlp, ("expert", "router"))
    _need(f"{where}.expert", mlp["expert"], ("ff",))
    _positive(f"{where}.expert", mlp["expert"], ("ff",))
    _need(f"{where}.router", mlp["router"], ("experts", "top"))
    _positive(f"{where}.router", mlp["router"], ("experts", "top"))
    if mlp["router"]["top"] > mlp["router"]["experts"]:
        raise ConfigError(f"{where}.router: top {mlp['router']['top']} of {mlp['router']['experts']} experts")
    if mlp.get("shared") is not None:
        _need(f"{where}.shared", mlp["shared"], ("ff",))
        _positive(f"{where}.shared", mlp["shared"], ("ff",))


@dataclass(frozen=True)
class RevupelConfig:
    model_type = "Revupel"

    vocab: int
    width: int
    norm_eps: float
    taps: int
    layers: tuple = field(default_factory=tuple)
    """The layer entries as config.json gives them (checked)."""
    side_dim: int = 0
    """Values of the tokens' second embedding that each layer takes (0: the model has none)."""
    loop: Mapping | None = None
    max_position: int = DEFAULT_MAX_POSITION
    eos_token_ids: tuple[int, ...] = field(default_factory=tuple)

    def __post_init__(self) -> None:
        for name in ("vocab", "width", "max_position", "taps"):
            if int(getattr(self, name)) <= 0:
                raise ConfigError(f"{name} must be positive, not {getattr(self, name)}")
        if self.side_dim < 0:
            raise ConfigError(f"token_side.dim must not be negative, not {self.side_dim}")
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
            if layer.get("mlp") is not None:
                _check_mlp(f"{where}.mlp", layer["mlp"])
        if self.loop is not None:
            _need("loop", self.loop, ("start", "stop", "times"))
            start, stop, times = self.loop["start"], self.loop["stop"], self.loop["times"]
            if not (isinstance(start, int) and isinstance(stop, int) and 0 <= start < stop <= len(self.layers)):
                raise ConfigError(f"loop: start {start!r} and stop {stop!r} must bound a stretch of the "
                                  f"{len(self.layers)} layers")
            if not isinstance(times, int) or isinstance(times, bool) or times < 1:
                raise ConfigError(f"loop.times must be a positive integer, not {times!r}")

    @classmethod
    def from_hf(cls, config: Mapping[str, Any], generation: Mapping[str, Any] | None = None) -> "RevupelConfig":
        if config.get("architecture") != "Revupel":
            raise ConfigError(f"architecture {config.get('architecture')!r} is not 'Revupel'")
        _need("config.json", config, ("vocab", "width", "norm", "canon", "layers"))
        _need("norm", config["norm"], ("eps",))
        _need("canon", config["canon"], ("taps",))
        if not isinstance(config["layers"], (list, tuple)):
            raise ConfigError("layers must be a list")
        side = config.get("token_side")
        if side is not None:
            _need("token_side", side, ("dim",))
        eos = config.get("eos_token_id")
        eos = [] if eos is None else ([int(t) for t in eos] if isinstance(eos, (list, tuple)) else [int(eos)])
        return cls(
            vocab=int(config["vocab"]), width=int(config["width"]), norm_eps=float(config["norm"]["eps"]),
            taps=int(config["canon"]["taps"]),
            layers=tuple(copy.deepcopy(layer) for layer in config["layers"]),
            side_dim=int(side["dim"]) if side is not None else 0,
            loop=copy.deepcopy(config["loop"]) if config.get("loop") is not None else None,
            max_position=int(config.get("max_position", DEFAULT_MAX_POSITION)),
            eos_token_ids=tuple(eos),
        )

    def to_hf(self) -> dict:
        """The config.json that reads back as this configuration."""
        out: dict[str, Any] = {
            "architecture": "Revupel", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
            "canon": {"taps": self.taps}, "layers": [copy.deepcopy(layer) for layer in self.layers],
        }
        if self.side_dim:
            out["token_side"] = {"dim": self.side_dim}
        if self.loop is not None:
            out["loop"] = copy.deepcopy(dict(self.loop))
        if self.max_position != DEFAULT_MAX_POSITION:
            out["max_position"] = self.max_position
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out
