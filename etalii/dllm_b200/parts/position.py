"""Rotary position encoding: frequencies from the base and the scaling rule in float64, the table of cosines and
sines per position in float64 rounded once to float32 (reference: src/etalii_dllm/numerics.py:267-311 for the
frequencies, cpp/include/dllm/nn.hpp:501-530 for the rotation of pairs (i, i + rotary_dim/2))."""
from __future__ import annotations

import math
from typing import Mapping

import torch

from .registry import register_part


def rotary_frequencies(rotary_dim: int, theta: float, scaling: Mapping | None) -> list[float]:
    log_theta = math.log(float(theta))
    freqs = [math.exp(-(2 * i / rotary_dim) * log_theta) for i in range(rotary_dim // 2)]
    kind = "default" if not scaling else str(scaling.get("rope_type", "default"))
    if kind == "linear":
        freqs = [f / float(scaling["factor"]) for f in freqs]
    elif kind == "llama3":
        factor = float(scaling["factor"])
        low = float(scaling.get("low_freq_factor", 1.0))
        high = float(scaling.get("high_freq_factor", 4.0))
        original = float(scaling.get("original_max_position_embeddings", 8192))
        out = []
        for f in freqs:
            wavelength = 2 * math.pi / f
            if wavelength < original / high:
                out.append(f)
            elif wavelength > original / low:
                out.append(f / factor)
            else:
                smooth = (original / wavelength - low) / (high - low)
                out.append((1 - smooth) * f / factor + smooth * f)
        freqs = out
    elif kind == "yarn":
        # Frequencies that turn fewer than `slow` times over the `original` positions are divided by `factor`, those
        # that turn more than `fast` times stay, and a ramp over the pair index joins the two: the pair whose
        # frequency turns t times is at index rotary_dim ln(original / (2 pi t)) / (2 ln theta).
        factor, original = float(scaling["factor"]), float(scaling["original"])

        def index_of(turns: float) -> float:
            return rotary_dim * math.log(original / (2 * math.pi * turns)) / (2 * log_theta)

        low = max(math.floor(index_of(float(scaling["fast"]))), 0)
        high = min(math.ceil(index_of(float(scaling["slow"]))), rotary_dim - 1)
        out = []
        for i, f in enumerate(freqs):
            ramp = min(max((i - low) / max(high - low, 0.001), 0.0), 1.0)
            out.append(f / factor * ramp + f * (1 - ramp))
        freqs = out
    elif kind != "default":
        raise ValueError(f"rotary scaling {kind!r} is not supported")
    return freqs


def rotary_magnitude(scaling: Mapping | None) -> float:
    """What the cosines and sines are multiplied by: 0.1 ln(factor) + 1 under the YaRN rule (a rotated vector grows by
    it, and so does its share of a score), else 1."""
    if scaling and str(scaling.get("rope_type", "default")) == "yarn":
        return 0.1 * math.log(float(scaling["factor"])) + 1.0
    return 1.0


class RotaryEmbedding:
    """Gives the mixer a table [positions, rotary_dim / 2, (cos, sin)] in float32 and the number of rotated
    dimensions. Another position encoding of this role provides the same two things (or `table() is None` for no
    rotation)."""

    def __init__(self, head_dim: int, theta: float, scaling: Mapping | None = None,
                 rotary_dim: int | None = None, pairing: str = "halves") -> None:
        """`pairing`: which dimensions of a head turn together. "halves": i with i + rotary_dim / 2; "interleaved":
        2i with 2i + 1. The kernels rotate halves; a mixer brings another pairing into that layout by reordering
        the rows of its q and k matrices once, at load time (`row_order`), which changes no q . k."""
        if pairing not in ("halves", "interleaved"):
            raise ValueError(f"rotary pairing {pairing!r} is not known (halves, interleaved)")
        self.pairing = pairing
        self.head_dim = int(head_dim)
        self.rotary_dim = int(rotary_dim) if rotary_dim else self.head_dim
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        self.rotated = self.rotary_dim
        """Dimensions of a head that turn. For interleaved pairs of an even head, the kernels are told that the
        whole head turns (`rotary_dim` = head_dim, which is what the products that end in the rotation take): the
        pairs beyond `rotated` get the angle zero, whose cosine and sine are exactly 1 and 0."""
        if pairing == "interleaved" and self.head_dim % 2 == 0:
            self.rotary_dim = self.head_dim
        self.theta = float(theta)
        self.scaling = dict(scaling) if scaling else None
        self._table = None

    @staticmethod
    def parameters(**_) -> dict:
        return {}

    def bind(self, tensors, rt) -> None:
        key = ("rotary", self.rotary_dim, self.rotated, self.theta, tuple(sorted((self.scaling or {}).items())),
               rt.max_length)

        def make() -> torch.Tensor:
            values = rotary_frequencies(self.rotated, self.theta, self.scaling)
            values += [0.0] * ((self.rotary_dim - self.rotated) // 2)  # (pairs that stay as they are)
            freqs = torch.tensor(values, dtype=torch.float64)
            angles = torch.arange(rt.max_length, dtype=torch.float64)[:, None] * freqs[None, :]
            table = (torch.stack([torch.cos(angles), torch.sin(angles)], dim=-1) * rotary_magnitude(self.scaling)) \
                .to(torch.float32)
            return table.contiguous().to(rt.device)

        self._table = rt.shared(key, make)

    def table(self) -> torch.Tensor | None:
        return self._table

    def row_order(self) -> list[int] | None:
        """For each place of a head as the kernels see it, the dimension of the model's head that belongs there (None:
        they are the same). Pair i of an interleaved head, dimensions (2i, 2i + 1), goes to the places
        (i, i + rotary_dim / 2)."""
        if self.pairing == "halves":
            return None
        half = self.rotated // 2
        rest = list(range(self.rotated, self.head_dim))
        if self.rotary_dim == self.rotated:  # (an odd head: the rest lies behind the rotated places)
            return [2 * i for i in range(half)] + [2 * i + 1 for i in range(half)] + rest
        # the whole head is a rotation of halves: the dimensions that do not turn fill both halves up, as pairs
        # with the angle zero
        return [2 * i for i in range(half)] + rest[:len(rest) // 2] + \
            [2 * i + 1 for i in range(half)] + rest[len(rest) // 2:]


register_part("position", "rotary", RotaryEmbedding)
