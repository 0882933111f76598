"""A short causal convolution over time between a norm and the part that reads it: every channel of the normed rows is
filtered over the sequence's own earlier tokens and added to the row itself,

    h_t = norm(x_t);   out_t = h_t + sum_j w[:, j] h_(t - taps + 1 + j)     (zeros before the sequence's start),

with one weight per channel and tap, the last tap on the token itself. The last taps - 1 normed rows of a sequence are
state: they live in the cache's fixed-size state (float32, zero when a slot is taken) and are carried from step to
step, so a prompt may be cut anywhere. Norm and filter are one kernel (elementwise.cu::norm_conv_kernel), float32,
rounded once to the activation type."""
from __future__ import annotations

import torch

from ..cache.paged import CacheNeed
from ..kernels import ops
from .registry import register_part
from .spec import ParamSpec


class ShortConvolution:
    MAX_TAPS = 8

    def __init__(self, hidden_size: int, taps: int) -> None:
        self.hidden_size, self.taps = int(hidden_size), int(taps)
        self.weight = None

    @staticmethod
    def parameters(hidden_size, taps) -> dict[str, ParamSpec]:
        return {"weight": ParamSpec((int(hidden_size), int(taps)))}

    def supports(self, rt) -> str | None:
        if not 1 <= self.taps <= self.MAX_TAPS:
            return f"a convolution of {self.taps} taps: the kernel takes 1 to {self.MAX_TAPS}"
        return None

    def cache_need(self) -> CacheNeed | None:
        if self.taps == 1:
            return None
        return CacheNeed("state", state_shape=(self.taps - 1, self.hidden_size))

    def bind(self, tensors, rt) -> None:
        self.weight = rt.to_device(tensors["weight"], torch.float32)

    def forward(self, norm, x: torch.Tensor, batch, history, rt, name: str = "filtered") -> torch.Tensor:
        """norm: an RMS norm with a weight (its `weight` and `eps` go into the kernel); x the float32 stream; history
        the state [slots, taps - 1, hidden] (None for one tap). Returns the filtered rows in the activation type."""
        out = rt.ws.buffer(name, (batch.n_tokens, self.hidden_size), rt.dtype)
        ops.norm_conv(out, x, norm.weight, self.weight, history, norm.eps, batch)
        return out

    def kernel_libraries(self, rt) -> set[str]:
        return {"elementwise"}


register_part("filter", "short_convolution", ShortConvolution)
