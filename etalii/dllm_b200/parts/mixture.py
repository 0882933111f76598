"""A mixture of gated feed-forward experts. A router gives every token a logit per expert, z = W_r h + b in float32;
the `top` experts with the largest logits run for the token, weighted by the softmax over those logits only, and the
weighted sum of their outputs is the part's output. Every expert is a clamped gated unit: g = min(W_gate h, limit),
u = clamp(W_up h, -limit, limit), W_down (g sigmoid(alpha g) (u + shift)). An optional shared expert (any registered
feed-forward) runs for every token and is added.

The experts' weights are stacked, [experts, 2 ff, width] with gate and up rows interleaved and [experts, width, ff],
and the kernels (csrc/moe.cu) find a token's experts on the device: a step has the same launches whatever the router
chooses, so a decode step with a mixture is captured in a CUDA graph like any other."""
from __future__ import annotations

import torch

from ..kernels import ops
from .norm import NormedInput, StreamOperand, row_rule
from .registry import build_part, part_factory, register_part
from .spec import ParamSpec, PartSpec


class ClampedGLUExperts:
    accepts_stream = True

    def __init__(self, hidden_size: int, intermediate_size: int, experts: int, top: int, limit: float,
                 alpha: float = 1.702, shift: float = 1.0, router_bias: bool = True,
                 shared: PartSpec | None = None) -> None:
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.experts, self.top = int(experts), int(top)
        if not 1 <= self.top <= self.experts:
            raise ValueError(f"top {top} of {experts} experts")
        self.limit, self.alpha, self.shift = float(limit), float(alpha), float(shift)
        self.router_bias = bool(router_bias)
        self.shared = build_part("feed_forward", shared) if shared is not None else None
        self.w_gate_up = self.w_down = self.router = self.bias = None

    @staticmethod
    def parameters(hidden_size, intermediate_size, experts, router_bias=True, shared=None, **_) -> dict[str, ParamSpec]:
        out = {"router": ParamSpec((int(experts), hidden_size))}
        if router_bias:
            out["router_bias"] = ParamSpec((int(experts),))
        for e in range(int(experts)):
            out[f"e{e}.gate"] = ParamSpec((intermediate_size, hidden_size))
            out[f"e{e}.up"] = ParamSpec((intermediate_size, hidden_size))
            out[f"e{e}.down"] = ParamSpec((hidden_size, intermediate_size))
        if shared is not None:
            declared = part_factory("feed_forward", shared.kind).parameters(**dict(shared.params))
            out.update({f"shared.{name}": param for name, param in declared.items()})
        return out

    def supports(self, rt) -> str | None:
        if self.experts > 256 or self.top > 16:
            return f"{self.experts} experts, top {self.top}: the router kernel takes at most 256 and 16"
        if self.shared is not None and hasattr(self.shared, "supports"):
            reason = self.shared.supports(rt)
            if reason:
                return f"shared: {reason}"
        return row_rule(rt, hidden_size=self.hidden_size)

    def bind(self, tensors, rt) -> None:
        ff, width = self.intermediate_size, self.hidden_size
        gate_up = torch.stack([torch.stack([tensors[f"e{e}.gate"].to(rt.dtype), tensors[f"e{e}.up"].to(rt.dtype)], dim=1)
                               .reshape(2 * ff, width) for e in range(self.experts)])
        down = torch.stack([tensors[f"e{e}.down"].to(rt.dtype) for e in range(self.experts)])
        self.w_gate_up = gate_up.contiguous().to(rt.device)
        self.w_down = down.contiguous().to(rt.device)
        self.router = rt.to_device(tensors["router"], torch.float32)
        self.bias = rt.to_device(tensors["router_bias"], torch.float32) if self.router_bias else None
        if self.shared is not None:
            self.shared.bind({name[len("shared."):]: t for name, t in tensors.items() if name.startswith("shared.")}, rt)

    def forward(self, h, residual: torch.Tensor, batch, rt, epilogue: int = ops.EPI_RESIDUAL) -> None:
        """h: the activations [tokens, hidden], or the stream still to be rounded (`StreamOperand`: the router then
        reads the float32 stream), or a pending norm. Adds into `residual` (float32), or writes it with
        `epilogue=ops.EPI_STORE_F32`."""
        if isinstance(h, NormedInput):
            h = h.tensor()
        if isinstance(h, StreamOperand):
            routed, h = h.x, h.tensor()
        else:
            routed = h
        n = h.shape[0]
        chosen = rt.ws.buffer("experts_chosen", (n, self.top), torch.int32)
        weights = rt.ws.buffer("experts_weights", (n, self.top), torch.float32)
        ops.moe_route(chosen, weights, routed, self.router, self.bias, self.top)
        act = rt.ws.buffer("experts_act", (n * self.top, self.intermediate_size), rt.dtype)
        adds = epilogue == ops.EPI_RESIDUAL
        if ops.moe_grouped_supported(n, rt.dtype, self.hidden_size, self.intermediate_size):
            # many tokens: the pairs in expert order, every expert's rows as tile products
            offsets = rt.ws.buffer("experts_offsets", (self.experts + 1,), torch.int32)
            places = rt.ws.buffer("experts_places", (n * self.top,), torch.int32)
            pairs_out = rt.ws.buffer("experts_out", (n * self.top, self.hidden_size), torch.float32)
            ops.moe_experts_grouped(residual, h, self.w_gate_up, self.w_down, chosen, weights, self.top, self.limit,
                                    self.alpha, self.shift, offsets, places, act, pairs_out, accumulate=adds)
        else:
            ops.moe_up(act, h, self.w_gate_up, chosen, self.top, self.limit, self.alpha, self.shift)
            ops.moe_down(residual, act, self.w_down, chosen, weights, self.top, accumulate=adds)
        if self.shared is not None:
            self.shared.forward(h, residual, batch, rt)  # (adds)

    def kernel_libraries(self, rt) -> set[str]:
        names = {"moe", "elementwise"}
        if rt.dtype == torch.bfloat16 and self.hidden_size % 8 == 0 and self.intermediate_size % 8 == 0:
            names.add("moe_grouped")
        if self.shared is not None and hasattr(self.shared, "kernel_libraries"):
            names |= set(self.shared.kernel_libraries(rt))
        return names


class ActivationExperts:
    """A mixture of experts without gate matrices: every expert is W_down act(W_up h) (the activation by name, no
    biases). `weights` says what a chosen expert counts for: "softmax_all", its share of the softmax over ALL
    experts' router logits, as it is (the chosen shares do not add up to one); "softmax_chosen", the softmax over the
    chosen logits only. The router has no bias unless `router_bias`. An optional shared feed-forward (any registered
    kind) runs for every token and is added. Stacked weights [experts, ff, width] and [experts, width, ff]; a token's
    experts are found on the device, so a step's launches do not depend on the router's choice."""

    accepts_stream = True

    def __init__(self, hidden_size: int, intermediate_size: int, experts: int, top: int,
                 activation: str = "relu_squared", weights: str = "softmax_all", router_bias: bool = False,
                 shared: PartSpec | None = None) -> None:
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.experts, self.top = int(experts), int(top)
        if not 1 <= self.top <= self.experts:
            raise ValueError(f"top {top} of {experts} experts")
        if ops.ACTIVATIONS.get(activation, 0) == 0:
            raise ValueError(f"activation {activation!r} is not known (gelu, gelu_tanh, relu_squared)")
        if weights not in ("softmax_all", "softmax_chosen"):
            raise ValueError(f"weights {weights!r}: softmax_all or softmax_chosen")
        self.activation, self.weights, self.router_bias = activation, weights, bool(router_bias)
        self.shared = build_part("feed_forward", shared) if shared is not None else None
        self.w_up = self.w_down = self.router = self.bias = None

    @staticmethod
    def parameters(hidden_size, intermediate_size, experts, router_bias=False, shared=None, **_) -> dict[str, ParamSpec]:
        out = {"router": ParamSpec((int(experts), hidden_size))}
        if router_bias:
            out["router_bias"] = ParamSpec((int(experts),))
        for e in range(int(experts)):
            out[f"e{e}.up"] = ParamSpec((intermediate_size, hidden_size))
            out[f"e{e}.down"] = ParamSpec((hidden_size, intermediate_size))
        if shared is not None:
            declared = part_factory("feed_forward", shared.kind).parameters(**dict(shared.params))
            out.update({f"shared.{name}": param for name, param in declared.items()})
        return out

    def supports(self, rt) -> str | None:
        if self.experts > 256 or self.top > 16:
            return f"{self.experts} experts, top {self.top}: the router kernel takes at most 256 and 16"
        if self.shared is not None and hasattr(self.shared, "supports"):
            reason = self.shared.supports(rt)
            if reason:
                return f"shared: {reason}"
        return row_rule(rt, hidden_size=self.hidden_size)

    def bind(self, tensors, rt) -> None:
        self.w_up = torch.stack([tensors[f"e{e}.up"].to(rt.dtype) for e in range(self.experts)]).contiguous() \
            .to(rt.device)
        self.w_down = torch.stack([tensors[f"e{e}.down"].to(rt.dtype) for e in range(self.experts)]).contiguous() \
            .to(rt.device)
        self.router = rt.to_device(tensors["router"], torch.float32)
        self.bias = rt.to_device(tensors["router_bias"], torch.float32) if self.router_bias else None
        if self.shared is not None:
            self.shared.bind({name[len("shared."):]: t for name, t in tensors.items() if name.startswith("shared.")}, rt)

    def forward(self, h, residual: torch.Tensor, batch, rt, epilogue: int = ops.EPI_RESIDUAL) -> None:
        """h: the activations [tokens, hidden], the stream still to be rounded (`StreamOperand`: the router then reads
        the float32 stream), or a pending norm. Adds into `residual` (float32), or writes it with
        `epilogue=ops.EPI_STORE_F32`."""
        if isinstance(h, NormedInput):
            h = h.tensor()
        if isinstance(h, StreamOperand):
            routed, h = h.x, h.tensor()
        else:
            routed = h
        n = h.shape[0]
        chosen = rt.ws.buffer("experts_chosen", (n, self.top), torch.int32)
        weights = rt.ws.buffer("experts_weights", (n, self.top), torch.float32)
        ops.moe_route(chosen, weights, routed, self.router, self.bias, self.top,
                      all_experts=self.weights == "softmax_all")
        act = rt.ws.buffer("experts_act", (n * self.top, self.intermediate_size), rt.dtype)
        adds = epilogue == ops.EPI_RESIDUAL
        kind = ops.ACTIVATIONS[self.activation]
        if ops.moe_grouped_supported(n, rt.dtype, self.hidden_size, self.intermediate_size) and \
                ops.moe_plain_grouped_built():
            offsets = rt.ws.buffer("experts_offsets", (self.experts + 1,), torch.int32)
            places = rt.ws.buffer("experts_places", (n * self.top,), torch.int32)
            pairs_out = rt.ws.buffer("experts_out", (n * self.top, self.hidden_size), torch.float32)
            ops.moe_plain_experts_grouped(residual, h, self.w_up, self.w_down, chosen, weights, self.top, kind, offsets,
                                          places, act, pairs_out, accumulate=adds)
        else:
            ops.moe_up_plain(act, h, self.w_up, chosen, self.top, kind)
            ops.moe_down(residual, act, self.w_down, chosen, weights, self.top, accumulate=adds)
        if self.shared is not None:
            self.shared.forward(h, residual, batch, rt)  # (adds)

    def kernel_libraries(self, rt) -> set[str]:
        names = {"moe", "elementwise"}
        if rt.dtype == torch.bfloat16 and self.hidden_size % 8 == 0 and self.intermediate_size % 8 == 0:
            names.add("moe_grouped")
        if self.shared is not None and hasattr(self.shared, "kernel_libraries"):
            names |= set(self.shared.kernel_libraries(rt))
        return names


register_part("feed_forward", "clamped_glu_experts", ClampedGLUExperts)
register_part("feed_forward", "activation_experts", ActivationExperts)
