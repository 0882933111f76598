"""The SwiGLU feed-forward: down(silu(gate(h)) * up(h)). Gate and up are one matrix product whose rows interleave
(row 2i = gate_i, row 2i + 1 = up_i) so the product's epilogue applies silu(gate) * up on the accumulators; the down
projection adds into the residual in its epilogue (reference: src/etalii_dllm/transformer.py:548-558,
cpp/include/dllm/nn.hpp:467-492)."""
from __future__ import annotations

import torch

from ..kernels import ops
from .norm import NormedInput, project, row_rule
from .registry import register_part
from .spec import ParamSpec


class SwiGLU:
    accepts_pending_norm = True

    def __init__(self, hidden_size: int, intermediate_size: int) -> None:
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.w_gate_up = self.w_down = None

    @staticmethod
    def parameters(hidden_size, intermediate_size) -> dict[str, ParamSpec]:
        return {"gate": ParamSpec((intermediate_size, hidden_size)), "up": ParamSpec((intermediate_size, hidden_size)),
                "down": ParamSpec((hidden_size, intermediate_size))}

    def supports(self, rt) -> str | None:
        return row_rule(rt, hidden_size=self.hidden_size, intermediate_size=self.intermediate_size)

    def bind(self, tensors, rt) -> None:
        gate, up = tensors["gate"].to(rt.dtype), tensors["up"].to(rt.dtype)
        fused = torch.stack([gate, up], dim=1).reshape(2 * self.intermediate_size, self.hidden_size)
        self.w_gate_up = fused.contiguous().to(rt.device)
        self.w_down = rt.to_device(tensors["down"], rt.dtype)

    def absorb_input_scale(self, scale: torch.Tensor) -> bool:
        """Takes a per-input-feature scale (the weight of the norm in front) into the columns of the gate/up
        matrix (bfloat16 only)."""
        if self.w_gate_up is None or self.w_gate_up.dtype != torch.bfloat16:
            return False
        self.w_gate_up = (self.w_gate_up.float() * scale.to(self.w_gate_up.device).float()[None, :]) \
            .to(torch.bfloat16).contiguous()
        return True

    def forward(self, h: torch.Tensor, residual: torch.Tensor, batch, rt) -> None:
        rows = h.shape[0]
        if ops.FUSED_FEED_FORWARD and isinstance(h, NormedInput) and h.x is residual and \
                rt.dtype == torch.bfloat16 and ops.mlp_decode_supported(rows, self.hidden_size, self.intermediate_size):
            # (an option, off by default: norm, gate/up, SwiGLU, down and the residual sum in one kernel)
            scratch = rt.ws.buffer("mlp_partial", (ops.mlp_decode_scratch(rows, self.hidden_size,
                                                                          self.intermediate_size),), torch.float32)
            ops.mlp_decode(residual, h.weight, h.eps, self.w_gate_up, self.w_down, scratch,
                           rt.ws.zeros("mlp_tickets", 8, torch.int32))
            return
        act = rt.ws.buffer("ffn_act", (h.shape[0], self.intermediate_size), rt.dtype)
        project(act, h, self.w_gate_up, ops.EPI_SWIGLU)
        ops.gemm(residual, act, self.w_down, ops.EPI_RESIDUAL)


    def kernel_libraries(self, rt) -> set[str]:
        if rt.dtype != torch.bfloat16:
            return {"gemm_simt"}
        names = {"gemv", "gemm_tcgen05"}
        if any(ops.splits_over_clusters(64, w.shape[0], w.shape[1]) for w in (self.w_gate_up, self.w_down)):
            names.add("gemv_cluster")  # (steps of 17 to 64 tokens with weights this small)
        if ops.FUSED_FEED_FORWARD and ops.mlp_decode_supported(1, self.hidden_size, self.intermediate_size):
            names.add("mlp_decode")
        if any(ops.streams_through_shared_memory(1, w.shape[0], w.shape[1]) for w in (self.w_gate_up, self.w_down)):
            names.add("gemv_tma")
        return names


class ClampedGLU:
    """A gated feed-forward whose pre-activations are clamped: g = min(gate(h), limit), u = clamp(up(h), -limit,
    limit); down(g * sigmoid(alpha * g) * (u + shift)). Gate and up are one product whose rows interleave (row 2i =
    gate_i, row 2i + 1 = up_i). A decode-sized bfloat16 step applies the activation in that product's epilogue (for
    alpha 1.702 and shift 1, which the epilogue has built in); larger steps and float32 store gate and up and run the
    activation as a kernel of its own. The activation is computed in float32 either way."""

    def __init__(self, hidden_size: int, intermediate_size: int, limit: float, alpha: float = 1.702,
                 shift: float = 1.0) -> None:
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.limit, self.alpha, self.shift = float(limit), float(alpha), float(shift)
        self.w_gate_up = self.w_down = None

    @staticmethod
    def parameters(hidden_size, intermediate_size, **_) -> dict[str, ParamSpec]:
        return {"gate": ParamSpec((intermediate_size, hidden_size)), "up": ParamSpec((intermediate_size, hidden_size)),
                "down": ParamSpec((hidden_size, intermediate_size))}

    def supports(self, rt) -> str | None:
        return row_rule(rt, hidden_size=self.hidden_size, intermediate_size=self.intermediate_size)

    def bind(self, tensors, rt) -> None:
        gate, up = tensors["gate"].to(rt.dtype), tensors["up"].to(rt.dtype)
        fused = torch.stack([gate, up], dim=1).reshape(2 * self.intermediate_size, self.hidden_size)
        self.w_gate_up = fused.contiguous().to(rt.device)
        self.w_down = rt.to_device(tensors["down"], rt.dtype)

    def forward(self, h: torch.Tensor, residual: torch.Tensor, batch, rt, epilogue: int = ops.EPI_RESIDUAL) -> None:
        """Adds into `residual` (float32), or with `epilogue=ops.EPI_STORE_F32` writes it."""
        if isinstance(h, NormedInput):
            h = h.tensor()
        rows = h.shape[0]
        act = rt.ws.buffer("ffn_act", (rows, self.intermediate_size), rt.dtype)
        if rt.dtype == torch.bfloat16 and self.alpha == 1.702 and self.shift == 1.0 and \
                ops.glu_clamped_fuses(rows, *self.w_gate_up.shape):
            ops.gemm(act, h, self.w_gate_up, ops.EPI_GLU_CLAMPED, eps=self.limit)
        else:
            both = rt.ws.buffer("ffn_gate_up", (rows, 2 * self.intermediate_size), rt.dtype)
            ops.gemm(both, h, self.w_gate_up, ops.EPI_STORE_T)
            ops.glu_clamped(act, both, self.limit, self.alpha, self.shift)
        ops.gemm(residual, act, self.w_down, epilogue)

    def kernel_libraries(self, rt) -> set[str]:
        if rt.dtype != torch.bfloat16:
            return {"gemm_simt", "elementwise"}
        return {"gemv", "gemv_cluster", "gemm_tcgen05", "elementwise"}


class ActivationMLP:
    """A feed-forward without a gate matrix: down(act(up(h) + b_up)) + b_down, the activation by name ("gelu": the exact
    erf form, "gelu_tanh", "relu_squared"), the biases optional. With `token_gate` the output is multiplied by
    sigmoid(w_g . h), one number per token: the gate's row rides as one more row of the up matrix and multiplies the
    activated values, which the down product is linear in. Bias, activation and gate are one float32 kernel between
    the two products."""

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "gelu", biases: bool = False,
                 token_gate: bool = False) -> None:
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        if ops.ACTIVATIONS.get(activation, 0) == 0:
            raise ValueError(f"activation {activation!r} is not known (gelu, gelu_tanh, relu_squared)")
        self.activation, self.biases, self.token_gate = activation, bool(biases), bool(token_gate)
        if self.biases and self.token_gate:
            raise ValueError("a token gate with biases is not built: the gate multiplies the activated values, and a "
                             "bias behind the down product would escape it")
        self.padded = -(-self.intermediate_size // 8) * 8  # (the down product reads rows in 16-byte pieces)
        self.w_up = self.w_down = self.b_up = self.b_down = None

    @staticmethod
    def parameters(hidden_size, intermediate_size, biases=False, token_gate=False, **_) -> dict[str, ParamSpec]:
        out = {"up": ParamSpec((int(intermediate_size), hidden_size)),
               "down": ParamSpec((hidden_size, int(intermediate_size)))}
        if biases:
            out.update({"up_bias": ParamSpec((int(intermediate_size),)), "down_bias": ParamSpec((hidden_size,))})
        if token_gate:
            out["gate"] = ParamSpec((1, hidden_size))
        return out

    def supports(self, rt) -> str | None:
        return row_rule(rt, hidden_size=self.hidden_size)

    def bind(self, tensors, rt) -> None:
        up = tensors["up"].to(rt.dtype)
        if self.token_gate:
            up = torch.cat([up, tensors["gate"].to(rt.dtype).reshape(1, self.hidden_size)], dim=0)
        self.w_up = up.contiguous().to(rt.device)
        down = torch.zeros(self.hidden_size, self.padded, dtype=rt.dtype)
        down[:, :self.intermediate_size] = tensors["down"].to(rt.dtype)
        self.w_down = down.contiguous().to(rt.device)
        if self.biases:
            self.b_up = rt.to_device(tensors["up_bias"], torch.float32)
            self.b_down = rt.to_device(tensors["down_bias"], torch.float32)

    def forward(self, h: torch.Tensor, residual: torch.Tensor, batch, rt, epilogue: int = ops.EPI_RESIDUAL) -> None:
        """Adds into `residual` (float32), or with `epilogue=ops.EPI_STORE_F32` writes it."""
        if isinstance(h, NormedInput):
            h = h.tensor()
        rows = h.shape[0]
        ff = self.intermediate_size
        pre = rt.ws.buffer("ffn_pre", (rows, self.w_up.shape[0]), torch.float32)
        ops.gemm(pre, h, self.w_up, ops.EPI_STORE_F32)
        act = rt.ws.buffer("ffn_act", (rows, self.padded), rt.dtype)
        ops.bias_act(act, pre, self.b_up, ops.ACTIVATIONS[self.activation], ff, self.token_gate)
        ops.gemm(residual, act, self.w_down, epilogue)
        if self.b_down is not None:
            ops.add_row(residual, self.b_down)

    def kernel_libraries(self, rt) -> set[str]:
        if rt.dtype != torch.bfloat16:
            return {"gemm_simt", "elementwise"}
        return {"gemv", "gemv_cluster", "gemm_tcgen05", "elementwise"}


class GatedMLP:
    """A gated feed-forward with the activation by name: down(act(gate(h)) * up(h)), without biases ("gelu_tanh": the
    tanh form of gelu; "gelu": the erf form; "relu_squared"). Gate and up are one product whose rows interleave (row 2i
    = gate_i, row 2i + 1 = up_i). A decode-sized bfloat16 step applies the activation in that product's epilogue (the
    tanh form of gelu, which the weight-streaming kernels have built in); larger steps and float32 keep the product's
    float32 rows and run the activation as a kernel of its own. The activation is computed in float32 either way."""

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "gelu_tanh") -> None:
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        if ops.ACTIVATIONS.get(activation, 0) == 0:
            raise ValueError(f"activation {activation!r} is not known (gelu, gelu_tanh, relu_squared)")
        self.activation = activation
        self.w_gate_up = self.w_down = None

    @staticmethod
    def parameters(hidden_size, intermediate_size, **_) -> dict[str, ParamSpec]:
        return {"gate": ParamSpec((intermediate_size, hidden_size)), "up": ParamSpec((intermediate_size, hidden_size)),
                "down": ParamSpec((hidden_size, intermediate_size))}

    def supports(self, rt) -> str | None:
        return row_rule(rt, hidden_size=self.hidden_size, intermediate_size=self.intermediate_size)

    def bind(self, tensors, rt) -> None:
        gate, up = tensors["gate"].to(rt.dtype), tensors["up"].to(rt.dtype)
        fused = torch.stack([gate, up], dim=1).reshape(2 * self.intermediate_size, self.hidden_size)
        self.w_gate_up = fused.contiguous().to(rt.device)
        self.w_down = rt.to_device(tensors["down"], rt.dtype)

    def forward(self, h: torch.Tensor, residual: torch.Tensor, batch, rt, epilogue: int = ops.EPI_RESIDUAL) -> None:
        """Adds into `residual` (float32), or with `epilogue=ops.EPI_STORE_F32` writes it."""
        if isinstance(h, NormedInput):
            h = h.tensor()
        rows = h.shape[0]
        act = rt.ws.buffer("ffn_act", (rows, self.intermediate_size), rt.dtype)
        if rt.dtype == torch.bfloat16 and self.activation == "gelu_tanh" and \
                ops.glu_clamped_fuses(rows, *self.w_gate_up.shape):
            ops.gemm(act, h, self.w_gate_up, ops.EPI_GLU_GELU_TANH)
        else:
            both = rt.ws.buffer("ffn_gate_up_f32", (rows, 2 * self.intermediate_size), torch.float32)
            ops.gemm(both, h, self.w_gate_up, ops.EPI_STORE_F32)
            ops.glu_act(act, both, ops.ACTIVATIONS[self.activation])
        ops.gemm(residual, act, self.w_down, epilogue)

    def kernel_libraries(self, rt) -> set[str]:
        if rt.dtype != torch.bfloat16:
            return {"gemm_simt", "elementwise"}
        return {"gemv", "gemv_cluster", "gemm_tcgen05", "elementwise"}


register_part("feed_forward", "gated_mlp", GatedMLP)
register_part("feed_forward", "swiglu", SwiGLU)
register_part("feed_forward", "activation_mlp", ActivationMLP)
register_part("feed_forward", "clamped_glu", ClampedGLU)
