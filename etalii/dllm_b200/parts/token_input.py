"""What a layer adds to the stream from the step's token ids themselves: a second embedding table gives every token a
row, of which this layer takes its own stretch e [dim]; gated by the stream and projected back,

    g = act(W_gate x) * e;   y = W_proj g;   x <- x + y / sqrt(mean(y^2) + eps) * weight,

x being the float32 stream as it is (no norm in front). The table is one tensor for all layers (every layer names it
and they share the device copy); the gate's activation, the stretch and eps are parameters. The two products are the
library's own; the reduction of the second one is the stretch's width, padded with zeros to what the products read in
one piece."""
from __future__ import annotations

import torch

from ..kernels import ops
from .norm import row_rule
from .registry import register_part
from .spec import ParamSpec


class GatedTokenInput:
    def __init__(self, hidden_size: int, vocab_size: int, dim: int, table_width: int, offset: int, eps: float,
                 activation: str = "gelu_tanh") -> None:
        self.hidden_size, self.vocab_size, self.dim = int(hidden_size), int(vocab_size), int(dim)
        self.table_width, self.offset, self.eps = int(table_width), int(offset), float(eps)
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation {activation!r} is not known ({', '.join(map(str, ops.ACTIVATIONS))})")
        if self.offset < 0 or self.offset + self.dim > self.table_width:
            raise ValueError(f"the stretch {self.offset} .. {self.offset + self.dim} is outside a table row of "
                             f"{self.table_width}")
        self.activation = activation
        self.padded = -(-self.dim // 8) * 8
        self.table = self.w_gate = self.w_proj = self.weight = None

    @staticmethod
    def parameters(hidden_size, vocab_size, dim, table_width, **_) -> dict[str, ParamSpec]:
        return {"table": ParamSpec((int(vocab_size), int(table_width))), "gate": ParamSpec((int(dim), hidden_size)),
                "proj": ParamSpec((hidden_size, int(dim))), "norm": ParamSpec((hidden_size,), "ones")}

    def supports(self, rt) -> str | None:
        return row_rule(rt, hidden_size=self.hidden_size)

    def bind(self, tensors, rt) -> None:
        self.table = rt.to_device(tensors["table"], rt.dtype)
        self.w_gate = rt.to_device(tensors["gate"], rt.dtype)
        proj = torch.zeros(self.hidden_size, self.padded, dtype=rt.dtype)
        proj[:, :self.dim] = tensors["proj"].to(rt.dtype)
        self.w_proj = proj.contiguous().to(rt.device)
        self.weight = rt.to_device(tensors["norm"], torch.float32)

    def forward(self, x: torch.Tensor, batch, rt) -> None:
        n = batch.n_tokens
        operand = x
        if rt.dtype != torch.float32:
            operand = rt.ws.buffer("stream_operand", tuple(x.shape), rt.dtype)
            ops.cast_rows(operand, x)
        z = rt.ws.buffer("token_gate", (n, self.dim), torch.float32)
        # (few rows of a long reduction: a block per 16 weight rows would be a handful of blocks, so the reduction is
        # split over the blocks of a cluster)
        narrow = rt.dtype == torch.bfloat16 and n <= 16 and self.dim <= 256 and self.hidden_size >= 1024
        ops.gemm(z, operand, self.w_gate, ops.EPI_STORE_F32, kernel=6 if narrow else 0)
        gated = rt.ws.buffer("token_gated", (n, self.padded), rt.dtype)
        ops.gate_embed(gated, z, self.table, self.offset, self.dim, batch.tokens, ops.ACTIVATIONS[self.activation])
        y = rt.ws.buffer("sublayer_out", tuple(x.shape), torch.float32)
        ops.gemm(y, gated, self.w_proj, ops.EPI_STORE_F32)
        ops.norm_add_residual(x, y, self.weight, self.eps)

    def kernel_libraries(self, rt) -> set[str]:
        if rt.dtype != torch.bfloat16:
            return {"gemm_simt", "elementwise"}
        return {"gemv", "gemv_cluster", "gemm_tcgen05", "elementwise"}


register_part("token_input", "gated_token_input", GatedTokenInput)
