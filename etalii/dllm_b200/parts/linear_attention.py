"""Mixers whose memory is one matrix per head, S [dim, vdim] in float32, instead of a list of keys and values. A token
writes an outer product k v^T into S and reads S^T q; what differs between the kinds is how S shrinks between tokens
and what the write is:

  "decay_linear_attention": S <- decay_h S + k v^T with a fixed decay per head (retention, lightning attention);
  "gated_delta_rule":       S <- g S; S <- S + k (beta (v - S^T k))^T with a decay g and a step size beta per token
                            and head, q and k unit vectors after a short causal convolution over time;
  "gated_matrix_memory":    S <- a_t S + b_t k v^T with exponential input gates held in range by a running maximum of the
                            log gates, a normaliser n carried beside S, the read-out divided by max(|n . q|, e^-m).

S lives in the cache's fixed-size state, one per slot and cache entry, starts at zero when a slot is taken and is
carried from step to step; the kernels (csrc/recurrent.cu) walk a step's tokens in order, so a prompt may be cut
anywhere. Projections run in the activation type and leave float32 rows; the recurrence, its inputs' scaling, the
decays, the norms of the read-out and the gates are float32."""
from __future__ import annotations

import torch

from ..cache.paged import CacheNeed
from ..kernels import ops
from .norm import row_rule
from .registry import register_part
from .spec import ParamSpec

_GATES = {"silu": ops.GATE_SILU, "sigmoid": ops.GATE_SIGMOID}


def _libraries(rt) -> set[str]:
    if rt.dtype != torch.bfloat16:
        return {"gemm_simt", "elementwise", "recurrent"}
    return {"gemv", "gemv_cluster", "gemm_tcgen05", "elementwise", "recurrent"}


class DecayLinearAttention:
    """q, k [heads x dim] and v [heads x vdim] projected from h (through silu if `input_activation` says so), k times
    `key_scale`; per head S <- decay_h S + k v^T, o = S^T q. The read-out is divided by its root mean square, per
    head (`norm` "head") or over all heads together ("all"), times a weight if `norm_weight` (one value per place of
    the group), times gate(W_g h) (`gate` "silu" or "sigmoid"), and projected by W_o."""

    def __init__(self, hidden_size: int, heads: int, dim: int, vdim: int, decay, eps: float,
                 input_activation: str | None = None, key_scale: float = 1.0, norm: str = "head",
                 norm_weight: bool = False, gate: str = "silu") -> None:
        self.hidden_size, self.heads, self.dim, self.vdim = int(hidden_size), int(heads), int(dim), int(vdim)
        self.decay_values = [float(d) for d in decay]
        if len(self.decay_values) != self.heads:
            raise ValueError(f"{len(self.decay_values)} decays for {self.heads} heads")
        if input_activation not in (None, "silu"):
            raise ValueError(f"input activation {input_activation!r}: none or silu")
        if norm not in ("head", "all") or gate not in _GATES:
            raise ValueError("norm: head or all; gate: silu or sigmoid")
        self.eps, self.input_activation, self.key_scale = float(eps), input_activation, float(key_scale)
        self.norm, self.norm_weight, self.gate = norm, bool(norm_weight), gate
        self.w_in = self.w_o = self.decay = self.weight = None

    @staticmethod
    def parameters(hidden_size, heads, dim, vdim, norm="head", norm_weight=False, **_) -> dict[str, ParamSpec]:
        qk, values = int(heads) * int(dim), int(heads) * int(vdim)
        out = {"q": ParamSpec((qk, hidden_size)), "k": ParamSpec((qk, hidden_size)),
               "v": ParamSpec((values, hidden_size)), "g": ParamSpec((values, hidden_size)),
               "o": ParamSpec((hidden_size, values))}
        if norm_weight:
            out["norm"] = ParamSpec((values if norm == "all" else int(vdim),), "ones")
        return out

    def supports(self, rt) -> str | None:
        if self.dim % 4 or self.dim > 256:
            return f"dim {self.dim}: the scan keeps a head's rows in 16-byte pieces, a multiple of 4 up to 256"
        return row_rule(rt, hidden_size=self.hidden_size, **{"heads x vdim": self.heads * self.vdim})

    def cache_need(self) -> CacheNeed:
        return CacheNeed("state", state_shape=(self.heads, self.vdim, self.dim))  # (a column's rows contiguous)

    def bind(self, tensors, rt) -> None:
        fused = torch.cat([tensors[name].to(rt.dtype) for name in ("q", "k", "v", "g")], dim=0)
        self.w_in = fused.contiguous().to(rt.device)
        self.w_o = rt.to_device(tensors["o"], rt.dtype)
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=rt.device)
        self.weight = rt.to_device(tensors["norm"], torch.float32) if self.norm_weight else None

    def forward(self, h: torch.Tensor, residual: torch.Tensor, batch, state, rt, write_cache: bool = True,
                epilogue: int = ops.EPI_RESIDUAL) -> None:
        n = batch.n_tokens
        qk, values = self.heads * self.dim, self.heads * self.vdim
        rows = rt.ws.buffer("mixer_rows", (n, 2 * qk + 2 * values), torch.float32)
        ops.gemm(rows, h, self.w_in, ops.EPI_STORE_F32)
        read = rt.ws.buffer("mixer_read", (n, values), torch.float32)
        ops.decay_scan(read, rows, 0, qk, 2 * qk, self.heads, self.dim, self.vdim, self.decay,
                       self.input_activation == "silu", self.key_scale, state, batch)
        gated = rt.ws.buffer("mixer_gated", (n, values), rt.dtype)
        ops.gated_norm(gated, read, self.weight, rows, 2 * qk + values, values if self.norm == "all" else self.vdim,
                       self.eps, _GATES[self.gate])
        ops.gemm(residual, gated, self.w_o, epilogue)

    def kernel_libraries(self, rt) -> set[str]:
        return _libraries(rt)


class GatedDeltaRule:
    """q, k [qk_heads x dim] and v [heads x vdim] projected from h; each passes a causal convolution over time per
    channel (`conv` taps, the last one on the token itself) and silu; q and k become unit vectors per head (q times
    dim^-1/2). beta = sigmoid(W_b h) and g = exp(-exp(A_log) softplus(W_a h + dt_bias)) per head. Head h uses q/k
    head h // (heads / qk_heads). Per head: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q. The read-out
    is divided by its root mean square per head, times a weight [vdim] shared by the heads, times silu(W_g h), and
    projected by W_o. Besides S the last conv - 1 inputs of the convolution are state."""

    UNIT_EPS = 1e-6  # (inside the kernel: x / sqrt(sum x^2 + 1e-6))

    def __init__(self, hidden_size: int, heads: int, qk_heads: int, dim: int, vdim: int, conv: int,
                 eps: float) -> None:
        self.hidden_size, self.heads, self.qk_heads = int(hidden_size), int(heads), int(qk_heads)
        self.dim, self.vdim, self.conv, self.eps = int(dim), int(vdim), int(conv), float(eps)
        if self.heads % self.qk_heads:
            raise ValueError(f"{self.heads} heads are not a multiple of {self.qk_heads} q/k heads")
        self.channels = 2 * self.qk_heads * self.dim + self.heads * self.vdim
        self.w_in = self.w_o = self.taps = self.a_log = self.dt_bias = self.weight = None

    @staticmethod
    def parameters(hidden_size, heads, qk_heads, dim, vdim, conv, **_) -> dict[str, ParamSpec]:
        qk, values = int(qk_heads) * int(dim), int(heads) * int(vdim)
        return {"q": ParamSpec((qk, hidden_size)), "k": ParamSpec((qk, hidden_size)),
                "v": ParamSpec((values, hidden_size)), "g": ParamSpec((values, hidden_size)),
                "b": ParamSpec((int(heads), hidden_size)), "a": ParamSpec((int(heads), hidden_size)),
                "q_conv": ParamSpec((qk, int(conv))), "k_conv": ParamSpec((qk, int(conv))),
                "v_conv": ParamSpec((values, int(conv))), "A_log": ParamSpec((int(heads),)),
                "dt_bias": ParamSpec((int(heads),)), "norm": ParamSpec((int(vdim),), "ones"),
                "o": ParamSpec((hidden_size, values))}

    def supports(self, rt) -> str | None:
        if self.dim % 4 or self.dim > 256:
            return f"dim {self.dim}: the scan keeps a head's rows in 16-byte pieces, a multiple of 4 up to 256"
        if not 1 <= self.conv <= 16:
            return f"a convolution of {self.conv} taps: the kernel takes 1 to 16"
        return row_rule(rt, hidden_size=self.hidden_size, **{"heads x vdim": self.heads * self.vdim})

    def cache_need(self) -> CacheNeed:
        matrix = CacheNeed("state", state_shape=(self.heads, self.vdim, self.dim))
        if self.conv == 1:
            return matrix
        return CacheNeed("several", parts=(matrix, CacheNeed("state", state_shape=(self.conv - 1, self.channels))))

    def bind(self, tensors, rt) -> None:
        fused = torch.cat([tensors[name].to(rt.dtype) for name in ("q", "k", "v", "g", "b", "a")], dim=0)
        self.w_in = fused.contiguous().to(rt.device)
        self.w_o = rt.to_device(tensors["o"], rt.dtype)
        taps = torch.cat([tensors[name].float() for name in ("q_conv", "k_conv", "v_conv")], dim=0)
        self.taps = taps.contiguous().to(rt.device)
        self.a_log = rt.to_device(tensors["A_log"], torch.float32)
        self.dt_bias = rt.to_device(tensors["dt_bias"], torch.float32)
        self.weight = rt.to_device(tensors["norm"], torch.float32)

    def forward(self, h: torch.Tensor, residual: torch.Tensor, batch, state, rt, write_cache: bool = True,
                epilogue: int = ops.EPI_RESIDUAL) -> None:
        n = batch.n_tokens
        matrix, history = (state, None) if self.conv == 1 else state
        values = self.heads * self.vdim
        rows = rt.ws.buffer("mixer_rows", (n, self.channels + values + 2 * self.heads), torch.float32)
        ops.gemm(rows, h, self.w_in, ops.EPI_STORE_F32)
        prepared = rt.ws.buffer("mixer_prepared", (n, self.channels), torch.float32)
        aux = rt.ws.buffer("mixer_aux", (n, 2 * self.heads + self.qk_heads), torch.float32)
        ops.delta_prepare(prepared, aux, rows, self.channels + values, self.channels + values + self.heads, self.taps,
                          self.a_log, self.dt_bias, history, self.heads, self.qk_heads, self.dim, self.vdim, batch)
        read = rt.ws.buffer("mixer_read", (n, values), torch.float32)
        ops.delta_scan(read, prepared, aux, self.heads, self.qk_heads, self.dim, self.vdim, matrix, batch)
        gated = rt.ws.buffer("mixer_gated", (n, values), rt.dtype)
        ops.gated_norm(gated, read, self.weight, rows, self.channels, self.vdim, self.eps, ops.GATE_SILU)
        ops.gemm(residual, gated, self.w_o, epilogue)

    def kernel_libraries(self, rt) -> set[str]:
        return _libraries(rt)


class GatedMatrixMemory:
    """q = W_q h * dim^-1/2, k = W_k h [heads x dim], v = W_v h [heads x vdim]. Per head a log input gate
    i = cap tanh((W_i h + b_i) / cap) and a log forget gate f = logsigmoid(cap tanh((W_f h + b_f) / cap)); with a running
    maximum m (zero at a sequence's start) m' = max(f + m, i):

        S' = exp(f + m - m') S + exp(i - m') k v^T,   n' likewise with k alone,
        o  = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6).

    Each head's o is divided by its root mean square, the heads together are multiplied by a weight [heads x vdim]
    and by sigmoid(W_g h), and projected by W_o. S and n are one state tensor [heads, vdim + 1, dim] (n is the column
    of S that a value of 1 writes), m a second one [heads]; both float32, zero when a slot is taken, carried from
    step to step. Gates, maximum, exponentials, state, read-out and norm are float32."""

    def __init__(self, hidden_size: int, heads: int, dim: int, vdim: int, gate_cap: float, eps: float) -> None:
        self.hidden_size, self.heads, self.dim, self.vdim = int(hidden_size), int(heads), int(dim), int(vdim)
        self.gate_cap, self.eps = float(gate_cap), float(eps)
        self.padded = -(-self.dim // 4) * 4
        """A head's q and k as the scan sees them: rows of zeros fill `dim` up to a multiple of 4 (they change no
        q . k and leave their rows of S zero)."""
        self.w_in = self.w_o = self.i_bias = self.f_bias = self.weight = None

    @staticmethod
    def parameters(hidden_size, heads, dim, vdim, **_) -> dict[str, ParamSpec]:
        qk, values = int(heads) * int(dim), int(heads) * int(vdim)
        return {"q": ParamSpec((qk, hidden_size)), "k": ParamSpec((qk, hidden_size)),
                "v": ParamSpec((values, hidden_size)), "g": ParamSpec((values, hidden_size)),
                "i": ParamSpec((int(heads), hidden_size)), "i_bias": ParamSpec((int(heads),)),
                "f": ParamSpec((int(heads), hidden_size)), "f_bias": ParamSpec((int(heads),)),
                "norm": ParamSpec((values,), "ones"), "o": ParamSpec((hidden_size, values))}

    def supports(self, rt) -> str | None:
        if self.dim > 256:
            return f"dim {self.dim}: the scan keeps a head's rows in registers, at most 256"
        return row_rule(rt, hidden_size=self.hidden_size, **{"heads x vdim": self.heads * self.vdim})

    def cache_need(self) -> CacheNeed:
        return CacheNeed("several", parts=(CacheNeed("state", state_shape=(self.heads, self.vdim + 1, self.padded)),
                                           CacheNeed("state", state_shape=(self.heads,))))

    def bind(self, tensors, rt) -> None:
        def heads_padded(w):
            if self.padded == self.dim:
                return w.to(rt.dtype)
            out = torch.zeros(self.heads, self.padded, self.hidden_size, dtype=rt.dtype)
            out[:, :self.dim] = w.to(rt.dtype).view(self.heads, self.dim, self.hidden_size)
            return out.view(self.heads * self.padded, self.hidden_size)

        fused = torch.cat([heads_padded(tensors["q"]), heads_padded(tensors["k"])] +
                          [tensors[name].to(rt.dtype) for name in ("v", "g", "i", "f")], dim=0)
        self.w_in = fused.contiguous().to(rt.device)
        self.w_o = rt.to_device(tensors["o"], rt.dtype)
        self.i_bias = rt.to_device(tensors["i_bias"], torch.float32)
        self.f_bias = rt.to_device(tensors["f_bias"], torch.float32)
        self.weight = rt.to_device(tensors["norm"], torch.float32)

    def forward(self, h: torch.Tensor, residual: torch.Tensor, batch, state, rt, write_cache: bool = True,
                epilogue: int = ops.EPI_RESIDUAL) -> None:
        n = batch.n_tokens
        matrix, maximum = state
        heads, qk, values = self.heads, self.heads * self.padded, self.heads * self.vdim
        rows = rt.ws.buffer("mixer_rows", (n, 2 * qk + 2 * values + 2 * heads), torch.float32)
        ops.gemm(rows, h, self.w_in, ops.EPI_STORE_F32)
        aux = rt.ws.buffer("mixer_aux", (n, 3 * heads), torch.float32)
        gates_at = 2 * qk + 2 * values
        ops.running_max_gates(aux, rows, gates_at, gates_at + heads, self.i_bias, self.f_bias, self.gate_cap, heads,
                              maximum, batch)
        read = rt.ws.buffer("mixer_read", (n, values), torch.float32)
        nq = rt.ws.buffer("mixer_nq", (n, heads), torch.float32)
        ops.gated_scan(read, nq, rows, 0, qk, 2 * qk, heads, self.padded, self.vdim, aux, self.dim ** -0.5, matrix,
                       batch)
        gated = rt.ws.buffer("mixer_gated", (n, values), rt.dtype)
        ops.normalised_readout(gated, read, nq, aux, 2 * heads, self.weight, rows, 2 * qk + values, heads, self.vdim,
                               self.eps)
        ops.gemm(residual, gated, self.w_o, epilogue)

    def kernel_libraries(self, rt) -> set[str]:
        return _libraries(rt)


register_part("mixer", "decay_linear_attention", DecayLinearAttention)
register_part("mixer", "gated_matrix_memory", GatedMatrixMemory)
register_part("mixer", "gated_delta_rule", GatedDeltaRule)
