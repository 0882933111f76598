"""Grouped-query attention without a softmax, over a sliding window that also keeps a sequence's first positions.

Per token, from the mixer's input h: q = W_q h, k = W_k h, v = W_v h (with `biases`, each plus its bias); with
`whole_norm`, q and k are each divided by the root mean square of the WHOLE projection, all heads at once, and
multiplied by a weight per coordinate. Query head a uses key/value head a / (heads / kv_heads); keys have `dim` values,
values `vdim`. There is no rotation. Position i sees j <= i with i - j < window, and the first `keep_first` positions of
the sequence at any distance (at their true distances). The weight of a visible key is
    w_a(i, j) = sigmoid(q_a . k_j * scale - slope_a (i - j) + b_a),
slope_a = 2^(-distance_exponent (a + 1) / heads) (`distance_exponent` None: no penalty), b_a a learned number per head
(`head_bias`); nothing is normalised over the keys. With `head_mixing` a matrix M [heads, heads] then mixes the heads'
weights, w_a <- sum_g M[a, g] w_g, and head a applies its mixed weights to the values of its own key/value head. With
`gate` the concatenated heads are multiplied element by element by sigmoid(W_g h); W_o follows.

One product makes everything a token needs of h: [q | k | v | gate]. Biases, norms, scores, weights, their mixing, the
sums and the gate are float32; the cache holds keys and values in the activation type."""
from __future__ import annotations

import torch

from ..cache.paged import CacheNeed
from ..kernels import ops
from .norm import row_rule
from .registry import register_part
from .spec import ParamSpec


class SigmoidAttention:
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, dim: int, vdim: int, scale: float,
                 eps: float = 1e-6, window: int | None = None, keep_first: int = 0,
                 distance_exponent: float | None = None, biases: bool = False, whole_norm: bool = False,
                 head_bias: bool = False, head_mixing: bool = False, gate: bool = False) -> None:
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are not a multiple of {num_kv_heads} kv heads")
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.dim, self.vdim, self.scale, self.eps = int(dim), int(vdim), float(scale), float(eps)
        self.window = int(window) if window else 0
        self.keep_first = int(keep_first) if self.window else 0
        self.distance_exponent = None if distance_exponent is None else float(distance_exponent)
        self.biases, self.whole_norm, self.head_bias = bool(biases), bool(whole_norm), bool(head_bias)
        self.head_mixing, self.gate = bool(head_mixing), bool(gate)
        self.w_in = self.w_o = self.bias_rows = self.norm_weights = self.mix = self.slopes = self.head_biases = None

    @staticmethod
    def parameters(hidden_size, num_heads, num_kv_heads, dim, vdim, biases=False, whole_norm=False, head_bias=False,
                   head_mixing=False, gate=False, **_) -> dict[str, ParamSpec]:
        heads, groups, dim, vdim = int(num_heads), int(num_kv_heads), int(dim), int(vdim)
        out = {"q": ParamSpec((heads * dim, hidden_size)), "k": ParamSpec((groups * dim, hidden_size)),
               "v": ParamSpec((groups * vdim, hidden_size)), "o": ParamSpec((hidden_size, heads * vdim))}
        if biases:
            out.update({"q_bias": ParamSpec((heads * dim,)), "k_bias": ParamSpec((groups * dim,)),
                        "v_bias": ParamSpec((groups * vdim,))})
        if whole_norm:
            out.update({"q_norm": ParamSpec((heads * dim,), "ones"), "k_norm": ParamSpec((groups * dim,), "ones")})
        if head_bias:
            out["pb"] = ParamSpec((heads,))
        if head_mixing:
            out["talk"] = ParamSpec((heads, heads))
        if gate:
            out["g"] = ParamSpec((heads * vdim, hidden_size))
        return out

    def supports(self, rt) -> str | None:
        if self.num_heads * self.vdim > 8192:
            return f"heads x vdim {self.num_heads * self.vdim}: the attention kernel holds at most 8192 sums a token"
        floats = self.num_heads * (self.dim + self.num_heads + 64)
        if floats * 4 > 200 * 1024:
            return (f"{self.num_heads} heads of {self.dim}: a token's queries, the mixing matrix and a tile's weights "
                    f"must fit a block's shared memory")
        return row_rule(rt, hidden_size=self.hidden_size, **{"heads x vdim": self.num_heads * self.vdim})

    def cache_need(self) -> CacheNeed:
        return CacheNeed("kv", kv_heads=self.num_kv_heads, head_dim=self.dim,
                         value_dim=0 if self.vdim == self.dim else self.vdim, window=self.window or None,
                         keep_first=self.keep_first)

    def bind(self, tensors, rt) -> None:
        names = ("q", "k", "v", "g") if self.gate else ("q", "k", "v")
        self.w_in = torch.cat([tensors[name].to(rt.dtype) for name in names], dim=0).contiguous().to(rt.device)
        self.w_o = rt.to_device(tensors["o"], rt.dtype)
        f32 = lambda name: tensors[name].to(torch.float32).contiguous().to(rt.device)  # noqa: E731
        self.bias_rows = (f32("q_bias"), f32("k_bias"), f32("v_bias")) if self.biases else None
        self.norm_weights = (f32("q_norm"), f32("k_norm")) if self.whole_norm else None
        self.head_biases = f32("pb") if self.head_bias else None
        self.mix = f32("talk") if self.head_mixing else None
        if self.distance_exponent is not None:
            heads = self.num_heads
            self.slopes = torch.tensor([2.0 ** (-self.distance_exponent * (a + 1) / heads) for a in range(heads)],
                                       dtype=torch.float64).to(torch.float32).to(rt.device)

    def forward(self, h: torch.Tensor, residual: torch.Tensor, batch, cache, rt, write_cache: bool = True,
                epilogue: int = ops.EPI_RESIDUAL) -> None:
        """h: the mixer's input [tokens, hidden] in the activation type. Adds the output to `residual` (float32), or
        with `epilogue=ops.EPI_STORE_F32` writes it there."""
        n = batch.n_tokens
        heads, groups, dim, vdim = self.num_heads, self.num_kv_heads, self.dim, self.vdim
        rows = rt.ws.buffer("mixer_rows", (n, self.w_in.shape[0]), torch.float32)
        ops.gemm(rows, h, self.w_in, ops.EPI_STORE_F32)
        q = rt.ws.buffer("sigmoid_q", (n, heads * dim), rt.dtype)
        k_at = heads * dim
        v_at = k_at + groups * dim
        ops.sigmoid_prepare(rows, 0, k_at, v_at, q, cache, heads, self.bias_rows, self.norm_weights, self.eps, batch,
                            write_cache)
        attended = rt.ws.buffer("attended", (n, heads * vdim), rt.dtype)
        gates, gate_at = (rows, v_at + groups * vdim) if self.gate else (None, 0)
        if ops.sigmoid_attention_tiles(rt.dtype, heads, groups, dim, vdim, cache.page_size):
            ops.sigmoid_attention_tiled(attended, q, cache, heads, self.scale, self.window, self.keep_first, self.mix,
                                        self.slopes, self.head_biases, gates, gate_at, batch, rt.ws)
        else:
            ops.sigmoid_attention(attended, q, cache, heads, self.scale, self.window, self.keep_first, self.mix,
                                  self.slopes, self.head_biases, gates, gate_at, batch, rt.ws)
        ops.gemm(residual, attended, self.w_o, epilogue)

    def kernel_libraries(self, rt) -> set[str]:
        if rt.dtype != torch.bfloat16:
            return {"gemm_simt", "elementwise", "sigmoid_attention"}
        names = {"gemv", "gemv_cluster", "gemm_tcgen05", "elementwise", "sigmoid_attention"}
        if ops.sigmoid_attention_tiles(rt.dtype, self.num_heads, self.num_kv_heads, self.dim, self.vdim):
            names.add("sigmoid_attention_tiled")
        return names


register_part("mixer", "sigmoid_attention", SigmoidAttention)
