"""Attention whose keys and values are made from a small latent per position instead of being kept themselves.

Per token, from the mixer's input h: the query goes through a latent of its own, c_q = rms(W_dq h) * w_q, q = W_uq c_q,
laid out head by head as [dim plain | rot_dim rotated]. W_dkv h gives kv_rank + rot_dim numbers: the first kv_rank,
divided by their root mean square and weighted, are the latent c; the last rot_dim, rotated by the position (pairs
i, i + rot_dim / 2; a position encoding that pairs 2i with 2i + 1 has the rotated rows of W_uq and W_dkv put into that
order once, when the weights are bound, which changes no q . k), are ONE key part r that all heads share. Head a has the keys [W_uk,a c | r] and the values
W_uv,a c; the score is (q_plain . W_uk,a c + q_rot . r) * scale, causal, ordinary softmax (with `sink`, a learned
number per head whose exponential also stands in the denominator: a score without a key or a value); the head's
output is multiplied by sigmoid(W_g h)_a (with `gate`) and W_o runs over the concatenated heads.

Only [c | r] is cached, one row per position for all heads (a keys-only cache entry). The kernels never build the
heads' keys and values: since q_plain . W_uk c = (W_uk^T q_plain) . c, a query is taken into the latent's coordinates
once and attention runs over the cached rows themselves, every head against the same rows; the weighted sum of c is
then mapped through W_uv. Norms, rotation, scores, softmax and the gate are float32; the cache holds the activation
type.

In bfloat16, with sizes the tile kernel takes, attention runs on the tensor cores (heads and tokens as rows of one
query matrix over the shared rows) with two merged weights made when the weights are bound:
W_qa,h = scale [W_uk,h^T W_uq,h,plain ; W_uq,h,rot] takes the query latent straight into the latent's coordinates (one
product for all heads, the rotation done as the attention kernel reads its queries), and W_ov = [W_o,h W_uv,h]_h takes
the gated sums of c of all heads straight to the output (the gate is a number per token and head, so it can sit in
front of both maps). That trades more multiply-adds and weight bytes (rank against dim and vdim) for two plain
products in place of four and two small per-head kernels; the separate maps are then not kept on the device."""
from __future__ import annotations

import torch

from ..cache.paged import CacheNeed
from ..kernels import ops
from .norm import row_rule
from .registry import build_part, register_part
from .spec import ParamSpec


class LatentAttention:
    def __init__(self, hidden_size: int, num_heads: int, dim: int, rot_dim: int, vdim: int, q_rank: int, kv_rank: int,
                 scale: float, eps: float, position=None, gate: bool = True, sink: bool = False) -> None:
        self.hidden_size, self.num_heads = int(hidden_size), int(num_heads)
        self.dim, self.rot_dim, self.vdim = int(dim), int(rot_dim), int(vdim)
        self.q_rank, self.kv_rank = int(q_rank), int(kv_rank)
        self.scale, self.eps, self.gate, self.sink = float(scale), float(eps), bool(gate), bool(sink)
        self.sinks = None
        if self.rot_dim and position is None:
            raise ValueError("a rotated key part needs a position encoding")
        self.position = build_part("position", position) if position is not None and self.rot_dim else None
        if self.position is not None and self.position.rotary_dim != self.rot_dim:
            raise ValueError(f"the position encoding turns {self.position.rotary_dim} values, the rotated part has "
                             f"{self.rot_dim}")
        self.w_down = self.w_uq = self.w_uk = self.w_uv = self.w_o = self.q_weight = self.c_weight = None
        self.w_qa = self.w_ov = None

    @staticmethod
    def parameters(hidden_size, num_heads, dim, rot_dim, vdim, q_rank, kv_rank, gate=True, sink=False,
                   **_) -> dict[str, ParamSpec]:
        heads = int(num_heads)
        out = {"dq": ParamSpec((int(q_rank), hidden_size)), "dq_norm": ParamSpec((int(q_rank),), "ones"),
               "uq": ParamSpec((heads * (int(dim) + int(rot_dim)), int(q_rank))),
               "dkv": ParamSpec((int(kv_rank) + int(rot_dim), hidden_size)),
               "dkv_norm": ParamSpec((int(kv_rank),), "ones"),
               "uk": ParamSpec((heads * int(dim), int(kv_rank))), "uv": ParamSpec((heads * int(vdim), int(kv_rank))),
               "o": ParamSpec((hidden_size, heads * int(vdim)))}
        if gate:
            out["g"] = ParamSpec((heads, hidden_size))
        if sink:
            out["sink"] = ParamSpec((heads,))
        return out

    def supports(self, rt) -> str | None:
        if self.kv_rank > 512:
            return f"kv_rank {self.kv_rank}: the attention kernels hold a head's sum in registers, at most 512"
        if ops.latent_tiles(rt.dtype, self.kv_rank, self.rot_dim) is None and (self.kv_rank + self.rot_dim) * 16 > 48 * 1024:
            return f"kv_rank + rot_dim {self.kv_rank + self.rot_dim}: the general kernel keeps four queries in 48 KB"
        return row_rule(rt, hidden_size=self.hidden_size, q_rank=self.q_rank,
                        **{"heads x vdim": self.num_heads * self.vdim})

    def cache_need(self) -> CacheNeed:
        return CacheNeed("kv", kv_heads=1, head_dim=self.kv_rank + self.rot_dim, keys_only=True)

    def bind(self, tensors, rt) -> None:
        # one product for everything a token needs of h: the two latents (with the shared key part) and the gates
        tensors = dict(tensors)
        order = self.position.row_order() if self.position is not None and hasattr(self.position, "row_order") \
            else None
        if order is not None:
            # the position encoding pairs other places than the kernels rotate: the rotated rows of the two maps that
            # make them are put in the kernels' order, the queries' and the shared key part's alike
            index = torch.tensor(order, dtype=torch.long)
            dkv, uq = tensors["dkv"], tensors["uq"]
            tensors["dkv"] = torch.cat([dkv[:self.kv_rank], dkv[self.kv_rank:][index]], dim=0)
            uq = uq.view(self.num_heads, self.dim + self.rot_dim, self.q_rank)
            tensors["uq"] = torch.cat([uq[:, :self.dim], uq[:, self.dim:][:, index]], dim=1).reshape(
                self.num_heads * (self.dim + self.rot_dim), self.q_rank).contiguous()
        if self.sink:
            self.sinks = tensors["sink"].to(torch.float32).contiguous().to(rt.device)
        names = ("dq", "dkv", "g") if self.gate else ("dq", "dkv")
        fused = torch.cat([tensors[name].to(rt.dtype) for name in names], dim=0)
        self.w_down = fused.contiguous().to(rt.device)
        self.q_weight = rt.to_device(tensors["dq_norm"], torch.float32)
        self.c_weight = rt.to_device(tensors["dkv_norm"], torch.float32)
        if self.position is not None:
            self.position.bind({}, rt)
        if ops.latent_tiles(rt.dtype, self.kv_rank, self.rot_dim) is not None:
            heads, dim, rot, vdim, rank = self.num_heads, self.dim, self.rot_dim, self.vdim, self.kv_rank
            uq = tensors["uq"].to(device=rt.device, dtype=torch.float32).view(heads, dim + rot, self.q_rank)
            uk = tensors["uk"].to(device=rt.device, dtype=torch.float32).view(heads, dim, rank)
            uv = tensors["uv"].to(device=rt.device, dtype=torch.float32).view(heads, vdim, rank)
            wo = tensors["o"].to(device=rt.device, dtype=torch.float32).view(self.hidden_size, heads, vdim)
            absorbed = torch.bmm(uk.transpose(1, 2), uq[:, :dim])                     # [heads, rank, q_rank]
            self.w_qa = (torch.cat([absorbed, uq[:, dim:]], dim=1) * self.scale).reshape(
                heads * (rank + rot), self.q_rank).to(rt.dtype).contiguous()
            self.w_ov = torch.einsum("whv,hvr->whr", wo, uv).reshape(self.hidden_size, heads * rank).to(
                rt.dtype).contiguous()
            return
        self.w_uq = rt.to_device(tensors["uq"], rt.dtype)
        self.w_uk = rt.to_device(tensors["uk"], rt.dtype)
        self.w_uv = rt.to_device(tensors["uv"], rt.dtype)
        self.w_o = rt.to_device(tensors["o"], rt.dtype)

    def forward(self, h: torch.Tensor, residual: torch.Tensor, batch, cache, rt, write_cache: bool = True,
                epilogue: int = ops.EPI_RESIDUAL) -> None:
        """h: the mixer's input [tokens, hidden] in the activation type. Adds the output to `residual` (float32), or
        with `epilogue=ops.EPI_STORE_F32` writes it there."""
        n = batch.n_tokens
        heads, dim, rot, vdim, rank = self.num_heads, self.dim, self.rot_dim, self.vdim, self.kv_rank
        rows = rt.ws.buffer("mixer_rows", (n, self.w_down.shape[0]), torch.float32)
        ops.gemm(rows, h, self.w_down, ops.EPI_STORE_F32)
        table = self.position.table() if self.position is not None else None
        cq = rt.ws.buffer("latent_cq", (n, self.q_rank), rt.dtype)
        ops.latent_prepare(rows, 0, self.q_rank, self.q_rank, rank, rot, self.q_weight, self.c_weight, self.eps, table,
                           cq, cache, batch, write_cache)
        gates, gate_at = (rows, self.q_rank + rank + rot) if self.gate else (None, 0)
        if self.w_qa is not None:
            if ops.latent_tiles(rt.dtype, rank, rot, cache.page_size) is None:
                raise ValueError(f"pages of {cache.page_size} positions: the tile kernel takes multiples of 32")
            q_lat = rt.ws.buffer("latent_q_abs", (n, heads * (rank + rot)), torch.float32)
            ops.gemm(q_lat, cq, self.w_qa, ops.EPI_STORE_F32)
            mixed = rt.ws.buffer("latent_mixed16", (n, heads * rank), rt.dtype)
            ops.latent_attention_tiled(mixed, q_lat, table, gates, gate_at, cache, heads, rank, rot, batch, rt.ws,
                                       sinks=self.sinks)
            ops.gemm(residual, mixed, self.w_ov, epilogue)
            return
        q = rt.ws.buffer("latent_q", (n, heads * (dim + rot)), torch.float32)
        ops.gemm(q, cq, self.w_uq, ops.EPI_STORE_F32)
        attended = rt.ws.buffer("attended", (n, heads * vdim), rt.dtype)
        q_lat = rt.ws.buffer("latent_q_abs", (n, heads * (rank + rot)), torch.float32)
        ops.latent_queries(q_lat, q, self.w_uk, table, heads, dim, rot, rank, self.scale, batch)
        mixed = rt.ws.buffer("latent_mixed", (n, heads * rank), torch.float32)
        ops.latent_attention(mixed, q_lat, cache, heads, rank, rot, batch, sinks=self.sinks)
        ops.latent_values(attended, mixed, self.w_uv, gates, gate_at, heads, rank, vdim)
        ops.gemm(residual, attended, self.w_o, epilogue)

    def kernel_libraries(self, rt) -> set[str]:
        if rt.dtype != torch.bfloat16:
            return {"gemm_simt", "elementwise", "latent_attention"}
        names = {"gemv", "gemv_cluster", "gemm_tcgen05", "elementwise", "latent_attention"}
        if ops.latent_tiles(rt.dtype, self.kv_rank, self.rot_dim) is not None:
            names.add("latent_attention_tiled")
        return names


register_part("mixer", "latent_attention", LatentAttention)
