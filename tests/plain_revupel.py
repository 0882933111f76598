"""A plain, slow implementation of the Revupel design in float64 on the CPU, one function per mechanism, written from
the design's equations and sharing no code with the library. Tests compare the library's results with it.

Notation: h is a sublayer's input [tokens, width] of ONE sequence; `start` is the position of its first token. What a
run of a layer keeps between calls is a dict `kept`: "conv" (the last taps - 1 inputs of the input convolution), and
of the mixer either "c" [positions, kv_rank] and "kr" [positions, rot_dim] (latent attention) or "S" [heads, dim, vdim],
"n" [heads, dim], "m" [heads] (matrix memory). Weights are applied as W x (stored [out, in])."""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def sigmoid(x: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-x))


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gelu_erf(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def relu_squared(z: torch.Tensor) -> torch.Tensor:
    return torch.clamp(z, min=0.0) ** 2


def rotate_halves(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x: [tokens, ..., dims]: place i turns with place i + dims/2 by the angle position * base^(-2i/dims)."""
    out = x.clone()
    half = dims // 2
    shape = [-1] + [1] * (x.dim() - 2)
    for i in range(half):
        angle = positions.to(F64) * (float(base) ** (-2.0 * i / dims))
        c, s = torch.cos(angle).view(shape), torch.sin(angle).view(shape)
        u, v = x[..., i], x[..., i + half]
        out[..., i] = u * c - v * s
        out[..., i + half] = v * c + u * s
    return out


def input_convolution(taps_w: torch.Tensor, h: torch.Tensor, kept: dict) -> torch.Tensor:
    """h + conv(h): conv(h)_t = sum_j w[:, j] h_(t - taps + 1 + j), the inputs before this call from kept["conv"]
    (zeros before the sequence's start). Leaves the last taps - 1 inputs in kept["conv"]."""
    width, taps = taps_w.shape
    before = kept.get("conv")
    if before is None:
        before = torch.zeros(taps - 1, width, dtype=F64)
    line = torch.cat([before, h], dim=0)  # line[taps - 1 + t] = h_t
    out = h.clone()
    for t in range(h.shape[0]):
        for j in range(taps):
            out[t] += taps_w[:, j].to(F64) * line[t + j]
    kept["conv"] = line[line.shape[0] - (taps - 1):].clone() if taps > 1 else line[:0]
    return out


def latent_attention(w: dict, p: dict, h: torch.Tensor, start: int, eps: float, kept: dict) -> torch.Tensor:
    """Attention whose keys and values are made from a latent of kv_rank numbers per position and one rotated key part
    of rot_dim numbers that all heads share; queries go through a latent of their own."""
    n = h.shape[0]
    heads, dim, rot_dim, vdim, kv_rank = p["heads"], p["dim"], p["rot_dim"], p["vdim"], p["kv_rank"]
    positions = torch.arange(start, start + n)
    cq = rms(h @ w["dq"].to(F64).T, eps) * w["dq.norm"].to(F64)
    q = (cq @ w["uq"].to(F64).T).view(n, heads, dim + rot_dim)
    q_plain = q[..., :dim]
    q_rot = rotate_halves(q[..., dim:], positions, p["rot"]["dims"], p["rot"]["base"])
    down = h @ w["dkv"].to(F64).T
    c = rms(down[:, :kv_rank], eps) * w["dkv.norm"].to(F64)
    kr = rotate_halves(down[:, kv_rank:], positions, p["rot"]["dims"], p["rot"]["base"])
    kept["c"] = torch.cat([kept["c"], c]) if "c" in kept else c
    kept["kr"] = torch.cat([kept["kr"], kr]) if "kr" in kept else kr
    all_c, all_kr = kept["c"], kept["kr"]
    k_plain = (all_c @ w["uk"].to(F64).T).view(-1, heads, dim)
    values = (all_c @ w["uv"].to(F64).T).view(-1, heads, vdim)
    gates = sigmoid(h @ w["g"].to(F64).T)  # [n, heads]
    out = torch.zeros(n, heads, vdim, dtype=F64)
    for t in range(n):
        see = start + t + 1
        for a in range(heads):
            scores = (k_plain[:see, a] @ q_plain[t, a] + all_kr[:see] @ q_rot[t, a]) * p["scale"]
            weights = torch.softmax(scores, dim=0)
            out[t, a] = (weights[:, None] * values[:see, a]).sum(dim=0) * gates[t, a]
    return out.reshape(n, heads * vdim) @ w["o"].to(F64).T


def logsigmoid(x: torch.Tensor) -> torch.Tensor:
    return -torch.log1p(torch.exp(-x.abs())) + torch.clamp(x, max=0.0)


def matrix_memory(w: dict, p: dict, h: torch.Tensor, eps: float, kept: dict) -> torch.Tensor:
    """Per head a matrix S and a vector n written with exponential input gates under a running maximum m of the log
    gates: m' = max(f + m, i); S' = exp(f + m - m') S + exp(i - m') k v^T; n' likewise with k; the read-out is
    S'^T q / (max(|n' . q|, exp(-m')) + 1e-6), then normed per head, weighted, gated and projected."""
    n_tokens = h.shape[0]
    heads, dim, vdim, cap = p["heads"], p["dim"], p["vdim"], float(p["gate_cap"])
    q = (h @ w["q"].to(F64).T).view(n_tokens, heads, dim) * dim ** -0.5
    k = (h @ w["k"].to(F64).T).view(n_tokens, heads, dim)
    v = (h @ w["v"].to(F64).T).view(n_tokens, heads, vdim)
    log_in = cap * torch.tanh((h @ w["i"].to(F64).T + w["i.b"].to(F64)) / cap)
    log_forget = logsigmoid(cap * torch.tanh((h @ w["f"].to(F64).T + w["f.b"].to(F64)) / cap))
    S = kept.get("S", torch.zeros(heads, dim, vdim, dtype=F64))
    n = kept.get("n", torch.zeros(heads, dim, dtype=F64))
    m = kept.get("m", torch.zeros(heads, dtype=F64))
    read = torch.zeros(n_tokens, heads, vdim, dtype=F64)
    for t in range(n_tokens):
        m_new = torch.maximum(log_forget[t] + m, log_in[t])
        keep = torch.exp(log_forget[t] + m - m_new)
        write = torch.exp(log_in[t] - m_new)
        S = keep[:, None, None] * S + write[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + write[:, None] * k[t]
        m = m_new
        top = torch.einsum("hdv,hd->hv", S, q[t])
        below = torch.maximum((n * q[t]).sum(dim=-1).abs(), torch.exp(-m)) + 1e-6
        read[t] = top / below[:, None]
    kept["S"], kept["n"], kept["m"] = S, n, m
    normed = rms(read, eps).reshape(n_tokens, heads * vdim) * w["norm"].to(F64)
    return (normed * sigmoid(h @ w["g"].to(F64).T)) @ w["o"].to(F64).T


def dense_feed_forward(w: dict, h: torch.Tensor) -> torch.Tensor:
    up = h @ w["up"].to(F64).T + w["up.b"].to(F64)
    return gelu_erf(up) @ w["down"].to(F64).T + w["down.b"].to(F64)


def expert(w: dict, prefix: str, h: torch.Tensor) -> torch.Tensor:
    return relu_squared(h @ w[prefix + "up"].to(F64).T) @ w[prefix + "down"].to(F64).T


def choose_experts(w: dict, p: dict, h: torch.Tensor):
    """(chosen [tokens, top], weights [tokens, top]): the softmax over ALL experts' logits, the `top` largest scores,
    the chosen scores as they are (the lower expert first on ties)."""
    scores = torch.softmax(h @ w["router"].to(F64).T, dim=-1)
    order = torch.sort(scores, dim=-1, descending=True, stable=True).indices[:, :p["router"]["top"]]
    return order, torch.gather(scores, 1, order)


def mixture(w: dict, p: dict, h: torch.Tensor) -> torch.Tensor:
    chosen, weights = choose_experts(w, p, h)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, weight in zip(chosen[t].tolist(), weights[t]):
            out[t] += weight * expert(w, f"e{e}.", h[t:t + 1])[0]
    if p.get("shared") is not None:
        out += expert(w, "shared.", h) * sigmoid(h @ w["shared.sg"].to(F64).T)
    return out


def token_input(w: dict, part: torch.Tensor, x: torch.Tensor, eps: float) -> torch.Tensor:
    """What a layer adds from the tokens themselves: `part` [tokens, dim] is the layer's part of the tokens' second
    embedding; y = W_proj (gelu_tanh(W_gate x) * part), and the return value is y / rms(y) * weight."""
    y = (gelu_tanh(x @ w["gate"].to(F64).T) * part) @ w["proj"].to(F64).T
    return rms(y, eps) * w["norm"].to(F64)


def sub(weights: dict, prefix: str) -> dict:
    return {name[len(prefix):]: t for name, t in weights.items() if name.startswith(prefix)}


def run_order(config: dict) -> list[int]:
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return list(range(n))
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))


def layer(config: dict, weights: dict, index: int, x: torch.Tensor, tokens, start: int, kept: dict) -> torch.Tensor:
    entry, eps, prefix = config["layers"][index], float(config["norm"]["eps"]), f"l{index}."
    h = rms(x, eps) * weights[prefix + "norm1"].to(F64)
    h = input_convolution(weights[prefix + "canon1"], h, kept)
    w = sub(weights, prefix + "mix.")
    if entry["type"] == "latent_attention":
        x = x + latent_attention(w, entry["mixer"], h, start, eps, kept)
    else:
        x = x + matrix_memory(w, entry["mixer"], h, eps, kept)
    mlp = entry.get("mlp")
    if mlp is not None:
        h = rms(x, eps) * weights[prefix + "norm2"].to(F64)
        w = sub(weights, prefix + "mlp.")
        x = x + (dense_feed_forward(w, h) if mlp["kind"] == "dense" else mixture(w, mlp, h))
    side = config.get("token_side")
    if side:
        dim = side["dim"]
        part = weights["side.embed"].to(F64)[torch.tensor(tokens)][:, index * dim:(index + 1) * dim]
        x = x + token_input(sub(weights, prefix + "side."), part, x, eps)
    return x


def forward(config: dict, weights: dict, tokens, state: list | None = None, start: int = 0, streams: list | None = None):
    """Logits [tokens, vocab] of `tokens` at positions start.. of one sequence. `state`: a list with one dict per run
    of a layer (made by `new_state`), carried between calls. `streams`: filled with the stream after every run."""
    if state is None:
        state = new_state(config)
    x = weights["embed"].to(F64)[torch.tensor(tokens)]
    for run, index in enumerate(run_order(config)):
        x = layer(config, weights, index, x, tokens, start, state[run])
        if streams is not None:
            streams.append(x.clone())
    x = rms(x, float(config["norm"]["eps"])) * weights["final.norm"].to(F64)
    return x @ weights["head"].to(F64).T


def new_state(config: dict) -> list:
    return [{} for _ in run_order(config)]


def greedy(config: dict, weights: dict, prompt, steps: int) -> list[int]:
    state = new_state(config)
    logits = forward(config, weights, prompt, state, 0)
    out, at = [], len(prompt)
    for _ in range(steps):
        out.append(int(torch.argmax(logits[-1])))
        logits = forward(config, weights, [out[-1]], state, at)
        at += 1
    return out
