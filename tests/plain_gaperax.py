"""A plain, slow implementation of the Gaperax design in float64 on the CPU, one function per mechanism, written from
the design's equations and sharing no code with the library.

Notation: x the residual stream [tokens, width]; a layer computes x += mixer(norm1(x)) and, where it has a
feed-forward, x += ff(norm2(x)); norm(x) = tanh(alpha x) w + b. Positions count from 0 in each sequence. A sequence's
state is, per layer run, what its mixer keeps of earlier positions."""
from __future__ import annotations

import math

import numpy as np


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def rms(x, eps):
    """x over its root mean square along the last axis, eps inside the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def dynamic_tanh(x, alpha, w, b):
    return np.tanh(alpha * x) * w + b


def stretched_frequencies(dims, base, scaling):
    """The rotation's frequencies f_i = base^(-2i / dims), i < dims / 2, and what cos and sin are multiplied by. With
    `scaling` (factor, original, fast, slow): the pair whose frequency turns t times in `original` positions sits at
    index d(t) = dims ln(original / (2 pi t)) / (2 ln base); between lo = d(fast) (rounded down, at least 0) and hi =
    d(slow) (rounded up, at most dims - 1) a ramp r_i goes from 0 to 1 and f_i becomes f_i / factor r_i + f_i (1 -
    r_i); cos and sin grow by 0.1 ln(factor) + 1."""
    half = dims // 2
    f = np.array([base ** (-2.0 * i / dims) for i in range(half)], dtype=np.float64)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def index_of(turns):
        return dims * math.log(original / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(index_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(index_of(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((np.arange(half) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x, positions, freqs, magnitude):
    """x [tokens, ..., 2 n]: the pair (x[2i], x[2i + 1]) = (u, v) at position p becomes (u c - v s, v c + u s) with
    c, s = magnitude cos(p f_i), magnitude sin(p f_i)."""
    out = np.array(x, dtype=np.float64)
    shape = [len(positions)] + [1] * (x.ndim - 2) + [len(freqs)]
    angles = (np.asarray(positions, dtype=np.float64)[:, None] * freqs[None, :]).reshape(shape)
    c, s = np.cos(angles) * magnitude, np.sin(angles) * magnitude
    u, v = x[..., 0::2], x[..., 1::2]
    out[..., 0::2] = u * c - v * s
    out[..., 1::2] = v * c + u * s
    return out


def latent_attention(w, m, h, positions, kept, eps):
    """h [tokens, width] of ONE sequence at `positions`; `kept` = (latents, shared key parts) of the positions before
    (None at the start). Returns the output and the new `kept`."""
    heads, dim, rot, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    n = len(h)
    cq = rms(h @ w["dq"].T, eps) * w["dq.norm"]
    q = (cq @ w["uq"].T).reshape(n, heads, dim + rot)
    down = h @ w["dkv"].T
    c = rms(down[:, :rank], eps) * w["dkv.norm"]
    r = down[:, rank:]
    q_rot = q[..., dim:]
    if rot:
        freqs, magnitude = stretched_frequencies(m["rot"]["dims"], float(m["rot"]["base"]), m["rot"].get("scaling"))
        q_rot = rotate_pairs(q_rot, positions, freqs, magnitude)
        r = rotate_pairs(r, positions, freqs, magnitude)
    if kept is not None:
        c, r = np.concatenate([kept[0], c]), np.concatenate([kept[1], r])
    keys = (c @ w["uk"].T).reshape(len(c), heads, dim)
    values = (c @ w["uv"].T).reshape(len(c), heads, vdim)
    scores = (np.einsum("tad,sad->ats", q[..., :dim], keys) + np.einsum("tad,sd->ats", q_rot, r)) * m["scale"]
    first = len(c) - n
    seen = np.arange(len(c))[None, :] <= (first + np.arange(n))[:, None]
    scores = np.where(seen[None], scores, -np.inf)
    sink = np.asarray(w["sink"], dtype=np.float64)[:, None, None]
    top = np.maximum(scores.max(axis=2, keepdims=True), sink)
    e = np.exp(scores - top)
    weights = e / (e.sum(axis=2, keepdims=True) + np.exp(sink - top))  # the sink: in the sum, without a value
    out = np.einsum("ats,sav->tav", weights, values).reshape(n, heads * vdim)
    return out @ w["o"].T, (c, r)


def visible(i, j, size, keep):
    """Whether position i sees position j: not ahead, and inside the window or among the first `keep`."""
    return (j <= i) & ((i - j < size) | (j < keep))


def sigmoid_attention(w, m, h, positions, kept, eps):
    """h [tokens, width] of ONE sequence; `kept` = (normed keys, values) of the positions before."""
    heads, groups, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    n = len(h)
    q = rms(h @ w["q"].T + w["q.b"], eps) * w["q.norm"]  # over the whole projection, all heads at once
    k = rms(h @ w["k"].T + w["k.b"], eps) * w["k.norm"]
    v = h @ w["v"].T + w["v.b"]
    if kept is not None:
        k, v = np.concatenate([kept[0], k]), np.concatenate([kept[1], v])
    total = len(k)
    first = total - n
    share = heads // groups
    q = q.reshape(n, heads, dim)
    keys = np.repeat(k.reshape(total, groups, dim), share, axis=1)
    values = np.repeat(v.reshape(total, groups, vdim), share, axis=1)
    i = (first + np.arange(n))[:, None]
    j = np.arange(total)[None, :]
    slopes = np.array([2.0 ** (-8.0 * (a + 1) / heads) for a in range(heads)])
    scores = np.einsum("tad,sad->ats", q, keys) * m["scale"] - slopes[:, None, None] * (i - j)[None]
    weights = sigmoid(scores + np.asarray(w["pb"], dtype=np.float64)[:, None, None])
    weights = np.where(visible(i, j, m["mask"]["size"], m["mask"]["keep_first"])[None], weights, 0.0)
    mixed = np.einsum("ag,gts->ats", w["talk"], weights)
    out = np.einsum("ats,sav->tav", mixed, values).reshape(n, heads * vdim)
    return (out * sigmoid(h @ w["g"].T)) @ w["o"].T, (k, v)


def feed_forward(w, h):
    return (gelu_tanh(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def weights_layer(config, index):
    while config["layers"][index].get("weights_of") is not None:
        index = config["layers"][index]["weights_of"]
    return index


def part(weights, prefix):
    return {name[len(prefix):]: np.asarray(value, dtype=np.float64) for name, value in weights.items()
            if name.startswith(prefix)}


def norm_of(weights, name):
    return tuple(np.asarray(weights[name + end], dtype=np.float64) for end in (".alpha", "", ".b"))


def new_state(config):
    return [None] * len(config["layers"])


def forward(config, weights, tokens, state=None, start=0, layers_out=None):
    """Logits [tokens, vocab] of `tokens` of one sequence whose first `start` tokens are in `state`."""
    state = new_state(config) if state is None else state
    eps = float(config["norm"]["eps"])
    x = np.asarray(weights["embed"], dtype=np.float64)[np.asarray(tokens, dtype=np.int64)]
    positions = np.arange(start, start + len(tokens))
    for index, layer in enumerate(config["layers"]):
        prefix = f"l{weights_layer(config, index)}."
        mixer = latent_attention if layer["type"] == "latent_attention" else sigmoid_attention
        h = dynamic_tanh(x, *norm_of(weights, prefix + "norm1"))
        y, state[index] = mixer(part(weights, prefix + "mix."), layer["mixer"], h, positions, state[index], eps)
        x = x + y
        if layer.get("mlp") is not None:
            x = x + feed_forward(part(weights, prefix + "mlp."), dynamic_tanh(x, *norm_of(weights, prefix + "norm2")))
        if layers_out is not None:
            layers_out.append(x.copy())
    return dynamic_tanh(x, *norm_of(weights, "final.norm")) @ np.asarray(weights["head"], dtype=np.float64).T


def greedy(config, weights, prompt, count):
    """The `count` tokens the model chooses greedily after `prompt`, through its own carried state."""
    state = new_state(config)
    logits = forward(config, weights, prompt, state, 0)
    out, at = [], len(prompt)
    for _ in range(count):
        out.append(int(np.argmax(logits[-1])))
        logits = forward(config, weights, [out[-1]], state, at)
        at += 1
    return out
