"""Small Gaperax configurations and random weights for the tests: sizes that are no powers of two, key, value and
latent sizes that all differ, fewer key/value heads than query heads and as many, one head and several, windows shorter
than a page and longer than two, first positions kept within a page, across a page border, and none, frequencies with
and without stretching, a layer without a feed-forward, layers that run with another layer's weights (an attention
layer and a latent layer, one of them twice)."""
from __future__ import annotations

import math

import torch


def latent(heads=3, dim=16, rot_dim=8, vdim=24, q_rank=40, kv_rank=32, base=1e4, scale=0.25, scaling="default",
           ff=40):
    rot = {"base": base, "dims": rot_dim}
    if scaling == "default":
        scaling = {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}
    if scaling is not None:
        rot["scaling"] = scaling
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
             "scale": scale, "rot": rot}
    return {"type": "latent_attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def attention(heads=4, kv_heads=2, dim=24, vdim=16, size=40, keep_first=3, scale=0.2, ff=48):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
             "mask": {"size": size, "keep_first": keep_first}}
    return {"type": "attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def shared(layer: dict, source: int) -> dict:
    return dict(layer, weights_of=source)


def config(layers, vocab=211, width=96, eps=1e-5) -> dict:
    return {"architecture": "Gaperax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


def _mixed():
    first, second = attention(), latent()
    return config([first, second, attention(heads=6, kv_heads=6, dim=8, vdim=12, size=70, keep_first=0, ff=0),
                   shared(first, 0), shared(second, 1), shared(first, 3)])


def _tiled():
    a = latent(heads=4, dim=32, rot_dim=16, vdim=32, q_rank=48, kv_rank=64, scale=0.15, base=5e5,
               scaling={"factor": 4.0, "original": 128, "fast": 8.0, "slow": 1.0}, ff=64)
    b = attention(heads=8, kv_heads=2, dim=32, vdim=16, size=150, keep_first=70, scale=0.1, ff=64)
    return config([a, b, shared(a, 0), attention(heads=2, kv_heads=2, dim=64, vdim=64, size=64, keep_first=64,
                                                 scale=0.08, ff=32)], width=128, vocab=157)


def _narrow():
    return config([latent(heads=1, dim=8, rot_dim=2, vdim=16, q_rank=8, kv_rank=24, scale=0.5, base=50.0,
                          scaling=None, ff=24),
                   attention(heads=1, kv_heads=1, dim=12, vdim=8, size=5, keep_first=1, scale=0.3, ff=0),
                   latent(heads=5, dim=24, rot_dim=0, vdim=8, q_rank=16, kv_rank=72, scale=0.18, ff=0)],
                  width=64, vocab=97, eps=3e-4)


CASES = {
    # both mixers, grouped key/value heads and one per head, a layer without a feed-forward, shared weights
    "mixed": _mixed,
    # sizes that tile for the tensor cores, a window over more than two pages, kept positions across a page border
    "tiled": _tiled,
    # one head, a window of five, a rotated part of one pair and of none, no stretching, a latent of 72
    "narrow": _narrow,
}


def own_layers(config_dict: dict) -> list[int]:
    return [i for i, layer in enumerate(config_dict["layers"]) if layer.get("weights_of") is None]


def random_weights(config_dict: dict, seed: int = 0) -> dict:
    """bfloat16 tensors by checkpoint name, scaled so that activations stay of order one through the layers."""
    g = torch.Generator().manual_seed(seed)
    width = config_dict["width"]
    t: dict[str, torch.Tensor] = {}

    def matrix(name, rows, cols, gain=1.0):
        t[name] = (torch.randn(rows, cols, generator=g) * gain / math.sqrt(cols)).to(torch.bfloat16)

    def vector(name, size, mean=1.0, spread=0.2):
        t[name] = (mean + spread * torch.randn(size, generator=g)).to(torch.bfloat16)

    def norm(name):
        vector(name, width, 1.0, 0.2)
        vector(name + ".b", width, 0.0, 0.1)
        t[name + ".alpha"] = (0.7 + 0.2 * torch.rand((), generator=g)).to(torch.bfloat16)

    matrix("embed", config_dict["vocab"], width, gain=math.sqrt(width))
    matrix("head", config_dict["vocab"], width)
    norm("final.norm")
    for i in own_layers(config_dict):
        layer = config_dict["layers"][i]
        p, m = f"l{i}.", layer["mixer"]
        norm(p + "norm1")
        heads = m["heads"]
        if layer["type"] == "latent_attention":
            matrix(p + "mix.dq", m["q_rank"], width, 1.5)
            vector(p + "mix.dq.norm", m["q_rank"], 1.2, 0.3)
            matrix(p + "mix.uq", heads * (m["dim"] + m["rot_dim"]), m["q_rank"], 2.0)
            matrix(p + "mix.dkv", m["kv_rank"] + m["rot_dim"], width, 1.5)
            vector(p + "mix.dkv.norm", m["kv_rank"], 1.2, 0.3)
            matrix(p + "mix.uk", heads * m["dim"], m["kv_rank"], 2.0)
            matrix(p + "mix.uv", heads * m["vdim"], m["kv_rank"], 1.5)
            vector(p + "mix.sink", heads, 0.5, 1.0)
            matrix(p + "mix.o", width, heads * m["vdim"], 0.5)
        else:
            groups = m["kv_heads"]
            matrix(p + "mix.q", heads * m["dim"], width, 1.5)
            vector(p + "mix.q.b", heads * m["dim"], 0.0, 0.3)
            matrix(p + "mix.k", groups * m["dim"], width, 1.5)
            vector(p + "mix.k.b", groups * m["dim"], 0.0, 0.3)
            matrix(p + "mix.v", groups * m["vdim"], width, 1.5)
            vector(p + "mix.v.b", groups * m["vdim"], 0.0, 0.3)
            vector(p + "mix.q.norm", heads * m["dim"], 1.5, 0.4)
            vector(p + "mix.k.norm", groups * m["dim"], 1.5, 0.4)
            t[p + "mix.talk"] = (torch.eye(heads) * 0.6 + 0.3 * torch.randn(heads, heads, generator=g)
                                 / math.sqrt(heads)).to(torch.bfloat16)
            vector(p + "mix.pb", heads, -2.0, 0.7)
            matrix(p + "mix.g", heads * m["vdim"], width, 2.0)
            matrix(p + "mix.o", width, heads * m["vdim"], 0.25)
        mlp = layer.get("mlp")
        if mlp is not None:
            norm(p + "norm2")
            matrix(p + "mlp.gate", mlp["ff"], width, 1.5)
            matrix(p + "mlp.up", mlp["ff"], width, 1.5)
            matrix(p + "mlp.down", width, mlp["ff"], 0.5)
    return t


def make_engine(config_dict: dict, tensors: dict, dtype: str, max_tokens: int = 2048, **kwargs):
    from etalii.dllm_b200.config.registry import config_from_dict
    from etalii.dllm_b200.engine.engine import Engine

    kwargs.setdefault("max_length", 1024)
    return Engine(config_from_dict(config_dict), tensors, dtype=dtype, device="cuda:0", max_tokens=max_tokens, **kwargs)


def tokens_for(config_dict: dict, lengths, seed: int = 5):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, config_dict["vocab"], (n,), generator=g).tolist() for n in lengths]


def as_numpy(tensors: dict) -> dict:
    return {name: value.to(torch.float64).numpy() for name, value in tensors.items()}
