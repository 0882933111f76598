"""Small Revupel configurations and random weights for the tests: sizes that are no powers of two, key, value and
latent sizes that all differ, one head and several, convolutions of one, two and four taps, a loop of two rounds, of
one, and none, layers without a feed-forward, dense and mixed feed-forwards with and without a shared expert, a model
without a second token embedding, a matrix memory whose head size is no multiple of four."""
from __future__ import annotations

import math

import torch


def latent(heads=3, dim=16, rot_dim=8, vdim=24, q_rank=40, kv_rank=32, base=1e4, scale=0.25, mlp="default"):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
             "scale": scale, "rot": {"base": base, "dims": rot_dim}}
    return {"type": "latent_attention", "mixer": mixer, "mlp": moe() if mlp == "default" else mlp}


def memory(heads=2, dim=20, vdim=12, gate_cap=8.0, mlp="default"):
    mixer = {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": gate_cap}
    return {"type": "mlstm", "mixer": mixer, "mlp": dense() if mlp == "default" else mlp}


def moe(ff=24, experts=5, top=2, shared_ff=16):
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared_ff:
        out["shared"] = {"ff": shared_ff}
    return out


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def config(layers, vocab=211, width=96, eps=1e-5, taps=4, side_dim=12, loop=None) -> dict:
    out = {"architecture": "Revupel", "vocab": vocab, "width": width, "norm": {"eps": eps}, "canon": {"taps": taps},
           "layers": layers}
    if side_dim:
        out["token_side"] = {"dim": side_dim}
    if loop is not None:
        out["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return out


CASES = {
    # both mixers, both feed-forwards, a layer without one, a loop of two rounds over an attention and a memory layer
    "mixed": lambda: config([
        latent(),
        memory(),
        latent(heads=2, dim=24, rot_dim=4, vdim=16, q_rank=24, kv_rank=48, base=77.0, scale=0.2, mlp=None),
        memory(heads=3, dim=8, vdim=24, gate_cap=15.0, mlp=moe(ff=16, experts=3, top=1, shared_ff=0))],
        loop=(1, 3, 2)),
    # sizes that tile for the tensor cores, two taps, no second embedding, no loop
    "tiled": lambda: config([
        latent(heads=4, dim=32, rot_dim=16, vdim=32, q_rank=48, kv_rank=64, scale=0.15, mlp=dense(64)),
        memory(heads=2, dim=32, vdim=64, mlp=moe(ff=32, experts=4, top=2, shared_ff=32)),
        latent(heads=8, dim=16, rot_dim=32, vdim=16, q_rank=64, kv_rank=32, scale=0.2, base=1e6,
               mlp=moe(ff=32, experts=4, top=3, shared_ff=0))], width=128, vocab=157, taps=2, side_dim=0),
    # one head, one tap, a memory head of six values (no 16-byte pieces), all experts chosen, a loop of one round from
    # the first layer on
    "narrow": lambda: config([
        latent(heads=1, dim=8, rot_dim=2, vdim=16, q_rank=8, kv_rank=24, scale=0.5, base=50.0,
               mlp=moe(ff=8, experts=2, top=2, shared_ff=8)),
        memory(heads=1, dim=6, vdim=24, gate_cap=3.0, mlp=None)], width=64, vocab=97, eps=3e-4, taps=1, side_dim=8,
        loop=(0, 2, 1)),
    # five heads over a latent of 72 (padded to 128 in the tile kernel), three memory heads of 12, seven experts, three
    # taps, a single layer run three times in the middle
    "uneven": lambda: config([
        memory(heads=3, dim=12, vdim=40, gate_cap=5.0, mlp=dense(56)),
        latent(heads=5, dim=24, rot_dim=8, vdim=40, q_rank=56, kv_rank=72, scale=0.18, base=3e4,
               mlp=moe(ff=40, experts=7, top=3, shared_ff=24)),
        latent(heads=2, dim=40, rot_dim=24, vdim=12, q_rank=16, kv_rank=16, scale=0.12, mlp=dense(24))],
        width=88, vocab=301, taps=3, side_dim=20, loop=(1, 2, 3)),
}


def random_weights(config_dict: dict, seed: int = 0) -> dict:
    """bfloat16 tensors by checkpoint name, scaled so that activations stay of order one through the layers."""
    g = torch.Generator().manual_seed(seed)
    width = config_dict["width"]
    t: dict[str, torch.Tensor] = {}

    def matrix(name, rows, cols, gain=1.0):
        t[name] = (torch.randn(rows, cols, generator=g) * gain / math.sqrt(cols)).to(torch.bfloat16)

    def vector(name, size, mean=1.0, spread=0.2):
        t[name] = (mean + spread * torch.randn(size, generator=g)).to(torch.bfloat16)

    def scalar(name, mean=1.0, spread=0.2):
        t[name] = (mean + spread * torch.randn((), generator=g)).to(torch.bfloat16)

    n_layers = len(config_dict["layers"])
    side = config_dict.get("token_side", {}).get("dim", 0)
    taps = config_dict["canon"]["taps"]
    matrix("embed", config_dict["vocab"], width, gain=math.sqrt(width))
    matrix("head", config_dict["vocab"], width)
    scalar("final.norm")
    if side:
        matrix("side.embed", config_dict["vocab"], n_layers * side, gain=math.sqrt(n_layers * side))
    for i, layer in enumerate(config_dict["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        scalar(p + "norm1")
        t[p + "canon1"] = (0.4 * torch.randn(width, taps, generator=g)).to(torch.bfloat16)
        if layer["type"] == "latent_attention":
            heads = m["heads"]
            matrix(p + "mix.dq", m["q_rank"], width, 1.5)
            vector(p + "mix.dq.norm", m["q_rank"], 1.2, 0.3)
            matrix(p + "mix.uq", heads * (m["dim"] + m["rot_dim"]), m["q_rank"], 2.0)
            matrix(p + "mix.dkv", m["kv_rank"] + m["rot_dim"], width, 1.5)
            vector(p + "mix.dkv.norm", m["kv_rank"], 1.2, 0.3)
            matrix(p + "mix.uk", heads * m["dim"], m["kv_rank"], 2.0)
            matrix(p + "mix.uv", heads * m["vdim"], m["kv_rank"], 1.5)
            matrix(p + "mix.g", heads, width, 2.0)
            matrix(p + "mix.o", width, heads * m["vdim"])
        else:
            heads = m["heads"]
            matrix(p + "mix.q", heads * m["dim"], width, 1.5)
            matrix(p + "mix.k", heads * m["dim"], width, 1.5)
            matrix(p + "mix.v", heads * m["vdim"], width, 1.5)
            matrix(p + "mix.g", heads * m["vdim"], width, 2.0)
            matrix(p + "mix.o", width, heads * m["vdim"])
            vector(p + "mix.norm", heads * m["vdim"], 1.0, 0.3)
            matrix(p + "mix.i", heads, width, 3.0)
            vector(p + "mix.i.b", heads, 0.0, 1.0)
            matrix(p + "mix.f", heads, width, 3.0)
            vector(p + "mix.f.b", heads, 2.0, 1.0)
        mlp = layer.get("mlp")
        if mlp is not None:
            scalar(p + "norm2")
            if mlp["kind"] == "dense":
                matrix(p + "mlp.up", mlp["ff"], width, 1.5)
                vector(p + "mlp.up.b", mlp["ff"], 0.0, 0.3)
                matrix(p + "mlp.down", width, mlp["ff"])
                vector(p + "mlp.down.b", width, 0.0, 0.3)
            else:
                matrix(p + "mlp.router", mlp["router"]["experts"], width, 4.0)
                for e in range(mlp["router"]["experts"]):
                    matrix(p + f"mlp.e{e}.up", mlp["expert"]["ff"], width, 1.5)
                    matrix(p + f"mlp.e{e}.down", width, mlp["expert"]["ff"], 1.0)
                if mlp.get("shared") is not None:
                    matrix(p + "mlp.shared.up", mlp["shared"]["ff"], width, 1.5)
                    matrix(p + "mlp.shared.down", width, mlp["shared"]["ff"], 2.0)
                    matrix(p + "mlp.shared.sg", 1, width, 2.0)
        if side:
            matrix(p + "side.gate", side, width, 0.3)
            matrix(p + "side.proj", width, side)
            vector(p + "side.norm", width, 0.5, 0.1)
    return t


def make_engine(config_dict: dict, tensors: dict, dtype: str, max_tokens: int = 2048, **kwargs):
    from etalii.dllm_b200.config.registry import config_from_dict
    from etalii.dllm_b200.engine.engine import Engine

    kwargs.setdefault("max_length", 1024)
    return Engine(config_from_dict(config_dict), tensors, dtype=dtype, device="cuda:0", max_tokens=max_tokens, **kwargs)


def tokens_for(config_dict: dict, lengths, seed: int = 5):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, config_dict["vocab"], (n,), generator=g).tolist() for n in lengths]
