"""The Gaperax design as data: which parts each layer has, the order they run in, and the checkpoint's tensor names.

Every layer is pre-norm, x += mixer(norm1(x)) and then (a layer may have none) x += feed_forward(norm2(x)), with norms
that compute no statistics: tanh(alpha x) w + b, alpha one number. The mixer is one of
  latent_attention: softmax attention whose keys and values are linear maps of a cached latent, with one rotated key
                    part shared by the heads (interleaved pairs, frequencies stretched by the YaRN rule), queries
                    through a latent of their own, and a learned sink per head in the softmax's denominator;
  attention:        grouped-query attention without a softmax: q, k and v with biases, q and k normed over the whole
                    projection, a distance penalty slope_h (i - j), a sliding window that also keeps the sequence's
                    first tokens, weights sigmoid(score + b_h) mixed across heads by a matrix, and a sigmoid gate on
                    the concatenated heads.
The feed-forward is down(gelu_tanh(gate(h)) * up(h)). A layer may run with another layer's tensors (`weights_of`) and
a cache of its own: the schedule then names the owning layer twice. Tensor names: `embed`, `head`, `final.norm{,.b,
.alpha}`, and per layer i `l<i>.norm1{,.b,.alpha}`, `l<i>.norm2{,.b,.alpha}`, `l<i>.mix.*`, `l<i>.mlp.{gate,up,down}`."""
from __future__ import annotations

from ..config.gaperax import GaperaxConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

DISTANCE_EXPONENT = 8.0
"""Head h of H takes slope 2^(-8 (h + 1) / H) off a score per position of distance."""


def norm_spec(width: int, name: str) -> PartSpec:
    return PartSpec("dynamic_tanh", {"hidden_size": width},
                    {"weight": name, "bias": name + ".b", "alpha": name + ".alpha"})


def mixer_spec(width: int, eps: float, layer: dict, prefix: str) -> PartSpec:
    m, p = layer["mixer"], prefix + "mix."
    if layer["type"] == "latent_attention":
        position = None
        if m["rot_dim"]:
            scaling = m["rot"].get("scaling")
            if scaling is not None:
                scaling = {"rope_type": "yarn", "factor": float(scaling["factor"]),
                           "original": float(scaling["original"]), "fast": float(scaling["fast"]),
                           "slow": float(scaling["slow"])}
            position = PartSpec("rotary", {"head_dim": m["rot_dim"], "theta": float(m["rot"]["base"]),
                                           "rotary_dim": int(m["rot"]["dims"]), "pairing": "interleaved",
                                           "scaling": scaling})
        names = {name: p + name for name in ("dq", "uq", "dkv", "uk", "uv", "o", "sink")}
        names.update({"dq_norm": p + "dq.norm", "dkv_norm": p + "dkv.norm"})
        return PartSpec("latent_attention", {
            "hidden_size": width, "num_heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"], "vdim": m["vdim"],
            "q_rank": m["q_rank"], "kv_rank": m["kv_rank"], "scale": float(m["scale"]), "eps": eps,
            "position": position, "gate": False, "sink": True}, names)
    names = {name: p + name for name in ("q", "k", "v", "g", "o", "talk", "pb")}
    names.update({"q_bias": p + "q.b", "k_bias": p + "k.b", "v_bias": p + "v.b", "q_norm": p + "q.norm",
                  "k_norm": p + "k.norm"})
    return PartSpec("sigmoid_attention", {
        "hidden_size": width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "dim": m["dim"],
        "vdim": m["vdim"], "scale": float(m["scale"]), "eps": eps, "window": int(m["mask"]["size"]),
        "keep_first": int(m["mask"]["keep_first"]), "distance_exponent": DISTANCE_EXPONENT, "biases": True,
        "whole_norm": True, "head_bias": True, "head_mixing": True, "gate": True}, names)


def build_spec(config: GaperaxConfig) -> ModelSpec:
    width, eps = config.width, config.norm_eps
    owners = [config.weights_layer(index) for index in range(len(config.layers))]
    own = sorted(set(owners))  # (layers that have tensors, by their index in the model)
    layers = []
    for index in own:
        layer, prefix = config.layers[index], f"l{index}."
        parts = {"mixer": mixer_spec(width, eps, layer, prefix), "mixer_norm": norm_spec(width, prefix + "norm1")}
        block = "pre_norm_mixer"
        if layer.get("mlp") is not None:
            block = "pre_norm"
            parts["feed_forward"] = PartSpec(
                "gated_mlp", {"hidden_size": width, "intermediate_size": int(layer["mlp"]["ff"]),
                              "activation": "gelu_tanh"},
                {"gate": prefix + "mlp.gate", "up": prefix + "mlp.up", "down": prefix + "mlp.down"})
            parts["feed_forward_norm"] = norm_spec(width, prefix + "norm2")
        layers.append(LayerSpec(block=block, parts=parts))
    schedule = tuple(ScheduleEntry(own.index(owner), cache, True) for cache, owner in enumerate(owners))
    return ModelSpec(
        vocab_size=config.vocab, hidden_size=width, max_position=config.max_position,
        embedding=PartSpec("token_embedding", {"vocab_size": config.vocab, "hidden_size": width}, {"weight": "embed"}),
        layers=tuple(layers), final_norm=norm_spec(width, "final.norm"),
        head=PartSpec("linear", {"vocab_size": config.vocab, "hidden_size": width}, {"weight": "head"}),
        schedule=schedule, stop_token_ids=tuple(config.eos_token_ids),
        # (a layer without a feed-forward has no use for a second norm; a checkpoint that stores one all the same loads)
        ignored_suffixes=tuple(f"l{i}.norm2{end}" for i in own if config.layers[i].get("mlp") is None
                               for end in ("", ".b", ".alpha")),
    )


register_architecture("Gaperax", GaperaxConfig, build_spec)
