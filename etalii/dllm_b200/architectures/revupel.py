"""The Revupel design as data: which parts each layer has, the order they run in, and the checkpoint's tensor names.

Every layer is pre-norm with RMS norms whose weight is one number: x += mixer(h + conv(h)) with h = norm1(x) and conv a
short causal convolution over time on every channel; then (a layer may have none) x += feed_forward(norm2(x)); then,
in a model with a second token embedding, x += the layer's gated token input. The mixer is one of
  latent_attention: softmax attention whose keys and values are linear maps of a cached latent, with one rotated key
                    part shared by the heads, queries through a latent of their own, a sigmoid gate per head;
  mlstm:            a matrix memory per head written with exponential gates under a running maximum.
The feed-forward is dense (erf gelu, biases) or a mixture of relu-squared experts weighted by their shares of the
softmax over all experts, with a shared expert behind a sigmoid gate per token. A stretch of layers may run several
times in a row with the same weights (`loop`): every run has a cache entry of its own. Tensor names: `embed`, `head`,
`final.norm`, `side.embed`, and per layer i `l<i>.norm1`, `l<i>.norm2`, `l<i>.canon1`, `l<i>.mix.*`, `l<i>.mlp.*`,
`l<i>.side.{gate,proj,norm}`."""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.revupel import RevupelConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def mixer_spec(width: int, eps: float, layer: dict, prefix: str) -> PartSpec:
    m, p = layer["mixer"], prefix + "mix."
    if layer["type"] == "latent_attention":
        position = None
        if m["rot_dim"]:
            position = PartSpec("rotary", {"head_dim": m["rot_dim"], "theta": float(m["rot"]["base"]),
                                           "rotary_dim": int(m["rot"]["dims"]), "pairing": "halves"})
        names = {name: p + name for name in ("dq", "uq", "dkv", "uk", "uv", "g", "o")}
        names.update({"dq_norm": p + "dq.norm", "dkv_norm": p + "dkv.norm"})
        return PartSpec("latent_attention", {
            "hidden_size": width, "num_heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"], "vdim": m["vdim"],
            "q_rank": m["q_rank"], "kv_rank": m["kv_rank"], "scale": float(m["scale"]), "eps": eps,
            "position": position, "gate": True}, names)
    names = {name: p + name for name in ("q", "k", "v", "g", "o", "norm", "i", "f")}
    names.update({"i_bias": p + "i.b", "f_bias": p + "f.b"})
    return PartSpec("gated_matrix_memory", {"hidden_size": width, "heads": m["heads"], "dim": m["dim"],
                                            "vdim": m["vdim"], "gate_cap": float(m["gate_cap"]), "eps": eps}, names)


def feed_forward_spec(width: int, mlp: dict, prefix: str) -> PartSpec:
    p = prefix + "mlp."
    if mlp["kind"] == "dense":
        return PartSpec("activation_mlp", {"hidden_size": width, "intermediate_size": int(mlp["ff"]),
                                           "activation": "gelu", "biases": True, "token_gate": False},
                        {"up": p + "up", "down": p + "down", "up_bias": p + "up.b", "down_bias": p + "down.b"})
    experts = int(mlp["router"]["experts"])
    names = {"router": p + "router"}
    for e in range(experts):
        names.update({f"e{e}.{part}": f"{p}e{e}.{part}" for part in ("up", "down")})
    shared = None
    if mlp.get("shared") is not None:
        shared = PartSpec("activation_mlp", {"hidden_size": width, "intermediate_size": int(mlp["shared"]["ff"]),
                                             "activation": "relu_squared", "biases": False, "token_gate": True})
        names.update({"shared.up": p + "shared.up", "shared.down": p + "shared.down", "shared.gate": p + "shared.sg"})
    return PartSpec("activation_experts", {
        "hidden_size": width, "intermediate_size": int(mlp["expert"]["ff"]), "experts": experts,
        "top": int(mlp["router"]["top"]), "activation": "relu_squared", "weights": "softmax_all",
        "router_bias": False, "shared": shared}, names)


def build_spec(config: RevupelConfig) -> ModelSpec:
    width, eps = config.width, config.norm_eps
    n_layers = len(config.layers)
    layers = []
    for index, layer in enumerate(config.layers):
        prefix = f"l{index}."
        norm = lambda name: PartSpec("rmsnorm", {"hidden_size": width, "eps": eps, "scalar": True},  # noqa: E731
                                     {"weight": prefix + name})
        parts = {"mixer": mixer_spec(width, eps, layer, prefix), "mixer_norm": norm("norm1"),
                 "mixer_filter": PartSpec("short_convolution", {"hidden_size": width, "taps": config.taps},
                                          {"weight": prefix + "canon1"})}
        if layer.get("mlp") is not None:
            parts["feed_forward"] = feed_forward_spec(width, layer["mlp"], prefix)
            parts["feed_forward_norm"] = norm("norm2")
        if config.side_dim:
            parts["token_input"] = PartSpec("gated_token_input", {
                "hidden_size": width, "vocab_size": config.vocab, "dim": config.side_dim,
                "table_width": n_layers * config.side_dim, "offset": index * config.side_dim, "eps": eps,
                "activation": "gelu_tanh"},
                {"table": "side.embed", "gate": prefix + "side.gate", "proj": prefix + "side.proj",
                 "norm": prefix + "side.norm"})
        layers.append(LayerSpec(block="filtered_pre_norm", parts=parts))

    schedule = []
    if config.loop is not None:
        start, stop, times = config.loop["start"], config.loop["stop"], config.loop["times"]
        runs = list(range(start)) + list(range(start, stop)) * times + list(range(stop, n_layers))
        schedule = [ScheduleEntry(layer, cache, True) for cache, layer in enumerate(runs)]
    return ModelSpec(
        vocab_size=config.vocab, hidden_size=width, max_position=config.max_position,
        embedding=PartSpec("token_embedding", {"vocab_size": config.vocab, "hidden_size": width}, {"weight": "embed"}),
        layers=tuple(layers),
        final_norm=PartSpec("rmsnorm", {"hidden_size": width, "eps": eps, "scalar": True}, {"weight": "final.norm"}),
        head=PartSpec("linear", {"vocab_size": config.vocab, "hidden_size": width}, {"weight": "head"}),
        schedule=tuple(schedule), stop_token_ids=tuple(config.eos_token_ids),
        # (a layer without a feed-forward has no use for a second norm; a checkpoint that stores one all the same loads)
        ignored_suffixes=tuple(f"l{i}.norm2" for i, layer in enumerate(config.layers) if layer.get("mlp") is None),
    )


register_architecture("Revupel", RevupelConfig, build_spec)
