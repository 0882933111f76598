"""Revupel without a GPU: the configuration reader, the model as data (run order of a loop, cache entries, tensor
names), the keys-only cache entry's accounting, and the plain implementation against itself and on hand-made inputs."""
import copy
import math

import pytest
import torch

import plain_revupel as P
import revupel_cases as C
from etalii.dllm_b200 import architectures  # noqa: F401
from etalii.dllm_b200.cache.paged import CacheNeed, PagedCache
from etalii.dllm_b200.config.registry import ConfigError, architecture, config_from_dict
from etalii.dllm_b200.weights.loader import expected_tensors


@pytest.mark.parametrize("case", sorted(C.CASES))
def test_config_reads_back_and_names_every_tensor(case):
    config_dict = C.CASES[case]()
    config = config_from_dict(config_dict)
    assert config.model_type == "Revupel" and config.to_hf() == config_dict
    assert config_from_dict(config.to_hf()) == config
    spec = architecture(config.model_type).build_spec(config)
    expected = expected_tensors(spec)
    made = C.random_weights(config_dict)
    assert set(expected) == set(made)
    assert all(tuple(expected[name].shape) == tuple(made[name].shape) for name in made)
    assert expected["final.norm"].shape == () and expected["l0.norm1"].shape == ()


def test_a_loop_runs_its_layers_again_with_cache_entries_of_their_own():
    config = config_from_dict(C.CASES["mixed"]())
    spec = architecture("Revupel").build_spec(config)
    order = spec.run_order()
    assert [e.layer for e in order] == [0, 1, 2, 1, 2, 3] == P.run_order(C.CASES["mixed"]())
    assert [e.cache for e in order] == list(range(6)) and all(e.writes_cache for e in order)
    assert all(layer.block == "filtered_pre_norm" for layer in spec.layers)
    assert "feed_forward" not in spec.layers[2].parts and "token_input" in spec.layers[2].parts
    names = expected_tensors(spec)
    assert "l2.norm2" not in names and "l3.mlp.shared.up" not in names and "l0.mlp.shared.sg" in names
    plain = architecture("Revupel").build_spec(config_from_dict(C.CASES["tiled"]()))
    assert plain.schedule == () and all("token_input" not in layer.parts for layer in plain.layers)
    assert "side.embed" not in expected_tensors(plain)


@pytest.mark.parametrize("change,text", [
    (lambda c: c["layers"][0].update(type="window"), "type 'window' is not supported"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=6), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"].update(rot_dim=7), "rot_dim"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "no kv_rank"),
    (lambda c: c["layers"][1]["mixer"].update(gate_cap=0.0), "gate_cap"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "mlp.kind"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=6), "top 6 of 5"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["loop"].update(times=0), "loop.times"),
    (lambda c: c["canon"].update(taps=0), "taps"),
    (lambda c: c.pop("norm"), "no norm"),
])
def test_refused_configurations(change, text):
    config_dict = copy.deepcopy(C.CASES["mixed"]())
    change(config_dict)
    with pytest.raises(ConfigError, match=text):
        config_from_dict(config_dict)


def test_a_keys_only_entry_takes_and_returns_pages_like_any_other():
    need = CacheNeed("kv", kv_heads=1, head_dim=40, keys_only=True)
    other = CacheNeed("kv", kv_heads=2, head_dim=16)
    cache = PagedCache([need, other, need, CacheNeed("state", state_shape=(3, 5))], max_tokens=64 * 6, max_length=256)
    assert [entries for _, entries in cache.groups()] == [[0, 2], [1]]
    a, b = cache.acquire(2)
    cache.reserve(a, 130)
    cache.advance(a, 130)
    cache.reserve(b, 64)
    cache.advance(b, 64)
    assert cache.pages_held() == 2 * (3 + 1)
    cache.release([a])
    cache.check()
    c = cache.acquire(1)[0]
    cache.reserve(c, 65)
    cache.check()
    cache.release([b, c])
    assert cache.pages_held() == 0


@pytest.mark.parametrize("case", sorted(C.CASES))
def test_the_plain_model_gives_the_same_logits_however_a_prompt_is_cut(case):
    config = C.CASES[case]()
    weights = C.random_weights(config, 3)
    tokens = C.tokens_for(config, [23])[0]
    whole = P.forward(config, weights, tokens)
    for cuts in ([23], [1] * 23, [2, 5, 1, 15], [22, 1]):
        state, at, rows = P.new_state(config), 0, []
        for n in cuts:
            rows.append(P.forward(config, weights, tokens[at:at + n], state, at))
            at += n
        assert torch.allclose(torch.cat(rows), whole, rtol=0, atol=1e-9 * float(whole.abs().max()))


def test_plain_convolution_by_hand():
    taps = torch.tensor([[0.5, -1.0, 2.0]], dtype=P.F64)  # one channel, three taps, the last on the token itself
    h = torch.tensor([[1.0], [10.0], [100.0], [1000.0]], dtype=P.F64)
    kept = {}
    out = P.input_convolution(taps, h[:3], kept)
    assert out[:, 0].tolist() == [1 + 2.0, 10 + 20 - 1, 100 + 200 - 10 + 0.5]
    assert kept["conv"][:, 0].tolist() == [10.0, 100.0]
    assert P.input_convolution(taps, h[3:], kept)[0, 0].item() == 1000 + 2000 - 100 + 5


def test_plain_matrix_memory_by_hand():
    """One head of one key dimension and one value: with W_i = W_f = 0 and biases chosen, the gates are constants."""
    p = {"heads": 1, "dim": 1, "vdim": 1, "gate_cap": 50.0}
    one = torch.ones(1, 1, dtype=P.F64)
    w = {"q": one, "k": one, "v": 2 * one, "g": 0 * one, "o": one, "norm": torch.ones(1, dtype=P.F64),
         "i": 0 * one, "i.b": torch.tensor([1.0], dtype=P.F64), "f": 0 * one, "f.b": torch.tensor([0.0], dtype=P.F64)}
    h = torch.ones(2, 1, dtype=P.F64)
    kept = {}
    P.matrix_memory(w, p, h, 0.0, kept)
    i, f = 50.0 * math.tanh(1 / 50.0), math.log(0.5)
    m1 = max(f + 0.0, i)
    m2 = max(f + m1, i)
    s1 = math.exp(i - m1) * 2.0
    s2 = math.exp(f + m1 - m2) * s1 + math.exp(i - m2) * 2.0
    assert abs(float(kept["m"]) - m2) < 1e-12 and abs(float(kept["S"]) - s2) < 1e-12
    assert abs(float(kept["n"]) - s2 / 2.0) < 1e-12


def test_plain_experts_keep_their_share_of_the_softmax_over_all():
    w = {"router": torch.tensor([[1.0], [3.0], [2.0], [3.0]], dtype=P.F64)}
    chosen, weights = P.choose_experts(w, {"router": {"top": 2}}, torch.ones(1, 1, dtype=P.F64))
    total = sum(math.exp(v) for v in (1.0, 3.0, 2.0, 3.0))
    assert chosen.tolist() == [[1, 3]]  # the lower expert first on ties
    assert torch.allclose(weights, torch.tensor([[math.exp(3.0) / total] * 2], dtype=P.F64))
    assert float(weights.sum()) < 1.0
