"""Gaperax without a GPU: the configuration reader, the model as data (layers that run with another layer's weights,
cache entries, tensor names), the accounting of a windowed cache entry that keeps a sequence's first pages, the
stretched rotary frequencies, and the plain implementation against itself and on hand-made inputs."""
import copy
import math

import numpy as np
import pytest

import gaperax_cases as C
import plain_gaperax as P
from etalii.dllm_b200 import architectures  # noqa: F401
from etalii.dllm_b200.cache.paged import CacheNeed, PagedCache
from etalii.dllm_b200.config.registry import ConfigError, architecture, config_from_dict
from etalii.dllm_b200.parts.position import rotary_frequencies, rotary_magnitude
from etalii.dllm_b200.weights.loader import expected_tensors


@pytest.mark.parametrize("case", sorted(C.CASES))
def test_config_reads_back_and_names_every_tensor(case):
    config_dict = C.CASES[case]()
    config = config_from_dict(config_dict)
    assert config.model_type == "Gaperax" and config.to_hf() == config_dict
    assert config_from_dict(config.to_hf()) == config
    spec = architecture(config.model_type).build_spec(config)
    expected = expected_tensors(spec)
    made = C.random_weights(config_dict)
    assert set(expected) == set(made)
    assert all(tuple(expected[name].shape) == tuple(made[name].shape) for name in made)
    assert expected["final.norm.alpha"].shape == ()


def test_layers_that_run_with_another_layers_weights_have_caches_of_their_own():
    config = config_from_dict(C.CASES["mixed"]())
    spec = architecture("Gaperax").build_spec(config)
    order = spec.run_order()
    assert len(spec.layers) == 3  # only three layers have tensors
    assert [e.layer for e in order] == [0, 1, 2, 0, 1, 0]  # (the last one's `weights_of` leads to 0 through 3)
    assert [e.cache for e in order] == list(range(6)) and all(e.writes_cache for e in order)
    assert [layer.block for layer in spec.layers] == ["pre_norm", "pre_norm", "pre_norm_mixer"]
    names = expected_tensors(spec)
    assert "l3.mix.q" not in names and "l2.norm2" not in names and "l2.mlp.up" not in names
    assert {"l0.mix.talk", "l0.mix.q.b", "l0.mix.k.norm", "l1.mix.sink", "l1.mix.dkv.norm", "l1.norm2.alpha"} <= set(names)
    needs = [spec.layers[e.layer].parts["mixer"] for e in order]
    assert needs[0].params["window"] == 40 and needs[0].params["keep_first"] == 3
    assert needs[1].params["position"].params["pairing"] == "interleaved"
    assert needs[1].params["position"].params["scaling"]["rope_type"] == "yarn"


@pytest.mark.parametrize("change,text", [
    (lambda c: c["layers"][0].update(type="mlstm"), "type 'mlstm' is not supported"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=6), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"].update(rot_dim=7), "rot_dim"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "no kv_rank"),
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].pop("slow"), "no slow"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "not a multiple"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "mask.size"),
    (lambda c: c["layers"][0]["mixer"]["mask"].pop("keep_first"), "no keep_first"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "mlp.kind"),
    (lambda c: c["layers"][3].update(weights_of=9), "weights_of 9"),
    (lambda c: c["layers"][0].update(weights_of=3), "leads back to itself"),
    (lambda c: c["layers"][3].update(weights_of=1), "other sizes"),
    (lambda c: c.pop("norm"), "no norm"),
])
def test_refused_configurations(change, text):
    config_dict = copy.deepcopy(C.CASES["mixed"]())
    change(config_dict)
    with pytest.raises(ConfigError, match=text):
        config_from_dict(config_dict)


def test_a_window_that_keeps_the_first_positions_keeps_their_pages():
    """A window of 100 with 70 kept first positions: pages 0 and 1 hold kept positions and stay; the pages between them
    and the window go back to the pool while the sequence runs."""
    need = CacheNeed("kv", kv_heads=2, head_dim=8, value_dim=12, window=100, keep_first=70)
    plain = CacheNeed("kv", kv_heads=2, head_dim=8, value_dim=12, window=100)
    cache = PagedCache([need, plain], max_tokens=64 * 40, max_length=1024, max_slots=2)
    (slot,) = cache.acquire(1)
    cache.reserve(slot, 600)
    cache.advance(slot, 600)
    for _ in range(5):
        cache.reserve(slot, 1)
        cache.advance(slot, 1)
    kept, windowed = (group for group in cache._groups)
    held = [i for i, page in enumerate(kept.pages_of[slot]) if page is not None]
    assert held == [0, 1, 7, 8, 9]  # 605 tokens: the window starts at 505, in page 7
    assert [i for i, page in enumerate(windowed.pages_of[slot]) if page is not None] == [7, 8, 9]
    cache.check()
    cache.release([slot])
    assert cache.pages_held() == 0


def test_stretched_frequencies_by_hand():
    """Eight pairs, base 100, 64 original positions: pair i turns 64 f_i / (2 pi) times; those that turn more than
    `fast` times stay, those that turn fewer than `slow` times are divided by the factor, a ramp joins them."""
    scaling = {"rope_type": "yarn", "factor": 4.0, "original": 64.0, "fast": 4.0, "slow": 0.5}
    got = rotary_frequencies(16, 100.0, scaling)
    plain = [100.0 ** (-2.0 * i / 16) for i in range(8)]
    index = lambda turns: 16 * math.log(64 / (2 * math.pi * turns)) / (2 * math.log(100.0))  # noqa: E731
    low, high = math.floor(index(4.0)), math.ceil(index(0.5))
    assert (low, high) == (1, 6)
    for i in range(8):
        ramp = min(max((i - low) / (high - low), 0.0), 1.0)
        assert got[i] == pytest.approx(plain[i] / 4.0 * ramp + plain[i] * (1 - ramp), rel=1e-15)
    assert got[0] == plain[0] and got[1] == plain[1] and got[7] == pytest.approx(plain[7] / 4)
    assert rotary_magnitude(scaling) == pytest.approx(0.1 * math.log(4.0) + 1.0)
    assert rotary_magnitude(None) == 1.0 and rotary_frequencies(16, 100.0, None) == pytest.approx(plain)
    ours, magnitude = P.stretched_frequencies(16, 100.0, {k: v for k, v in scaling.items() if k != "rope_type"})
    assert list(ours) == pytest.approx(got, rel=1e-15) and magnitude == pytest.approx(rotary_magnitude(scaling))


@pytest.mark.parametrize("case", sorted(C.CASES))
def test_the_plain_model_gives_the_same_logits_however_a_prompt_is_cut(case):
    config = C.CASES[case]()
    weights = C.as_numpy(C.random_weights(config, 3))
    tokens = C.tokens_for(config, [90])[0]
    whole = P.forward(config, weights, tokens)
    for cuts in ([90], [1] * 90, [2, 5, 1, 82], [89, 1]):
        state, at, rows = P.new_state(config), 0, []
        for n in cuts:
            rows.append(P.forward(config, weights, tokens[at:at + n], state, at))
            at += n
        assert np.allclose(np.concatenate(rows), whole, rtol=0, atol=1e-9 * float(np.abs(whole).max()))


def test_plain_norm_and_feed_forward_by_hand():
    x = np.array([[0.5, -2.0]])
    out = P.dynamic_tanh(x, 2.0, np.array([3.0, 1.0]), np.array([0.25, -1.0]))
    assert out[0] == pytest.approx([3 * math.tanh(1.0) + 0.25, math.tanh(-4.0) - 1.0])
    w = {"gate": np.array([[1.0, 0.0]]), "up": np.array([[0.0, 2.0]]), "down": np.array([[1.0], [-1.0]])}
    g = 0.5 * 0.5 * (1 + math.tanh(math.sqrt(2 / math.pi) * (0.5 + 0.044715 * 0.125)))
    assert P.feed_forward(w, x)[0] == pytest.approx([g * -4.0, g * 4.0])


def test_plain_sink_counts_once_and_has_no_value():
    """One head, identity maps, one position: the only key's weight is e^s / (e^s + e^sink)."""
    m = {"heads": 1, "dim": 1, "rot_dim": 0, "vdim": 1, "q_rank": 1, "kv_rank": 1, "scale": 1.0}
    one = np.ones((1, 1))
    w = {"dq": one, "dq.norm": np.ones(1), "uq": 3 * one, "dkv": one, "dkv.norm": np.ones(1), "uk": one, "uv": 5 * one,
         "o": one, "sink": np.array([0.7])}
    out, kept = P.latent_attention(w, m, np.ones((1, 1)), [0], None, 0.0)
    assert out[0, 0] == pytest.approx(5.0 * math.exp(3.0) / (math.exp(3.0) + math.exp(0.7)))
    out, _ = P.latent_attention(w, m, np.ones((1, 1)), [1], kept, 0.0)  # two equal keys share what the sink leaves
    assert out[0, 0] == pytest.approx(5.0 * 2 * math.exp(3.0) / (2 * math.exp(3.0) + math.exp(0.7)))


def test_plain_window_keeps_the_first_positions_at_their_true_distance():
    assert [int(j) for j in range(10) if P.visible(np.int64(9), np.int64(j), 3, 2)] == [0, 1, 7, 8, 9]
    assert [int(j) for j in range(10) if P.visible(np.int64(2), np.int64(j), 3, 2)] == [0, 1, 2]
    # one head, key = query = 1 after the norm, no mixing: the weight of key j is sigmoid(scale - slope (i - j) + b)
    m = {"heads": 1, "kv_heads": 1, "dim": 1, "vdim": 1, "scale": 2.0, "mask": {"size": 2, "keep_first": 1}}
    one = np.ones((1, 1))
    w = {"q": one, "q.b": np.zeros(1), "k": one, "k.b": np.zeros(1), "v": one, "v.b": np.array([1.0]),
         "q.norm": np.ones(1), "k.norm": np.ones(1), "talk": 0.5 * one, "pb": np.array([-1.0]), "g": 0 * one, "o": one}
    out, _ = P.sigmoid_attention(w, m, np.ones((4, 1)), range(4), None, 0.0)
    slope = 2.0 ** -8
    weight = lambda d: 1 / (1 + math.exp(-(2.0 - slope * d - 1.0)))  # noqa: E731
    # position 3 sees 0 (kept, three away), 2 and 3; values are 2; mixing halves; the gate is sigmoid(0)
    assert out[3, 0] == pytest.approx((weight(3) + weight(1) + weight(0)) * 2.0 * 0.5 * 0.5)
    assert out[0, 0] == pytest.approx(weight(0) * 2.0 * 0.5 * 0.5)
