"""Gaperax on the GPU against the plain implementation (tests/plain_gaperax.py): every mechanism alone through its part
or kernel, then whole models through the engine's step function, decode graph and generation loop, cut and batched in
every way a server would."""
import math

import numpy as np
import pytest
import torch

import gaperax_cases as C
import plain_gaperax as P
from helpers import TOL, host, rel_error
from test_revupel_gpu import PartHarness, _bf16, _feed, _inputs, _mixer_call, _pointing_weights, _runtime, _vector

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [("float32", torch.float32), ("bfloat16", torch.bfloat16)]
PART_TOL = {torch.float32: 2e-5, torch.bfloat16: 3e-2}
SHARP_TOL = {torch.float32: 5e-5, torch.bfloat16: 0.14}
"""For the tests whose weights make one score stand out: such sharp maps amplify the rounding of bfloat16 rows, and
what the tests decide (a key seen or not) moves the output by more than 0.2."""
SCHEDULE = [[(0, 70), (1, 2), (2, 17)], [(0, 1), (1, 1), (2, 1)], [(0, 1), (1, 1), (2, 1)], [(0, 2), (2, 65)],
            [(0, 1), (2, 1)], [(2, 1)]]


def _np(weights, renames=()):
    out = {}
    for name, value in weights.items():
        for old, new in renames:
            name = name.replace(old, new)
        out[name] = value.to(torch.float64).numpy()
    return out


# ---- the small parts --------------------------------------------------------------------------------------------------


@pytest.mark.parametrize("name,dtype", DTYPES)
@pytest.mark.parametrize("rows,width", [(1, 72), (5, 200), (70, 1000), (3, 4100), (9, 50), (4, 7)])
def test_norm_without_statistics(name, dtype, rows, width):
    from etalii.dllm_b200.parts import PartSpec, build_part

    rt = _runtime(dtype)
    g = torch.Generator().manual_seed(rows + width)
    norm = build_part("norm", PartSpec("dynamic_tanh", {"hidden_size": width}))
    weights = {"weight": _vector(g, width, 1.0, 0.3), "bias": _vector(g, width, 0.0, 0.3),
               "alpha": torch.tensor(0.8, dtype=torch.bfloat16)}
    norm.bind(weights, rt)
    x = (2.0 * torch.randn(rows, width, generator=g))
    w = _np(weights)
    want = P.dynamic_tanh(x.double().numpy(), w["alpha"], w["weight"], w["bias"])
    assert rel_error(host(norm.forward(x.to(DEV), rt)), want) <= (1e-6 if dtype == torch.float32 else 6e-3)
    some = torch.tensor([rows - 1, 0], dtype=torch.int32, device=DEV)
    got = host(norm.forward(x.to(DEV), rt, rows=some, n_rows=2, name="gathered"))
    assert rel_error(got, want[[rows - 1, 0]]) <= (1e-6 if dtype == torch.float32 else 6e-3)


@pytest.mark.parametrize("name,dtype", DTYPES)
@pytest.mark.parametrize("rows,width,ff", [(1, 72, 40), (5, 96, 56), (150, 200, 328), (70, 64, 8), (33, 256, 1024)])
def test_gated_feed_forward_with_the_tanh_form_of_gelu(name, dtype, rows, width, ff):
    """Steps of one, a few and many rows: the activation inside the first product's epilogue and as a kernel of its
    own."""
    from etalii.dllm_b200.parts import PartSpec, build_part

    rt = _runtime(dtype)
    g = torch.Generator().manual_seed(rows + ff)
    part = build_part("feed_forward", PartSpec("gated_mlp", {"hidden_size": width, "intermediate_size": ff,
                                                             "activation": "gelu_tanh"}))
    weights = {"gate": _bf16(g, ff, width, 2.5), "up": _bf16(g, ff, width, 1.5), "down": _bf16(g, width, ff)}
    part.bind(weights, rt)
    h = torch.randn(rows, width, generator=g).to(dtype).float()
    stream = torch.zeros(rows, width, device=DEV)
    part.forward(h.to(DEV).to(dtype), stream, None, rt)
    want = P.feed_forward(_np(weights), h.double().numpy())
    assert rel_error(host(stream), want) <= PART_TOL[dtype]


# ---- latent attention with a sink, interleaved pairs and stretched frequencies ------------------------------------------


def _shape(heads, dim, rot_dim, vdim, q_rank, kv_rank, base=1e4, scale=0.25, scaling="default"):
    rot = dict(base=base, dims=rot_dim)
    if scaling == "default":
        scaling = {"factor": 6.0, "original": 48, "fast": 12.0, "slow": 1.5}
    if scaling is not None:
        rot["scaling"] = scaling
    return dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, q_rank=q_rank, kv_rank=kv_rank, scale=scale, rot=rot)


def _latent(width, p, eps=1e-5):
    from etalii.dllm_b200.parts import PartSpec, build_part

    position = None
    if p["rot_dim"]:
        scaling = p["rot"].get("scaling")
        position = PartSpec("rotary", {"head_dim": p["rot_dim"], "theta": p["rot"]["base"], "rotary_dim": p["rot_dim"],
                                       "pairing": "interleaved",
                                       "scaling": dict(scaling, rope_type="yarn") if scaling else None})
    return build_part("mixer", PartSpec("latent_attention", {
        "hidden_size": width, "num_heads": p["heads"], "dim": p["dim"], "rot_dim": p["rot_dim"], "vdim": p["vdim"],
        "q_rank": p["q_rank"], "kv_rank": p["kv_rank"], "scale": p["scale"], "eps": eps, "position": position,
        "gate": False, "sink": True}))


def _latent_weights(g, width, p, sink=(0.5, 1.0)):
    heads = p["heads"]
    return {"dq": _bf16(g, p["q_rank"], width, 1.5), "dq_norm": _vector(g, p["q_rank"], 1.2, 0.3),
            "uq": _bf16(g, heads * (p["dim"] + p["rot_dim"]), p["q_rank"], 2.0),
            "dkv": _bf16(g, p["kv_rank"] + p["rot_dim"], width, 1.5), "dkv_norm": _vector(g, p["kv_rank"], 1.2, 0.3),
            "uk": _bf16(g, heads * p["dim"], p["kv_rank"], 2.0), "uv": _bf16(g, heads * p["vdim"], p["kv_rank"], 1.5),
            "sink": _vector(g, heads, *sink), "o": _bf16(g, width, heads * p["vdim"])}


def _plain_latent(w, p, h, eps=1e-5):
    names = _np(w, (("dq_norm", "dq.norm"), ("dkv_norm", "dkv.norm")))
    return P.latent_attention(names, p, h.double().numpy(), range(len(h)), None, eps)[0]


LATENT_SHAPES = {
    "unequal": _shape(3, 16, 8, 24, 40, 32),
    "one_head": _shape(1, 8, 2, 16, 8, 24, base=50.0, scale=0.5, scaling=None),
    "tiles": _shape(7, 48, 24, 40, 72, 128, base=1e5, scale=0.12),
    "nothing_rotated": _shape(2, 20, 0, 12, 24, 40, scale=0.3),
    "wide_rotation": _shape(4, 32, 64, 16, 48, 256, scale=0.08, scaling={"factor": 2.0, "original": 32, "fast": 4.0,
                                                                        "slow": 4.0}),
    "heads_across_tiles": _shape(40, 16, 16, 8, 32, 64, scale=0.2),
}


@pytest.mark.parametrize("name,dtype", DTYPES)
@pytest.mark.parametrize("shape", sorted(LATENT_SHAPES))
def test_latent_attention_part_in_pieces(name, dtype, shape):
    """Three sequences fed as a server would: a prompt portion that crosses a page border, portions of two tokens,
    single tokens beside neighbours, a sequence that ends early; against the plain mixer on each whole sequence."""
    rt = _runtime(dtype)
    p, width = LATENT_SHAPES[shape], 72
    part = _latent(width, p)
    g = torch.Generator().manual_seed(len(shape))
    weights = _latent_weights(g, width, p)
    part.bind(weights, rt)
    sequences = _inputs(dtype, width, 3)
    got = _feed(PartHarness(part.cache_need(), dtype, 3), _mixer_call(part, rt), sequences, SCHEDULE, width)
    for rows, h in zip(got, sequences):
        assert rel_error(rows, _plain_latent(weights, p, h)) <= PART_TOL[dtype]


@pytest.mark.parametrize("name,dtype", DTYPES)
@pytest.mark.parametrize("sink", [-30.0, 0.0, 4.0, 30.0])
def test_a_sink_takes_its_share_and_gives_nothing(name, dtype, sink):
    """A sink far below every score changes nothing, one far above leaves next to nothing for the keys, and between the
    two it takes exactly its share: in a prompt (the tile kernel in bfloat16), in portions and in tokens decoded alone
    (keys dealt to several blocks), at the first token too, whose only key is itself."""
    rt = _runtime(dtype)
    p, width = _shape(5, 16, 8, 24, 40, 64, scale=0.3), 72
    part = _latent(width, p)
    g = torch.Generator().manual_seed(7)
    weights = _latent_weights(g, width, p, sink=(sink, 0.5))
    part.bind(weights, rt)
    h = _inputs(dtype, width, 4, [230])[0]
    schedule = [[(0, 1)], [(0, 129)], [(0, 3)]] + [[(0, 1)]] * 97
    got = _feed(PartHarness(part.cache_need(), dtype, 1), _mixer_call(part, rt), [h], schedule, width)[0]
    want = _plain_latent(weights, p, h)
    assert rel_error(got, want) <= PART_TOL[dtype]
    without = _plain_latent(dict(weights, sink=torch.full((5,), -80.0)), p, h)
    if sink <= -30:
        assert rel_error(want, without) < 1e-9
    else:
        assert rel_error(want, without) > 0.1  # the test's premise: the sink matters


@pytest.mark.parametrize("name,dtype", DTYPES)
@pytest.mark.parametrize("far", [0, 1, 63, 64, 65, 127, 128, 300])
def test_a_far_key_among_hundreds(name, dtype, far):
    """One key far back, at the sequence's first places and at and around page borders, takes the weight of the last
    tokens, in the prompt and in a token decoded alone; without it the output differs by far more than the tolerance."""
    rt = _runtime(dtype)
    width = 48
    p = _shape(3, 16, 4, 24, 24, 24, base=1e6, scale=1.0, scaling=None)
    part = _latent(width, p)
    g = torch.Generator().manual_seed(20 + far)
    weights = _latent_weights(g, width, p)
    _pointing_weights(g, width, p, weights, 0.05)
    part.bind(weights, rt)
    n, half = 420, width // 2
    h = torch.randn(n + 1, width, generator=g)
    u = torch.randn(half, generator=g)
    h[far, half:] = u
    h[n - 1, :half] = h[n, :half] = u
    h = h.to(dtype).float()
    got = _feed(PartHarness(part.cache_need(), dtype, 1), _mixer_call(part, rt), [h], [[(0, n)], [(0, 1)]], width)[0]
    want = _plain_latent(weights, p, h)
    without = h.clone()
    without[far, half:] = torch.randn(half, generator=g).to(dtype).float()
    other = _plain_latent(weights, p, without)
    for row in (n - 1, n):
        assert rel_error(want[row], other[row]) > 0.2  # the test's premise: that key matters
        assert rel_error(got[row], want[row]) <= SHARP_TOL[dtype]


@pytest.mark.parametrize("name,dtype", DTYPES)
def test_pairs_turn_with_their_neighbours_and_by_the_stretched_angles(name, dtype):
    """Only the rotated part decides here (queries and keys have no other part worth speaking of), with a base so small
    that every pair turns visibly within the sequence: pairing i with i + half, plain frequencies or a magnitude of one
    would each give other weights."""
    rt = _runtime(dtype)
    width = 64
    p = _shape(2, 8, 16, 16, 32, 32, base=20.0, scale=0.6,
               scaling={"factor": 5.0, "original": 16, "fast": 2.0, "slow": 0.25})
    part = _latent(width, p)
    g = torch.Generator().manual_seed(3)
    weights = _latent_weights(g, width, p)
    uq = weights["uq"].float().view(2, 24, 32)
    uq[:, :8] *= 0.05
    uq[:, 8:] *= 3.0
    weights["uq"] = uq.view(48, 32).to(torch.bfloat16)
    dkv = weights["dkv"].float()
    dkv[32:] *= 3.0
    weights["dkv"] = dkv.to(torch.bfloat16)
    part.bind(weights, rt)
    h = _inputs(dtype, width, 9, [150])[0]
    schedule = [[(0, 100)]] + [[(0, 1)]] * 50
    got = _feed(PartHarness(part.cache_need(), dtype, 1), _mixer_call(part, rt), [h], schedule, width)[0]
    want = _plain_latent(weights, p, h)
    assert rel_error(got, want) <= SHARP_TOL[dtype]
    plain_angles = dict(p, rot=dict(base=20.0, dims=16))
    assert rel_error(want, _plain_latent(weights, plain_angles, h)) > 0.2  # the premise: the stretching matters


# ---- attention with sigmoid weights ---------------------------------------------------------------------------------


def _attention_shape(heads, kv_heads, dim, vdim, size, keep_first, scale=0.2):
    return dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale,
                mask=dict(size=size, keep_first=keep_first))


def _attention(width, p, eps=1e-5):
    from etalii.dllm_b200.parts import PartSpec, build_part

    return build_part("mixer", PartSpec("sigmoid_attention", {
        "hidden_size": width, "num_heads": p["heads"], "num_kv_heads": p["kv_heads"], "dim": p["dim"],
        "vdim": p["vdim"], "scale": p["scale"], "eps": eps, "window": p["mask"]["size"],
        "keep_first": p["mask"]["keep_first"], "distance_exponent": 8.0, "biases": True, "whole_norm": True,
        "head_bias": True, "head_mixing": True, "gate": True}))


def _attention_weights(g, width, p, head_bias=-2.0):
    heads, groups, dim, vdim = p["heads"], p["kv_heads"], p["dim"], p["vdim"]
    mix = (torch.eye(heads) * 0.6 + 0.4 * torch.randn(heads, heads, generator=g) / math.sqrt(heads)).to(torch.bfloat16)
    return {"q": _bf16(g, heads * dim, width, 1.5), "q_bias": _vector(g, heads * dim, 0.0, 0.3),
            "k": _bf16(g, groups * dim, width, 1.5), "k_bias": _vector(g, groups * dim, 0.0, 0.3),
            "v": _bf16(g, groups * vdim, width, 1.5), "v_bias": _vector(g, groups * vdim, 0.0, 0.3),
            "q_norm": _vector(g, heads * dim, 1.5, 0.4), "k_norm": _vector(g, groups * dim, 1.5, 0.4),
            "talk": mix, "pb": _vector(g, heads, head_bias, 0.7), "g": _bf16(g, heads * vdim, width, 2.0),
            "o": _bf16(g, width, heads * vdim, 0.5)}


def _plain_attention(w, p, h, eps=1e-5):
    names = _np(w, (("q_bias", "q.b"), ("k_bias", "k.b"), ("v_bias", "v.b"), ("q_norm", "q.norm"),
                    ("k_norm", "k.norm")))
    return P.sigmoid_attention(names, p, h.double().numpy(), range(len(h)), None, eps)[0]


ATTENTION_SHAPES = {
    "grouped": _attention_shape(4, 2, 24, 16, 40, 3),
    "one_head": _attention_shape(1, 1, 12, 8, 5, 1, scale=0.3),
    "tiles": _attention_shape(8, 2, 32, 16, 150, 70, scale=0.1),
    "nothing_kept": _attention_shape(6, 6, 8, 12, 70, 0),
    "all_seen": _attention_shape(3, 1, 20, 24, 500, 0, scale=0.15),
    "kept_beyond_the_window": _attention_shape(2, 2, 64, 64, 16, 100, scale=0.08),
    "many_heads": _attention_shape(24, 8, 16, 40, 33, 31),
    # (queries, a tile and the weights of 32 heads of 128 do not fit one block: two blocks of a cluster share them)
    "two_blocks": _attention_shape(32, 8, 128, 128, 90, 10, scale=0.05),
    "two_blocks_two_kv_heads": _attention_shape(32, 2, 112, 96, 40, 70, scale=0.05),
}


@pytest.mark.parametrize("name,dtype", DTYPES)
@pytest.mark.parametrize("shape", sorted(ATTENTION_SHAPES))
def test_sigmoid_attention_part_in_pieces(name, dtype, shape):
    rt = _runtime(dtype)
    p, width = ATTENTION_SHAPES[shape], 72
    part = _attention(width, p)
    g = torch.Generator().manual_seed(len(shape))
    weights = _attention_weights(g, width, p)
    part.bind(weights, rt)
    sequences = _inputs(dtype, width, 3)
    got = _feed(PartHarness(part.cache_need(), dtype, 3), _mixer_call(part, rt), sequences, SCHEDULE, width)
    for rows, h in zip(got, sequences):
        assert rel_error(rows, _plain_attention(weights, p, h)) <= PART_TOL[dtype]


@pytest.mark.parametrize("name,dtype", DTYPES)
@pytest.mark.parametrize("size,keep_first,marked", [(120, 24, 23), (120, 24, 24), (64, 1, 0), (64, 64, 63), (64, 65, 64),
                                                    (200, 0, 150), (33, 130, 129)])
def test_one_marked_value_shows_exactly_where_it_is_seen(name, dtype, size, keep_first, marked):
    """One position's value is made a hundred times the others' and every weight close to one: the rows that see the
    position (inside the window, or because it is one of the kept first positions) differ from the run without the
    mark, all others do not, in a prompt of 300 tokens and in 150 tokens decoded alone behind it. The position is the
    last kept one, the first that is not kept, at a page's border, or deep in the sequence."""
    rt = _runtime(dtype)
    width = 48
    p = _attention_shape(3, 3, 16, 16, size, keep_first)
    part = _attention(width, p)
    g = torch.Generator().manual_seed(size + marked)
    weights = _attention_weights(g, width, p, head_bias=5.0)
    v = torch.zeros(3 * 16, width)
    v[:, 0] = 1.0  # every value coordinate reads the input's first place
    weights["v"] = v.to(torch.bfloat16)
    weights["v_bias"] = (0.1 * weights["v_bias"].float()).to(torch.bfloat16)
    part.bind(weights, rt)
    n = 450
    h = torch.randn(n, width, generator=g)
    h[:, 0] = 0.0
    plain = h.to(dtype).float().clone()
    h[marked, 0] = 100.0
    h = h.to(dtype).float()
    schedule = [[(0, 300)]] + [[(0, 1)]] * 150
    got = _feed(PartHarness(part.cache_need(), dtype, 1), _mixer_call(part, rt), [h], schedule, width)[0]
    want, without = _plain_attention(weights, p, h), _plain_attention(weights, p, plain)
    seen = [i for i in range(n) if i >= marked and (i - marked < size or marked < keep_first)]
    unseen = [i for i in range(n) if i not in seen]
    moved = np.abs(want - without).max(axis=1) / np.abs(without).max()
    assert all(moved[i] > 0.2 for i in seen) and all(moved[i] == 0 for i in unseen)  # the test's premise
    assert seen and (marked < keep_first or unseen[-1] > marked)
    assert rel_error(got, want) <= PART_TOL[dtype]
    # the rows that do not see the mark equal the run without it, to rounding of their own sums
    if unseen:
        assert np.abs(got[unseen] - without[unseen]).max() <= PART_TOL[dtype] * np.abs(without).max()


@pytest.mark.parametrize("name,dtype", DTYPES)
def test_many_sequences_decode_side_by_side_over_pages_used_before(name, dtype):
    """Forty sequences of unequal lengths take slots and pages that other sequences have just given back, then decode
    together for eighty steps while their windows pass over what they decoded."""
    rt = _runtime(dtype)
    p, width, count = _attention_shape(4, 2, 16, 24, 50, 6), 64, 40
    part = _attention(width, p)
    g = torch.Generator().manual_seed(11)
    weights = _attention_weights(g, width, p)
    part.bind(weights, rt)
    harness = PartHarness(part.cache_need(), dtype, count, pages=200)
    lengths = [1 + (7 * i) % 90 for i in range(count)]
    waste = _inputs(dtype, width, 5, [100] * count)
    _feed(harness, _mixer_call(part, rt), waste, [[(i, 100) for i in range(count)]], width)
    for i in range(count):
        harness.again(i)
    sequences = _inputs(dtype, width, 6, [n + 80 for n in lengths])
    schedule = [[(i, n) for i, n in enumerate(lengths)]] + [[(i, 1) for i in range(count)]] * 80
    got = _feed(harness, _mixer_call(part, rt), sequences, schedule, width)
    for rows, h in zip(got, sequences):
        assert rel_error(rows, _plain_attention(weights, p, h)) <= PART_TOL[dtype]
    harness.cache.check()


# ---- whole models through the engine -------------------------------------------------------------------------------------


class Case:
    def __init__(self, case, seed=1):
        self.config = C.CASES[case]()
        self.tensors = C.random_weights(self.config, seed)
        self.weights = C.as_numpy(self.tensors)
        self._memo = {}

    def logits(self, tokens):
        key = tuple(tokens)
        if key not in self._memo:
            self._memo[key] = P.forward(self.config, self.weights, list(tokens))
        return self._memo[key]


_CASES = {}


def _case(name) -> Case:
    if name not in _CASES:
        _CASES[name] = Case(name)
    return _CASES[name]


def _run(engine, prompts, schedule):
    """Feeds `prompts` by `schedule` (steps of (prompt, count)); a prompt's slot is given back with its last token.
    Returns every position's logits per prompt."""
    at = [0] * len(prompts)
    slots = {}
    rows = [[] for _ in prompts]
    for step in schedule:
        for i, _ in step:
            if i not in slots:
                slots[i] = engine.open(1)[0]
        pieces = [prompts[i][at[i]:at[i] + n] for i, n in step]
        out = host(engine.step([slots[i] for i, _ in step], pieces, [list(range(len(p))) for p in pieces]))
        engine.check()
        offset = 0
        for (i, n) in step:
            rows[i].append(out[offset:offset + n])
            offset += n
            at[i] += n
            if at[i] == len(prompts[i]):
                engine.close([slots.pop(i)])
    assert not slots
    return [np.concatenate(r) for r in rows]


def _compare(case, got, prompts, dtype_name):
    """Every logit of every position within the tolerance in float32. bfloat16: nine of ten positions within the
    tolerance, the median within half of it and none beyond twice it (sums of up to a hundred and fifty sigmoid weights
    that nothing normalises carry the rounding of every key and value they read; what a lost key or a stale page does
    is decided in float32, where the same schedules run through the same cache and step function, and by the tests
    with weights made to point)."""
    errors = []
    for rows, tokens in zip(got, prompts):
        want = case.logits(tokens)
        assert rows.shape == want.shape
        errors += list(np.abs(rows - want).max(axis=1) / np.abs(want).max())
    errors = np.sort(np.asarray(errors))
    if dtype_name == "float32":
        assert errors[-1] <= TOL[dtype_name]
    else:
        assert errors[int(0.9 * (len(errors) - 1))] <= TOL[dtype_name] and errors[-1] <= 2 * TOL[dtype_name]
        assert np.median(errors) <= TOL[dtype_name] / 2


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(C.CASES))
def test_whole_prompts_alone_and_as_one_batch(name, dtype_name):
    case = _case(name)
    engine = C.make_engine(case.config, case.tensors, dtype_name)
    prompts = C.tokens_for(case.config, [1, 2, 70, 231, 5])
    alone = _run(engine, prompts, [[(i, len(p))] for i, p in enumerate(prompts)])
    _compare(case, alone, prompts, dtype_name)
    together = _run(engine, prompts, [[(i, len(p)) for i, p in enumerate(prompts)]])
    _compare(case, together, prompts, dtype_name)
    if dtype_name == "float32":  # batch mates change nothing beyond rounding; in float32 that is very little
        assert all(rel_error(a, b) <= 1e-5 for a, b in zip(alone, together))
    engine.cache.check()


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(C.CASES))
def test_portions_and_single_tokens(name, dtype_name):
    """One prompt cut into portions of 64, 2, 65, 3 and 1, 1, ...: the pieces cross page borders and window edges and
    end in token-by-token decoding; then the first tokens one by one from an empty cache."""
    case = _case(name)
    engine = C.make_engine(case.config, case.tensors, dtype_name)
    prompt = C.tokens_for(case.config, [250], seed=6)[0]
    schedule = [[(0, 64)], [(0, 2)], [(0, 65)], [(0, 3)]] + [[(0, 1)]] * 116
    _compare(case, _run(engine, [prompt], schedule), [prompt], dtype_name)
    schedule = [[(0, 1)]] * 5 + [[(0, 245)]]
    _compare(case, _run(engine, [prompt], schedule), [prompt], dtype_name)
    engine.cache.check()
    assert engine.cache.pages_held() == 0


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(C.CASES))
def test_unequal_batches_early_finishers_and_slots_used_again(name, dtype_name):
    """Requests of unequal length start together and decode together; the shorter ones end earlier and give their
    slots and pages back; later requests take those slots and pages (which still hold the old rows) and run beside the
    survivors."""
    case = _case(name)
    engine = C.make_engine(case.config, case.tensors, dtype_name, max_tokens=64 * 10, max_slots=4)
    prompts = C.tokens_for(case.config, [40, 9, 75, 30, 12], seed=8)
    schedule = [[(0, 30), (1, 6), (2, 66)]]
    schedule += [[(0, 1), (1, 1), (2, 1)]] * 3          # request 1 ends here
    schedule += [[(0, 1), (2, 1)]] * 6                  # request 2 ends here
    schedule += [[(3, 25), (4, 10)]]                    # two new requests take the freed slots
    schedule += [[(0, 1), (3, 1), (4, 1)]]              # ... and decode beside the survivor
    schedule += [[(3, 1), (4, 1)], [(3, 3)]]
    got = _run(engine, prompts, schedule)
    _compare(case, got, prompts, dtype_name)
    engine.cache.check()
    assert engine.cache.pages_held() == 0


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_long_decoding_through_the_decode_graph(dtype_name):
    """A hundred and fifty single-token steps of three sequences as the generation loop runs them (one captured graph
    replayed), across page borders and with every window passing over decoded tokens; then the last step's logits
    against the plain implementation on the whole history."""
    case = _case("mixed")
    engine = C.make_engine(case.config, case.tensors, dtype_name, decode_logits=True)
    prompts = C.tokens_for(case.config, [7, 20, 66], seed=9)
    slots = engine.open(3)
    first = host(engine.step(slots, prompts)).argmax(axis=1).tolist()
    chosen = engine.decode(slots, first, 150)
    histories = [p + [f] + [step[i] for step in chosen] for i, (p, f) in enumerate(zip(prompts, first))]
    graph_logits = host(engine.last_decode_graph.logits)  # of the last step: history without its last token
    for i, history in enumerate(histories):
        want = case.logits(history[:-1])[-1]
        assert rel_error(graph_logits[i], want) <= TOL[dtype_name] * (2.0 if dtype_name == "bfloat16" else 1.0)
        if dtype_name == "float32":
            assert int(np.argmax(want)) == history[-1]
    engine.close(slots)
    engine.cache.check()


def test_greedy_generation_through_the_generation_loop():
    """`Engine.generate` (batches planned by the scheduler, prompt step, decode graphs, early finishers) gives the
    tokens the plain implementation chooses greedily through its own carried state, in float32."""
    from etalii.dllm_b200 import SamplingOptions

    case = _case("mixed")
    engine = C.make_engine(case.config, case.tensors, "float32")
    prompts = C.tokens_for(case.config, [3, 18, 70], seed=10)
    results = engine.generate(prompts, 12, SamplingOptions(), ignore_eos=True)
    for prompt, result in zip(prompts, results):
        assert list(result.tokens) == P.greedy(case.config, case.weights, prompt, 12)
    again = engine.generate(prompts[:2], 5, SamplingOptions(), ignore_eos=True)  # the slots are used again
    assert [list(r.tokens) for r in again] == [list(r.tokens)[:5] for r in results[:2]]


def test_sampled_generation_runs_in_bfloat16():
    from etalii.dllm_b200 import SamplingOptions

    case = _case("tiled")
    engine = C.make_engine(case.config, case.tensors, "bfloat16")
    prompts = C.tokens_for(case.config, [5, 33], seed=11)
    a = engine.generate(prompts, 20, SamplingOptions(temperature=0.8, top_k=20, seed=3), ignore_eos=True)
    b = engine.generate(prompts, 20, SamplingOptions(temperature=0.8, top_k=20, seed=3), ignore_eos=True)
    assert [list(r.tokens) for r in a] == [list(r.tokens) for r in b] and all(len(r.tokens) == 20 for r in a)


def test_trace_replay_and_command_line_on_a_gaperax_folder(tmp_path):
    """bin/trace_run and `dllm-b200 generate` as subprocesses on a model folder the library wrote."""
    import json
    import os
    import subprocess
    import sys

    from etalii.dllm_b200.weights.random_init import write_model

    case = _case("narrow")
    folder = write_model(str(tmp_path / "model"), case.config, case.tensors)
    tokens = C.tokens_for(case.config, [20], seed=12)[0]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": tokens[:17], "want": [0, 16]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": tokens[17:18], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": tokens[18:20], "want": [1]}], "end": ["a"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    done = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype",
                           "float32", "--out", str(out), "--max-tokens", "128"],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                          timeout=900)
    assert done.returncode == 0, done.stderr[-2000:]
    assert [line for line in done.stdout.split("\n") if line.startswith("done")] == ["done 0", "done 1", "done 2"]
    want = case.logits(tokens)
    first = np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1)
    last = np.fromfile(out / "2.f32", dtype="<f4").reshape(1, -1)
    assert not (out / "1.f32").exists()
    assert rel_error(first, want[[0, 16]]) <= TOL["float32"] and rel_error(last, want[[19]]) <= TOL["float32"]

    tool = [sys.executable, os.path.join(root, "bin", "dllm-b200")]
    done = subprocess.run(tool + ["--model", folder, "info"], capture_output=True, text=True, timeout=600)
    assert done.returncode == 0 and json.loads(done.stdout)["architecture"] == "Gaperax"
    prompt = tokens[:9]
    done = subprocess.run(tool + ["--model", folder, "--dtype", "float32", "--cache-tokens", "256", "generate",
                                  "--prompt-ids", ",".join(map(str, prompt)), "--max-tokens", "6", "--ignore-eos"],
                          capture_output=True, text=True, timeout=900)
    assert done.returncode == 0, done.stderr[-2000:]
    assert [int(t) for t in done.stdout.split()] == P.greedy(case.config, case.weights, prompt, 6)
