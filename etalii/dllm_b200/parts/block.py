"""Arrangements of a layer's parts. A block class declares the parts it takes as `PARTS` (name -> role), is built
with them as keyword arguments, exposes them as `parts` (name -> part) and its one mixer as `mixer`, and runs them
in `forward(x, batch, cache, rt, write_cache)` on the float32 residual stream x.

"pre_norm": x += mixer(norm(x)); x += feed_forward(norm(x)) (reference: src/etalii_dllm/transformer.py:493-558).
"output_norm": x += norm(mixer(x)); x += norm(feed_forward(x)): the sublayers read the stream itself and the norm sits
on what they return.
"filtered_pre_norm": x += mixer(filter(norm(x))); x += feed_forward(norm(x)); x += token_input(x): a filter over time
sits between the first norm and the mixer; the feed-forward and the token input are optional."""
from __future__ import annotations

import torch

from ..kernels import ops
from .norm import StreamOperand
from .registry import register_part


def normed(norm, consumer, x, rt):
    """The norm's output for `consumer`: a consumer that says so gets the norm still pending and may apply it
    inside its own kernel."""
    if getattr(consumer, "accepts_pending_norm", False) and hasattr(norm, "lazy"):
        return norm.lazy(x, rt)
    return norm.forward(x, rt)


class PreNormBlock:
    PARTS = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "feed_forward_norm": "norm"}

    def __init__(self, mixer, feed_forward, mixer_norm, feed_forward_norm) -> None:
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm
        self.parts = {"mixer": mixer, "feed_forward": feed_forward, "mixer_norm": mixer_norm,
                      "feed_forward_norm": feed_forward_norm}
        # each norm feeds exactly one part here, so its weight may move into that part's first product
        for norm, consumer in ((mixer_norm, mixer), (feed_forward_norm, feed_forward)):
            if hasattr(norm, "give_weight_to"):
                norm.give_weight_to(consumer)

    def forward(self, x, batch, cache, rt, write_cache: bool = True) -> None:
        self.mixer.forward(normed(self.mixer_norm, self.mixer, x, rt), x, batch, cache, rt, write_cache)
        self.feed_forward.forward(normed(self.feed_forward_norm, self.feed_forward, x, rt), x, batch, rt)


class PreNormMixerBlock:
    """A layer without a feed-forward: x += mixer(norm(x))."""

    PARTS = {"mixer": "mixer", "mixer_norm": "norm"}

    def __init__(self, mixer, mixer_norm) -> None:
        self.mixer, self.mixer_norm = mixer, mixer_norm
        self.parts = {"mixer": mixer, "mixer_norm": mixer_norm}
        if hasattr(mixer_norm, "give_weight_to"):
            mixer_norm.give_weight_to(mixer)

    def forward(self, x, batch, cache, rt, write_cache: bool = True) -> None:
        self.mixer.forward(normed(self.mixer_norm, self.mixer, x, rt), x, batch, cache, rt, write_cache)


def stream_input(consumer, x, rt):
    """The stream as `consumer`'s input: a consumer that says so (`accepts_stream`) gets it still in float32 with
    the rounding pending, anyone else the rounded activations. Where the kernel that last wrote the stream also left
    its rounding (`leave_rounded`) and no kernel has run since, that copy is the rounding."""
    ready = None
    kept = getattr(rt, "stream_rounded", None)
    if kept is not None and kept[0] == x.data_ptr() and kept[1] == tuple(x.shape) and kept[2] == ops.launches:
        ready = kept[3]
    operand = StreamOperand(x, rt, ready)
    return operand if getattr(consumer, "accepts_stream", False) else operand.tensor()


def add_normed_output(norm, x, out, rt) -> None:
    """x += norm(out); in bfloat16 the same kernel leaves the new rows rounded for whoever reads the stream next."""
    copy = rt.ws.buffer("stream_operand", tuple(x.shape), rt.dtype) if rt.dtype == torch.bfloat16 else None
    norm.add_normed(x, out, rt, copy)
    rt.stream_rounded = (x.data_ptr(), tuple(x.shape), ops.launches, copy) if copy is not None else None


class OutputNormBlock:
    """x += mixer_norm(mixer(x)); x += feed_forward_norm(feed_forward(x)). Each sublayer writes its float32 output to
    a work buffer (`epilogue=ops.EPI_STORE_F32`) and the norm adds the normed rows into the stream in one kernel
    (`add_normed`), which also leaves the stream's rounding for the next sublayer's products."""

    PARTS = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "feed_forward_norm": "norm"}

    def __init__(self, mixer, feed_forward, mixer_norm, feed_forward_norm) -> None:
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm
        self.parts = {"mixer": mixer, "feed_forward": feed_forward, "mixer_norm": mixer_norm,
                      "feed_forward_norm": feed_forward_norm}

    def forward(self, x, batch, cache, rt, write_cache: bool = True) -> None:
        out = rt.ws.buffer("sublayer_out", tuple(x.shape), torch.float32)
        self.mixer.forward(stream_input(self.mixer, x, rt), out, batch, cache, rt, write_cache,
                           epilogue=ops.EPI_STORE_F32)
        add_normed_output(self.mixer_norm, x, out, rt)
        self.feed_forward.forward(stream_input(self.feed_forward, x, rt), out, batch, rt, epilogue=ops.EPI_STORE_F32)
        add_normed_output(self.feed_forward_norm, x, out, rt)


class OutputNormMixerBlock:
    """A layer without a feed-forward: x += mixer_norm(mixer(x))."""

    PARTS = {"mixer": "mixer", "mixer_norm": "norm"}

    def __init__(self, mixer, mixer_norm) -> None:
        self.mixer, self.mixer_norm = mixer, mixer_norm
        self.parts = {"mixer": mixer, "mixer_norm": mixer_norm}

    def forward(self, x, batch, cache, rt, write_cache: bool = True) -> None:
        out = rt.ws.buffer("sublayer_out", tuple(x.shape), torch.float32)
        self.mixer.forward(stream_input(self.mixer, x, rt), out, batch, cache, rt, write_cache,
                           epilogue=ops.EPI_STORE_F32)
        add_normed_output(self.mixer_norm, x, out, rt)


class FilteredPreNormBlock:
    """x += mixer(filter(mixer_norm(x))); then, where the layer has them, x += feed_forward(feed_forward_norm(x)) and
    x += token_input(x). The filter (a short convolution over time) keeps a history of its own beside what the mixer
    keeps: the block answers for the layer's cache need and hands each part its view."""

    PARTS = {"mixer": "mixer", "mixer_norm": "norm", "mixer_filter": "filter"}
    OPTIONAL_PARTS = {"feed_forward": "feed_forward", "feed_forward_norm": "norm", "token_input": "token_input"}

    def __init__(self, mixer, mixer_norm, mixer_filter, feed_forward=None, feed_forward_norm=None,
                 token_input=None) -> None:
        if (feed_forward is None) != (feed_forward_norm is None):
            raise ValueError("a feed-forward and its norm come together")
        self.mixer, self.mixer_norm, self.mixer_filter = mixer, mixer_norm, mixer_filter
        self.feed_forward, self.feed_forward_norm, self.token_input = feed_forward, feed_forward_norm, token_input
        self.parts = {name: part for name, part in (
            ("mixer", mixer), ("mixer_norm", mixer_norm), ("mixer_filter", mixer_filter),
            ("feed_forward", feed_forward), ("feed_forward_norm", feed_forward_norm), ("token_input", token_input))
            if part is not None}
        if feed_forward is not None and hasattr(feed_forward_norm, "give_weight_to"):
            feed_forward_norm.give_weight_to(feed_forward)
        self._filter_keeps = mixer_filter.cache_need() is not None
        self._mixer_keeps = hasattr(mixer, "cache_need") and mixer.cache_need() is not None

    def cache_need(self):
        from ..cache.paged import CacheNeed

        needs = []
        if self._mixer_keeps:
            needs.append(self.mixer.cache_need())
        if self._filter_keeps:
            needs.append(self.mixer_filter.cache_need())
        if not needs:
            return None
        return CacheNeed("several", parts=tuple(needs))

    def forward(self, x, batch, cache, rt, write_cache: bool = True) -> None:
        views = list(cache) if cache is not None else []
        mixer_view = views.pop(0) if self._mixer_keeps else None
        history = views.pop(0) if self._filter_keeps else None
        h = self.mixer_filter.forward(self.mixer_norm, x, batch, history, rt)
        self.mixer.forward(h, x, batch, mixer_view, rt, write_cache)
        if self.feed_forward is not None:
            self.feed_forward.forward(normed(self.feed_forward_norm, self.feed_forward, x, rt), x, batch, rt)
        if self.token_input is not None:
            self.token_input.forward(x, batch, rt)


register_part("block", "pre_norm", PreNormBlock)
register_part("block", "filtered_pre_norm", FilteredPreNormBlock)
register_part("block", "output_norm", OutputNormBlock)
register_part("block", "output_norm_mixer", OutputNormMixerBlock)
register_part("block", "pre_norm_mixer", PreNormMixerBlock)
