"""Arrangements of parts into a layer. "prenorm": h += mixer(norm(h)); h += feed_forward(norm(h))
(src/forward.cpp:200-244), over the slots mixer_norm, mixer, feed_forward_norm, feed_forward. The residual stream h
is float32; the sums happen in the parts' last matrix product, in float32.

"parallel_gated": ONE norm, whose rows n = norm(h) every sublayer reads, and one sum:
h += sigmoid(G1 n + g1) * mixer(n) + sigmoid(G2 n + g2) * feed_forward(n); the feed-forward (and its gate) may be
absent. Slots: norm, mixer, gate (family "gate": the logits of both gates in one product), feed_forward. A mixer
that is two mixers side by side hands over both results and their constants, so that the weighing, the gating and
the residual sum are one float32 kernel."""
from __future__ import annotations

from .base import Block, DeferredNorm, register_block


def normed_input(norm, consumer, h):
    """norm(h), or, for as few rows as the streaming product takes and a consumer that can normalise inside its
    first kernel, the norm deferred. How many rows that is, is the kernel library's answer, not a constant here."""
    if consumer.accepts_deferred_norm and getattr(norm, "fusable", False) and norm.rt.fast("norm"):
        from .. import fast_ops
        if h.shape[0] <= fast_ops.skinny_limits()[0]:
            return DeferredNorm(norm, h)
    return norm.forward(h)


@register_block("prenorm")
class PreNormBlock(Block):
    def __init__(self, mixer_norm, mixer, feed_forward_norm, feed_forward):
        super().__init__(mixer_norm=mixer_norm, mixer=mixer, feed_forward_norm=feed_forward_norm, feed_forward=feed_forward)

    def forward(self, h, step, cache, write_cache=True):
        h = self.mixer.forward(normed_input(self.mixer_norm, self.mixer, h), step, cache, h, write_cache)
        return self.feed_forward.forward(normed_input(self.feed_forward_norm, self.feed_forward, h), h)


@register_block("parallel_gated")
class ParallelGatedBlock(Block):
    def __init__(self, norm, mixer, gate=None, feed_forward=None):
        parts = {"norm": norm, "mixer": mixer}
        if gate is not None:
            parts["gate"] = gate
        if feed_forward is not None:
            parts["feed_forward"] = feed_forward
        super().__init__(**parts)
        self.gate, self.feed_forward = gate, feed_forward

    def forward(self, h, step, cache, write_cache=True):
        from .. import ops
        n = self.norm.forward(h)
        if hasattr(self.mixer, "forward_sides"):
            p, q, a, b = self.mixer.forward_sides(n, step, cache, write_cache)
        else:
            p, q, a, b = self.mixer.forward(n, step, cache, None, write_cache), None, 1.0, 1.0
        r = self.feed_forward.forward(n, None) if self.feed_forward is not None else None
        gates = self.gate.forward(n) if self.gate is not None else None
        return ops.gated_sum(h, gates, p, a, q, b, r)
