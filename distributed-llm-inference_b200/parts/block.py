"""Arrangements: how a layer's norms, mixer and feed-forward sit around the residual."""

from __future__ import annotations

from .base import BuildEnv, Part, ResidualStream, build_part, can_fuse, normed_input, register_part


@register_part("arrangement", "prenorm")
class PreNormBlock(Part):
    """x = x + mixer(norm(x)); x = x + ffn(norm(x)) (src/dli/model/llama.py:211-212).
    Roles: mixer_norm, mixer, ffn_norm, ffn.  The feed-forward's output stays pending on the
    stream; the next norm adds it."""

    graph_capturable = True

    def __init__(self, spec, env: BuildEnv) -> None:
        self.spec, self.env = spec, env
        self.mixer_norm = build_part("norm", spec.parts["mixer_norm"], env)
        self.mixer = build_part("mixer", spec.parts["mixer"], env)
        self.ffn_norm = build_part("norm", spec.parts["ffn_norm"], env)
        self.ffn = build_part("feed_forward", spec.parts["ffn"], env)

        if hasattr(self.mixer, "defer_output"):
            self.mixer.defer_output = can_fuse(self.ffn_norm, self.ffn)

    def children(self):
        return [self.mixer_norm, self.mixer, self.ffn_norm, self.ffn]

    def cache_need(self):
        """What this layer's run step keeps between steps: whatever its one mixer needs."""
        return self.mixer.cache_need()

    def first_consumer(self):
        """The norm that takes the stream's pending delta, and the part that reads its output."""
        return self.mixer_norm, self.mixer

    def defer_last_product(self, flag: bool) -> None:
        """Whether whoever runs after this layer can take the feed-forward's last product uncomputed."""
        if hasattr(self.ffn, "defer_output"):
            self.ffn.defer_output = bool(flag)

    def forward(self, stream: ResidualStream, batch, cache) -> None:
        y = normed_input(self.mixer_norm, stream.h, stream.take_pending(), self.mixer)
        a = self.mixer.forward(y, batch, cache)
        y = normed_input(self.ffn_norm, stream.h, a, self.ffn)
        stream.pending = self.ffn.forward(y)
