"""Arrangements of a layer's parts.

``prenorm_residual`` (engine/model/layers.py:301-303): ``h = x + m * mixer(norm(x))``, then
``out = h + m * feed_forward(norm(h))``; ``m`` is the parameter ``residual_mult`` (1 unless the
model description says otherwise), and a layer without a feed-forward stops after its mixer.  The residual stream ``h`` is 32-bit and is updated in
place; each add is fused into the norm that follows it, so a block returns its
feed-forward's output as a pending ``delta`` for the next norm to add.

``sandwich_residual``: a norm before and after each sublayer, ``x <- x + post(mixer(pre(x)))`` and
``x <- x + post'(feed_forward(pre'(x)))``.  The norm after a sublayer, the add and the norm before the
next sublayer are one kernel: the block hands its last sublayer's raw output on as the pending delta
together with what is to be done to it before the add (``output_post``: an output bias, if the
sublayer has one, and the norm).
"""

from __future__ import annotations

from .base import Block, BuildEnv, CacheBinding
from .norm import PostNorm
from .registry import build_part, register_part


@register_part("block", "prenorm_residual")
class PreNormResidualBlock(Block):
    def __init__(self, mixer, feed_forward, pre_mixer, pre_feed_forward, residual_mult: float = 1.0) -> None:
        self.mixer, self.feed_forward = mixer, feed_forward
        self.pre_mixer, self.pre_feed_forward = pre_mixer, pre_feed_forward
        self.residual_mult = float(residual_mult)

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, *, layer, **_):
        has_ff = layer.feed_forward is not None
        return cls(
            build_part("mixer", layer.mixer, env),
            build_part("feed_forward", layer.feed_forward, env) if has_ff else None,
            build_part("norm", layer.norms["pre_mixer"], env),
            build_part("norm", layer.norms["pre_feed_forward"], env) if has_ff else None,
            params.get("residual_mult", 1.0),
        )

    def parts(self):
        both = [self.pre_mixer, self.mixer, self.pre_feed_forward, self.feed_forward]
        return [p for p in both if p is not None]

    def forward(self, h, delta, ctx, binding: CacheBinding | None, delta_scale: float = 1.0):
        x = self.pre_mixer.add_norm(h, delta, ctx, tag="norm.mixer", delta_scale=delta_scale)
        mixed = self.mixer.forward(x, ctx, binding)
        if self.feed_forward is None:
            return mixed
        x = self.pre_feed_forward.add_norm(h, mixed, ctx, tag="norm.ffn", delta_scale=self.residual_mult)
        return self.feed_forward.forward(x, ctx)


@register_part("block", "sandwich_residual")
class SandwichResidualBlock(Block):
    """Norms ``pre_mixer``, ``post_mixer`` and, with a feed-forward, ``pre_feed_forward`` and
    ``post_feed_forward``.  A feed-forward with an output bias leaves it to the post norm's kernel
    (``output_bias``)."""

    def __init__(self, mixer, feed_forward, norms: dict) -> None:
        self.mixer, self.feed_forward, self.norms = mixer, feed_forward, norms
        self.residual_mult = 1.0

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, *, layer, **_):
        has_ff = layer.feed_forward is not None
        names = ["pre_mixer", "post_mixer"] + (["pre_feed_forward", "post_feed_forward"] if has_ff else [])
        return cls(build_part("mixer", layer.mixer, env),
                   build_part("feed_forward", layer.feed_forward, env) if has_ff else None,
                   {n: build_part("norm", layer.norms[n], env) for n in names})

    def parts(self):
        return [*self.norms.values(), self.mixer] + ([self.feed_forward] if self.feed_forward is not None else [])

    @property
    def output_post(self) -> PostNorm:
        if self.feed_forward is None:
            return PostNorm(self.norms["post_mixer"])
        return PostNorm(self.norms["post_feed_forward"], getattr(self.feed_forward, "output_bias", None))

    def forward(self, h, delta, ctx, binding, delta_scale: float = 1.0, delta_post: PostNorm | None = None):
        x = self.norms["pre_mixer"].add_norm(h, delta, ctx, tag="norm.mixer", delta_scale=delta_scale,
                                             delta_post=delta_post)
        mixed = self.mixer.forward(x, ctx, binding)
        if self.feed_forward is None:
            return mixed
        x = self.norms["pre_feed_forward"].add_norm(h, mixed, ctx, tag="norm.ffn",
                                                    delta_post=PostNorm(self.norms["post_mixer"]))
        return self.feed_forward.forward(x, ctx)
