"""Mixers made of other mixers.

``parallel_sum``: several mixers side by side that read the same input; the result is the sum of
their outputs, each times its own factor.  Every branch keeps its own cache (a tuple of requests,
a tuple of bindings).
"""

from __future__ import annotations

from ..config.spec import PartSpec
from .base import BuildEnv, Mixer
from .registry import build_part, register_part


def _part_spec(raw) -> PartSpec:
    return raw if isinstance(raw, PartSpec) else PartSpec(raw["kind"], dict(raw.get("params", {})))


@register_part("mixer", "parallel_sum")
class ParallelSum(Mixer):
    def __init__(self, branches: list[Mixer], scales: list[float], hidden_size: int) -> None:
        if len(branches) < 2 or len(branches) != len(scales):
            raise ValueError("a sum of mixers needs at least two branches, each with its factor")
        self.branches, self.scales, self.hidden_size = branches, [float(s) for s in scales], hidden_size
        for b in branches:
            b.allow_split = False  # the sum below takes whole outputs

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, **_):
        branches = [build_part("mixer", _part_spec(b["mixer"]), env) for b in params["branches"]]
        return cls(branches, [b["scale"] for b in params["branches"]], params.get("hidden_size", env.hidden_size))

    @property
    def captures(self) -> bool:
        return all(getattr(b, "captures", True) for b in self.branches)

    def parts(self):
        return list(self.branches)

    def cache_request(self):
        return tuple(b.cache_request() for b in self.branches)

    def forward(self, x, ctx, binding):
        import torch

        outs = [b.forward(x, ctx, bind) for b, bind in zip(self.branches, binding)]
        total = ctx.ws.buffer("parallel.sum", x.shape[0], self.hidden_size, torch.float32)
        ctx.ops.weighted_sum(outs[0], self.scales[0], outs[1], self.scales[1], total)
        for o, s in zip(outs[2:], self.scales[2:]):
            ctx.ops.weighted_sum(total, 1.0, o, s, total)
        return total
