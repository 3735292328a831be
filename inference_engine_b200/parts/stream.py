"""Operations on the whole residual stream between layers (category ``stream``).

``reinject``: ``x <- W [x; x0]`` with ``x0`` the embedding's output of the same token and ``W`` of
shape ``[width, 2 width]`` (the stream's part first).  A model whose layers run several times in a
row with the same weights applies it before each pass.  The product runs in the compute dtype with
32-bit sums; its result is the new 32-bit stream.
"""

from __future__ import annotations

from .base import BuildEnv, Part, WeightDecl
from .registry import register_part


@register_part("stream", "reinject")
class Reinject(Part):
    category = "stream"
    needs_embedding = True  # the model keeps the embedding's output of the step for this part

    def __init__(self, weight: str, hidden_size: int, dtype) -> None:
        self.weight_name, self.hidden_size, self.dtype = weight, int(hidden_size), dtype
        self.weight = None

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, **_):
        return cls(params["weight"], params.get("hidden_size", env.hidden_size), env.torch_dtype)

    def weights(self) -> dict[str, WeightDecl]:
        return {self.weight_name: WeightDecl((self.hidden_size, 2 * self.hidden_size))}

    def bind(self, tensors, env: BuildEnv) -> None:
        self.weight = tensors[self.weight_name].to(self.dtype).contiguous()

    def forward(self, h, x0, ctx) -> None:
        both = ctx.ws.buffer("stream.both", h.shape[0], 2 * self.hidden_size, self.dtype)
        ctx.ops.concat_cast(h, x0, both)
        ctx.ops.linear(both, self.weight, out=h, tag="stream.reinject")
