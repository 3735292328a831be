"""Grouped-query attention without a softmax, over the paged cache.

``q = W_q h``, ``k = W_k h``, ``v = W_v h`` (no biases; value rows may have another size than key
rows).  Every query and key head is divided by its root mean square over ``dim`` and multiplied by
a weight of size ``dim`` that the heads share (one for queries, one for keys), then rotated by its
position on the first ``rotary_dim`` entries.  The weight of a visible key is ``sigmoid(q . k *
scale + bias[head])``; the weights are not normalised over the keys.  A query sees the keys at or
before it; with ``chunk`` only those of its own chunk of that many positions, counted from the
request's position 0 (pages before the current chunk are given back).  Query head ``h`` uses
key/value head ``h // (heads / kv_heads)``.  Scores and weights are 32-bit.
"""

from __future__ import annotations

from .base import BuildEnv, CacheBinding, Mixer, PagedKVRequest, WeightDecl
from .registry import register_part


@register_part("mixer", "sigmoid_attention")
class SigmoidAttention(Mixer):
    allow_split = True

    def __init__(self, *, names: dict, hidden_size: int, heads: int, kv_heads: int, dim: int, vdim: int,
                 scale: float, chunk: int | None, eps: float, position, dtype) -> None:
        if heads % kv_heads:
            raise ValueError(f"heads ({heads}) not divisible by kv_heads ({kv_heads})")
        if chunk is not None and chunk < 1:
            raise ValueError("a chunk holds at least one position")
        self.names, self.hidden_size = dict(names), hidden_size
        self.heads, self.kv_heads, self.dim, self.vdim = heads, kv_heads, dim, vdim
        self.scale, self.chunk, self.eps = float(scale), chunk, float(eps)
        self.position, self.dtype = position, dtype
        self.w_qkv = None

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, **_):
        position = env.positions[params["position"]] if params.get("position") else None
        return cls(names=params["names"], hidden_size=params.get("hidden_size", env.hidden_size),
                   heads=params["heads"], kv_heads=params["kv_heads"], dim=params["dim"], vdim=params["vdim"],
                   scale=params["scale"], chunk=params.get("chunk"), eps=params["eps"], position=position,
                   dtype=env.torch_dtype)

    def weights(self) -> dict[str, WeightDecl]:
        n, h = self.names, self.hidden_size
        return {
            n["q"]: WeightDecl((self.heads * self.dim, h)), n["k"]: WeightDecl((self.kv_heads * self.dim, h)),
            n["v"]: WeightDecl((self.kv_heads * self.vdim, h)),
            n["q_norm"]: WeightDecl((self.dim,), "vector", "ones_plus_normal"),
            n["k_norm"]: WeightDecl((self.dim,), "vector", "ones_plus_normal"),
            n["head_bias"]: WeightDecl((self.heads,), "vector"),
            n["o"]: WeightDecl((h, self.heads * self.vdim)),
        }

    def bind(self, tensors, env: BuildEnv) -> None:
        import torch

        n = self.names
        self.w_qkv = torch.cat([tensors[n[k]].to(self.dtype) for k in "qkv"]).contiguous()
        self.w_o = tensors[n["o"]].to(self.dtype).contiguous()
        self.q_norm = tensors[n["q_norm"]].float().contiguous()
        self.k_norm = tensors[n["k_norm"]].float().contiguous()
        self.head_bias = tensors[n["head_bias"]].float().contiguous()

    def cache_request(self) -> PagedKVRequest:
        return PagedKVRequest(self.kv_heads, self.dim, None, value_dim=self.vdim, chunk=self.chunk)

    def forward(self, x, ctx, binding: CacheBinding):
        import torch

        n = x.shape[0]
        group = ctx.groups[binding.group]
        k_cache, v_cache = group.k[binding.slot], group.v[binding.slot]
        ops, ws = ctx.ops, ctx.ws
        proj = ops.linear(x, self.w_qkv, ws=ws, tag="sigattn.qkv", out_dtype=torch.float32)
        q = ws.buffer("sigattn.q", n, self.heads * self.dim, self.dtype)
        table = self.position.rotary_table() if self.position is not None else None
        rot_dims = self.position.rotary_dim if self.position is not None else 0
        ops.qk_norm_rope_write(proj, ctx.positions, table, rot_dims, self.q_norm, self.k_norm, self.eps, q,
                               k_cache, v_cache, group.slot_mapping if binding.writes else None,
                               self.heads, self.kv_heads, self.dim, self.vdim, group.page_size)
        out = ws.buffer("sigattn.out", n, self.heads * self.vdim, self.dtype)
        ops.sigmoid_attention(q, k_cache, v_cache, group.block_tables, ctx, self.heads, self.kv_heads, self.dim,
                              self.vdim, group.page_size, self.scale, self.chunk, self.head_bias, out)
        return ops.linear(out, self.w_o, ws=ws, tag="sigattn.delta", out_dtype=torch.float32,
                          allow_split=self.allow_split)
