"""Attention over a shared low-rank latent: every token caches one latent vector and one rotated
key part, from which all heads' keys and values follow.

Per token, with ``h`` the mixer's input: ``q = W_q h`` is laid out head by head as ``dim``
unrotated then ``rot_dim`` rotated entries.  ``W_dkv h`` has ``kv_rank + rot_dim`` rows: the first
``kv_rank``, divided by their root mean square (eps inside the root) and multiplied by a weight,
are the latent ``c``; the rest is one key part shared by all heads.  The rotated query and key
parts are turned by the position's angles (pairs ``2i, 2i+1``; the first ``rot.dims`` entries of
the part, the rest pass).  Head ``n``'s key is ``[W_uk[n] c, rotated part]``, its value
``W_uv[n] c``; scores are scaled by ``scale``, masked causally and soft-maxed; each head's output
is multiplied by ``sigmoid(W_g h)[n]``, and ``W_o`` maps the concatenated heads back.

Only ``c`` and the rotated key part are cached (one row of ``kv_rank + rot_dim`` numbers per
token and layer, shared by the heads).  The products with ``W_uk`` and ``W_uv`` are moved to the
query side: ``q_unrotated[n] . (W_uk[n] c) = (W_uk[n]^T q_unrotated[n]) . c``, and
``sum_j p_j W_uv[n] c_j = W_uv[n] sum_j p_j c_j``.  So the attention runs with one shared
key/value head whose key rows are the cached rows and whose value rows are their first
``kv_rank`` entries, in prompts and in decoding alike, and nothing is expanded per cached token.
"""

from __future__ import annotations

from .base import BuildEnv, CacheBinding, Mixer, PagedKVRequest, WeightDecl
from .registry import register_part


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    def __init__(self, *, names: dict, hidden_size: int, heads: int, dim: int, rot_dim: int, vdim: int,
                 kv_rank: int, scale: float, eps: float, position, dtype) -> None:
        self.names, self.hidden_size, self.heads = dict(names), hidden_size, heads
        self.dim, self.rot_dim, self.vdim, self.kv_rank = dim, rot_dim, vdim, kv_rank
        self.scale, self.eps, self.position, self.dtype = float(scale), float(eps), position, dtype
        if position is not None:
            if getattr(position, "layout", "halves") != "interleaved":
                raise ValueError("the latent attention rotates interleaved pairs: give it a rotary "
                                 "encoding with layout='interleaved'")
            if position.rotary_dim > rot_dim:
                raise ValueError(f"rotary dims ({position.rotary_dim}) exceed the rotated part ({rot_dim})")
        self.q_size = heads * (dim + rot_dim)
        self.row = kv_rank + rot_dim  # a cached row
        self.w_in = self.w_uk_t = self.w_uv = self.w_o = self.latent_norm = None

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, **_):
        position = env.positions[params["position"]] if params.get("position") else None
        return cls(names=params["names"], hidden_size=params.get("hidden_size", env.hidden_size),
                   heads=params["heads"], dim=params["dim"], rot_dim=params["rot_dim"],
                   vdim=params["vdim"], kv_rank=params["kv_rank"], scale=params["scale"],
                   eps=params["eps"], position=position, dtype=env.torch_dtype)

    def weights(self) -> dict[str, WeightDecl]:
        n, h = self.names, self.hidden_size
        return {
            n["q"]: WeightDecl((self.q_size, h)),
            n["dkv"]: WeightDecl((self.row, h)),
            n["latent_norm"]: WeightDecl((self.kv_rank,), "vector", "ones_plus_normal"),
            n["uk"]: WeightDecl((self.heads * self.dim, self.kv_rank)),
            n["uv"]: WeightDecl((self.heads * self.vdim, self.kv_rank)),
            n["gate"]: WeightDecl((self.heads, h)),
            n["o"]: WeightDecl((h, self.heads * self.vdim)),
        }

    def bind(self, tensors, env: BuildEnv) -> None:
        import torch

        n = self.names
        # one product for the query, the latent with the shared key part, and the gate
        self.w_in = torch.cat([tensors[n[k]].to(self.dtype) for k in ("q", "dkv", "gate")]).contiguous()
        self.latent_norm = tensors[n["latent_norm"]].float().contiguous()
        uk = tensors[n["uk"]].to(self.dtype).view(self.heads, self.dim, self.kv_rank)
        self.w_uk_t = uk.transpose(1, 2).contiguous()  # [heads, kv_rank, dim]: query side of the key product
        self.w_uv = tensors[n["uv"]].to(self.dtype).view(self.heads, self.vdim, self.kv_rank).contiguous()
        self.w_o = tensors[n["o"]].to(self.dtype).contiguous()

    def cache_request(self) -> PagedKVRequest:
        return PagedKVRequest(1, self.row, None, value_dim=0)

    def forward(self, x, ctx, binding: CacheBinding):
        import torch

        n, H = x.shape[0], self.heads
        group = ctx.groups[binding.group]
        cache = group.k[binding.slot]
        proj = ctx.ops.linear(x, self.w_in, ws=ctx.ws, tag="latent.in", out_dtype=torch.float32)
        q_plain = ctx.ws.buffer("latent.q_plain", n, H * self.dim, self.dtype)
        q_abs = ctx.ws.buffer("latent.q", n, H * self.row, self.dtype)
        gate = ctx.ws.buffer("latent.gate", n, H, torch.float32)
        table = self.position.rotary_table() if self.position is not None else None
        rot_dims = self.position.rotary_dim if self.position is not None else 0
        ctx.ops.latent_prep(proj, ctx.positions, table, rot_dims, self.latent_norm, self.eps,
                            q_plain, q_abs, gate, cache, group.slot_mapping if binding.writes else None,
                            H, self.dim, self.rot_dim, self.kv_rank, group.page_size)
        q_rows = q_abs.view(n, H, self.row)
        ctx.ops.headwise_linear(q_plain.view(n, H, self.dim), self.w_uk_t, q_rows[:, :, : self.kv_rank])
        mixed = ctx.ws.buffer("latent.mixed", n, H * self.kv_rank, self.dtype)
        ctx.ops.paged_attention(q_abs, cache, cache, group.block_tables, ctx, H, 1, self.row,
                                group.page_size, self.scale, 0, mixed, ragged=group.ragged,
                                value_dim=self.kv_rank)
        out = ctx.ws.buffer("latent.out", n, H * self.vdim, self.dtype)
        ctx.ops.headwise_linear(mixed.view(n, H, self.kv_rank), self.w_uv, out.view(n, H, self.vdim),
                                row_scale=gate)
        return ctx.ops.linear(out, self.w_o, ws=ctx.ws, tag="mixer.delta", out_dtype=torch.float32,
                              allow_split=True)
