"""A recurrent mixer: the gated delta rule with one decay per head and key channel.

Per token, with ``h`` the mixer's input: ``q = W_q h`` and ``k = W_k h`` (``kv_heads x dim``),
``v = W_v h`` (``heads x vdim``); each passes a short causal convolution over time per channel
(``taps`` taps, the last one weighs the current token, zeros before the start) and silu.  ``q``
and ``k`` are made unit vectors per head (``x / sqrt(sum x^2 + 1e-6)``), ``q`` is also scaled by
``dim^-1/2``; head ``n`` uses q/k head ``n // (heads / kv_heads)``.  ``beta = sigmoid(W_b h)`` per
head; the decay is ``g = exp(-exp(A_log[n]) * softplus(W_a2 W_a1 h + dt_bias))`` per head and key
channel.  The state ``S`` (``dim x vdim`` per head, 32-bit, zero at the start) moves as

    S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q

so the read-out sees the token's own write.  Each head's ``o`` is divided by its root mean
square over ``vdim`` (eps inside the root), multiplied by a weight of size ``vdim`` and by
``sigmoid(W_g2 W_g1 h)``; ``W_o`` maps the heads back.

What a request keeps between steps is one state slot: per head ``S`` (stored column by column),
then the last ``taps - 1`` inputs of the convolutions.  Decays, step sizes, unit norms, the state
and the read-out norm are 32-bit in every precision; the projections run in the compute dtype
with 32-bit sums.
"""

from __future__ import annotations

from .base import BuildEnv, CacheBinding, Mixer, StateRequest, WeightDecl
from .registry import register_part


@register_part("mixer", "channel_delta")
class ChannelDeltaRule(Mixer):
    def __init__(self, *, names: dict, hidden_size: int, heads: int, kv_heads: int, dim: int, vdim: int,
                 taps: int, eps: float, dtype) -> None:
        if heads % kv_heads:
            raise ValueError(f"heads ({heads}) not divisible by kv_heads ({kv_heads})")
        if taps < 1:
            raise ValueError("the convolution needs at least one tap")
        self.names, self.hidden_size = dict(names), hidden_size
        self.heads, self.kv_heads, self.dim, self.vdim, self.taps = heads, kv_heads, dim, vdim, taps
        self.eps, self.dtype = float(eps), dtype
        self.qk_size, self.v_size = kv_heads * dim, heads * vdim
        self.channels = 2 * self.qk_size + self.v_size  # what the convolutions see
        self.matrix_floats = heads * dim * vdim
        self.rank_a = self.rank_g = None
        self.w_in = None

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, **_):
        obj = cls(names=params["names"], hidden_size=params.get("hidden_size", env.hidden_size),
                  heads=params["heads"], kv_heads=params["kv_heads"], dim=params["dim"],
                  vdim=params["vdim"], taps=params["taps"], eps=params["eps"], dtype=env.torch_dtype)
        obj.rank_a, obj.rank_g = params["decay_rank"], params["gate_rank"]
        return obj

    def weights(self) -> dict[str, WeightDecl]:
        n, h = self.names, self.hidden_size
        return {
            n["q"]: WeightDecl((self.qk_size, h)), n["k"]: WeightDecl((self.qk_size, h)),
            n["v"]: WeightDecl((self.v_size, h)),
            n["q_conv"]: WeightDecl((self.qk_size, self.taps), "vector"),
            n["k_conv"]: WeightDecl((self.qk_size, self.taps), "vector"),
            n["v_conv"]: WeightDecl((self.v_size, self.taps), "vector"),
            n["beta"]: WeightDecl((self.heads, h)),
            n["A_log"]: WeightDecl((self.heads,), "vector", "zeros"),
            n["dt_bias"]: WeightDecl((self.heads * self.dim,), "vector"),
            n["a1"]: WeightDecl((self.rank_a, h)), n["a2"]: WeightDecl((self.heads * self.dim, self.rank_a)),
            n["g1"]: WeightDecl((self.rank_g, h)), n["g2"]: WeightDecl((self.v_size, self.rank_g)),
            n["out_norm"]: WeightDecl((self.vdim,), "vector", "ones_plus_normal"),
            n["o"]: WeightDecl((h, self.v_size)),
        }

    def bind(self, tensors, env: BuildEnv) -> None:
        import torch

        n = self.names
        mat = lambda key: tensors[n[key]].to(self.dtype).contiguous()  # noqa: E731
        vec = lambda key: tensors[n[key]].float().contiguous()  # noqa: E731
        self.w_in = torch.cat([mat("q"), mat("k"), mat("v"), mat("beta")]).contiguous()
        self.w_a1, self.w_a2, self.w_g1, self.w_g2, self.w_o = mat("a1"), mat("a2"), mat("g1"), mat("g2"), mat("o")
        self.conv = torch.cat([vec("q_conv"), vec("k_conv"), vec("v_conv")]).contiguous()  # [channels, taps]
        self.A_log, self.dt_bias, self.out_norm = vec("A_log"), vec("dt_bias"), vec("out_norm")

    def cache_request(self) -> StateRequest:
        return StateRequest((self.matrix_floats + (self.taps - 1) * self.channels,))

    def forward(self, x, ctx, binding: CacheBinding):
        import torch

        f32, n = torch.float32, x.shape[0]
        group = ctx.groups[binding.group]
        state = group.state[binding.slot]  # [slots + 1, floats]
        ops, ws = ctx.ops, ctx.ws
        qkvb = ops.linear(x, self.w_in, ws=ws, tag="delta.in", out_dtype=f32)
        a_low = ops.linear(x, self.w_a1, ws=ws, tag="delta.a1", out_dtype=self.dtype)
        a = ops.linear(a_low, self.w_a2, ws=ws, tag="delta.a2", out_dtype=f32)
        g_low = ops.linear(x, self.w_g1, ws=ws, tag="delta.g1", out_dtype=self.dtype)
        gate = ops.linear(g_low, self.w_g2, ws=ws, tag="delta.g2", out_dtype=f32)
        q = ws.buffer("delta.q", n, self.qk_size, f32)
        k = ws.buffer("delta.k", n, self.qk_size, f32)
        v = ws.buffer("delta.v", n, self.v_size, f32)
        beta = ws.buffer("delta.beta", n, self.heads, f32)
        decay = ws.buffer("delta.decay", n, self.heads * self.dim, f32)
        ops.delta_prep(qkvb, a, self.conv, self.A_log, self.dt_bias, state, group.slots, ctx,
                       q, k, v, beta, decay, self.heads, self.kv_heads, self.dim, self.vdim, self.taps)
        o = ws.buffer("delta.o", n, self.v_size, f32)
        ops.delta_rule(q, k, v, beta, decay, state, group.slots, ctx, o,
                       self.heads, self.kv_heads, self.dim, self.vdim)
        out = ws.buffer("delta.out", n, self.v_size, self.dtype)
        ops.gated_rms_heads(o, self.out_norm, self.eps, gate, out, self.heads, self.vdim)
        return ops.linear(out, self.w_o, ws=ws, tag="mixer.delta", out_dtype=f32, allow_split=True)
