"""Small Rugedra configurations and random weights for the tests.  Sizes are odd on purpose:
head counts that are not powers of two, key and value sizes that differ, rotated parts only
partly rotated, rows that are not multiples of 8, several kinds of layers in several orders,
a layer without a feed-forward, and values that are 1 in one model and not in another."""

from __future__ import annotations

import torch


def latent(heads, dim, rot_dim, vdim, rank, rot_dims=None, base=10000.0):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank,
            "scale": (dim + rot_dim) ** -0.5,
            "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}}


def delta(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def moe(ff, experts, top, groups, keep, limit=1.25):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit},
            "router": {"experts": experts, "top": top, "groups": {"count": groups, "keep": keep}}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def config(width, vocab, layers, max_positions=256, eps=1e-5, mult=0.8, logit_scale=0.6):
    return {"architecture": "Rugedra", "vocab": vocab, "width": width, "max_positions": max_positions,
            "norm": {"eps": eps}, "residual_mult": mult, "logit_scale": logit_scale,
            "layers": [{"type": t, "mixer": m, "mlp": f} for t, m, f in layers]}


# delta first, a layer without feed-forward, grouped routing, partly rotated part, rows of 28 numbers
MIXED = config(72, 131, [
    ("channel_delta", delta(6, 2, 12, 20, 4), moe(40, 6, 3, 3, 2)),
    ("latent_attention", latent(3, 12, 8, 20, 20, rot_dims=4), None),
    ("latent_attention", latent(5, 8, 16, 8, 24, base=500.0), dense(100)),
    ("channel_delta", delta(2, 2, 40, 8, 2), dense(56)),
])
# attention only (no state slots), one group of experts, every expert chosen
LATENT_ONLY = config(64, 97, [
    ("latent_attention", latent(4, 16, 16, 16, 32), moe(24, 4, 4, 1, 1, limit=0.75)),
    ("latent_attention", latent(1, 24, 8, 40, 16), dense(96)),
], mult=1.0, logit_scale=1.0)
# recurrence only (no pages): one tap, one head, top 1
DELTA_ONLY = config(48, 61, [
    ("channel_delta", delta(1, 1, 24, 24, 1), moe(32, 5, 1, 5, 1)),
    ("channel_delta", delta(4, 4, 8, 12, 3), None),
], mult=0.5)

# nothing a multiple of 4: widths, rows, sizes of heads, experts
ODD = config(50, 53, [
    ("latent_attention", latent(3, 10, 6, 14, 18, rot_dims=2), moe(12, 3, 2, 1, 1)),
    ("channel_delta", delta(3, 1, 10, 14, 2), dense(30)),
], max_positions=200)

CONFIGS = {"mixed": MIXED, "latent_only": LATENT_ONLY, "delta_only": DELTA_ONLY, "odd": ODD}
RANKS = {"decay_rank": 6, "gate_rank": 10}


def with_ranks(cfg: dict) -> dict:
    """The configuration with the delta rule's low ranks spelled out (a folder's tensors give them
    otherwise)."""
    out = dict(cfg)
    out["layers"] = [dict(layer, mixer=dict(layer["mixer"], **RANKS)) if layer["type"] == "channel_delta" else layer
                     for layer in cfg["layers"]]
    return out


def make_weights(cfg: dict, seed: int = 0) -> dict:
    """Random bfloat16-valued weights, drawn so that faults show: queries and the latent's
    projections are large (peaked attention: a lost or misplaced key moves the output), the
    recurrence forgets slowly (decays near one: a lost state shows many tokens later), the
    convolutions weigh every tap, routers are sharp."""
    from inference_engine_b200.config import build_model_spec, config_from_dict
    from inference_engine_b200.engine.model import declared_weights

    decl = declared_weights(build_model_spec(config_from_dict(with_ranks(cfg))))
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, d in decl.items():
        t = torch.randn(d.shape, generator=g) * 0.08
        leaf = name.split(".", 1)[1] if name.startswith("l") else name
        if leaf.endswith("norm1") or leaf.endswith("norm2") or leaf in ("norm", "mix.dkv.norm", "mix.norm"):
            t = t + 1.0
        elif leaf in ("mix.q", "mix.dkv", "mix.uk"):
            t = t * 3.0
        elif leaf == "mix.A_log":
            t = t - 2.5
        elif leaf.endswith(".conv"):
            t = t * 4.0 + 0.5
        elif leaf == "mlp.router":
            t = t * 6.0
        elif leaf in ("embed", "pos"):
            t = t * 6.0
        elif leaf in ("mix.a2", "mix.g2"):
            t = t * 4.0
        out[name] = t.to(torch.bfloat16)
    out["final.norm"] = (out["final.norm"].float() + 1.0).to(torch.bfloat16)
    return out
