"""Small Ravapel configurations and random weights for the tests.  Sizes are odd on purpose: head
counts that are not powers of two, key and value sizes that differ, heads rotated in part, in full
or not at all, chunks of a few positions (and of one), one tap and several, a loop that runs once,
three times or is absent, a layer without a feed-forward, nothing a multiple of four."""

from __future__ import annotations

import torch


def hgrn2(heads, dim, vdim):
    return "hgrn2", {"heads": heads, "dim": dim, "vdim": vdim}


def parallel(left, right, left_scale=0.7, right_scale=1.2):
    return "parallel", {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}


def left(heads, kv_heads, dim, vdim, chunk=None, rot_dims=0, base=1000.0, scale=None):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
           "scale": dim ** -0.5 if scale is None else scale}
    if chunk:
        out["mask"] = {"size": chunk}
    if rot_dims:
        out["rot"] = {"dims": rot_dims, "base": base}
    return out


def right(heads, dim, vdim, cap=9.0):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def config(width, vocab, layers, *, taps=3, bigram=(37, 5, 3), loop=None, max_positions=256, eps=1e-5):
    cfg = {"architecture": "Ravapel", "vocab": vocab, "width": width, "max_positions": max_positions,
           "norm": {"eps": eps}, "layers": [{"type": t, "mixer": m, "mlp": f} for (t, m), f in layers]}
    if taps:
        cfg["canon"] = {"taps": taps}
    if bigram:
        cfg["embedding"] = {"bigram": {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


# a loop of two layers run three times; chunks of 10 and 7 positions; partly and fully rotated heads;
# a layer without a feed-forward; grouped and ungrouped key/value heads
MIXED = config(72, 131, [
    (hgrn2(3, 12, 20), dense(40)),
    (parallel(left(6, 2, 16, 24, chunk=10, rot_dims=8), right(3, 8, 12)), None),
    (hgrn2(2, 20, 8), dense(56)),
    (parallel(left(3, 3, 8, 8, chunk=7, rot_dims=8, base=50.0), right(5, 4, 20, cap=5.0), 1.1, 0.4), dense(48)),
    (hgrn2(6, 4, 12), dense(40)),
], taps=3, loop=(1, 3, 3))
# no loop, one tap, no bigram, no chunks, no rotation: every key is seen
PLAIN = config(64, 97, [
    (parallel(left(4, 1, 16, 8), right(2, 16, 16)), dense(96)),
    (hgrn2(1, 24, 40), None),
], taps=1, bigram=None, loop=None)
# nothing a multiple of four; a chunk of one position (a query sees itself only); the loop is all
# layers, once; five taps; a bucket count of 1 (every pair of tokens falls into row 0)
ODD = config(50, 53, [
    (parallel(left(3, 1, 10, 14, chunk=1, rot_dims=6), right(1, 6, 10)), dense(30)),
    (hgrn2(5, 6, 10), dense(22)),
], taps=5, bigram=(1, 7, 11), loop=(0, 2, 1), max_positions=200)
# recurrent layers only (no pages), no input convolution
RECURRENT = config(48, 61, [
    (hgrn2(4, 12, 12), dense(32)),
    (hgrn2(2, 24, 6), None),
], taps=None, loop=(1, 2, 2))

# larger than the others: key and value sizes that the tensor-core attention takes (48 and 80, 96 and 96),
# key sizes of the recurrences with more than one row group per lane, chunks of 100 and 64 positions
# (longer than, and as long as, a key tile), a loop over the first two layers
WIDE = config(160, 301, [
    (parallel(left(6, 3, 48, 80, chunk=100, rot_dims=24), right(4, 24, 40)), dense(256)),
    (hgrn2(5, 40, 56), dense(200)),
    (parallel(left(8, 2, 96, 96, chunk=64, rot_dims=96, base=300.0), right(2, 72, 24), 0.5, 0.9), dense(128)),
], taps=4, bigram=(211, 31, 7), loop=(0, 2, 2), max_positions=512)

CONFIGS = {"mixed": MIXED, "plain": PLAIN, "odd": ODD, "recurrent": RECURRENT}


def make_weights(cfg: dict, seed: int = 0) -> dict:
    """Random bfloat16-valued weights, drawn so that faults show: queries and keys are large and the
    head biases negative (peaked sigmoid weights: a lost, misplaced or wrongly visible key moves the
    output), the recurrences forget slowly (lower bounds and forget biases high: a lost state shows
    many tokens later), the convolutions weigh every tap, bigram and position rows are large."""
    from inference_engine_b200.config import build_model_spec, config_from_dict
    from inference_engine_b200.engine.model import declared_weights

    decl = declared_weights(build_model_spec(config_from_dict(cfg)))
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, d in decl.items():
        t = torch.randn(d.shape, generator=g) * 0.08
        leaf = name.split(".", 1)[1] if name.startswith("l") and name[1].isdigit() else name
        if leaf in ("mix.norm", "mix.right.norm", "mix.left.q.norm", "mix.left.k.norm"):
            t = t + 1.0
        elif leaf in ("mix.left.q", "mix.left.k"):
            t = t * 4.0
        elif leaf == "mix.left.pb":
            t = t * 10.0 - 2.0
        elif leaf == "mix.lower":
            t = torch.sigmoid(t * 20.0 + 2.0)  # lower bounds of the forget gate between 0.5 and 1
        elif leaf in ("mix.f.b", "mix.right.f.b"):
            t = t * 10.0 + 2.0
        elif leaf == "mix.right.i.b":
            t = t * 10.0
        elif leaf in ("mix.right.i", "mix.right.f"):
            t = t * 6.0
        elif leaf == "canon1":
            t = t * 4.0 + 0.4
        elif leaf.endswith(".b"):
            t = t * 4.0
        elif leaf in ("embed", "pos", "bigram"):
            t = t * 6.0
        elif leaf == "loop.in":
            t = t * 1.5
        out[name] = t.to(torch.bfloat16)
    return out
