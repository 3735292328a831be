"""Ravapel: a decoder-only model of recurrent layers and layers with two mixers side by side.

Configuration keys: ``vocab``, ``width``, ``max_positions``, ``norm.eps``, ``canon.taps``,
``embedding.bigram`` (``buckets``, ``mul_prev``, ``mul_cur``), ``loop`` (``start``, ``stop``,
``times``) and ``layers``; each layer gives its ``type`` (``hgrn2`` or ``parallel``), the mixer's
sizes under ``mixer`` and its feed-forward under ``mlp`` (``null``: none; ``kind`` ``dense``: a
gated feed-forward with biases).  Tensors: ``embed``, ``bigram``, ``pos``, ``loop.in``,
``l<i>.norm1`` / ``norm1b`` / ``norm2`` / ``norm2b``, ``l<i>.canon1``, ``l<i>.mix.*``,
``l<i>.mlp.*``, ``final.norm``, ``head``.

The model: token embedding plus a hashed bigram embedding (the previous token is request state)
plus a learned position vector.  Every layer has an RMS norm (weights stored around zero) before
and after each sublayer; what the mixer reads first passes a short causal convolution over time
(its last inputs are request state).  ``hgrn2`` layers are linear attention whose forget gate also
decides what is written; ``parallel`` layers add, each with its factor, a grouped-query attention
with normalised and rotated queries and keys, sigmoid weights instead of a softmax and a chunked
mask, and a matrix memory with exponential gates.  Layers ``loop.start .. loop.stop - 1`` run
``loop.times`` times in a row with the same weights and a cache of their own per pass; before each
pass the stream is mixed again with the embedding's output (``loop.in``).  Keys that are absent
switch their mechanism off (no ``canon``: no convolution; no ``embedding.bigram``: token embedding
only; no ``loop``: every layer once; no ``rot`` or ``mask``: no rotation, no chunks).
No torch import here.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any

from ..config.model_config import ConfigError, Footprint, id_tuple
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

NAME = "Ravapel"
LAYER_TYPES = ("hgrn2", "parallel")


def _need(raw, key: str, kind, where: str):
    if not isinstance(raw, dict) or key not in raw or raw[key] is None:
        raise ConfigError(f"config.json: {where} is missing the key {key!r}")
    try:
        return kind(raw[key])
    except (TypeError, ValueError) as exc:
        raise ConfigError(f"config.json: {where}.{key} = {raw[key]!r} is not a {kind.__name__}") from exc


def _parse_mixer(kind: str, raw: dict, where: str) -> dict:
    if kind == "hgrn2":
        return {k: _need(raw, k, int, where) for k in ("heads", "dim", "vdim")}
    left, right = raw.get("left"), raw.get("right")
    lw, rw = where + ".left", where + ".right"
    out_left = {k: _need(left, k, int, lw) for k in ("heads", "kv_heads", "dim", "vdim")}
    out_left["scale"] = _need(left, "scale", float, lw)
    if out_left["heads"] % out_left["kv_heads"]:
        raise ConfigError(f"config.json: {lw}.heads is not a multiple of kv_heads")
    rot, mask = left.get("rot") or {}, left.get("mask") or {}
    out_left["rot_dims"] = int(rot.get("dims", 0) or 0)
    out_left["rot_base"] = _need(rot, "base", float, lw + ".rot") if out_left["rot_dims"] else 0.0
    if out_left["rot_dims"] % 2 or not 0 <= out_left["rot_dims"] <= out_left["dim"]:
        raise ConfigError(f"config.json: {lw}.rot.dims must be even and at most dim")
    out_left["chunk"] = int(mask["size"]) if mask.get("size") else None
    if out_left["chunk"] is not None and out_left["chunk"] < 1:
        raise ConfigError(f"config.json: {lw}.mask.size must be at least 1")
    out_right = {k: _need(right, k, int, rw) for k in ("heads", "dim", "vdim")}
    out_right["gate_cap"] = _need(right, "gate_cap", float, rw)
    return {"left": out_left, "right": out_right,
            "left_scale": _need(raw, "left_scale", float, where),
            "right_scale": _need(raw, "right_scale", float, where)}


def _parse_mlp(raw, where: str):
    if raw is None:
        return None
    kind = _need(raw, "kind", str, where)
    if kind != "dense":
        raise ConfigError(f"config.json: {where}.kind = {kind!r} is not 'dense'")
    return {"kind": "dense", "ff": _need(raw, "ff", int, where)}


@dataclass(frozen=True)
class RavapelLayer:
    type: str
    mixer: dict
    mlp: dict | None


@dataclass(frozen=True)
class RavapelConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_position_embeddings: int
    norm_eps: float
    conv_taps: int | None  # None: no input convolution
    bigram: tuple[int, int, int] | None  # (buckets, mul_prev, mul_cur); None: no bigram embedding
    loop: tuple[int, int, int] | None  # (start, stop, times)
    layers: tuple[RavapelLayer, ...]
    eos_token_ids: tuple[int, ...] = ()
    torch_dtype: str = "bfloat16"

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "RavapelConfig":
        listed = raw.get("layers")
        if not isinstance(listed, list) or not listed:
            raise ConfigError("config.json: 'layers' must list at least one layer")
        layers = []
        for i, entry in enumerate(listed):
            where = f"layers[{i}]"
            kind = _need(entry, "type", str, where)
            if kind not in LAYER_TYPES:
                raise ConfigError(f"config.json: {where}.type = {kind!r} is not one of {LAYER_TYPES}")
            layers.append(RavapelLayer(kind, _parse_mixer(kind, entry.get("mixer") or {}, where + ".mixer"),
                                       _parse_mlp(entry.get("mlp"), where + ".mlp")))
        canon = raw.get("canon")
        bigram = (raw.get("embedding") or {}).get("bigram")
        loop = raw.get("loop")
        cfg = cls(
            architecture=str(raw.get("architecture", NAME)),
            vocab_size=_need(raw, "vocab", int, "the model"),
            hidden_size=_need(raw, "width", int, "the model"),
            max_position_embeddings=_need(raw, "max_positions", int, "the model"),
            norm_eps=_need(raw.get("norm") or {}, "eps", float, "norm"),
            conv_taps=_need(canon, "taps", int, "canon") if canon else None,
            bigram=(_need(bigram, "buckets", int, "embedding.bigram"),
                    _need(bigram, "mul_prev", int, "embedding.bigram"),
                    _need(bigram, "mul_cur", int, "embedding.bigram")) if bigram else None,
            loop=(_need(loop, "start", int, "loop"), _need(loop, "stop", int, "loop"),
                  _need(loop, "times", int, "loop")) if loop else None,
            layers=tuple(layers),
            eos_token_ids=id_tuple(raw.get("eos_token_id")),
            torch_dtype=str(raw.get("torch_dtype", "bfloat16")),
        )
        for key in ("vocab_size", "hidden_size", "max_position_embeddings"):
            if getattr(cfg, key) < 1:
                raise ConfigError(f"config.json: {key} must be >= 1")
        if not cfg.norm_eps > 0 or not math.isfinite(cfg.norm_eps):
            raise ConfigError("config.json: norm.eps must be a positive number")
        if cfg.conv_taps is not None and cfg.conv_taps < 1:
            raise ConfigError("config.json: canon.taps must be at least 1")
        if cfg.bigram is not None and cfg.bigram[0] < 1:
            raise ConfigError("config.json: embedding.bigram.buckets must be at least 1")
        if cfg.loop is not None:
            start, stop, times = cfg.loop
            if not 0 <= start <= stop <= len(layers) or times < 0:
                raise ConfigError("config.json: loop needs 0 <= start <= stop <= number of layers and times >= 0")
        return cfg

    def run_order(self) -> list[tuple[int, bool]]:
        """(layer, whether a pass of the loop starts with it), in the order the layers run."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, False) for i in range(n)]
        start, stop, times = self.loop
        order = [(i, False) for i in range(start)]
        for _ in range(times):
            order += [(i, i == start) for i in range(start, stop)]
        return order + [(i, False) for i in range(stop, n)]


def _rotary_name(m: dict) -> str:
    return f"rotary_{m['rot_dims']}_{m['rot_base']!r}"


def _hgrn2_spec(cfg: RavapelConfig, p: str, m: dict) -> PartSpec:
    return PartSpec("hgrn2", {
        "names": {"q": f"{p}.q", "f": f"{p}.f", "f_bias": f"{p}.f.b", "lower": f"{p}.lower", "v": f"{p}.v",
                  "out_norm": f"{p}.norm", "o": f"{p}.o"},
        "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"], "eps": cfg.norm_eps})


def _parallel_spec(cfg: RavapelConfig, p: str, m: dict) -> PartSpec:
    left, right = m["left"], m["right"]
    lp, rp = p + ".left", p + ".right"
    attention = PartSpec("sigmoid_attention", {
        "names": {"q": f"{lp}.q", "k": f"{lp}.k", "v": f"{lp}.v", "q_norm": f"{lp}.q.norm",
                  "k_norm": f"{lp}.k.norm", "head_bias": f"{lp}.pb", "o": f"{lp}.o"},
        "heads": left["heads"], "kv_heads": left["kv_heads"], "dim": left["dim"], "vdim": left["vdim"],
        "scale": left["scale"], "chunk": left["chunk"], "eps": cfg.norm_eps,
        "position": _rotary_name(left) if left["rot_dims"] else None})
    memory = PartSpec("mlstm", {
        "names": {"q": f"{rp}.q", "k": f"{rp}.k", "v": f"{rp}.v", "g": f"{rp}.g", "i": f"{rp}.i",
                  "i_bias": f"{rp}.i.b", "f": f"{rp}.f", "f_bias": f"{rp}.f.b", "out_norm": f"{rp}.norm",
                  "o": f"{rp}.o"},
        "heads": right["heads"], "dim": right["dim"], "vdim": right["vdim"], "gate_cap": right["gate_cap"],
        "eps": cfg.norm_eps})
    return PartSpec("parallel_sum", {"branches": [{"mixer": attention, "scale": m["left_scale"]},
                                                  {"mixer": memory, "scale": m["right_scale"]}]})


def _mixer_spec(cfg: RavapelConfig, i: int, layer: RavapelLayer) -> PartSpec:
    p = f"l{i}.mix"
    inner = _hgrn2_spec(cfg, p, layer.mixer) if layer.type == "hgrn2" else _parallel_spec(cfg, p, layer.mixer)
    if cfg.conv_taps is None:
        return inner
    return PartSpec("conv_input", {"weight": f"l{i}.canon1", "taps": cfg.conv_taps, "inner": inner})


def _mlp_spec(i: int, mlp: dict | None) -> PartSpec | None:
    if mlp is None:
        return None
    p = f"l{i}.mlp"
    return PartSpec("swiglu", {
        "gate_proj": f"{p}.gate", "up_proj": f"{p}.up", "down_proj": f"{p}.down", "gate_bias": f"{p}.gate.b",
        "up_bias": f"{p}.up.b", "down_bias": f"{p}.down.b", "intermediate_size": mlp["ff"]})


def ravapel_spec(cfg: RavapelConfig) -> ModelSpec:
    positions: dict[str, PartSpec] = {
        "learned": PartSpec("learned", {"weight": "pos", "positions": cfg.max_position_embeddings})}
    layers = []
    for i, layer in enumerate(cfg.layers):
        if layer.type == "parallel" and layer.mixer["left"]["rot_dims"]:
            left = layer.mixer["left"]
            positions.setdefault(_rotary_name(left), PartSpec("rotary", {
                "rotary_dim": left["rot_dims"], "theta": left["rot_base"], "layout": "halves",
                "angles": "float64"}))

        def norm(name: str) -> PartSpec:
            return PartSpec("rms", {"weight": f"l{i}.{name}", "eps": cfg.norm_eps, "offset": 1.0})

        norms = {"pre_mixer": norm("norm1"), "post_mixer": norm("norm1b")}
        if layer.mlp is not None:
            norms.update(pre_feed_forward=norm("norm2"), post_feed_forward=norm("norm2b"))
        layers.append(LayerSpec(prefix=f"l{i}", block=PartSpec("sandwich_residual", {}),
                                mixer=_mixer_spec(cfg, i, layer), feed_forward=_mlp_spec(i, layer.mlp),
                                norms=norms))
    schedule = tuple(ScheduleEntry(i, before="loop_in" if starts else None) for i, starts in cfg.run_order())
    if cfg.bigram is not None:
        embedding = PartSpec("token_bigram", {"weight": "embed", "bigram": "bigram", "vocab_size": cfg.vocab_size,
                                              "buckets": cfg.bigram[0], "mul_prev": cfg.bigram[1],
                                              "mul_cur": cfg.bigram[2]})
    else:
        embedding = PartSpec("token", {"weight": "embed", "vocab_size": cfg.vocab_size})
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
        max_position_embeddings=cfg.max_position_embeddings, embedding=embedding, positions=positions,
        layers=tuple(layers), schedule=schedule,
        final_norm=PartSpec("rms", {"weight": "final.norm", "eps": cfg.norm_eps, "offset": 1.0}),
        head=PartSpec("linear", {"weight": "head", "vocab_size": cfg.vocab_size}),
        eos_token_ids=cfg.eos_token_ids,
        stream_parts={"loop_in": PartSpec("reinject", {"weight": "loop.in"})} if cfg.loop is not None else {})


def ravapel_footprint(cfg: RavapelConfig) -> Footprint:
    h = cfg.hidden_size
    params = cfg.vocab_size * h * 2 + cfg.max_position_embeddings * h + h
    if cfg.bigram is not None:
        params += (cfg.bigram[0] + 1) * h
    if cfg.loop is not None:
        params += 2 * h * h
    runs = [0] * len(cfg.layers)
    for i, _ in cfg.run_order():
        runs[i] += 1
    per_token = 0
    per_request = 1 if cfg.bigram is not None else 0
    for layer, times in zip(cfg.layers, runs):
        m = layer.mixer
        params += 2 * h + (h * cfg.conv_taps if cfg.conv_taps else 0)
        if cfg.conv_taps:
            per_request += times * max((cfg.conv_taps - 1) * h, 1)
        if layer.type == "hgrn2":
            qk, v = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            params += 2 * qk * h + 2 * qk + v * h + m["vdim"] + h * v
            per_request += times * qk * m["vdim"]
        else:
            left, right = m["left"], m["right"]
            params += (left["heads"] + left["kv_heads"]) * left["dim"] * h + left["kv_heads"] * left["vdim"] * h
            params += 2 * left["dim"] + left["heads"] + h * left["heads"] * left["vdim"]
            per_token += times * left["kv_heads"] * (left["dim"] + left["vdim"])
            qk, v = right["heads"] * right["dim"], right["heads"] * right["vdim"]
            params += 2 * qk * h + 2 * v * h + 2 * right["heads"] * (h + 1) + v + h * v
            per_request += times * (right["heads"] * (right["vdim"] + 1) * right["dim"] + right["heads"])
        if layer.mlp is not None:
            params += 2 * h + 3 * layer.mlp["ff"] * h + 2 * layer.mlp["ff"] + h
    return Footprint(params, per_token, per_request)


def describe_ravapel(cfg: RavapelConfig) -> list[str]:
    kinds = [layer.type + ("" if layer.mlp is None else "+" + layer.mlp["kind"]) for layer in cfg.layers]
    fp = ravapel_footprint(cfg)
    loop = "none" if cfg.loop is None else f"layers {cfg.loop[0]}..{cfg.loop[1] - 1} x {cfg.loop[2]}"
    return [
        f"architecture        {cfg.architecture}",
        f"layers / width      {len(cfg.layers)} / {cfg.hidden_size}",
        f"layer kinds         {', '.join(kinds)}",
        f"loop                {loop}",
        f"parameters          {fp.parameters / 1e9:.3f} B",
        f"cache per token     {fp.cache_bytes_per_token(2)} B (bf16), state per request {fp.state_values_per_request * 4} B",
    ]


register_architecture(NAME, RavapelConfig, ravapel_spec, describe_ravapel, ravapel_footprint)
