"""Rugedra: a decoder-only model whose layers are listed one by one in ``config.json``.

Configuration keys: ``vocab``, ``width``, ``max_positions``, ``norm.eps``, ``residual_mult``,
``logit_scale`` and ``layers``; each layer gives its ``type`` (``latent_attention`` or
``channel_delta``), the mixer's sizes under ``mixer`` and its feed-forward under ``mlp``
(``null``: none; ``kind`` ``dense``: up, squared relu, down; ``kind`` ``moe``: routed gated
experts).  Tensors: ``embed``, ``pos``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``,
``l<i>.mlp.*``, ``final.norm``, ``head``.

The model: token embedding plus a learned position vector; pre-norm residual layers with layer
norms (weight, no bias) whose mixer and feed-forward outputs enter the residual stream times
``residual_mult``; a final layer norm; logits times ``logit_scale``.  Sizes that a tensor's shape
fixes but the configuration does not name (the ranks of the delta rule's two low-rank
projections) are taken from ``model.safetensors``'s header when a folder is loaded, or from the
optional keys ``decay_rank`` / ``gate_rank`` of the mixer.  No torch import here.
"""

from __future__ import annotations

import json
import math
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Any

from ..config.model_config import ConfigError, Footprint, id_tuple
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

NAME = "Rugedra"
MIXERS = ("latent_attention", "channel_delta")


def _need(raw: dict, key: str, kind, where: str):
    if not isinstance(raw, dict) or key not in raw or raw[key] is None:
        raise ConfigError(f"config.json: {where} is missing the key {key!r}")
    try:
        return kind(raw[key])
    except (TypeError, ValueError) as exc:
        raise ConfigError(f"config.json: {where}.{key} = {raw[key]!r} is not a {kind.__name__}") from exc


@dataclass(frozen=True)
class RugedraLayer:
    type: str
    mixer: dict  # the sizes as plain numbers (see `_parse_mixer`)
    mlp: dict | None


def _parse_mixer(kind: str, raw: dict, where: str) -> dict:
    if kind == "latent_attention":
        rot = raw.get("rot") or {}
        out = {k: _need(raw, k, int, where) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank")}
        out["scale"] = _need(raw, "scale", float, where)
        out["rot_base"] = _need(rot, "base", float, where + ".rot")
        out["rot_dims"] = _need(rot, "dims", int, where + ".rot")
        if out["rot_dims"] % 2 or not 0 <= out["rot_dims"] <= out["rot_dim"]:
            raise ConfigError(f"config.json: {where}.rot.dims must be even and at most rot_dim")
        return out
    out = {k: _need(raw, k, int, where) for k in ("heads", "kv_heads", "dim", "vdim")}
    out["taps"] = _need(raw, "conv", int, where)
    if out["heads"] % out["kv_heads"]:
        raise ConfigError(f"config.json: {where}.heads is not a multiple of kv_heads")
    for k in ("decay_rank", "gate_rank"):
        out[k] = int(raw[k]) if raw.get(k) is not None else None
    return out


def _parse_mlp(raw: dict | None, where: str) -> dict | None:
    if raw is None:
        return None
    kind = _need(raw, "kind", str, where)
    if kind == "dense":
        return {"kind": "dense", "ff": _need(raw, "ff", int, where)}
    if kind != "moe":
        raise ConfigError(f"config.json: {where}.kind = {kind!r} is neither 'dense' nor 'moe'")
    expert, router = raw.get("expert") or {}, raw.get("router") or {}
    groups = router.get("groups") or {}
    out = {
        "kind": "moe",
        "ff": _need(expert, "ff", int, where + ".expert"),
        "limit": _need(expert, "limit", float, where + ".expert"),
        "experts": _need(router, "experts", int, where + ".router"),
        "top": _need(router, "top", int, where + ".router"),
        "groups": int(groups.get("count", 1)),
        "keep_groups": int(groups.get("keep", groups.get("count", 1))),
    }
    if out["groups"] < 1 or out["experts"] % out["groups"] or not 1 <= out["keep_groups"] <= out["groups"]:
        raise ConfigError(f"config.json: {where}.router.groups does not divide the experts")
    return out


@dataclass(frozen=True)
class RugedraConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_position_embeddings: int
    norm_eps: float
    residual_mult: float
    logit_scale: float
    layers: tuple[RugedraLayer, ...]
    eos_token_ids: tuple[int, ...] = ()
    torch_dtype: str = "bfloat16"

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "RugedraConfig":
        layers = []
        listed = raw.get("layers")
        if not isinstance(listed, list) or not listed:
            raise ConfigError("config.json: 'layers' must list at least one layer")
        for i, entry in enumerate(listed):
            where = f"layers[{i}]"
            kind = _need(entry, "type", str, where)
            if kind not in MIXERS:
                raise ConfigError(f"config.json: {where}.type = {kind!r} is not one of {MIXERS}")
            layers.append(RugedraLayer(kind, _parse_mixer(kind, entry.get("mixer") or {}, where + ".mixer"),
                                       _parse_mlp(entry.get("mlp"), where + ".mlp")))
        cfg = cls(
            architecture=str(raw.get("architecture", NAME)),
            vocab_size=_need(raw, "vocab", int, "the model"),
            hidden_size=_need(raw, "width", int, "the model"),
            max_position_embeddings=_need(raw, "max_positions", int, "the model"),
            norm_eps=_need(raw.get("norm") or {}, "eps", float, "norm"),
            residual_mult=float(raw.get("residual_mult", 1.0)),
            logit_scale=float(raw.get("logit_scale", 1.0)),
            layers=tuple(layers),
            eos_token_ids=id_tuple(raw.get("eos_token_id")),
            torch_dtype=str(raw.get("torch_dtype", "bfloat16")),
        )
        for key in ("vocab_size", "hidden_size", "max_position_embeddings"):
            if getattr(cfg, key) < 1:
                raise ConfigError(f"config.json: {key} must be >= 1")
        if not cfg.norm_eps > 0 or not math.isfinite(cfg.norm_eps):
            raise ConfigError("config.json: norm.eps must be a positive number")
        return cfg

    def complete_from_folder(self, model_dir) -> "RugedraConfig":
        return self.with_tensor_shapes(read_tensor_shapes(model_dir))

    def with_tensor_shapes(self, shapes: dict[str, tuple[int, ...]]) -> "RugedraConfig":
        """Fill in the sizes only a tensor's shape gives (the delta rule's low ranks)."""
        layers = []
        for i, layer in enumerate(self.layers):
            mixer = dict(layer.mixer)
            if layer.type == "channel_delta":
                for key, name in (("decay_rank", f"l{i}.mix.a1"), ("gate_rank", f"l{i}.mix.g1")):
                    if mixer.get(key) is None and name in shapes:
                        mixer[key] = int(shapes[name][0])
            layers.append(RugedraLayer(layer.type, mixer, layer.mlp))
        return RugedraConfig(**{**self.__dict__, "layers": tuple(layers)})


def read_tensor_shapes(model_dir: str | Path) -> dict[str, tuple[int, ...]]:
    """Names and shapes from the header of ``model.safetensors`` (8 bytes of length, then JSON)."""
    path = Path(model_dir) / "model.safetensors"
    if not path.exists():
        return {}
    with open(path, "rb") as f:
        (size,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(size))
    return {k: tuple(v["shape"]) for k, v in header.items() if k != "__metadata__"}


def _mixer_spec(cfg: RugedraConfig, i: int, layer: RugedraLayer) -> PartSpec:
    p, m = f"l{i}.mix", layer.mixer
    if layer.type == "latent_attention":
        return PartSpec("latent_attention", {
            "names": {"q": f"{p}.q", "dkv": f"{p}.dkv", "latent_norm": f"{p}.dkv.norm", "uk": f"{p}.uk",
                      "uv": f"{p}.uv", "gate": f"{p}.g", "o": f"{p}.o"},
            "heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"], "vdim": m["vdim"],
            "kv_rank": m["kv_rank"], "scale": m["scale"], "eps": cfg.norm_eps,
            "position": _rotary_name(m) if m["rot_dims"] else None})
    if m.get("decay_rank") is None or m.get("gate_rank") is None:
        raise ConfigError(f"layers[{i}].mixer: the ranks of a1 and g1 are known neither from the tensors' "
                          "shapes nor from 'decay_rank' / 'gate_rank'")
    return PartSpec("channel_delta", {
        "names": {"q": f"{p}.q", "k": f"{p}.k", "v": f"{p}.v", "q_conv": f"{p}.q.conv", "k_conv": f"{p}.k.conv",
                  "v_conv": f"{p}.v.conv", "beta": f"{p}.b", "A_log": f"{p}.A_log", "dt_bias": f"{p}.dt_bias",
                  "a1": f"{p}.a1", "a2": f"{p}.a2", "g1": f"{p}.g1", "g2": f"{p}.g2", "out_norm": f"{p}.norm",
                  "o": f"{p}.o"},
        "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"], "taps": m["taps"],
        "decay_rank": m["decay_rank"], "gate_rank": m["gate_rank"], "eps": cfg.norm_eps})


def _rotary_name(m: dict) -> str:
    return f"rotary_{m['rot_dims']}_{m['rot_base']!r}"


def _mlp_spec(i: int, mlp: dict | None) -> PartSpec | None:
    if mlp is None:
        return None
    p = f"l{i}.mlp"
    if mlp["kind"] == "dense":
        return PartSpec("relu2", {"up_proj": f"{p}.up", "down_proj": f"{p}.down", "intermediate_size": mlp["ff"]})
    return PartSpec("routed_experts", {
        "router": f"{p}.router", "expert_prefix": f"{p}.e", "experts": mlp["experts"], "top": mlp["top"],
        "groups": mlp["groups"], "keep_groups": mlp["keep_groups"], "intermediate_size": mlp["ff"],
        "limit": mlp["limit"], "alpha": 1.702, "up_offset": 1.0})


def rugedra_spec(cfg: RugedraConfig) -> ModelSpec:
    positions: dict[str, PartSpec] = {
        "learned": PartSpec("learned", {"weight": "pos", "positions": cfg.max_position_embeddings})}
    layers = []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if layer.type == "latent_attention" and m["rot_dims"]:
            positions.setdefault(_rotary_name(m), PartSpec("rotary", {
                "rotary_dim": m["rot_dims"], "theta": m["rot_base"], "layout": "interleaved"}))
        norms = {"pre_mixer": PartSpec("layer", {"weight": f"l{i}.norm1", "eps": cfg.norm_eps})}
        if layer.mlp is not None:
            norms["pre_feed_forward"] = PartSpec("layer", {"weight": f"l{i}.norm2", "eps": cfg.norm_eps})
        layers.append(LayerSpec(
            prefix=f"l{i}", block=PartSpec("prenorm_residual", {"residual_mult": cfg.residual_mult}),
            mixer=_mixer_spec(cfg, i, layer), feed_forward=_mlp_spec(i, layer.mlp), norms=norms))
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
        max_position_embeddings=cfg.max_position_embeddings,
        embedding=PartSpec("token", {"weight": "embed", "vocab_size": cfg.vocab_size}),
        positions=positions, layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=PartSpec("layer", {"weight": "final.norm", "eps": cfg.norm_eps}),
        head=PartSpec("linear", {"weight": "head", "vocab_size": cfg.vocab_size,
                                 "logit_scale": cfg.logit_scale}),
        eos_token_ids=cfg.eos_token_ids)


def rugedra_footprint(cfg: RugedraConfig) -> Footprint:
    h = cfg.hidden_size
    params = cfg.vocab_size * h * 2 + cfg.max_position_embeddings * h + h
    per_token = per_request = 0
    for layer in cfg.layers:
        m = layer.mixer
        params += h
        if layer.type == "latent_attention":
            row = m["kv_rank"] + m["rot_dim"]
            params += (m["heads"] * (m["dim"] + m["rot_dim"]) + row + m["heads"]) * h + m["kv_rank"]
            params += m["heads"] * (m["dim"] + m["vdim"]) * m["kv_rank"] + h * m["heads"] * m["vdim"]
            per_token += row
        else:
            qk, v = m["kv_heads"] * m["dim"], m["heads"] * m["vdim"]
            ra, rg = m.get("decay_rank") or 0, m.get("gate_rank") or 0
            params += (2 * qk + v + m["heads"]) * h + (2 * qk + v) * m["taps"] + m["heads"]
            params += m["heads"] * m["dim"] * (1 + ra) + ra * h + rg * h + v * rg + m["vdim"] + h * v
            per_request += m["heads"] * m["dim"] * m["vdim"] + (m["taps"] - 1) * (2 * qk + v)
        if layer.mlp is not None:
            params += h
            if layer.mlp["kind"] == "dense":
                params += 2 * layer.mlp["ff"] * h
            else:
                params += layer.mlp["experts"] * (3 * layer.mlp["ff"] * h + h)
    return Footprint(params, per_token, per_request)


def describe_rugedra(cfg: RugedraConfig) -> list[str]:
    kinds = [layer.type + ("" if layer.mlp is None else "+" + layer.mlp["kind"]) for layer in cfg.layers]
    fp = rugedra_footprint(cfg)
    return [
        f"architecture        {cfg.architecture}",
        f"layers / width      {len(cfg.layers)} / {cfg.hidden_size}",
        f"layer kinds         {', '.join(kinds)}",
        f"parameters          {fp.parameters / 1e9:.3f} B",
        f"cache per token     {fp.cache_bytes_per_token(2)} B (bf16), state per request {fp.state_values_per_request * 4} B",
    ]


register_architecture(NAME, RugedraConfig, rugedra_spec, describe_rugedra, rugedra_footprint)
