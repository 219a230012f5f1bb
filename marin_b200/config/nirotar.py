"""Configuration of the Nirotar decoder: a list of layers, each with one of two attention mixers (grouped-query attention
with a sliding window, or attention over a latent that keys and values share) and a feed-forward of experts that a table
over the token ids chooses, plus the norm's eps.

Every size and constant comes from ``config.json``; what a part needs is checked here, so that a folder with a missing or
mistyped key is refused before any weight is read.  Optional keys switch a mechanism off when they are absent: no ``mask``
(every earlier position is seen), no ``rot`` (no rotation), no ``rot.scaling`` (plain frequencies), no ``kv_from`` (the layer
keeps a latent of its own), no ``mlp.shared`` (no shared expert), ``mlp`` null (a layer without feed-forward).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .base import ConfigError, ModelConfig, eos_ids, optional
from .fegarax import DEFAULT_MAX_POSITIONS, _int, _num, _obj

MIXER_TYPES = ("attention", "latent_attention")
SCALING_KEYS = ("factor", "low", "high", "original")


def _rot(m: Dict[str, Any], where: str, width: int) -> Optional[Dict[str, Any]]:
    rot = _obj(m, "rot", where, needed=False)
    if rot is None:
        return None
    r: Dict[str, Any] = {"base": _num(rot, "base", where + "rot: ", True), "dims": _int(rot, "dims", where + "rot: ", 2), "scaling": None}
    if r["dims"] % 2 or r["dims"] > width:
        raise ConfigError(f"config.json: {where}`rot.dims` {r['dims']} must be even and at most {width}")
    sc = _obj(rot, "scaling", where + "rot: ", needed=False)
    if sc is not None:
        r["scaling"] = {k: _num(sc, k, where + "rot.scaling: ", True) for k in SCALING_KEYS}
        if r["scaling"]["high"] <= r["scaling"]["low"]:
            raise ConfigError(f"config.json: {where}`rot.scaling.high` must be above `rot.scaling.low`")
    return r


def _rot_json(rot: Optional[Dict[str, Any]]) -> Optional[Dict[str, Any]]:
    if rot is None:
        return None
    out = {"base": rot["base"], "dims": rot["dims"]}
    if rot["scaling"] is not None:
        out["scaling"] = dict(rot["scaling"])
    return out


@dataclass
class NirotarLayer:
    type: str
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]]

    @classmethod
    def parse(cls, raw: Any, index: int) -> "NirotarLayer":
        where = f"layers[{index}]: "
        if not isinstance(raw, dict):
            raise ConfigError(f"config.json: {where}must be an object")
        kind = raw.get("type")
        if kind not in MIXER_TYPES:
            raise ConfigError(f"config.json: {where}`type` {kind!r} is not one of {list(MIXER_TYPES)}")
        m = _obj(raw, "mixer", where)
        mixer: Dict[str, Any] = {"heads": _int(m, "heads", where), "dim": _int(m, "dim", where), "vdim": _int(m, "vdim", where),
                                 "scale": _num(m, "scale", where)}
        if kind == "attention":
            mixer["kv_heads"] = _int(m, "kv_heads", where)
            if mixer["heads"] % mixer["kv_heads"] != 0:
                raise ConfigError(f"config.json: {where}{mixer['heads']} heads cannot share {mixer['kv_heads']} kv heads evenly")
            mask = _obj(m, "mask", where, needed=False)
            mixer["mask"] = {"size": _int(mask, "size", where + "mask: ")} if mask is not None else None
            mixer["rot"] = _rot(m, where, mixer["dim"])
        else:
            mixer["kv_rank"], mixer["rot_dim"] = _int(m, "kv_rank", where), _int(m, "rot_dim", where, 0)
            mixer["rot"] = _rot(m, where, mixer["rot_dim"]) if mixer["rot_dim"] else None
            mixer["kv_from"] = None
            if m.get("kv_from") is not None:
                mixer["kv_from"] = _int(m, "kv_from", where, 0)
                if mixer["kv_from"] >= index:
                    raise ConfigError(f"config.json: {where}`kv_from` {mixer['kv_from']} must name an earlier layer")
        mlp = raw.get("mlp")
        if mlp is not None:
            if not isinstance(mlp, dict):
                raise ConfigError(f"config.json: {where}`mlp` must be an object or null")
            if mlp.get("kind") != "moe":
                raise ConfigError(f"config.json: {where}`mlp.kind` {mlp.get('kind')!r} is not supported (moe)")
            expert, router = _obj(mlp, "expert", where + "mlp: "), _obj(mlp, "router", where + "mlp: ")
            shared = _obj(mlp, "shared", where + "mlp: ", needed=False)
            mlp = {"kind": "moe", "expert": {"ff": _int(expert, "ff", where + "mlp.expert: ")},
                   "router": {"experts": _int(router, "experts", where + "mlp.router: "), "top": _int(router, "top", where + "mlp.router: ")},
                   "shared": {"ff": _int(shared, "ff", where + "mlp.shared: ")} if shared is not None else None}
            if mlp["router"]["top"] > mlp["router"]["experts"]:
                raise ConfigError(f"config.json: {where}`mlp.router.top` exceeds `mlp.router.experts`")
        return cls(kind, mixer, mlp)

    def to_json_dict(self) -> Dict[str, Any]:
        m = {k: v for k, v in self.mixer.items() if k not in ("mask", "rot", "kv_from")}
        if self.mixer.get("mask") is not None:
            m["mask"] = dict(self.mixer["mask"])
        if self.mixer.get("rot") is not None:
            m["rot"] = _rot_json(self.mixer["rot"])
        if self.mixer.get("kv_from") is not None:
            m["kv_from"] = self.mixer["kv_from"]
        mlp = None
        if self.mlp is not None:
            mlp = {"kind": "moe", "expert": dict(self.mlp["expert"]), "router": dict(self.mlp["router"])}
            if self.mlp["shared"] is not None:
                mlp["shared"] = dict(self.mlp["shared"])
        return {"type": self.type, "mixer": m, "mlp": mlp}


@dataclass
class NirotarConfig(ModelConfig):
    layers: List[NirotarLayer] = field(default_factory=list)
    norm_eps: float = 0.0

    ARCHITECTURE = "Nirotar"
    MODEL_TYPE = "nirotar"

    @classmethod
    def from_dict(cls, raw: Dict[str, Any], generation: Optional[Dict[str, Any]] = None) -> "NirotarConfig":
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: `layers` must be a non-empty list")
        layers = [NirotarLayer.parse(layer, i) for i, layer in enumerate(layers_raw)]
        for i, layer in enumerate(layers):
            src = layer.mixer.get("kv_from")
            if src is None:
                continue
            other = layers[src]
            if other.type != "latent_attention" or other.mixer.get("kv_from") is not None:
                raise ConfigError(f"config.json: layers[{i}]: `kv_from` {src} must name a latent-attention layer that keeps its own latent")
            for key in ("kv_rank", "rot_dim", "rot"):
                if other.mixer[key] != layer.mixer[key]:
                    raise ConfigError(f"config.json: layers[{i}]: `{key}` differs from layer {src}'s, whose latent it reads")
        norm = _obj(raw, "norm", "")
        eos = eos_ids(raw.get("eos_token_id"))
        if generation is not None and generation.get("eos_token_id") is not None:
            eos = eos_ids(generation.get("eos_token_id"))
        return cls(architecture=cls.ARCHITECTURE, model_type=cls.MODEL_TYPE, vocab_size=_int(raw, "vocab", ""),
                   hidden_size=_int(raw, "width", ""),
                   max_position_embeddings=optional(raw, "max_positions", int, DEFAULT_MAX_POSITIONS),
                   eos_token_ids=eos, raw=dict(raw), layers=layers, norm_eps=_num(norm, "eps", "norm: "))

    def to_json_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": self.ARCHITECTURE, "vocab": self.vocab_size, "width": self.hidden_size,
                               "norm": {"eps": self.norm_eps}, "layers": [layer.to_json_dict() for layer in self.layers]}
        if self.max_position_embeddings != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_position_embeddings
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out
