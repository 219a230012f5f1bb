"""Configuration of the Vogunex decoder: a list of layers, each with one of three mixers (grouped-query attention over a
window of single positions and pooled blocks before it; attention over a latent that keys and values share, with queries
through a latent of their own; a selective state space layer), a dense or routed feed-forward, a token shift in front of
every mixer, the embedding's scale and the norm's eps.  A layer may name another layer whose weights it uses
(``weights_of``); it then brings no tensors and keeps a cache or state of its own.

Every size and constant comes from ``config.json``; what a part needs is checked here, so that a folder with a missing or
mistyped key is refused before any weight is read.  Optional keys switch a mechanism off when they are absent: no ``mask``
(every earlier position is seen), no ``mask.pool`` (nothing before the window is seen), no ``rot``, no ``softcap``, no
``mlp.shared``, ``mlp`` null.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .base import ConfigError, ModelConfig, eos_ids, optional
from .fegarax import DEFAULT_MAX_POSITIONS, _int, _num, _obj

MIXER_TYPES = ("attention", "latent_attention", "mamba2")
MLP_KINDS = ("dense", "moe")


def _rot(m: Dict[str, Any], where: str, width: int) -> Optional[Dict[str, Any]]:
    rot = _obj(m, "rot", where, needed=False)
    if rot is None:
        return None
    r = {"base": _num(rot, "base", where + "rot: ", True), "dims": _int(rot, "dims", where + "rot: ", 2)}
    if r["dims"] % 2 or r["dims"] > width:
        raise ConfigError(f"config.json: {where}`rot.dims` {r['dims']} must be even and at most {width}")
    return r


def _mask(m: Dict[str, Any], where: str, pooled: bool) -> Optional[Dict[str, Any]]:
    mask = _obj(m, "mask", where, needed=False)
    if mask is None:
        return None
    out: Dict[str, Any] = {"size": _int(mask, "size", where + "mask: ")}
    if pooled and mask.get("pool") is not None:
        out["pool"] = _int(mask, "pool", where + "mask: ")
    return out


def _mixer(kind: str, m: Dict[str, Any], where: str) -> Dict[str, Any]:
    if kind == "mamba2":
        out = {k: _int(m, k, where) for k in ("heads", "vdim", "state", "groups", "conv", "norm_groups")}
        if out["heads"] % out["groups"] != 0:
            raise ConfigError(f"config.json: {where}{out['heads']} heads cannot share {out['groups']} groups evenly")
        if (out["heads"] * out["vdim"]) % out["norm_groups"] != 0:
            raise ConfigError(f"config.json: {where}`norm_groups` {out['norm_groups']} does not divide heads * vdim")
        return out
    out = {"heads": _int(m, "heads", where), "dim": _int(m, "dim", where), "vdim": _int(m, "vdim", where), "scale": _num(m, "scale", where)}
    if kind == "attention":
        out["kv_heads"] = _int(m, "kv_heads", where)
        if out["heads"] % out["kv_heads"] != 0:
            raise ConfigError(f"config.json: {where}{out['heads']} heads cannot share {out['kv_heads']} kv heads evenly")
        out["mask"] = _mask(m, where, True)
        out["rot"] = _rot(m, where, out["dim"])
        out["softcap"] = _num(m, "softcap", where, True) if m.get("softcap") is not None else None
    else:
        out["kv_rank"], out["q_rank"], out["rot_dim"] = _int(m, "kv_rank", where), _int(m, "q_rank", where), _int(m, "rot_dim", where, 0)
        out["mask"] = _mask(m, where, False)
        out["rot"] = _rot(m, where, out["rot_dim"]) if out["rot_dim"] else None
        if out["rot"] is not None and out["rot"]["dims"] != out["rot_dim"]:
            raise ConfigError(f"config.json: {where}`rot.dims` must equal `rot_dim`: the whole rotated part turns")
    return out


def _expert(raw: Dict[str, Any], where: str) -> Dict[str, Any]:
    return {"ff": _int(raw, "ff", where), "limit": _num(raw, "limit", where, True)}


def _mlp(mlp: Any, where: str) -> Optional[Dict[str, Any]]:
    if mlp is None:
        return None
    if not isinstance(mlp, dict):
        raise ConfigError(f"config.json: {where}`mlp` must be an object or null")
    kind = mlp.get("kind")
    if kind not in MLP_KINDS:
        raise ConfigError(f"config.json: {where}`mlp.kind` {kind!r} is not one of {list(MLP_KINDS)}")
    if kind == "dense":
        return {"kind": "dense", "ff": _int(mlp, "ff", where + "mlp: ")}
    router = _obj(mlp, "router", where + "mlp: ")
    shared = _obj(mlp, "shared", where + "mlp: ", needed=False)
    out = {"kind": "moe", "expert": _expert(_obj(mlp, "expert", where + "mlp: "), where + "mlp.expert: "),
           "router": {"experts": _int(router, "experts", where + "mlp.router: "), "top": _int(router, "top", where + "mlp.router: ")},
           "shared": _expert(shared, where + "mlp.shared: ") if shared is not None else None}
    if out["router"]["top"] > out["router"]["experts"]:
        raise ConfigError(f"config.json: {where}`mlp.router.top` exceeds `mlp.router.experts`")
    return out


@dataclass
class VogunexLayer:
    type: str
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]]
    weights_of: Optional[int] = None

    @classmethod
    def parse(cls, raw: Any, index: int) -> "VogunexLayer":
        where = f"layers[{index}]: "
        if not isinstance(raw, dict):
            raise ConfigError(f"config.json: {where}must be an object")
        kind = raw.get("type")
        if kind not in MIXER_TYPES:
            raise ConfigError(f"config.json: {where}`type` {kind!r} is not one of {list(MIXER_TYPES)}")
        source = None
        if raw.get("weights_of") is not None:
            source = _int(raw, "weights_of", where, 0)
        return cls(kind, _mixer(kind, _obj(raw, "mixer", where), where), _mlp(raw.get("mlp"), where), source)

    def to_json_dict(self) -> Dict[str, Any]:
        m = {k: (dict(v) if isinstance(v, dict) else v) for k, v in self.mixer.items() if v is not None}
        mlp = None
        if self.mlp is not None:
            mlp = {k: (dict(v) if isinstance(v, dict) else v) for k, v in self.mlp.items() if v is not None}
        out: Dict[str, Any] = {"type": self.type, "mixer": m, "mlp": mlp}
        if self.weights_of is not None:
            out["weights_of"] = self.weights_of
        return out


@dataclass
class VogunexConfig(ModelConfig):
    layers: List[VogunexLayer] = field(default_factory=list)
    norm_eps: float = 0.0
    embedding_scale: float = 1.0

    ARCHITECTURE = "Vogunex"
    MODEL_TYPE = "vogunex"

    @classmethod
    def from_dict(cls, raw: Dict[str, Any], generation: Optional[Dict[str, Any]] = None) -> "VogunexConfig":
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: `layers` must be a non-empty list")
        layers = [VogunexLayer.parse(layer, i) for i, layer in enumerate(layers_raw)]
        for i, layer in enumerate(layers):
            j = layer.weights_of
            if j is None:
                continue
            if not 0 <= j < len(layers) or j == i or layers[j].weights_of is not None:
                raise ConfigError(f"config.json: layers[{i}]: `weights_of` {j} must name another layer that has weights of its own")
            if (layers[j].type, layers[j].mixer, layers[j].mlp) != (layer.type, layer.mixer, layer.mlp):
                raise ConfigError(f"config.json: layers[{i}]: differs from layer {j}, whose weights it uses")
        norm = _obj(raw, "norm", "")
        emb = _obj(raw, "embedding", "", needed=False)
        eos = eos_ids(raw.get("eos_token_id"))
        if generation is not None and generation.get("eos_token_id") is not None:
            eos = eos_ids(generation.get("eos_token_id"))
        return cls(architecture=cls.ARCHITECTURE, model_type=cls.MODEL_TYPE, vocab_size=_int(raw, "vocab", ""),
                   hidden_size=_int(raw, "width", ""),
                   max_position_embeddings=optional(raw, "max_positions", int, DEFAULT_MAX_POSITIONS),
                   eos_token_ids=eos, raw=dict(raw), layers=layers, norm_eps=_num(norm, "eps", "norm: "),
                   embedding_scale=_num(emb, "scale", "embedding: ") if emb is not None and emb.get("scale") is not None else 1.0)

    def to_json_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": self.ARCHITECTURE, "vocab": self.vocab_size, "width": self.hidden_size,
                               "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
                               "layers": [layer.to_json_dict() for layer in self.layers]}
        if self.max_position_embeddings != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_position_embeddings
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out
