"""Nirotar as data: pre-norm layers over one residual stream, each with one of two mixers and a feed-forward of experts.

* ``attention``: grouped-query softmax attention with neighbouring elements rotated in pairs (frequencies slowed by
  wavelength bands where ``rot.scaling`` is given), a sliding window and a learned sink per head.
* ``latent_attention``: attention over a latent that keys and values share, with one rotated key part for all heads and a
  learned sink; a layer with ``kv_from`` keeps nothing itself and reads an earlier layer's page rows.
* feed-forward: experts without a gate (the square of relu) named by a table over the token ids, each with weight
  ``1 / top``, and a shared expert of the same form that every token uses.

Tensor names: ``embed``, ``l<i>.norm1`` / ``norm2``, ``l<i>.mix.{q,k,v,o,sink}`` or ``l<i>.mix.{q,dkv,dkv.norm,uk,uv,o,sink}``,
``l<i>.mlp.table``, ``l<i>.mlp.e<j>.{up,down}``, ``l<i>.mlp.shared.{up,down}``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from typing import Optional

from ..config.nirotar import NirotarConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .registry import register_architecture

ATTENTION_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "sink": "sink"}
EXPERT_NAMES = {"table": "table", "up": "e{e}.up", "down": "e{e}.down", "shared_up": "shared.up", "shared_down": "shared.down"}


def _position(rot: Optional[dict], width: int) -> PartSpec:
    """The rotation of a part ``width`` wide: neighbouring elements in pairs, over its first ``rot.dims``."""
    if rot is None:
        return PartSpec("none", {})
    params = {"head_dim": width, "theta": rot["base"], "rotary_dim": rot["dims"], "interleaved": True}
    if rot["scaling"] is None:
        return PartSpec("rope", params)
    return PartSpec("rope_llama3", dict(params, **rot["scaling"]))


def build_spec(cfg: NirotarConfig) -> ModelSpec:
    h = cfg.hidden_size
    norm = PartSpec("rmsnorm", {"dim": h, "eps": cfg.norm_eps, "tensor": ""})
    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if layer.type == "attention":
            mixer = PartSpec("sink_attention", {
                "hidden": h, "heads": m["heads"], "kv_heads": m["kv_heads"], "head_dim": m["dim"], "v_head_dim": m["vdim"],
                "scale": m["scale"], "bias": False, "qk_norm": None, "position": _position(m["rot"], m["dim"]),
                "window": m["mask"]["size"] if m["mask"] is not None else None, "sink": "learned", "names": ATTENTION_NAMES})
            schedule.append(ScheduleEntry(i))
        else:
            mixer = PartSpec("latent_attention", {
                "hidden": h, "heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"], "v_head_dim": m["vdim"],
                "kv_rank": m["kv_rank"], "scale": m["scale"], "norm_eps": cfg.norm_eps, "position": _position(m["rot"], m["rot_dim"]),
                "sink": "learned", "own_latent": m["kv_from"] is None})
            schedule.append(ScheduleEntry(i, cache_of=m["kv_from"]))
        ffn = None
        if layer.mlp is not None:
            ffn = PartSpec("routed_experts", {
                "hidden": h, "intermediate": layer.mlp["expert"]["ff"], "experts": layer.mlp["router"]["experts"],
                "top": layer.mlp["router"]["top"], "router": "table", "vocab": cfg.vocab_size, "activation": "relu2",
                "weight_on": "output", "shared_intermediate": layer.mlp["shared"]["ff"] if layer.mlp["shared"] is not None else None,
                "names": EXPERT_NAMES})
        layers.append(LayerSpec(block="prenorm", norm=norm, mixer=mixer, feedforward=ffn, prefix=f"l{i}",
                                names={"norm1": "norm1", "mixer": "mix", "norm2": "norm2", "feedforward": "mlp"}))
    return ModelSpec(
        hidden_size=h,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("token_table", {"vocab": cfg.vocab_size, "hidden": h, "name": "embed", "tensor": "embed"}),
        final_norm=PartSpec("rmsnorm", {"dim": h, "eps": cfg.norm_eps, "name": "final.norm", "tensor": ""}),
        head=PartSpec("linear", {"vocab": cfg.vocab_size, "hidden": h, "name": "head", "tied": False, "tensor": "head"}),
        layers=layers,
        schedule=schedule,
    )


register_architecture(NirotarConfig.ARCHITECTURE, NirotarConfig.MODEL_TYPE, NirotarConfig, build_spec)
